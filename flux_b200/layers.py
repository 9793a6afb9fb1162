"""Tensor-parallel layers on top of the fused ops.

Megatron-style sequence-parallel linear layers and MLP blocks that call `AGKernel`, `GemmRS`,
`GemmGroupedV3AGScatter` and `GemmGroupedV3GatherRS` the way the reference's examples do
(examples/moe.py:141-211, examples/moe_flux_only.py:85-131, docs/moe_usage.md), so that a model
keeps its layer structure and only swaps the linear layers.

Layout (TP = size of the tensor-parallel group, activations are sharded along the token axis):

    ColumnParallelLinear   x_shard [M/TP, K]  ->  y [M, N/TP]     = all_gather(x_shard) @ W[N/TP, K].T
    RowParallelLinear      x [M, K/TP]        ->  y_shard [M/TP, N] = reduce_scatter(x @ W[N, K/TP].T)

The two ops are each other's transposes, so the backward passes use the same two kernels:

    ColumnParallelLinear   dx_shard = reduce_scatter(dy @ W)       GemmRS with the weight read as [K_local, N]
                           dW       = dy.T @ all_gather(x_shard)   the gathered input is kept from the forward
    RowParallelLinear      dx       = all_gather(dy_shard) @ W     AGKernel with the weight read as [K, N_local]
                           dW       = all_gather(dy_shard).T @ x   the gathered gradient comes out of the same call

Weight gradients are plain GEMMs (torch.matmul). The op objects own symmetric buffers and must be constructed
by every rank of the group in the same order; the backward ops are built at the first backward pass.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import moe as _moe
from . import ops as _ops
from .shm import get_comm


def _world(group) -> int:
    return dist.get_world_size(group) if group is not None and dist.is_initialized() else 1


# Factories of the fused ops. Tests replace them with CPU stand-ins of the same interface.
def _make_ag(group, full_m, n_dim, k_dim, dtype):
    return _ops.AGKernel(group, 1, full_m, n_dim, k_dim, dtype)


def _make_rs(group, max_m, n_dim, dtype, transpose_weight=False):
    return _ops.GemmRS(group, 1, max_m, n_dim, dtype, transpose_weight=transpose_weight)


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, bias, layer):
        need_w = weight.requires_grad
        gathered = None
        if need_w:
            gathered = torch.empty((x_shard.shape[0] * layer.world, x_shard.shape[1]), dtype=x_shard.dtype,
                                   device=x_shard.device)
        y = layer._ag().forward(x_shard.contiguous(), weight, bias=bias, gathered_input=gathered)
        ctx.layer = layer
        ctx.has_bias = bias is not None
        ctx.save_for_backward(gathered if need_w else None, weight)
        return y

    @staticmethod
    def backward(ctx, dy):
        gathered, weight = ctx.saved_tensors
        layer = ctx.layer
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # [M, N/TP] @ [N/TP, K] summed over ranks, rows scattered: the weight is the [K_local, N] operand
            dx = layer._rs_bwd().forward(dy, weight)
        if ctx.needs_input_grad[1]:
            dw = torch.matmul(dy.t(), gathered)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.sum(dim=0)
        return dx, dw, db, None


class ColumnParallelLinear(torch.nn.Module):
    """y[M, out_features/TP] = all_gather(x_shard)[M, in_features] @ W.T (+ bias), one fused kernel.

    `max_tokens` is the largest M (tokens over all ranks) the layer will see; it sizes the symmetric buffers.
    """

    def __init__(self, in_features: int, out_features: int, max_tokens: int, group=None, bias: bool = False,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        super().__init__()
        self.group = group
        self.world = _world(group)
        if out_features % self.world != 0:
            raise RuntimeError(f"ColumnParallelLinear: out_features={out_features} is not a multiple of TP={self.world}")
        self.in_features, self.out_features, self.max_tokens = int(in_features), int(out_features), int(max_tokens)
        self.out_local = self.out_features // self.world
        self.weight = torch.nn.Parameter(torch.empty((self.out_local, self.in_features), dtype=dtype, device=device))
        self.bias = torch.nn.Parameter(torch.zeros((self.out_local,), dtype=dtype, device=device)) if bias else None
        torch.nn.init.normal_(self.weight, std=0.02)
        self._fwd_op = None
        self._bwd_op = None

    def _ag(self):
        if self._fwd_op is None:
            self._fwd_op = _make_ag(self.group, self.max_tokens, self.out_local, self.in_features, self.weight.dtype)
        return self._fwd_op

    def _rs_bwd(self):
        if self._bwd_op is None:
            self._bwd_op = _make_rs(self.group, self.max_tokens, self.in_features, self.weight.dtype,
                                    transpose_weight=True)
        return self._bwd_op

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """`x_shard` is [tokens/TP, in_features] or sequence-first [s/TP, b, in_features] (the gather runs
        along the first axis, so the output is [s, b, out_features/TP])."""
        lead = x_shard.shape[:-1]
        y = _ColumnParallelFn.apply(x_shard.reshape(-1, x_shard.shape[-1]), self.weight, self.bias, self)
        return y if len(lead) == 1 else y.view(lead[0] * self.world, *lead[1:], y.shape[-1])


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, layer):
        y_shard = layer._rs().forward(x.contiguous(), weight)
        ctx.layer = layer
        ctx.save_for_backward(x, weight)
        return y_shard

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        layer = ctx.layer
        dy_shard = dy_shard.contiguous()
        need_w = ctx.needs_input_grad[1]
        gathered = None
        if need_w:
            gathered = torch.empty((dy_shard.shape[0] * layer.world, dy_shard.shape[1]), dtype=dy_shard.dtype,
                                   device=dy_shard.device)
        dx = dw = None
        if ctx.needs_input_grad[0] or need_w:
            # all_gather(dy_shard)[M, N] @ W[N, K/TP]: the weight is the [K, N_local] operand of the all-gather GEMM
            dx = layer._ag_bwd().forward(dy_shard, weight, transpose_weight=True, gathered_input=gathered)
        if need_w:
            dw = torch.matmul(gathered.t(), x)
        return (dx if ctx.needs_input_grad[0] else None), dw, None


class RowParallelLinear(torch.nn.Module):
    """y_shard[M/TP, out_features] = reduce_scatter(x[M, in_features/TP] @ W.T) (+ bias), one fused kernel.

    The bias is replicated and added to the scattered rows after the reduction; as with any sequence-parallel
    layer its gradient is a sum over the token shards, which the caller's gradient synchronisation has to
    all-reduce over the tensor-parallel group (`RowParallelLinear.bias.sequence_parallel` is set for that).
    """

    def __init__(self, in_features: int, out_features: int, max_tokens: int, group=None, bias: bool = False,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        super().__init__()
        self.group = group
        self.world = _world(group)
        if in_features % self.world != 0:
            raise RuntimeError(f"RowParallelLinear: in_features={in_features} is not a multiple of TP={self.world}")
        self.in_features, self.out_features, self.max_tokens = int(in_features), int(out_features), int(max_tokens)
        self.in_local = self.in_features // self.world
        self.weight = torch.nn.Parameter(torch.empty((self.out_features, self.in_local), dtype=dtype, device=device))
        torch.nn.init.normal_(self.weight, std=0.02)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros((self.out_features,), dtype=dtype, device=device))
            self.bias.sequence_parallel = True
        else:
            self.bias = None
        self._fwd_op = None
        self._bwd_op = None

    def _rs(self):
        if self._fwd_op is None:
            self._fwd_op = _make_rs(self.group, self.max_tokens, self.out_features, self.weight.dtype)
        return self._fwd_op

    def _ag_bwd(self):
        if self._bwd_op is None:
            self._bwd_op = _make_ag(self.group, self.max_tokens, self.in_local, self.out_features, self.weight.dtype)
        return self._bwd_op

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """`x` is [tokens, in_features/TP] or sequence-first [s, b, in_features/TP] (rows are scattered along
        the first axis: the output is [s/TP, b, out_features])."""
        lead = x.shape[:-1]
        y = _RowParallelFn.apply(x.reshape(-1, x.shape[-1]), self.weight, self)
        if len(lead) > 1:
            if lead[0] % self.world != 0:
                raise RuntimeError(f"RowParallelLinear: sequence length {lead[0]} is not a multiple of TP={self.world}")
            y = y.view(lead[0] // self.world, *lead[1:], y.shape[-1])
        return y if self.bias is None else y + self.bias


class TensorParallelMLP(torch.nn.Module):
    """Sequence-parallel MLP block: tokens sharded in, tokens sharded out.

    `x_shard [M/TP, hidden] -> fc1 (all-gather + GEMM) -> activation -> fc2 (GEMM + reduce-scatter) -> [M/TP, hidden]`;
    at TP=8 with hidden 12288 and ffn 49152 these are the two GEMMs of the dense benchmark.
    """

    def __init__(self, hidden: int, ffn_hidden: int, max_tokens: int, group=None, bias: bool = False,
                 activation: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        super().__init__()
        self.fc1 = ColumnParallelLinear(hidden, ffn_hidden, max_tokens, group, bias, dtype, device)
        self.fc2 = RowParallelLinear(ffn_hidden, hidden, max_tokens, group, bias, dtype, device)
        self.activation = activation if activation is not None else torch.nn.functional.gelu

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return self.fc2(self.activation(self.fc1(x_shard)))


# Routing helpers and grouped-op factories of the MoE block (replaced by CPU stand-ins in tests).
def _scatter_index(chosen, nexperts):
    splits = torch.empty(nexperts, dtype=torch.int32, device=chosen.device)
    return _moe.calc_scatter_index(chosen, splits, return_splits=True)


def _gather_index(scatter_index):
    return _moe.calc_gather_index(scatter_index)


def _make_moe_l0(group, max_tokens, hidden, ffn_hidden, nexperts, topk, dtype):
    env = _ops.DistEnvTPWithEP(group, 1, None)
    return _moe.GemmGroupedV3AGScatter(env, _ops.MoeArguments(max_tokens, hidden, ffn_hidden, nexperts, topk, dtype))


def _make_moe_l1(group, max_tokens, hidden, nexperts, topk, dtype):
    world = _world(group)
    rank = dist.get_rank(group) if world > 1 else 0
    get_comm(group)  # the op binds to the communicator of the most recent set-up call
    return _moe.GemmGroupedV3GatherRS(nexperts, max_tokens * topk, hidden, topk, rank, world, world, 1,
                                      input_dtype=dtype)


class MoEMLP(torch.nn.Module):
    """Tensor-parallel mixture-of-experts MLP (inference forward), tokens sharded in and out.

    Every expert's up projection is split along ffn (`w_up [E, ffn/TP, hidden]`) and its down projection along
    its input (`w_down [E, hidden, ffn/TP]`), as in examples/moe_flux_only.py:66-77. Per call:

      1. router: logits of this rank's tokens, top-k with softmax weights over the chosen experts; the choices
         and weights of all ranks are all-gathered (T x topk numbers) because the routing is global;
      2. `calc_scatter_index` / `calc_gather_index` give each (token, k) pair its row in expert order;
      3. layer 0: all-gather of the tokens + scatter + grouped GEMM in one kernel (`GemmGroupedV3AGScatter`);
      4. activation; with `gated=True` (SwiGLU-style) a second up projection `w_gate` runs over the same gathered
         tokens (`forward_multiple_weights`: the all-gather happens once) and the activation is
         `act(gate) * up`;
      5. layer 1: grouped GEMM + weighted top-k sum + reduce-scatter (`GemmGroupedV3GatherRS`), the routing
         weight of every row applied in fp32 through `output_vec_scale`.
    """

    def __init__(self, hidden: int, ffn_hidden: int, nexperts: int, topk: int, max_tokens: int, group=None,
                 activation: Optional[Callable[[torch.Tensor], torch.Tensor]] = None, gated: bool = False,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        super().__init__()
        self.group = group
        self.world = _world(group)
        if ffn_hidden % self.world != 0:
            raise RuntimeError(f"MoEMLP: ffn_hidden={ffn_hidden} is not a multiple of TP={self.world}")
        if max_tokens % self.world != 0:
            raise RuntimeError(f"MoEMLP: max_tokens={max_tokens} is not a multiple of TP={self.world}")
        self.hidden, self.ffn_hidden, self.nexperts, self.topk = int(hidden), int(ffn_hidden), int(nexperts), int(topk)
        self.max_tokens = int(max_tokens)
        ffn_local = self.ffn_hidden // self.world
        self.router = torch.nn.Parameter(torch.empty((self.nexperts, self.hidden), dtype=torch.float32, device=device))
        self.w_up = torch.nn.Parameter(torch.empty((self.nexperts, ffn_local, self.hidden), dtype=dtype, device=device))
        self.w_down = torch.nn.Parameter(torch.empty((self.nexperts, self.hidden, ffn_local), dtype=dtype, device=device))
        self.w_gate = None
        if gated:
            self.w_gate = torch.nn.Parameter(torch.empty((self.nexperts, ffn_local, self.hidden), dtype=dtype,
                                                         device=device))
        for w in (self.router, self.w_up, self.w_down, self.w_gate):
            if w is not None:
                torch.nn.init.normal_(w, std=0.02)
        if activation is None:
            activation = torch.nn.functional.silu if gated else torch.nn.functional.gelu
        self.activation = activation
        self._l0 = None
        self._l1 = None

    def route(self, x_shard: torch.Tensor):
        """(chosen experts [T, topk] int32, routing weights [T, topk] fp32) for the tokens of all ranks."""
        logits = x_shard.float() @ self.router.t()
        top_logits, chosen = torch.topk(logits, self.topk, dim=1)
        weights = torch.softmax(top_logits, dim=1)
        chosen = chosen.to(torch.int32)
        if self.world > 1:
            all_chosen = torch.empty((chosen.shape[0] * self.world, self.topk), dtype=chosen.dtype, device=chosen.device)
            all_weights = torch.empty((weights.shape[0] * self.world, self.topk), dtype=weights.dtype,
                                      device=weights.device)
            dist.all_gather_into_tensor(all_chosen, chosen.contiguous(), group=self.group)
            dist.all_gather_into_tensor(all_weights, weights.contiguous(), group=self.group)
            chosen, weights = all_chosen, all_weights
        return chosen, weights

    @torch.no_grad()
    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        if self._l0 is None:
            self._l0 = _make_moe_l0(self.group, self.max_tokens, self.hidden, self.ffn_hidden, self.nexperts, self.topk,
                                    self.w_up.dtype)
            self._l1 = _make_moe_l1(self.group, self.max_tokens, self.hidden, self.nexperts, self.topk,
                                    self.w_up.dtype)
        chosen, weights = self.route(x_shard)
        scatter_index, splits = _scatter_index(chosen, self.nexperts)
        gather_index, topk_index = _gather_index(scatter_index)
        # routing weight of every expert-sorted row
        row_scale = weights.reshape(-1)[gather_index.long() * self.topk + topk_index.long()].contiguous()
        if self.w_gate is None:
            act = self.activation(self._l0.forward(x_shard.contiguous(), self.w_up, splits, scatter_index))
        else:
            gate, up = self._l0.forward_multiple_weights(x_shard.contiguous(), [self.w_gate, self.w_up], splits,
                                                         scatter_index)
            act = self.activation(gate) * up
        return self._l1.forward_gather_rs(act, self.w_down, splits.cpu(), scatter_index.reshape(-1),
                                          output_vec_scale=row_scale)
