"""MoE grouped ops with the reference's names and arguments.

  GemmGroupedV3AGScatter - src/pybind/gemm_grouped_v3_ag_scatter.cc:29-68
                           (GemmGroupedV3AGScatterOp, src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc)
  GemmGroupedV3GatherRS  - src/pybind/gemm_grouped_v3_gather_rs.cc:35-126
                           (src/moe_gather_rs/ths_op/gemm_grouped_v3_gather_rs.cc)
  calc_scatter_index     - src/pybind/ths_op.cc:59-76 (stable order here)
Tensor parallelism over the ffn dimension; with an `ep_group` the experts are additionally split over
`ep_size` groups of `world / ep_size` ranks (DistEnvTPWithEP, src/ths_op/ths_op.cc:334-346).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib
from . import tune as _tune
from .ops import (DistEnvTPWithEP, MoeArguments, _check, _cur_stream, _out_dtype, _profile, _ptr, _tuning,
                  is_fp8_dtype)
from .shm import SymmBuffer, default_comm, fluxb_dtype, get_comm


def calc_scatter_index(choosed_experts: torch.Tensor, splits: Optional[torch.Tensor] = None,
                       return_splits: bool = False):
    """`flux.calc_scatter_index(choosed_experts, splits)`: row of every (token, k) pair in the
    expert-sorted order. Stable (ties keep token order), i.e. the reference's
    `calc_scatter_index_stable` (python/flux/testing/moe_utils.py:141-144); the number of experts is
    taken from `splits`."""
    _check(choosed_experts.is_cuda and choosed_experts.dtype == torch.int32 and choosed_experts.dim() == 2,
           "calc_scatter_index: choosed_experts must be a CUDA int32 [ntokens, topk] tensor")
    ntokens, topk = choosed_experts.shape
    if splits is not None:
        nexperts = int(splits.numel())
    else:
        nexperts = int(choosed_experts.max().item()) + 1 if choosed_experts.numel() else 1
    chosen = choosed_experts.contiguous()
    out = torch.empty_like(chosen)
    counts = torch.empty(nexperts, dtype=torch.int32, device=chosen.device)
    _lib.check(_lib.load().fluxb_moe_scatter_index(chosen.data_ptr(), ntokens, topk, nexperts, counts.data_ptr(),
                                                   out.data_ptr(), _cur_stream()))
    return (out, counts) if return_splits else out


def calc_gather_index(scatter_index: torch.Tensor):
    """Inverse permutation of `scatter_index` [ntokens, topk]: (gather_index, topk_index), each
    [ntokens*topk] int32 (src/moe_ag_scatter/sort_util.cu:39-92)."""
    _check(scatter_index.is_cuda and scatter_index.dtype == torch.int32 and scatter_index.dim() == 2,
           "calc_gather_index: scatter_index must be a CUDA int32 [ntokens, topk] tensor")
    ntokens, topk = scatter_index.shape
    si = scatter_index.contiguous()
    gi = torch.empty(ntokens * topk, dtype=torch.int32, device=si.device)
    ti = torch.empty(ntokens * topk, dtype=torch.int32, device=si.device)
    _lib.check(_lib.load().fluxb_moe_gather_index(si.data_ptr(), ntokens, topk, gi.data_ptr(), ti.data_ptr(),
                                                  _cur_stream()))
    return gi, ti


class GemmGroupedV3AGScatter:
    """MoE layer 0: all-gather of the token shards + scatter to expert order + grouped GEMM.
    out[scatter_index[t, k], :] = token_t . W[expert(t,k)]^T * output_scale[expert]."""

    def __init__(self, tp_env: DistEnvTPWithEP, moe_args: MoeArguments):
        self.comm = get_comm(tp_env.tp_group)
        self.args = moe_args
        w = self.comm.world
        self.ep_rank, self.ep_size = int(tp_env.ep_rank), int(tp_env.ep_size)
        _check(w % self.ep_size == 0 and moe_args.nexperts % self.ep_size == 0,
               "GemmGroupedV3AGScatter: the EP size must divide the world size and the number of experts")
        ffn_tp = w // self.ep_size
        _check(moe_args.ffn_hidden % ffn_tp == 0, "GemmGroupedV3AGScatter: ffn_hidden must divide by the ffn TP size")
        self.ffn_local = moe_args.ffn_hidden // ffn_tp
        self.nexperts_local = moe_args.nexperts // self.ep_size
        self.input_dtype = moe_args.input_dtype
        self.output_dtype = torch.bfloat16 if is_fp8_dtype(moe_args.input_dtype) and moe_args.output_dtype == moe_args.input_dtype \
            else moe_args.output_dtype
        lib = _lib.load()
        in_dt = fluxb_dtype(self.input_dtype)
        self._gather = SymmBuffer(self.comm, lib.fluxb_ag_gemm_gather_bytes(moe_args.max_ntokens, moe_args.hidden, in_dt))
        self._flags = SymmBuffer(self.comm, lib.fluxb_ag_gemm_flag_bytes(moe_args.max_ntokens, w))
        self._ws = torch.zeros(lib.fluxb_moe_ag_scatter_workspace_bytes(moe_args.max_ntokens, moe_args.topk, moe_args.nexperts,
                                                                      moe_args.hidden, in_dt),
                               dtype=torch.uint8, device=self.comm.device)
        h = C.c_void_p()
        _lib.check(lib.fluxb_moe_ag_scatter_create(
            self.comm.handle, moe_args.max_ntokens, moe_args.hidden, self.ffn_local, moe_args.nexperts, moe_args.topk,
            in_dt, fluxb_dtype(self.output_dtype), self._gather.table(), self._flags.table(), self._ws.data_ptr(),
            C.byref(h)))
        self._h = h
        if self.ep_size > 1:
            _lib.check(lib.fluxb_moe_ag_scatter_set_ep(h, self.ep_rank, self.ep_size))
        self.comm.host_barrier()

    def __del__(self):
        try:
            _lib.load().fluxb_moe_ag_scatter_destroy(self._h)
        except Exception:
            pass

    def _one(self, inputs_shard, weights, splits_gpu, scatter_index, output_scale, outputs_buf, allgather_output,
             tuning, reuse):
        a = self.args
        w = self.comm.world
        # shape rules of src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc:239-265
        _check(weights.is_cuda and weights.dim() == 3 and weights.is_contiguous(), "weights must be a contiguous CUDA [E, ffn/TP, hidden] tensor")
        _check(weights.dtype == self.input_dtype, "weights dtype mismatch")
        _check(tuple(weights.shape) == (self.nexperts_local, self.ffn_local, a.hidden),
               f"weights shape {tuple(weights.shape)} != {(self.nexperts_local, self.ffn_local, a.hidden)}")
        _check(splits_gpu.is_cuda and splits_gpu.dtype == torch.int32 and splits_gpu.numel() >= a.nexperts,
               "splits_gpu must be a CUDA int32 tensor with at least nexperts entries")
        _check(scatter_index.is_cuda and scatter_index.dtype == torch.int32 and scatter_index.dim() == 2
               and scatter_index.shape[1] == a.topk and scatter_index.is_contiguous(),
               "scatter_index must be a contiguous CUDA int32 [ntokens, topk] tensor")
        ntokens = scatter_index.shape[0]
        _check(ntokens % w == 0 and ntokens <= a.max_ntokens, f"ntokens={ntokens} must divide by TP and be <= max_ntokens")
        nlocal = ntokens // w
        if not reuse:
            _check(inputs_shard.is_cuda and inputs_shard.is_contiguous() and inputs_shard.dtype == self.input_dtype
                   and tuple(inputs_shard.shape) == (nlocal, a.hidden),
                   f"inputs_shard must be a contiguous [{nlocal}, {a.hidden}] tensor")
        if output_scale is not None:
            _check(output_scale.dtype == torch.float32 and output_scale.numel() == self.nexperts_local
                   and output_scale.is_contiguous(), "output_scale must be a float32 tensor with one entry per local expert")
        rows = ntokens * a.topk
        if self.ep_size > 1:
            # only the rows of this rank's experts are produced; their number is a device value (the reference
            # reads the splits back on every call, gemm_grouped_v3_ag_scatter.cc:323-363): callers who know it
            # pass an `outputs_buf` of that many rows and no read-back happens
            if outputs_buf is not None:
                rows = min(rows, outputs_buf.shape[0])
            else:
                e0 = self.ep_rank * self.nexperts_local
                rows = int(splits_gpu[e0:e0 + self.nexperts_local].sum().item())
        if outputs_buf is None:
            outputs_buf = torch.empty((rows, self.ffn_local), dtype=self.output_dtype, device=weights.device)
        else:
            _check(outputs_buf.dtype == self.output_dtype and outputs_buf.is_contiguous() and outputs_buf.shape[0] >= rows
                   and outputs_buf.dim() == 2 and outputs_buf.shape[1] == self.ffn_local,
                   "outputs_buf has the wrong shape, dtype or layout")
        if allgather_output is not None:
            _check(tuple(allgather_output.shape) == (ntokens, a.hidden) and allgather_output.dtype == self.input_dtype
                   and allgather_output.is_contiguous(), "allgather_output has the wrong shape, dtype or layout")
        _lib.check(_lib.load().fluxb_moe_ag_scatter_forward(
            self._h, None if reuse else inputs_shard.data_ptr(), nlocal, weights.data_ptr(), splits_gpu.data_ptr(),
            scatter_index.data_ptr(), _ptr(output_scale), outputs_buf.data_ptr(), _ptr(allgather_output),
            _tuning(tuning), _cur_stream()))
        return outputs_buf[:rows]

    def forward(self, inputs_shard, weights, splits_gpu, scatter_index, output_scale=None, outputs_buf=None,
                allgather_output=None, fast_accum=False, sm_margin=0, tuning=None):
        if tuning is None and _tune.TABLE.records:
            tuning = _tune.TABLE.get(_tune.record_key("moe_ag_scatter", scatter_index.shape[0] * self.args.topk,
                                                      self.ffn_local, self.args.hidden, self.input_dtype, self.comm.world))
        return self._one(inputs_shard, weights, splits_gpu, scatter_index, output_scale, outputs_buf,
                         allgather_output, tuning, reuse=False)

    def forward_multiple_weights(self, inputs_shard, weights: Sequence[torch.Tensor], splits_gpu, scatter_index,
                                 output_scale: Optional[Sequence[torch.Tensor]] = None,
                                 outputs_buf: Optional[Sequence[torch.Tensor]] = None, allgather_output=None,
                                 fast_accum=False, sm_margin=0, tuning=None) -> List[torch.Tensor]:
        """Several weight groups over the same gathered tokens (SwiGLU gate/up): the all-gather runs once."""
        outs = []
        for i, wt in enumerate(weights):
            outs.append(self._one(
                inputs_shard, wt, splits_gpu, scatter_index,
                None if output_scale is None else output_scale[i],
                None if outputs_buf is None else outputs_buf[i],
                allgather_output if i == 0 else None, tuning, reuse=(i > 0)))
        return outs

    def clear_buffers(self):
        """`clear_buffers` of the reference op: clears the arrival counters of both buffer parities and restarts
        the parity sequence (the recovery call after a bounded wait expired; in normal operation the counters are
        cleared by the calls themselves). Collective; ends with a host barrier."""
        _lib.check(_lib.load().fluxb_moe_ag_scatter_reset(self._h, _cur_stream()))
        self.comm.host_barrier()

    def profiling(self, inputs_shard, weights, splits_gpu, scatter_index, output_scale=None, outputs_buf=None,
                  allgather_output=None, fast_accum=False, sm_margin=0, prof_ctx=None):
        """Sweep tile shapes and all-gather transports for this problem (every rank times every candidate, the
        slowest rank decides), remember the winner for later `forward` calls of the same shape and return its
        output (src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc:450-604)."""
        a = self.args
        key = _tune.record_key("moe_ag_scatter", scatter_index.shape[0] * a.topk, self.ffn_local, a.hidden,
                               self.input_dtype, self.comm.world)

        def run(t):
            return self.forward(inputs_shard, weights, splits_gpu, scatter_index, output_scale, outputs_buf,
                                allgather_output, tuning=t if t else {})

        return _profile(run, self.comm.group, key, prof_ctx)


class GemmGroupedV3GatherRS:
    """MoE layer 1: grouped GEMM + top-k gather/reduce + reduce-scatter over the token dimension.
    The constructor takes no process group (the reference relies on the global NVSHMEM state set up by
    `init_flux_shm`); it binds to the communicator of the last `init_flux_shm(pg)` call, whose rank
    and size must match the `rank` / `world_size` arguments."""

    def __init__(self, total_num_experts, max_m, n_dim, topk, rank, world_size, tp_world_size, ep_world_size,
                 max_input_groups=1, ep_in_dp=False, input_dtype=torch.bfloat16, output_dtype=None):
        _check(int(tp_world_size) * int(ep_world_size) == int(world_size),
               "GemmGroupedV3GatherRS: tp_world_size * ep_world_size must equal world_size")
        _check(not ep_in_dp, "GemmGroupedV3GatherRS: ep_in_dp is not built")
        self.ep_size = int(ep_world_size)
        self.ep_rank = int(rank) // int(tp_world_size)  # ranks of one ffn-TP group are consecutive
        self.comm = default_comm()
        _check(self.comm.rank == int(rank) and self.comm.world == int(world_size),
               f"GemmGroupedV3GatherRS: rank/world_size ({rank}/{world_size}) do not match the communicator of "
               f"init_flux_shm ({self.comm.rank}/{self.comm.world})")
        self.nexperts, self.max_m, self.n_dim, self.topk = int(total_num_experts), int(max_m), int(n_dim), int(topk)
        self.max_input_groups = int(max_input_groups)
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        lib = _lib.load()
        w = self.comm.world
        self._stage = SymmBuffer(self.comm, lib.fluxb_moe_gather_rs_stage_bytes(self.max_m, self.n_dim, self.topk, w))
        self._cnt = SymmBuffer(self.comm, lib.fluxb_moe_gather_rs_cnt_bytes(self.max_m, self.n_dim, self.topk, w))
        self._ws = torch.zeros(lib.fluxb_moe_gather_rs_workspace_bytes(self.max_m, self.n_dim, self.topk, self.nexperts),
                               dtype=torch.uint8, device=self.comm.device)
        h = C.c_void_p()
        _lib.check(lib.fluxb_moe_gather_rs_create(
            self.comm.handle, self.nexperts, self.max_m, self.n_dim, self.topk, fluxb_dtype(self.input_dtype),
            fluxb_dtype(self.output_dtype), self._stage.table(), self._cnt.table(), self._ws.data_ptr(), C.byref(h)))
        self._h = h
        if self.ep_size > 1:
            _check(self.nexperts % self.ep_size == 0, "GemmGroupedV3GatherRS: the EP size must divide the number of experts")
            _lib.check(lib.fluxb_moe_gather_rs_set_ep(h, self.ep_rank, self.ep_size))
        self.comm.host_barrier()

    def __del__(self):
        try:
            _lib.load().fluxb_moe_gather_rs_destroy(self._h)
        except Exception:
            pass

    def forward_gather_rs(self, input, weight, splits_cpu, routing_idx=None, n_tokens_per_rank=None, input_scale=None,
                          weight_scale=None, output_vec_scale=None, fast_accum=False, sm_margin=0,
                          with_stream_sync=False, scatter_idx=None, tuning=None):
        if routing_idx is None:
            routing_idx = scatter_idx  # keyword used by examples/moe.py:204-209
        _check(routing_idx is not None, "forward_gather_rs: routing_idx is required")
        # argument rules of src/moe_gather_rs/ths_op/gemm_grouped_v3_gather_rs.cc:632-676
        _check(input.is_cuda and input.dim() == 2 and input.is_contiguous() and input.dtype == self.input_dtype,
               "input must be a contiguous CUDA [M, K] tensor of the op's dtype")
        _check(weight.is_cuda and weight.dim() == 3 and weight.is_contiguous() and weight.dtype == self.input_dtype,
               "weight must be a contiguous CUDA [E, N, K] tensor of the op's dtype")
        m, k = input.shape
        e_local = self.nexperts // self.ep_size
        _check(tuple(weight.shape) == (e_local, self.n_dim, k), f"weight shape {tuple(weight.shape)} != {(e_local, self.n_dim, k)}")
        _check(not splits_cpu.is_cuda and splits_cpu.dtype == torch.int32 and splits_cpu.numel() >= self.nexperts,
               "splits_cpu must be a CPU int32 tensor with at least nexperts entries")
        # the reference's extra splits[E] slot counts dropped tokens (gemm_grouped_v3_gather_rs.cc:668-674)
        _check(splits_cpu.numel() == self.nexperts or int(splits_cpu[self.nexperts:].sum()) == 0,
               "forward_gather_rs: token dropping (a non-zero splits[E] slot) is not built")
        _check(routing_idx.is_cuda and routing_idx.dtype == torch.int32, "routing_idx must be a CUDA int32 tensor")
        rows_all = routing_idx.numel()  # ntokens * topk; with expert parallelism `input` holds this rank's experts' rows
        _check(rows_all % self.topk == 0 and rows_all <= self.max_m and (self.ep_size > 1 or rows_all == m),
               f"routing_idx has {rows_all} entries for M={m} rows (max_m={self.max_m}, topk={self.topk})")
        w = self.comm.world
        for name, s, numel in (("input_scale", input_scale, 1), ("weight_scale", weight_scale, e_local),
                               ("output_vec_scale", output_vec_scale, m)):
            if s is not None:
                _check(s.is_cuda and s.dtype == torch.float32 and s.numel() == numel and s.is_contiguous(),
                       f"{name} must be a contiguous CUDA float32 tensor with {numel} element(s)")
        ntokens = rows_all // self.topk
        out = torch.empty((ntokens // w, self.n_dim), dtype=self.output_dtype, device=input.device)
        splits = splits_cpu.contiguous()
        if tuning is None and _tune.TABLE.records:
            tuning = _tune.TABLE.get(_tune.record_key("moe_gather_rs", m, self.n_dim, k, self.input_dtype, w))
        _lib.check(_lib.load().fluxb_moe_gather_rs_forward_ep(
            self._h, input.data_ptr(), m, ntokens, k, weight.data_ptr(), splits.data_ptr(),
            routing_idx.contiguous().data_ptr(), _ptr(input_scale), _ptr(weight_scale), _ptr(output_vec_scale),
            out.data_ptr(), _tuning(tuning), _cur_stream()))
        if with_stream_sync:
            torch.cuda.current_stream().synchronize()
        return out

    forward_gather_rs_no_zerobuffer = forward_gather_rs

    def forward_gather_rs_multiple(self, inputs, weights, splits_cpu, routing_idx=None, n_tokens_per_rank=None,
                                   input_scales=None, weight_scales=None, output_vec_scales=None, fast_accum=False,
                                   sm_margin=0, with_stream_sync=False, scatter_idx=None):
        """Sum over several input groups (python/flux/testing/moe_gather_rs_utils.py:59-106)."""
        total = None
        for i, (x, wt) in enumerate(zip(inputs, weights)):
            o = self.forward_gather_rs(
                x, wt, splits_cpu, routing_idx, n_tokens_per_rank,
                None if input_scales is None else input_scales[i],
                None if weight_scales is None else weight_scales[i],
                None if output_vec_scales is None else output_vec_scales[i], scatter_idx=scatter_idx)
            total = o.float() if total is None else total + o.float()
        out = total.to(self.output_dtype)
        if with_stream_sync:
            torch.cuda.current_stream().synchronize()
        return out

    def ep_zero_buffer(self):
        """Clears the per-token-block arrival counters (the recovery call after a bounded wait expired).
        Collective; ends with a host barrier."""
        _lib.check(_lib.load().fluxb_moe_gather_rs_reset(self._h, _cur_stream()))
        self.comm.host_barrier()

    def profiling(self, input, weight, splits_cpu, routing_idx, *args, prof_ctx=None, **kwargs):
        """Sweep the tile shapes of the grouped GEMM for this problem; see `GemmGroupedV3AGScatter.profiling`
        (src/moe_gather_rs/ths_op/gemm_grouped_v3_gather_rs.cc:822-1040)."""
        key = _tune.record_key("moe_gather_rs", input.shape[0], self.n_dim, input.shape[1], self.input_dtype,
                               self.comm.world)

        def run(t):
            return self.forward_gather_rs(input, weight, splits_cpu, routing_idx, *args, tuning=t if t else {}, **kwargs)

        return _profile(run, self.comm.group, key, prof_ctx)
