"""Wiring of the tensor-parallel layers (flux_b200/layers.py), checked on CPU.

The fused ops are replaced by stand-ins with the same call interface that compute through gloo and fp32
matmuls (the golden path of test/python/ag_gemm/test_ag_kernel.py:88-176 and
test/python/gemm_rs/test_gemm_rs.py:57-157), so what is tested here is which op a layer calls with which
operand in which layout, forward and backward, against an unsharded torch model.
"""
import torch
import torch.distributed as dist

from _dist import run_distributed


class FakeAG:
    """Interface of AGKernel.forward: all_gather(input) @ weight.T, or @ weight for a [K, N] weight."""

    def __init__(self, group, full_m, n_dim, k_dim, dtype):
        self.group, self.full_m, self.n_dim, self.k_dim = group, full_m, n_dim, k_dim

    def forward(self, input, weight, bias=None, transpose_weight=False, gathered_input=None):
        world = dist.get_world_size(self.group) if self.group is not None else 1
        if world > 1:
            full = torch.empty((input.shape[0] * world, input.shape[1]), dtype=input.dtype)
            dist.all_gather_into_tensor(full, input.contiguous(), group=self.group)
        else:
            full = input
        assert full.shape[0] <= self.full_m and full.shape[1] == self.k_dim
        if gathered_input is not None:
            gathered_input.copy_(full)
        w = weight if transpose_weight else weight.t()
        assert w.shape == (self.k_dim, self.n_dim)
        out = full.float() @ w.float()
        if bias is not None:
            out = out + bias.float()
        return out.to(input.dtype)


class FakeRS:
    """Interface of GemmRS.forward: reduce_scatter(input @ weight.T) over rows ([K_local, N] weight if transposed)."""

    def __init__(self, group, max_m, n_dim, dtype, transpose_weight=False):
        self.group, self.max_m, self.n_dim, self.transpose_weight = group, max_m, n_dim, transpose_weight

    def forward(self, input, weight):
        world = dist.get_world_size(self.group) if self.group is not None else 1
        w = weight if self.transpose_weight else weight.t()
        assert w.shape[1] == self.n_dim and input.shape[0] <= self.max_m
        part = (input.float() @ w.float()).contiguous()
        if world > 1:
            dist.all_reduce(part, group=self.group)
            rank = dist.get_rank(self.group)
            mpr = part.shape[0] // world
            part = part[rank * mpr:(rank + 1) * mpr]
        return part.to(input.dtype)


def _patch(layers):
    layers._make_ag = lambda group, full_m, n_dim, k_dim, dtype: FakeAG(group, full_m, n_dim, k_dim, dtype)
    layers._make_rs = lambda group, max_m, n_dim, dtype, transpose_weight=False: FakeRS(group, max_m, n_dim, dtype,
                                                                                        transpose_weight)


def _gather_rows(t, group, world):
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


def _mlp_case(rank, world, with_bias):
    from flux_b200 import layers

    _patch(layers)
    group = dist.group.WORLD if world > 1 else None
    hidden, ffn, tokens = 32, 64, 8 * world
    dtype = torch.float32
    torch.manual_seed(11 + rank)
    mlp = layers.TensorParallelMLP(hidden, ffn, tokens, group, bias=with_bias, dtype=dtype, device="cpu")
    if with_bias:
        with torch.no_grad():
            mlp.fc1.bias.normal_()
            mlp.fc2.bias.copy_(torch.arange(hidden, dtype=dtype) * 0.01)  # replicated: same on every rank
    x_shard = torch.randn(tokens // world, hidden, dtype=dtype, requires_grad=True)
    g_shard = torch.randn(tokens // world, hidden, dtype=dtype)
    y_shard = mlp(x_shard)
    (y_shard * g_shard).sum().backward()

    # unsharded reference with the full weights
    if world > 1:
        w1 = torch.cat(_gather_rows(mlp.fc1.weight.detach(), group, world), dim=0)              # [ffn, hidden]
        w2 = torch.cat(_gather_rows(mlp.fc2.weight.detach(), group, world), dim=1)              # [hidden, ffn]
        x = torch.cat(_gather_rows(x_shard.detach(), group, world), dim=0)
        g = torch.cat(_gather_rows(g_shard, group, world), dim=0)
        b1 = torch.cat(_gather_rows(mlp.fc1.bias.detach(), group, world), dim=0) if with_bias else None
    else:
        w1, w2, x, g = mlp.fc1.weight.detach(), mlp.fc2.weight.detach(), x_shard.detach(), g_shard
        b1 = mlp.fc1.bias.detach() if with_bias else None
    b2 = mlp.fc2.bias.detach() if with_bias else None
    w1 = w1.clone().requires_grad_(True)
    w2 = w2.clone().requires_grad_(True)
    x = x.clone().requires_grad_(True)
    h = x @ w1.t()
    if b1 is not None:
        b1 = b1.clone().requires_grad_(True)
        h = h + b1
    y = torch.nn.functional.gelu(h) @ w2.t()
    if b2 is not None:
        y = y + b2
    (y * g).sum().backward()
    mpr = tokens // world
    rows = slice(rank * mpr, (rank + 1) * mpr)
    fl = ffn // world
    cols = slice(rank * fl, (rank + 1) * fl)
    torch.testing.assert_close(y_shard.detach(), y.detach()[rows], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(x_shard.grad, x.grad[rows], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(mlp.fc1.weight.grad, w1.grad[cols], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(mlp.fc2.weight.grad, w2.grad[:, cols], rtol=1e-4, atol=1e-5)
    if with_bias:
        torch.testing.assert_close(mlp.fc1.bias.grad, b1.grad[cols], rtol=1e-4, atol=1e-5)
        # fc2's bias gradient is per token shard; summed over ranks it is the full gradient
        bg = mlp.fc2.bias.grad.clone()
        if world > 1:
            dist.all_reduce(bg, group=group)
        torch.testing.assert_close(bg, g.sum(dim=0), rtol=1e-4, atol=1e-5)
        assert mlp.fc2.bias.sequence_parallel


def test_tp_mlp_world2():
    run_distributed(_mlp_case, 2, False, use_cuda=False)


def test_tp_mlp_world2_bias():
    run_distributed(_mlp_case, 2, True, use_cuda=False)


def test_tp_mlp_world1():
    run_distributed(_mlp_case, 1, True, use_cuda=False)


def test_layer_argument_errors():
    import pytest
    from flux_b200 import layers

    class G:  # stands for a 2-rank group without initialising one
        pass

    old = layers._world
    layers._world = lambda group: 2
    try:
        with pytest.raises(RuntimeError):
            layers.ColumnParallelLinear(8, 7, 16, G(), device="cpu")
        with pytest.raises(RuntimeError):
            layers.RowParallelLinear(7, 8, 16, G(), device="cpu")
        with pytest.raises(RuntimeError):
            layers.MoEMLP(8, 7, 2, 1, 16, G(), device="cpu")
    finally:
        layers._world = old


class FakeL0:
    """Interface of GemmGroupedV3AGScatter.forward, computed by the oracle."""

    def __init__(self, group):
        self.group = group

    def forward(self, inputs_shard, weights, splits_gpu, scatter_index):
        from oracle import golden

        world = dist.get_world_size(self.group) if self.group is not None else 1
        shards = _gather_rows(inputs_shard, self.group, world) if world > 1 else [inputs_shard]
        out, _ = golden.moe_ag_scatter_single(shards, weights.detach(), splits_gpu, scatter_index)
        return out

    def forward_multiple_weights(self, inputs_shard, weights, splits_gpu, scatter_index):
        return [self.forward(inputs_shard, w, splits_gpu, scatter_index) for w in weights]


class FakeL1:
    """Interface of GemmGroupedV3GatherRS.forward_gather_rs, computed by the oracle."""

    def __init__(self, group, topk):
        self.group, self.topk = group, topk

    def forward_gather_rs(self, input, weight, splits_cpu, routing_idx, output_vec_scale=None):
        from oracle import golden

        si = routing_idx.view(-1, self.topk)
        if self.group is None:
            return golden.moe_gather_rs_single([input], [weight.detach()], splits_cpu, si, self.topk,
                                               output_vec_scales=[output_vec_scale])[0]
        return golden.moe_gather_rs_dist(self.group, input, weight.detach(), splits_cpu, si, self.topk,
                                         output_vec_scale=output_vec_scale)


def _moe_case(rank, world, gated=False):
    from flux_b200 import layers
    from oracle import golden

    group = dist.group.WORLD if world > 1 else None
    layers._scatter_index = lambda chosen, e: (golden.calc_scatter_index_stable(chosen), golden.calc_splits(chosen, e))
    layers._gather_index = golden.calc_gather_index
    layers._make_moe_l0 = lambda group, *a: FakeL0(group)
    layers._make_moe_l1 = lambda group, max_tokens, hidden, nexperts, topk, dtype: FakeL1(group, topk)
    hidden, ffn, nexperts, topk, tokens = 16, 24, 4, 2, 6 * world
    torch.manual_seed(5 + rank)
    blk = layers.MoEMLP(hidden, ffn, nexperts, topk, tokens, group, gated=gated, dtype=torch.float32, device="cpu")
    with torch.no_grad():
        g = torch.Generator().manual_seed(99)  # the router is replicated
        blk.router.copy_(torch.randn(nexperts, hidden, generator=g))
    x_shard = torch.randn(tokens // world, hidden)
    y_shard = blk(x_shard)

    if world > 1:
        x = torch.cat(_gather_rows(x_shard, group, world), dim=0)
        w_up = torch.cat(_gather_rows(blk.w_up.detach(), group, world), dim=1)      # [E, ffn, hidden]
        w_down = torch.cat(_gather_rows(blk.w_down.detach(), group, world), dim=2)  # [E, hidden, ffn]
        w_gate = torch.cat(_gather_rows(blk.w_gate.detach(), group, world), dim=1) if gated else None
    else:
        x, w_up, w_down = x_shard, blk.w_up.detach(), blk.w_down.detach()
        w_gate = blk.w_gate.detach() if gated else None
    logits = x @ blk.router.detach().t()
    top, chosen = torch.topk(logits, topk, dim=1)
    wts = torch.softmax(top, dim=1)
    ref = torch.zeros(tokens, hidden)
    for t in range(tokens):
        for k in range(topk):
            e = int(chosen[t, k])
            if gated:
                h = torch.nn.functional.silu(x[t] @ w_gate[e].t()) * (x[t] @ w_up[e].t())
            else:
                h = torch.nn.functional.gelu(x[t] @ w_up[e].t())
            ref[t] += wts[t, k] * (h @ w_down[e].t())
    mpr = tokens // world
    torch.testing.assert_close(y_shard, ref[rank * mpr:(rank + 1) * mpr], rtol=1e-4, atol=1e-5)


def test_moe_block_world2():
    run_distributed(_moe_case, 2, use_cuda=False)


def test_moe_block_world1():
    run_distributed(_moe_case, 1, use_cuda=False)


def test_moe_block_gated_world2():
    run_distributed(_moe_case, 2, True, use_cuda=False)


def _seq_first_case(rank, world):
    """Sequence-first [s, b, h] activations go through the same layers: flattening keeps the gather / scatter on
    the sequence axis."""
    from flux_b200 import layers

    _patch(layers)
    group = dist.group.WORLD
    hidden, ffn, seq, batch = 16, 32, 4 * world, 3
    torch.manual_seed(31 + rank)
    mlp = layers.TensorParallelMLP(hidden, ffn, seq * batch, group, dtype=torch.float32, device="cpu")
    x_shard = torch.randn(seq // world, batch, hidden)
    y_shard = mlp(x_shard)
    assert y_shard.shape == (seq // world, batch, hidden)
    h = mlp.fc1(x_shard)
    assert h.shape == (seq, batch, ffn // world)
    w1 = torch.cat(_gather_rows(mlp.fc1.weight.detach(), group, world), dim=0)
    w2 = torch.cat(_gather_rows(mlp.fc2.weight.detach(), group, world), dim=1)
    x = torch.cat(_gather_rows(x_shard, group, world), dim=0)  # [s, b, h]
    y = torch.nn.functional.gelu(x @ w1.t()) @ w2.t()
    sl = seq // world
    torch.testing.assert_close(y_shard.detach(), y[rank * sl:(rank + 1) * sl], rtol=1e-4, atol=1e-5)


def test_sequence_first_activations_world2():
    run_distributed(_seq_first_case, 2, use_cuda=False)
