"""Tensor-parallel layers (flux_b200/layers.py) on the GPU: forward and backward of the sequence-parallel MLP
and the forward of the MoE block against unsharded fp32 torch models built from the same bf16 parameters
(tolerance 1e-2 of the largest reference value for single GEMMs, 2e-2 for chained ones, as the reference's
own bf16 tests use: test/python/moe_gather_rs/test_moe_gather_rs.py:397-411)."""
import pytest
import torch

import dist_cases
from _dist import run_distributed
from conftest import gpu_count

pytestmark = pytest.mark.gpu


def _rel(x, ref):
    return float((x.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-12))


@pytest.mark.parametrize("with_bias", [False, True])
def test_tp_mlp_world1(with_bias):
    import flux_b200 as flux

    flux.init_flux_shm(None)
    hidden, ffn, tokens = 512, 1024, 384
    torch.manual_seed(3)
    mlp = flux.TensorParallelMLP(hidden, ffn, tokens, None, bias=with_bias)
    if with_bias:
        with torch.no_grad():
            mlp.fc1.bias.normal_(std=0.1)
            mlp.fc2.bias.normal_(std=0.1)
    x = torch.randn(tokens, hidden, device="cuda").bfloat16().requires_grad_(True)
    g = torch.randn(tokens, hidden, device="cuda").bfloat16()
    y = mlp(x)
    (y.float() * g.float()).sum().backward()
    torch.cuda.synchronize()
    flux.get_comm(None).check_status()

    w1 = mlp.fc1.weight.detach().float().requires_grad_(True)
    w2 = mlp.fc2.weight.detach().float().requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    h = xr @ w1.t()
    if with_bias:
        h = h + mlp.fc1.bias.detach().float()
    yr = torch.nn.functional.gelu(h.bfloat16().float()) @ w2.t()
    if with_bias:
        yr = yr + mlp.fc2.bias.detach().float()
    (yr * g.float()).sum().backward()
    assert y.shape == (tokens, hidden) and y.dtype == torch.bfloat16
    assert _rel(y, yr) <= 2e-2
    assert _rel(x.grad, xr.grad) <= 2e-2
    assert _rel(mlp.fc1.weight.grad, w1.grad) <= 2e-2
    assert _rel(mlp.fc2.weight.grad, w2.grad) <= 2e-2


@pytest.mark.parametrize("gated", [False, True])
def test_moe_block_world1(gated):
    import flux_b200 as flux

    flux.init_flux_shm(None)
    hidden, ffn, nexperts, topk, tokens = 512, 1024, 4, 2, 256
    torch.manual_seed(4)
    blk = flux.MoEMLP(hidden, ffn, nexperts, topk, tokens, None, gated=gated)
    x = torch.randn(tokens, hidden, device="cuda").bfloat16()
    y = blk(x)
    torch.cuda.synchronize()
    flux.get_comm(None).check_status()
    chosen, wts = blk.route(x)
    ref = torch.zeros(tokens, hidden, device="cuda")
    for e in range(nexperts):
        for k in range(topk):
            rows = (chosen[:, k] == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            up = (x[rows].float() @ blk.w_up[e].detach().float().t()).bfloat16()
            if gated:
                gate = (x[rows].float() @ blk.w_gate[e].detach().float().t()).bfloat16()
                h = (torch.nn.functional.silu(gate) * up).float()
            else:
                h = torch.nn.functional.gelu(up).float()
            ref[rows] += wts[rows, k:k + 1] * (h @ blk.w_down[e].detach().float().t())
    assert y.shape == (tokens, hidden)
    assert _rel(y, ref) <= 2e-2


def test_tp_mlp_multi_rank():
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    w = min(gpu_count(), 8)
    w = 1 << (w.bit_length() - 1)
    run_distributed(dist_cases.tp_mlp_case, w)


def test_profiling_records_a_tuning():
    """`profiling()` sweeps the tile shapes, returns a correct output and leaves a record that later
    `forward` calls of the same shape pick up (src/ag_gemm/ths_op/all_gather_gemm_op.cc:361-474)."""
    import flux_b200 as flux
    from flux_b200 import tune
    from oracle import golden

    flux.init_flux_shm(None)
    m, n, k = 512, 768, 1024
    g = torch.Generator().manual_seed(8)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    ref, _ = golden.ag_gemm_single([a], b)
    ctx = flux.ProfilingContext("ag_gemm")
    try:
        ag = flux.AGKernel(None, 1, m, n, k, torch.bfloat16)
        out = ag.profiling(a.cuda(), b.cuda(), prof_ctx=ctx)
        torch.cuda.synchronize()
        assert golden.max_rel_err(out, ref) <= 1e-2
        key = tune.record_key("ag_gemm", m, n, k, torch.bfloat16, 1)
        rec = ctx.get_latest_record()
        assert key in tune.TABLE.records and rec.key == key and repr(rec).startswith(f"fluxb_tuning[{key}]")
        assert ctx.get_latest_prof_result().startswith(key) and " * TopK=1" in ctx.get_latest_prof_result()
        # a record travels: forget it, load it again, and forward() picks it up
        tune.TABLE.records.clear()
        flux.load_tuning_record(rec)
        assert tune.TABLE.get(key) == rec.tuning
        out2 = ag.forward(a.cuda(), b.cuda())
        torch.cuda.synchronize()
        assert golden.max_rel_err(out2, ref) <= 1e-2
        rs = flux.GemmRS(None, 1, m, n, torch.bfloat16)
        out3 = rs.profiling(a.cuda(), b.cuda(), prof_ctx=ctx)
        torch.cuda.synchronize()
        assert golden.max_rel_err(out3, ref) <= 1e-2 and len(ctx.get_all_record_codes()) == 2
        assert len(ctx.get_all_records()) == 2 and len(ctx.get_all_prof_results()) == 2
    finally:
        tune.TABLE.records.clear()


@pytest.mark.parametrize("transpose_weight", [False, True])
def test_gemm_only_op(transpose_weight):
    """`flux.GemmOnly` (python/flux/cpp_mod.pyi:215-253): plain GEMM with [N,K] or [K,N] weights and a [1,N] bias."""
    import flux_b200 as flux
    from oracle import golden

    flux.init_flux_shm(None)
    m, n, k = 384, 640, 512
    g = torch.Generator().manual_seed(12)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    bias = (torch.randn(1, n, generator=g) * 0.1).bfloat16()
    ref, _ = golden.ag_gemm_single([a], b, bias=bias)
    op = flux.GemmOnly(torch.bfloat16, transpose_weight=transpose_weight)
    w = b.t().contiguous().cuda() if transpose_weight else b.cuda()
    out = op.forward(a.cuda(), w, bias=bias.cuda())
    torch.cuda.synchronize()
    op.comm.check_status()
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    assert golden.max_rel_err(out, ref) <= 1e-2
