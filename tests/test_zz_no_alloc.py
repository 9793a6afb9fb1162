"""GPU test of `fluxb_moe_scatter_gemm_static`, the entry point for callers that must not allocate.

Who needs it: a serving process that has handed all free device memory to its own pool at start-up
(a later cudaMalloc would fail or fragment the pool), or a latency-critical loop that cannot afford
the device-wide synchronisation an allocation may imply. Such a caller still owns its input and
output buffers; what it cannot provide on demand is the scratch workspace the grouped kernel needs
for its routing tables. This entry point keeps those tables in a fixed device array inside the
library and allocates nothing itself.

The test calls it through the C ABI twice in a row (the second call has fewer routed rows and a
different routing, so stale table contents of the first call would show) and compares each result
with the existing workspace-based entry point on the same inputs and with the CPU oracle, within
the 1e-2 relative tolerance the other bf16 tests use. It also checks that sizes beyond the built-in
capacity are rejected with a clear error. The file name sorts last so that a run that stops at the
first failure has already run every other test; it also passes when run alone in a fresh process.
"""
import ctypes as C
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from oracle import golden  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _case(ntokens, topk, nexperts, hidden, ffn, seed, skew):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(ntokens, nexperts, generator=g)
    if skew:
        logits[:, 1] = -1e9  # one expert without tokens
    chosen, _ = golden.topk_routing(logits, topk)
    si = golden.calc_scatter_index_stable(chosen)
    splits = golden.calc_splits(chosen, nexperts)
    tok = torch.randn(ntokens, hidden, generator=g).to(torch.bfloat16)
    w = (torch.randn(nexperts, ffn, hidden, generator=g) * 0.02).to(torch.bfloat16)
    scale = torch.rand(nexperts, generator=g) + 0.5
    return tok, w, splits, si, scale


def test_static_entry_point_matches_workspace_entry_point():
    import flux_b200 as flux
    from flux_b200 import _lib

    lib = _lib.load()
    flux.init_flux_shm(None)
    comm = flux.get_comm(None)
    comm.set_timeout_ms(5000)
    nexperts, hidden, ffn, topk = 8, 256, 384, 2
    env = flux.DistEnvTPWithEP(None, 1, None)
    ref_op = flux.GemmGroupedV3AGScatter(env, flux.MoeArguments(1024, hidden, ffn, nexperts, topk, torch.bfloat16))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (ntokens, seed, skew) in enumerate([(1024, 11, False), (384, 12, True)]):
        tok, w, splits, si, scale = _case(ntokens, topk, nexperts, hidden, ffn, seed, skew)
        d_tok, d_w, d_splits, d_si, d_scale = tok.cuda(), w.cuda(), splits.cuda(), si.cuda(), scale.cuda()
        out = torch.full((ntokens * topk, ffn), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.fluxb_moe_scatter_gemm_static(
            comm.handle, d_tok.data_ptr(), ntokens, hidden, d_w.data_ptr(), nexperts, ffn, topk, d_splits.data_ptr(),
            d_si.data_ptr(), d_scale.data_ptr(), out.data_ptr(), _lib.BF16, _lib.BF16, None, stream)
        assert rc == _lib.FLUXB_OK, _lib.last_error()
        expect = ref_op.forward(d_tok, d_w, d_splits, d_si, output_scale=d_scale)
        torch.cuda.synchronize()
        comm.check_status()
        assert not torch.isnan(out.float()).any(), f"call {call}: rows were left unwritten"
        assert golden.max_rel_err(out, expect) <= TOL, f"call {call}: differs from the workspace entry point"
        oracle, _ = golden.moe_ag_scatter_single([tok], w, splits, si, scale)
        assert golden.max_rel_err(out, oracle) <= TOL, f"call {call}: differs from the oracle"


def _call_static(lib, comm, d_tok, ntokens, hidden, d_w, nexperts, ffn, topk, d_splits, d_si, d_scale, out, in_dt, tuning=None):
    from flux_b200 import _lib

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.fluxb_moe_scatter_gemm_static(
        comm.handle, d_tok.data_ptr(), ntokens, hidden, d_w.data_ptr(), nexperts, ffn, topk, d_splits.data_ptr(),
        d_si.data_ptr(), d_scale.data_ptr(), out.data_ptr(), in_dt, _lib.BF16,
        C.byref(_lib.make_tuning(tuning)) if tuning else None, stream)
    assert rc == _lib.FLUXB_OK, _lib.last_error()


def test_static_entry_point_allocates_no_device_memory():
    """The property the entry point exists for, observed rather than read: the device's free memory
    (cudaMemGetInfo) is the same before and after the calls. The first call on a device does the one-time
    set-up (address look-up, kernel attributes), so the window opens after a warm call."""
    import flux_b200 as flux
    from flux_b200 import _lib

    lib = _lib.load()
    flux.init_flux_shm(None)
    comm = flux.get_comm(None)
    comm.set_timeout_ms(5000)
    nexperts, hidden, ffn, topk, ntokens = 8, 256, 384, 2, 512
    tok, w, splits, si, scale = _case(ntokens, topk, nexperts, hidden, ffn, 21, False)
    d = [t.cuda() for t in (tok, w, splits, si, scale)]
    out = torch.empty((ntokens * topk, ffn), dtype=torch.bfloat16, device="cuda")
    _call_static(lib, comm, d[0], ntokens, hidden, d[1], nexperts, ffn, topk, d[2], d[3], d[4], out, _lib.BF16)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        _call_static(lib, comm, d[0], ntokens, hidden, d[1], nexperts, ffn, topk, d[2], d[3], d[4], out, _lib.BF16)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    comm.check_status()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes across the calls"
    oracle, _ = golden.moe_ag_scatter_single([tok], w, splits, si, scale)
    assert golden.max_rel_err(out, oracle) <= TOL


def test_static_entry_point_fp8_and_cta_pairs():
    """e4m3 inputs, and the CTA-pair tile shape (256-row tiles whose second half may hold no rows)."""
    import flux_b200 as flux
    from flux_b200 import _lib

    lib = _lib.load()
    flux.init_flux_shm(None)
    comm = flux.get_comm(None)
    comm.set_timeout_ms(5000)
    nexperts, hidden, ffn, topk, ntokens = 4, 256, 256, 2, 160  # 320 routed rows over 4 experts: <= 128 rows for some
    tok, w, splits, si, scale = _case(ntokens, topk, nexperts, hidden, ffn, 31, False)
    out = torch.empty((ntokens * topk, ffn), dtype=torch.bfloat16, device="cuda")
    d = [t.cuda() for t in (tok, w, splits, si, scale)]
    oracle, _ = golden.moe_ag_scatter_single([tok], w, splits, si, scale)
    for cg in (1, 2):
        out.fill_(float("nan"))
        _call_static(lib, comm, d[0], ntokens, hidden, d[1], nexperts, ffn, topk, d[2], d[3], d[4], out, _lib.BF16,
                     tuning={"cta_group": cg})
        torch.cuda.synchronize()
        comm.check_status()
        assert not torch.isnan(out.float()).any(), f"cta_group {cg}: rows were left unwritten"
        assert golden.max_rel_err(out, oracle) <= TOL, f"cta_group {cg}"
    f8 = torch.float8_e4m3fn
    tok8, w8 = tok.to(f8), (w.float() * 16).to(f8)  # weights scaled into e4m3's normal range
    oracle8, _ = golden.moe_ag_scatter_single([tok8.to(torch.bfloat16)], w8.to(torch.bfloat16), splits, si, scale)
    out.fill_(float("nan"))
    _call_static(lib, comm, tok8.cuda(), ntokens, hidden, w8.cuda(), nexperts, ffn, topk, d[2], d[3], d[4], out, _lib.E4M3)
    torch.cuda.synchronize()
    comm.check_status()
    assert golden.max_rel_err(out, oracle8) <= 3e-2


def test_static_entry_point_rejects_oversized_problems():
    import flux_b200 as flux
    from flux_b200 import _lib

    lib = _lib.load()
    flux.init_flux_shm(None)
    comm = flux.get_comm(None)
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    too_many_rows = _lib.STATIC_MAX_ROWS // 2 + 1  # times topk = 2
    rc = lib.fluxb_moe_scatter_gemm_static(
        comm.handle, dummy.data_ptr(), too_many_rows, 64, dummy.data_ptr(), 8, 64, 2, dummy.data_ptr(),
        dummy.data_ptr(), None, dummy.data_ptr(), _lib.BF16, _lib.BF16, None, stream)
    assert rc == _lib.FLUXB_ERR_INVALID
    assert "capacity" in _lib.last_error()
    rc = lib.fluxb_moe_scatter_gemm_static(
        comm.handle, dummy.data_ptr(), 16, 64, dummy.data_ptr(), _lib.STATIC_MAX_EXPERTS + 1, 64, 2,
        dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), _lib.BF16, _lib.BF16, None, stream)
    assert rc == _lib.FLUXB_ERR_INVALID
    assert "capacity" in _lib.last_error()
