"""GPU tests of the runtime surface: the all-rank barrier, symmetric tensor lists, and failure detection.

Failure detection is tested without faulting anything: a wait whose flag nobody sets is given a 200-300 ms
budget; the kernel gives up, writes its code into the host-mapped status word and RETURNS; the host reads the
code, clears it, re-arms the op and carries on in the same context. (The reference's waits are unbounded:
include/flux/cuda/system_barrier.hpp:66-103, src/cuda/cudaipc_barrier_all.cu:55-61.)"""
import ctypes as C
import os
import sys
import time

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from ranks_on_gpu import Ranks, _p, _stream  # noqa: E402

from oracle import golden  # noqa: E402

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def flux():
    import flux_b200

    flux_b200.init_flux_shm(None)
    flux_b200.get_comm(None).set_timeout_ms(5000)
    return flux_b200


def test_group_barrier_world1(flux):
    """reference test: test/python/util/test_flux_ring_barrier.py (barrier_all on a stream, repeated)."""
    gb = flux.GroupBarrier(None)
    for _ in range(5):
        gb.barrier_all()
    side = torch.cuda.Stream()
    gb.barrier_all(side.cuda_stream)
    torch.cuda.synchronize()
    comm = flux.get_comm(None)
    assert comm.status() == 0


def test_create_tensor_list_world1(flux):
    ts = flux.flux_create_tensor_list((3, 5), torch.float32, None)
    assert len(ts) == 1 and ts[0].shape == (3, 5) and ts[0].dtype == torch.float32 and ts[0].is_cuda
    assert float(ts[0].abs().sum()) == 0.0  # symmetric memory starts zeroed
    ts[0].fill_(2.0)
    assert float(ts[0].sum()) == 30.0
    tb = flux.create_tensor_list((7,), torch.bfloat16, None, init_zero=True)
    assert tb[0].numel() == 7


def test_tensor_list_and_barrier_multi_rank():
    from conftest import gpu_count
    import dist_cases
    from _dist import run_distributed

    w = min(gpu_count(), 8)
    if w < 2:
        pytest.skip("needs >= 2 GPUs")
    run_distributed(dist_cases.runtime_case, 1 << (w.bit_length() - 1))


def _status(lib, h):
    s = C.c_int(-1)
    assert lib.fluxb_status_peek(h, C.byref(s)) == 0
    return s.value


def test_barrier_wait_runs_out_and_context_survives(flux):
    """A 2-rank barrier whose peer never arrives: the kernel returns after its budget with status 6."""
    from flux_b200 import _lib

    lib = _lib.load()
    h = C.c_void_p()
    _lib.check(lib.fluxb_comm_create(0, 2, C.byref(h)))
    try:
        _lib.check(lib.fluxb_comm_set_timeout_ms(h, 200))
        sync = [torch.zeros(2 * _lib.MAX_WORLD, dtype=torch.int32, device="cuda") for _ in range(2)]
        table = _lib.ptr_table([t.data_ptr() for t in sync])
        t0 = time.perf_counter()
        _lib.check(lib.fluxb_barrier_all(h, table, _stream()))
        torch.cuda.synchronize()  # returns: the wait is bounded
        waited = time.perf_counter() - t0
        assert 0.15 <= waited < 5.0, waited
        assert _status(lib, h) == 6  # kStatusTimeoutBarrier
        assert int(sync[1][0]) == 1  # this rank did announce itself to the peer
        _lib.check(lib.fluxb_status_clear(h))
        assert _status(lib, h) == 0
        # now the "peer" arrives (its slot is written by hand): the next barrier, epoch 2, completes at once
        sync[0][1] = 2
        _lib.check(lib.fluxb_barrier_all(h, table, _stream()))
        torch.cuda.synchronize()
        assert _status(lib, h) == 0
    finally:
        lib.fluxb_comm_destroy(h)
    # the context is intact: one more GEMM through the normal communicator, checked against the oracle
    g = torch.Generator().manual_seed(3)
    a = torch.randn(256, 512, generator=g).to(BF16)
    b = (torch.randn(384, 512, generator=g) * 0.02).to(BF16)
    op = flux.AGKernel(None, 1, 256, 384, 512, BF16)
    out = op.gemm_only(a.cuda(), b.cuda())
    torch.cuda.synchronize()
    op.comm.check_status()
    assert golden.max_rel_err(out, golden.ag_gemm_single([a], b)[0]) <= 1e-2


@pytest.mark.parametrize("m_local", [128, 256])  # one CTA per tile / CTA pairs
def test_fused_kernel_flag_wait_runs_out_then_recovers(flux, m_local):
    """Rank 0 of a 2-rank AG-GEMM runs alone: its own shard's tiles finish, the tiles of the absent peer wait
    for arrival counters nobody bumps, the budget (300 ms) expires, every role leaves its loop, the CTAs free
    their tensor memory and the kernel returns with status 5. After `reset` on both ranks the same op handles
    run a complete 2-rank call (both ranks in one launch) and match the oracle."""
    from flux_b200 import _lib

    world, n, k = 2, 256, 512
    rk = Ranks(world, timeout_ms=300)
    lib = rk.lib
    try:
        ops = rk.ag_gemm_ops(m_local * world, n, k, BF16, BF16)
        g = torch.Generator().manual_seed(11)
        shards = [torch.randn(m_local, k, generator=g).to(BF16) for _ in range(world)]
        ws = [(torch.randn(n, k, generator=g) * 0.02).to(BF16) for _ in range(world)]
        d_sh, d_w = [s.cuda() for s in shards], [w.cuda() for w in ws]
        outs = [torch.zeros((m_local * world, n), dtype=BF16, device="cuda") for _ in range(world)]
        # ---- rank 0 alone, as an ordinary launch
        _lib.check(lib.fluxb_comm_set_ranks_on_gpu(rk.comms[0], 1))
        t0 = time.perf_counter()
        _lib.check(lib.fluxb_ag_gemm_forward(ops[0], _p(d_sh[0]), m_local, _p(d_w[0]), n, k, _p(outs[0]), None, 0, None,
                                             None, 1.0, 0, None, None, _stream()))
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 0.25 <= waited < 10.0, waited
        assert _status(lib, rk.comms[0]) == 5  # kStatusTimeoutFlag
        # the rows of rank 0's own shard were computed before the wait began
        ref0, _ = golden.ag_gemm_single(shards, ws[0])
        assert golden.max_rel_err(outs[0][:m_local], ref0[:m_local]) <= 1e-2
        # ---- recovery: clear the status, re-arm both ranks, run the full 2-rank call
        _lib.check(lib.fluxb_status_clear(rk.comms[0]))
        for r in range(world):
            _lib.check(lib.fluxb_ag_gemm_reset(ops[r], _stream()))
        torch.cuda.synchronize()
        _lib.check(lib.fluxb_comm_set_ranks_on_gpu(rk.comms[0], world))
        for call in range(2):
            rk.ag_gemm_forward(ops, d_sh, d_w, outs)
            for r in range(world):
                ref, _ = golden.ag_gemm_single(shards, ws[r])
                assert golden.max_rel_err(outs[r], ref) <= 1e-2, (call, r)
    finally:
        rk.close()
