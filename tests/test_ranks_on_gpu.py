"""Multi-rank parity on ONE GPU: all ranks of a fused op run side by side in one cooperative launch
(`fluxb_run_ranks`), so the all-gather push, the arrival counters, the reduce-scatter push and the owner-side
sum run through the same device code as on n GPUs - on a machine that has a single one.

Small cases are checked against the CPU oracle in full; the BASELINE shapes (dense D0 / D1, fp8 F, MoE X, each
at their TP=8 per-rank sizes) are checked by fp64 dot products on sampled entries, rows of every source rank
included. Tolerances: max|x-ref| / max|ref| <= 1e-2 (bf16), 2e-2 (MoE layer 1), 3e-2 (fp8); and the reference
tests' elementwise |x-y| <= t + t*|y| with t = 1e-2 (AG bf16), 2e-2 (RS bf16), 3e-2 (fp8)
(test/python/ag_gemm/test_ag_kernel.py:610-616,765-785; test/python/gemm_rs/test_gemm_rs.py:588-599)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from ranks_on_gpu import Ranks, _stream  # noqa: E402

from oracle import golden  # noqa: E402

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _close(out, ref, tol_rel, tol_elem, what):
    err = golden.max_rel_err(out, ref)
    assert err <= tol_rel, f"{what}: max rel err {err}"
    assert golden.torch_allclose(out, ref, rtol=tol_elem, atol=tol_elem), f"{what}: elementwise {tol_elem} check failed"


def _cpu_inputs(rank, rows, n, k, dtype, seed):
    g = torch.Generator().manual_seed(seed + rank)
    a = torch.randn(rows, k, generator=g).to(dtype)
    b = (torch.randn(n, k, generator=g) * 0.02).to(dtype)
    return a, b


# transport of the all-gather: 1 = pushed by the kernel's communication warps in units of 32 rows (3: 64 rows,
# 4: 128 rows), 2 = copy engines
@pytest.mark.parametrize("ag_mode", [1, 2, 3, 4])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ag_gemm_all_ranks_on_one_gpu(world, ag_mode):
    shapes = [(256, 512, 512), (200, 264, 512), (128, 136, 512), (256, 512, 512), (37, 72, 512)]
    rk = Ranks(world)
    try:
        ops = rk.ag_gemm_ops(256 * world, 512, 512, BF16, BF16)
        for it, (m_local, n, k) in enumerate(shapes):
            ab = [_cpu_inputs(r, m_local, n, k, BF16, 1234 + 17 * it) for r in range(world)]
            shards = [a for a, _ in ab]
            biases = None
            if it == 1:
                g = torch.Generator().manual_seed(5)
                biases = [(torch.randn(m_local * world, n, generator=g) * 0.1).to(BF16) for _ in range(world)]
            outs = [torch.empty((m_local * world, n), dtype=BF16, device="cuda") for _ in range(world)]
            gathered = [torch.empty((m_local * world, k), dtype=BF16, device="cuda") for _ in range(world)]
            rk.ag_gemm_forward(ops, [a.cuda() for a in shards], [b.cuda() for _, b in ab], outs,
                               biases=[b.cuda() for b in biases] if biases else None,
                               bias_mode=1 if biases else 0, gathered=gathered, tuning={"ag_mode": ag_mode})
            for r in range(world):
                ref, ref_g = golden.ag_gemm_single(shards, ab[r][1], bias=biases[r] if biases else None)
                _close(outs[r], ref, 1e-2, 1e-2, f"AG-GEMM world {world} call {it} rank {r}")
                assert torch.equal(gathered[r].cpu().view(torch.int16), ref_g.view(torch.int16)), \
                    f"world {world} call {it} rank {r}: gathered input differs from all_gather"
    finally:
        rk.close()


@pytest.mark.parametrize("world,fp32_wire", [(2, False), (4, False), (8, False), (4, True)])
def test_gemm_rs_all_ranks_on_one_gpu(world, fp32_wire):
    from flux_b200 import _lib

    n = 520
    shapes = [(256 * world, n, 256), (128 * world, n, 512), (40 * world, n, 136), (256 * world, n, 256)]
    rk = Ranks(world)
    try:
        ops = rk.gemm_rs_ops(256 * world, n, BF16, BF16)
        for it, (m, _, k_local) in enumerate(shapes):
            ab = [_cpu_inputs(r, m, n, k_local, BF16, 4321 + 17 * it) for r in range(world)]
            biases = None
            if it == 1:
                g = torch.Generator().manual_seed(6)
                biases = [(torch.randn(m, n, generator=g) * 0.1).to(BF16) for _ in range(world)]
            outs = [torch.empty((m // world, n), dtype=BF16, device="cuda") for _ in range(world)]
            rk.gemm_rs_forward(ops, [a.cuda() for a, _ in ab], [b.cuda() for _, b in ab], outs,
                               biases=[b.cuda() for b in biases] if biases else None,
                               flags=_lib.RS_FP32_WIRE if fp32_wire else 0)
            refs = golden.gemm_rs_single([a for a, _ in ab], [b for _, b in ab], biases)
            for r in range(world):
                _close(outs[r], refs[r], 1e-2, 2e-2, f"GEMM-RS world {world} call {it} rank {r}")
    finally:
        rk.close()


@pytest.mark.parametrize("ag_mode", [1, 2])
def test_fp8_all_ranks_on_one_gpu(ag_mode):
    world, m_local, n, k = 4, 256, 392, 1024
    f8 = torch.float8_e4m3fn
    rk = Ranks(world)
    try:
        qa, sa, qb, sb = [], [], [], []
        for r in range(world):
            g = torch.Generator().manual_seed(555 + r)
            q, s = golden.quantize_fp8_rows(torch.randn(m_local, k, generator=g))
            qa.append(q), sa.append(s)
            q, s = golden.quantize_fp8_rows(torch.randn(n, k, generator=g) * 0.02)
            qb.append(q), sb.append(s)
        ops = rk.ag_gemm_ops(m_local * world, n, k, f8, BF16, with_scales=True)
        outs = [torch.empty((m_local * world, n), dtype=BF16, device="cuda") for _ in range(world)]
        for _ in range(2):  # both buffer parities
            rk.ag_gemm_forward(ops, [q.cuda() for q in qa], [q.cuda() for q in qb], outs,
                               scales_a=[s.cuda() for s in sa], scales_b=[s.cuda() for s in sb],
                               tuning={"ag_mode": ag_mode})
            for r in range(world):
                ref, _ = golden.ag_gemm_single(qa, qb[r], input_scales=sa, weight_scale=sb[r])
                _close(outs[r], ref, 3e-2, 3e-2, f"fp8 AG-GEMM rank {r}")
        # fp8 GEMM-RS: every rank holds [M, k] with per-row scales
        m = m_local * world
        qa2, sa2 = [], []
        for r in range(world):
            g = torch.Generator().manual_seed(777 + r)
            q, s = golden.quantize_fp8_rows(torch.randn(m, k, generator=g))
            qa2.append(q), sa2.append(s)
        rs = rk.gemm_rs_ops(m, n, f8, BF16)
        outs2 = [torch.empty((m_local, n), dtype=BF16, device="cuda") for _ in range(world)]
        rk.gemm_rs_forward(rs, [q.cuda() for q in qa2], [q.cuda() for q in qb], outs2,
                           scales_a=[s.cuda() for s in sa2], scales_b=[s.cuda() for s in sb])
        refs = golden.gemm_rs_single(qa2, qb, None, sa2, sb)
        for r in range(world):
            _close(outs2[r], refs[r], 3e-2, 3e-2, f"fp8 GEMM-RS rank {r}")
    finally:
        rk.close()


def _int8_inputs(world, m_rows, n, k, seed):
    xs, ws, sxs, sws = [], [], [], []
    for r in range(world):
        g = torch.Generator().manual_seed(seed + r)
        xs.append(torch.randint(-127, 128, (m_rows, k), generator=g, dtype=torch.int32).to(torch.int8))
        ws.append(torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int32).to(torch.int8))
        sxs.append(torch.rand(m_rows, 1, generator=g) * 0.01 + 0.001)
        sws.append(torch.rand(1, n, generator=g) * 0.01 + 0.001)
    return xs, ws, sxs, sws


@pytest.mark.parametrize("ag_mode", [1, 2])
def test_int8_ag_gemm_bitwise_all_ranks_on_one_gpu(ag_mode):
    """w8a8 AG-GEMM: int8 operands, int32 accumulation, per-row x per-channel dequantisation, bias [1,N]. The
    reference's test demands a bitwise match with its golden path (test/python/ag_gemm/test_ag_kernel.py:615)."""
    world, m_local, n, k = 4, 256, 392, 1024
    rk = Ranks(world)
    try:
        xs, ws, sxs, sws = _int8_inputs(world, m_local, n, k, 31)
        g = torch.Generator().manual_seed(9)
        biases = [(torch.randn(1, n, generator=g) * 0.5).to(BF16) for _ in range(world)]
        ops = rk.ag_gemm_ops(m_local * world, n, k, torch.int8, BF16, with_scales=True)
        outs = [torch.empty((m_local * world, n), dtype=BF16, device="cuda") for _ in range(world)]
        for with_bias in (False, True):
            rk.ag_gemm_forward(ops, [x.cuda() for x in xs], [w.cuda() for w in ws], outs,
                               biases=[b.cuda() for b in biases] if with_bias else None, bias_mode=2 if with_bias else 0,
                               scales_a=[s.reshape(-1).cuda() for s in sxs], scales_b=[s.reshape(-1).cuda() for s in sws],
                               tuning={"ag_mode": ag_mode})
            for r in range(world):
                ref, _ = golden.ag_gemm_single(xs, ws[r], bias=biases[r] if with_bias else None, input_scales=sxs,
                                               weight_scale=sws[r])
                assert torch.equal(outs[r].cpu().view(torch.int16), ref.view(torch.int16)), \
                    f"int8 AG-GEMM rank {r} bias {with_bias}: not bit-identical to the golden path " \
                    f"(max rel err {golden.max_rel_err(outs[r], ref)})"
    finally:
        rk.close()


def test_int8_gemm_rs_all_ranks_on_one_gpu():
    """w8a8 GEMM-RS: every rank's dequantised partial in bf16, bias [1,N] on rank 0 only
    (src/gemm_rs/ths_op/gemm_reduce_scatter.cc:596-599), reduce-scatter."""
    world, m, n, k_local = 4, 512, 264, 512
    rk = Ranks(world)
    try:
        xs, ws, sxs, sws = _int8_inputs(world, m, n, k_local, 77)
        g = torch.Generator().manual_seed(10)
        bias = (torch.randn(1, n, generator=g) * 0.5).to(BF16)
        ops = rk.gemm_rs_ops(m, n, torch.int8, BF16)
        outs = [torch.empty((m // world, n), dtype=BF16, device="cuda") for _ in range(world)]
        from flux_b200 import _lib

        d_x, d_w = [x.cuda() for x in xs], [w.cuda() for w in ws]
        d_sx, d_sw = [s.reshape(-1).cuda() for s in sxs], [s.reshape(-1).cuda() for s in sws]
        d_bias = bias.cuda()
        for r in range(world):  # every rank passes the bias; only rank 0 applies it
            _lib.check(rk.lib.fluxb_gemm_rs_forward(
                ops[r], d_x[r].data_ptr(), d_w[r].data_ptr(), m, n, k_local, outs[r].data_ptr(), d_bias.data_ptr(),
                _lib.BIAS_1N, d_sx[r].data_ptr(), d_sw[r].data_ptr(), 1.0, 0, None, _stream()))
        rk.run()
        refs = golden.gemm_rs_single(xs, ws, [bias if r == 0 else None for r in range(world)], sxs, sws)
        for r in range(world):
            # the reference's own bar for w8a8 GEMM-RS is 2e-1 elementwise (test/python/gemm_rs/test_gemm_rs.py:593);
            # the rounding points are the golden path's, so nearly every element is bit-identical as well
            _close(outs[r], refs[r], 1e-2, 2e-1, f"int8 GEMM-RS rank {r}")
            same = (outs[r].cpu().view(torch.int16) == refs[r].view(torch.int16)).float().mean().item()
            assert same >= 0.99, f"rank {r}: only {same:.4f} of the elements are bit-identical to the golden path"
    finally:
        rk.close()


def test_gemm_rs_ring_reduction_all_ranks_on_one_gpu():
    """`ring_reduction`: partials summed in the order rank+1, ..., own last, rounded to bf16 after every addition
    (src/gemm_rs/ring_reduce.cu:54-80)."""
    from flux_b200 import _lib

    world, m, n, k_local = 4, 1024, 520, 256
    rk = Ranks(world)
    try:
        ab = [_cpu_inputs(r, m, n, k_local, BF16, 2468) for r in range(world)]
        ops = rk.gemm_rs_ops(m, n, BF16, BF16)
        outs = [torch.empty((m // world, n), dtype=BF16, device="cuda") for _ in range(world)]
        rk.gemm_rs_forward(ops, [a.cuda() for a, _ in ab], [b.cuda() for _, b in ab], outs, flags=_lib.RS_RING_ORDER)
        parts = [golden._rs_partial(a, b, None, None, None) for a, b in ab]
        for r in range(world):
            ref = golden.ring_reduce_single(parts, r)
            _close(outs[r], ref, 1e-2, 2e-2, f"ring-order GEMM-RS rank {r}")
            # the roundings are the reference's: nearly every element is bit-identical (the partials themselves may
            # differ in their last bit, because the GPU accumulates K in another order than the CPU matmul)
            same = (outs[r].cpu().view(torch.int16) == ref.view(torch.int16)).float().mean().item()
            assert same >= 0.95, f"rank {r}: only {same:.3f} of the elements match the ring reduction bit for bit"
    finally:
        rk.close()


@pytest.mark.parametrize("ag_mode", [1, 2, 4])
@pytest.mark.parametrize("world", [2, 4])
def test_moe_all_ranks_on_one_gpu(world, ag_mode):
    ntokens, topk, nexperts, hidden, ffn = 128 * world, 2, 4, 256, 128 * world
    ffn_local = ffn // world
    rk = Ranks(world)
    try:
        l0, l1 = rk.moe_ops(ntokens, hidden, ffn_local, nexperts, topk, BF16)
        for it in range(3):
            g = torch.Generator().manual_seed(1234 + it)
            logits = torch.randn(ntokens, nexperts, generator=g)
            if it == 1:
                logits[:, 0] = -1e9  # an expert that receives no tokens
            chosen, rw = golden.topk_routing(logits, topk)
            si = golden.calc_scatter_index_stable(chosen)
            splits = golden.calc_splits(chosen, nexperts)
            gi, ti = golden.calc_gather_index(si)
            toks, w0s, w1s = [], [], []
            for r in range(world):
                gr = torch.Generator().manual_seed(999 + r + 7 * it)
                toks.append(torch.randn(ntokens // world, hidden, generator=gr).to(BF16))
                w0s.append((torch.randn(nexperts, ffn_local, hidden, generator=gr) * 0.02).to(BF16))
                w1s.append((torch.randn(nexperts, hidden, ffn_local, generator=gr) * 0.02).to(BF16))
            oscale = torch.rand(nexperts, generator=g) + 0.5
            out0 = [torch.empty((ntokens * topk, ffn_local), dtype=BF16, device="cuda") for _ in range(world)]
            gathered = [torch.empty((ntokens, hidden), dtype=BF16, device="cuda") for _ in range(world)]
            rk.moe_l0_forward(l0, [t.cuda() for t in toks], [w.cuda() for w in w0s], splits.cuda(), si.cuda(), out0,
                              out_scales=[oscale.cuda()] * world, gathered=gathered, tuning={"ag_mode": ag_mode})
            ref0 = []
            for r in range(world):
                ref, ref_g = golden.moe_ag_scatter_single(toks, w0s[r], splits, si, oscale)
                ref0.append(ref)
                _close(out0[r], ref, 1e-2, 1e-2, f"MoE layer 0 world {world} call {it} rank {r}")
                assert torch.equal(gathered[r].cpu().view(torch.int16), ref_g.view(torch.int16))
            # layer 1 on the oracle's layer-0 output, so that errors do not compound
            vec = rw.reshape(-1)[(gi.long() * topk + ti.long())].contiguous()
            out1 = [torch.empty((ntokens // world, hidden), dtype=BF16, device="cuda") for _ in range(world)]
            rk.moe_l1_forward(l1, [x.cuda() for x in ref0], [w.cuda() for w in w1s], splits, si.reshape(-1).cuda(), out1,
                              vec_scale=vec.cuda())
            refs1 = golden.moe_gather_rs_single(ref0, w1s, splits, si, topk, output_vec_scales=[vec] * world)
            for r in range(world):
                _close(out1[r], refs1[r], 2e-2, 2e-2, f"MoE layer 1 world {world} call {it} rank {r}")
    finally:
        rk.close()


@pytest.mark.parametrize("world,ep_size", [(4, 2), (4, 4), (2, 2)])
def test_moe_expert_parallel_all_ranks_on_one_gpu(world, ep_size):
    """TP x EP (DistEnvTPWithEP with an ep_group, src/ths_op/ths_op.cc:334-346): `ep_size` groups of world / ep_size
    ranks; a group holds nexperts / ep_size experts with the ffn dimension sharded inside the group. Tokens are gathered
    from all ranks; layer 0 produces only the rows of the rank's experts, layer 1 combines every rank's share."""
    ntokens, topk, nexperts, hidden = 128 * world, 2, 8, 256
    ffn_tp = world // ep_size
    ffn_local, e_local = 128, nexperts // ep_size
    rk = Ranks(world)
    try:
        l0, l1 = rk.moe_ops(ntokens, hidden, ffn_local, nexperts, topk, BF16, ep_size=ep_size)
        for it in range(2):
            g = torch.Generator().manual_seed(4321 + it)
            logits = torch.randn(ntokens, nexperts, generator=g)
            if it == 1:
                logits[:, 5] = -1e9  # an expert that receives no tokens
            chosen, rw = golden.topk_routing(logits, topk)
            si = golden.calc_scatter_index_stable(chosen)
            splits = golden.calc_splits(chosen, nexperts)
            gi, ti = golden.calc_gather_index(si)
            vec_all = rw.reshape(-1)[(gi.long() * topk + ti.long())].contiguous()
            toks, w0s, w1s, ref0, vecs = [], [], [], [], []
            for r in range(world):
                gr = torch.Generator().manual_seed(555 + r + 9 * it)
                toks.append(torch.randn(ntokens // world, hidden, generator=gr).to(BF16))
                w0s.append((torch.randn(e_local, ffn_local, hidden, generator=gr) * 0.02).to(BF16))
                w1s.append((torch.randn(e_local, hidden, ffn_local, generator=gr) * 0.02).to(BF16))
            out0 = []
            for r in range(world):
                ep_rank = r // ffn_tp
                ref, _ = golden.moe_ag_scatter_single(toks, w0s[r], splits, si, None, ep_rank=ep_rank, ep_size=ep_size)
                ref0.append(ref)
                m_start = int(splits[:ep_rank * e_local].sum())
                vecs.append(vec_all[m_start:m_start + ref.shape[0]].contiguous())
                out0.append(torch.full((max(ref.shape[0], 1), ffn_local), float("nan"), dtype=BF16, device="cuda"))
            rk.moe_l0_forward(l0, [t.cuda() for t in toks], [w.cuda() for w in w0s], splits.cuda(), si.cuda(), out0)
            for r in range(world):
                if ref0[r].shape[0] > 0:
                    _close(out0[r][:ref0[r].shape[0]], ref0[r], 1e-2, 1e-2, f"EP layer 0 world {world} ep {ep_size} call {it} rank {r}")
            out1 = [torch.empty((ntokens // world, hidden), dtype=BF16, device="cuda") for _ in range(world)]
            d_x = [x.cuda() if x.shape[0] > 0 else torch.zeros((1, ffn_local), dtype=BF16, device="cuda")[:0] for x in ref0]
            rk.moe_l1_forward(l1, d_x, [w.cuda() for w in w1s], splits, si.reshape(-1).cuda(), out1,
                              vec_scales=[v.cuda() for v in vecs])
            refs1 = golden.moe_gather_rs_single(ref0, w1s, splits, si, topk, output_vec_scales=vecs, ep_size=ep_size)
            for r in range(world):
                _close(out1[r], refs1[r], 2e-2, 2e-2, f"EP layer 1 world {world} ep {ep_size} call {it} rank {r}")
    finally:
        rk.close()


# ------------------------------------------------------------------------------------------------
# BASELINE shapes at TP=8 (per-rank sizes), all eight ranks on one GPU, fp64 samples
# ------------------------------------------------------------------------------------------------
def _spread(n, count):
    return torch.tensor([round(i * (n - 1) / (count - 1)) for i in range(count)], dtype=torch.long, device="cuda")


def _cmp64(got, exact, tol_rel, tol_elem, what):
    got, exact = got.double(), exact.double()
    rel = float((got - exact).abs().max() / exact.abs().max())
    assert rel <= tol_rel, f"{what}: max rel err {rel}"
    bad = (got - exact).abs() > tol_elem + tol_elem * exact.abs()
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} of {bad.numel()} samples outside the elementwise {tol_elem} bar"


def _gpu_randn(g, rows, cols, scale, dtype=BF16):
    # drawn on the GPU: the check below is made of fp64 dots of these very tensors, no CPU copy is involved
    return (torch.randn(rows, cols, generator=g, device="cuda") * scale).to(dtype)


def test_dense_baseline_shapes_tp8_on_one_gpu():
    world, M, N0, K0 = 8, 4096, 49152, 12288
    m_local, n_local = M // world, N0 // world
    g = torch.Generator(device="cuda").manual_seed(1234)
    rk = Ranks(world)
    try:
        # D0: AG-GEMM, per rank A shard [512, 12288], B [6144, 12288] -> C [4096, 6144]
        shards = [_gpu_randn(g, m_local, K0, 1.0) for _ in range(world)]
        b0 = [_gpu_randn(g, n_local, K0, 0.02) for _ in range(world)]
        c0 = [torch.empty((M, n_local), dtype=BF16, device="cuda") for _ in range(world)]
        ops = rk.ag_gemm_ops(M, n_local, K0, BF16, BF16)
        rows_l, cols = _spread(m_local, 8), _spread(n_local, 16)
        grows = (torch.arange(world, device="cuda")[:, None] * m_local + rows_l[None, :]).reshape(-1)
        a_rows = torch.cat([s[rows_l] for s in shards]).double()
        for call in range(2):  # all-gather pushed by the kernel, then carried by the copy engines
            for t in c0:
                t.zero_()
            rk.ag_gemm_forward(ops, shards, b0, c0, tuning={"ag_mode": 1 + call})
            for r in range(world):
                _cmp64(c0[r][grows][:, cols], a_rows @ b0[r][cols].double().t(), 1e-2, 1e-2, f"D0 call {call} rank {r}")
        del ops, b0
        # D1: GEMM-RS on the AG output, per rank A [4096, 6144], B [12288, 6144] -> out [512, 12288]
        N1 = 12288
        b1 = [_gpu_randn(g, N1, n_local, 0.02) for _ in range(world)]
        outs = [torch.empty((m_local, N1), dtype=BF16, device="cuda") for _ in range(world)]
        rs = rk.gemm_rs_ops(M, N1, BF16, BF16)
        cols1 = _spread(N1, 16)
        exact = sum(c0[r][grows].double() @ b1[r][cols1].double().t() for r in range(world))
        # the reference's golden path rounds every rank's partial product to bf16 before the reduce-scatter
        # (torch.matmul in bf16, test/python/gemm_rs/test_gemm_rs.py:113-135), sums and rounds once more
        golden_path = sum((c0[r][grows].double() @ b1[r][cols1].double().t()).to(BF16).double() for r in range(world))
        for call in range(2):
            rk.gemm_rs_forward(rs, c0, b1, outs)
            got = torch.cat([outs[r][rows_l][:, cols1] for r in range(world)])
            rel = float((got.double() - exact).abs().max() / exact.abs().max())
            assert rel <= 1e-2, f"D1 call {call}: max rel err vs fp64 {rel}"
            _cmp64(got, golden_path.to(BF16), 1e-2, 2e-2, f"D1 call {call} vs the golden path")
    finally:
        rk.close()


def test_fp8_baseline_shape_tp8_on_one_gpu():
    world, M, N, K = 8, 8192, 28672, 8192
    m_local, n_local = M // world, N // world
    f8 = torch.float8_e4m3fn
    g = torch.Generator(device="cuda").manual_seed(99)
    rk = Ranks(world)
    try:
        qa, sa, qb, sb = [], [], [], []
        for r in range(world):
            a = torch.randn(m_local, K, generator=g, device="cuda")
            s = (a.abs().amax(1).clamp_min(1e-12) / 448.0).float()
            qa.append((a / s[:, None]).to(f8)), sa.append(s)
            b = torch.randn(n_local, K, generator=g, device="cuda") * 0.02
            s = (b.abs().amax(1).clamp_min(1e-12) / 448.0).float()
            qb.append((b / s[:, None]).to(f8)), sb.append(s)
        ops = rk.ag_gemm_ops(M, n_local, K, f8, BF16, with_scales=True)
        outs = [torch.empty((M, n_local), dtype=BF16, device="cuda") for _ in range(world)]
        rk.ag_gemm_forward(ops, qa, qb, outs, scales_a=sa, scales_b=sb)
        rows_l, cols = _spread(m_local, 8), _spread(n_local, 16)
        grows = (torch.arange(world, device="cuda")[:, None] * m_local + rows_l[None, :]).reshape(-1)
        a_rows = torch.cat([qa[r][rows_l].double() * sa[r][rows_l].double()[:, None] for r in range(world)])
        for r in range(world):
            exact = a_rows @ (qb[r][cols].double() * sb[r][cols].double()[:, None]).t()
            _cmp64(outs[r][grows][:, cols], exact, 3e-2, 3e-2, f"F rank {r}")
    finally:
        rk.close()


def test_moe_baseline_shape_tp8_on_one_gpu():
    from flux_b200 import calc_gather_index, calc_scatter_index

    world, T, H, E, FFN, TOPK = 8, 8192, 4096, 8, 14336, 2
    ffn_l, t_local = FFN // world, T // world
    g = torch.Generator(device="cuda").manual_seed(1234)
    rk = Ranks(world)
    try:
        logits = torch.randn(T, E, generator=g, device="cuda")
        w, chosen = torch.topk(torch.softmax(logits, -1), TOPK, dim=-1)
        chosen = chosen.to(torch.int32)
        # routing through the library's index kernels, checked bit for bit against the oracle
        import flux_b200

        flux_b200.init_flux_shm(None)
        si, splits = calc_scatter_index(chosen, torch.empty(E), return_splits=True)
        gi, ti = calc_gather_index(si)
        assert torch.equal(si.cpu(), golden.calc_scatter_index_stable(chosen.cpu()))
        assert torch.equal(splits.cpu(), golden.calc_splits(chosen.cpu(), E))
        ogi, oti = golden.calc_gather_index(si.cpu())
        assert torch.equal(gi.cpu(), ogi) and torch.equal(ti.cpu(), oti)
        vec = w.reshape(-1)[(gi.long() * TOPK + ti.long())].contiguous().float()
        toks = [_gpu_randn(g, t_local, H, 1.0) for _ in range(world)]
        w0 = [_gpu_randn(g, E * ffn_l, H, 0.02).view(E, ffn_l, H) for _ in range(world)]
        w1 = [_gpu_randn(g, E * H, ffn_l, 0.02).view(E, H, ffn_l) for _ in range(world)]
        l0, l1 = rk.moe_ops(T, H, ffn_l, E, TOPK, BF16)
        act = [torch.empty((T * TOPK, ffn_l), dtype=BF16, device="cuda") for _ in range(world)]
        gathered = [torch.empty((T, H), dtype=BF16, device="cuda") for _ in range(world)]
        rk.moe_l0_forward(l0, toks, w0, splits, si, act, gathered=gathered)
        x_all = torch.cat(toks)
        tok_s = (torch.arange(world, device="cuda")[:, None] * t_local + _spread(t_local, 4)[None, :]).reshape(-1)
        rows0 = si[tok_s].reshape(-1).long()
        tok_of_row = tok_s.repeat_interleave(TOPK)
        exp_of_row = chosen[tok_s].reshape(-1).long()
        cols0, cols1 = _spread(ffn_l, 16), _spread(H, 16)
        for r in range(world):
            assert torch.equal(gathered[r], x_all), f"rank {r}: gathered tokens differ from all_gather"
            exact0 = torch.einsum("rh,rch->rc", x_all[tok_of_row].double(), w0[r][exp_of_row[:, None], cols0[None, :]].double())
            _cmp64(act[r][rows0][:, cols0], exact0, 1e-2, 1e-2, f"X layer 0 rank {r}")
        out1 = [torch.empty((t_local, H), dtype=BF16, device="cuda") for _ in range(world)]
        rk.moe_l1_forward(l1, act, w1, splits.cpu(), si.view(-1), out1, vec_scale=vec)
        # exact value, and the reference's golden path on the same samples: per-expert matmul rounded to bf16, times
        # the row scale, rounded, top-k sum rounded, reduce-scatter (python/flux/testing/moe_gather_rs_utils.py:59-119)
        exact = torch.zeros((tok_s.numel(), cols1.numel()), dtype=torch.float64, device="cuda")
        gold = torch.zeros_like(exact)
        for r in range(world):
            tk = torch.zeros_like(exact)
            for k in range(TOPK):
                rr = si[tok_s][:, k].long()
                e = chosen[tok_s][:, k].long()
                d = torch.einsum("rf,rcf->rc", act[r][rr].double(), w1[r][e[:, None], cols1[None, :]].double())
                exact += vec[rr].double()[:, None] * d
                tk += (d.to(BF16).float() * vec[rr][:, None]).to(BF16).double()
            gold += tk.to(BF16).double()
        got = torch.cat([out1[r][_spread(t_local, 4)][:, cols1] for r in range(world)])
        rel = float((got.double() - exact).abs().max() / exact.abs().max())
        assert rel <= 2e-2, f"X layer 1: max rel err vs fp64 {rel}"
        _cmp64(got, gold.to(BF16), 2e-2, 2e-2, "X layer 1 vs the golden path")
    finally:
        rk.close()
