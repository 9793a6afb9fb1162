"""CPU tests of the oracle (`oracle/golden.py`): pinned against vectors produced by the reference's
own helpers (tests/golden/*.pt, made by tests/golden/make_golden.py), against the hand-computable
`--debug` inputs of the reference's tests, and for self-consistency between its distributed (gloo)
and single-process forms."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist import run_distributed  # noqa: E402

from oracle import golden  # noqa: E402

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return torch.load(os.path.join(GOLD, name), weights_only=False)


# ------------------------------------------------------------------ pinned: routing (bit-exact)
def test_routing_matches_reference_vectors():
    for case in _load("routing.pt"):
        chosen = case["chosen"]
        si = golden.calc_scatter_index_stable(chosen)
        assert torch.equal(si, case["scatter_index"])
        assert torch.equal(golden.calc_splits(chosen, case["nexperts"]), case["splits"])
        gi, ti = golden.calc_gather_index(si)
        # inverse permutation: row scatter_index[t,k] holds token t, slot k
        ntokens, topk = chosen.shape
        for t in range(ntokens):
            for k in range(topk):
                assert gi[si[t, k]] == t and ti[si[t, k]] == k
        # rows are grouped by expert in expert order, sizes = splits
        experts_by_row = chosen.reshape(-1)[(gi.long() * topk + ti.long())]
        assert torch.equal(experts_by_row, torch.sort(chosen.reshape(-1), stable=True).values)


# ------------------------------------------------------------------ pinned: MoE layer 0
def test_moe_l0_matches_reference_vectors():
    for case in _load("moe_l0.pt"):
        out, gathered = golden.moe_ag_scatter_single(
            [case["tokens"]], case["weights"], case["splits"], case["scatter_index"], case["output_scale"])
        assert torch.equal(gathered, case["tokens"])
        # same torch ops on the same machine: identical bits
        assert torch.equal(out, case["out"]), float((out.float() - case["out"].float()).abs().max())


# ------------------------------------------------------------------ pinned: MoE layer 1
def test_moe_l1_matches_reference_vectors():
    for case in _load("moe_l1.pt"):
        ntokens, topk, nexperts, kloc, n, dtype = case["case"]
        ranks = case["ranks"]
        outs = golden.moe_gather_rs_single(
            [r["x"] for r in ranks], [r["w"] for r in ranks], case["splits"], case["scatter_index"], topk,
            input_scales=[torch.ones(1)] * len(ranks), weight_scales=[torch.ones(nexperts)] * len(ranks),
            output_vec_scales=[r["vec"] for r in ranks])
        for r, o in enumerate(outs):
            ref = ranks[r]["out"]
            # the reference all-reduces rounded partials over gloo; the single-process form sums in fp32
            tol = 1e-6 if dtype == torch.float32 else 1e-2
            assert golden.max_rel_err(o, ref) <= tol


# ------------------------------------------------------------------ pinned: expert parallelism
def test_moe_expert_parallel_matches_reference_vectors():
    """The reference's golden path with ep_size = 2 (tests/golden/make_golden.py --only-ep): layer 0 computes only the
    rows of the rank's experts; layer 1 scatters them into the full result, the reduce-scatter adds the ranks."""
    for case in _load("moe_l0_ep.pt"):
        out, _ = golden.moe_ag_scatter_single(
            [case["tokens"]], case["weights"], case["splits"], case["scatter_index"], case["output_scale"],
            ep_rank=case["ep_rank"], ep_size=case["ep_size"])
        assert out.shape == case["out"].shape and torch.equal(out, case["out"])
    case = _load("moe_l1_ep.pt")
    ranks = case["ranks"]
    e_local = ranks[0]["w"].shape[0]
    outs = golden.moe_gather_rs_single(
        [r["x"] for r in ranks], [r["w"] for r in ranks], case["splits"], case["scatter_index"], case["topk"],
        input_scales=[torch.ones(1)] * len(ranks), weight_scales=[torch.ones(e_local)] * len(ranks),
        output_vec_scales=[r["vec"] for r in ranks], ep_size=case["ep_size"])
    for r, o in enumerate(outs):
        assert golden.max_rel_err(o, ranks[r]["out"]) <= 1e-2


# ------------------------------------------------------------------ known answers of the --debug inputs
def test_ag_gemm_debug_known_answer():
    """test/python/ag_gemm/test_ag_kernel.py:670-678: input zero except column 0 = rank+1, weight = 1
    => every element of row block r of the output equals r+1."""
    world, m_local, k, n = 4, 8, 32, 16
    inputs = []
    for r in range(world):
        a = torch.zeros(m_local, k, dtype=torch.bfloat16)
        a[:, 0] = r + 1
        inputs.append(a)
    w = torch.ones(n, k, dtype=torch.bfloat16)
    out, gathered = golden.ag_gemm_single(inputs, w)
    for r in range(world):
        assert torch.all(out[r * m_local:(r + 1) * m_local] == r + 1)
    assert torch.equal(gathered, torch.cat(inputs))


def test_gemm_rs_debug_known_answer():
    """test/python/gemm_rs/test_gemm_rs.py:495-504: input column 0 = rank+1, weight = 1 =>
    every output element = sum_r (r+1) (36 at TP=8)."""
    world, m, k, n = 8, 16, 32, 8
    inputs, weights = [], []
    for r in range(world):
        a = torch.zeros(m, k, dtype=torch.bfloat16)
        a[:, 0] = r + 1
        inputs.append(a)
        weights.append(torch.ones(n, k, dtype=torch.bfloat16))
    outs = golden.gemm_rs_single(inputs, weights)
    assert len(outs) == world
    for o in outs:
        assert o.shape == (m // world, n)
        assert torch.all(o == 36)


def test_fp8_dequant_rule():
    """fp8 golden = bf16 matmul of the e4m3 values times row scale times channel scale
    (test_ag_kernel.py:119-124,143-147); it must track the unquantised fp32 product within the
    quantisation noise, and equal the explicit dequantised product within bf16 rounding."""
    g = torch.Generator().manual_seed(5)
    a = torch.randn(64, 128, generator=g)
    b = torch.randn(32, 128, generator=g) * 0.02
    qa, sa = golden.quantize_fp8_rows(a)
    qb, sb = golden.quantize_fp8_rows(b)
    out, _ = golden.ag_gemm_single([qa], qb, input_scales=[sa], weight_scale=sb)
    deq = (qa.float() * sa[:, None]) @ (qb.float() * sb[:, None]).t()
    assert out.dtype == torch.bfloat16
    assert golden.max_rel_err(out, deq) <= 1e-2
    assert golden.max_rel_err(out, a @ b.t()) <= 6e-2


# ------------------------------------------------------------------ gloo (world 2) == single process
def _dist_vs_single(rank, world, tmpdir):
    import torch.distributed as dist

    grp = dist.group.WORLD
    # the CPU-runnable reference configuration: M=256 K=512 N_local=512 fp32, A,B ~ N(0,1)/sqrt(512)
    shards, weights = [], []
    for r in range(world):
        g = torch.Generator().manual_seed(1234 + r)
        shards.append(torch.randn(128, 512, generator=g) / 512 ** 0.5)
        weights.append(torch.randn(512, 512, generator=g) / 512 ** 0.5)
    out, gathered = golden.ag_gemm_dist(grp, shards[rank], weights[rank])
    ref, ref_g = golden.ag_gemm_single(shards, weights[rank])
    assert out.shape == (256, 512)
    assert torch.equal(gathered, ref_g)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
    # GEMM-RS: A [256, 256] per rank (K sharded), B [512, 256]
    ins, ws = [], []
    for r in range(world):
        g = torch.Generator().manual_seed(4321 + r)
        ins.append(torch.randn(256, 256, generator=g) / 16)
        ws.append(torch.randn(512, 256, generator=g) / 16)
    o = golden.gemm_rs_dist(grp, ins[rank], ws[rank])
    refs = golden.gemm_rs_single(ins, ws)
    assert o.shape == (128, 512)
    assert torch.allclose(o, refs[rank], rtol=1e-5, atol=1e-5)


def test_oracle_gloo_world2(tmp_path):
    run_distributed(_dist_vs_single, 2, str(tmp_path), use_cuda=False)


def test_moe_identity_weights_roundtrip():
    """Layer 0 with identity expert weights returns the gathered tokens in expert-sorted order; layer 1
    with identity weights and routing weights returns sum_k w[t,k] * token_t."""
    g = torch.Generator().manual_seed(9)
    ntokens, topk, nexperts, h = 24, 2, 4, 16
    logits = torch.randn(ntokens, nexperts, generator=g)
    chosen, rw = golden.topk_routing(logits, topk)
    si = golden.calc_scatter_index_stable(chosen)
    splits = golden.calc_splits(chosen, nexperts)
    tokens = torch.randn(ntokens, h, generator=g)
    eye = torch.eye(h).repeat(nexperts, 1, 1)
    out0, _ = golden.moe_ag_scatter_single([tokens], eye, splits, si)
    gi, ti = golden.calc_gather_index(si)
    assert torch.equal(out0, tokens[gi.long()])
    vec = rw.reshape(-1)[(gi.long() * topk + ti.long())]
    out1 = golden.moe_gather_rs_single([out0], [eye], splits, si, topk, output_vec_scales=[vec])[0]
    assert torch.allclose(out1, tokens * rw.sum(1, keepdim=True), rtol=1e-5, atol=1e-6)


def test_dense_matches_reference_vectors():
    """Dense AG-GEMM and GEMM-RS: the oracle against outputs of the reference's own golden functions
    (`perf_torch` of test/python/ag_gemm/test_ag_kernel.py:88-176 and test/python/gemm_rs/test_gemm_rs.py:57-157,
    executed unmodified on 2 gloo ranks by tests/golden/make_golden.py). fp32 agrees to rounding of a
    different summation order; 16-bit outputs to one rounding of the output format."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLD, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    cases = _load("dense.pt")
    assert len(cases) == 4
    for c in cases:
        case, ranks = c["case"], c["ranks"]
        world = len(ranks)
        dtype = case[3]
        ins = [mg.dense_inputs(case, r, world) for r in range(world)]
        fp8 = golden.is_fp8(dtype)
        tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else \
            dict(rtol=2e-3, atol=2e-3) if dtype == torch.float16 else dict(rtol=1.6e-2, atol=1e-2)
        rs_outs = None if fp8 else golden.gemm_rs_single(
            [i["rs_input"] for i in ins], [i["rs_weight"] for i in ins],
            biases=[i["rs_bias"] for i in ins] if case[4] else None)
        for r in range(world):
            out, gathered = golden.ag_gemm_single(
                [i["ag_input"] for i in ins], ins[r]["ag_weight"], bias=ins[r]["ag_bias"],
                input_scales=[i["input_scale"] for i in ins] if fp8 else None, weight_scale=ins[r]["weight_scale"])
            assert out.dtype == ranks[r]["ag_out"].dtype and out.shape == ranks[r]["ag_out"].shape
            torch.testing.assert_close(out.float(), ranks[r]["ag_out"].float(), **tol)
            assert abs(gathered.double().sum().item() - ranks[r]["ag_gathered_sum"]) <= 1e-6 * gathered.numel()
            if fp8:
                assert out.dtype == torch.bfloat16 and ranks[r]["rs_out"] is None
                continue
            assert rs_outs[r].dtype == ranks[r]["rs_out"].dtype and rs_outs[r].shape == ranks[r]["rs_out"].shape
            torch.testing.assert_close(rs_outs[r].float(), ranks[r]["rs_out"].float(), **tol)
