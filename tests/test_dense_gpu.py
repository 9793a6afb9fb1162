"""GPU parity tests of the dense path (plain GEMM, AG-GEMM, GEMM-RS) against the oracle.

Every case calls through the C ABI (`libfluxb.so`), on seeded inputs generated on the CPU so the oracle
and the kernel see identical values. Tolerance: max relative error <= 1e-2 for 16-bit inputs (fp32
accumulation), <= 3e-2 for fp8 against the dequantised oracle. Multi-rank cases need >= 2 GPUs."""
import ctypes as C
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import dist_cases  # noqa: E402
from _dist import run_distributed  # noqa: E402
from conftest import gpu_count  # noqa: E402

from oracle import golden  # noqa: E402

pytestmark = pytest.mark.gpu
BF16_TOL = 1e-2
FP8_TOL = 3e-2


@pytest.fixture(scope="module")
def flux():
    import flux_b200

    flux_b200.init_flux_shm(None)
    flux_b200.get_comm(None).set_timeout_ms(5000)
    return flux_b200


def _mk(m, n, k, dtype, seed=1):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(dtype)
    b = (torch.randn(n, k, generator=g) * 0.02).to(dtype)
    return a, b


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (256, 512, 1024), (200, 264, 136),
                                   (1, 8, 8), (129, 72, 520), (1024, 1024, 1024), (4096, 1536, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_only_matches_oracle(flux, m, n, k, dtype):
    a, b = _mk(m, n, k, dtype)
    op = flux.AGKernel(None, 1, m, n, k, dtype)
    out = op.gemm_only(a.cuda(), b.cuda())
    torch.cuda.synchronize()
    op.comm.check_status()
    ref, _ = golden.ag_gemm_single([a], b)
    assert out.shape == (m, n) and out.dtype == dtype
    assert golden.max_rel_err(out, ref) <= BF16_TOL


@pytest.mark.parametrize("m,n,k,cta_group", [(256, 264, 512, 1), (512, 520, 1024, 2), (200, 72, 136 * 2, 1), (1024, 1536, 4096, 2)])
def test_int8_gemm_is_bit_identical_to_the_golden_path(flux, m, n, k, cta_group):
    """w8a8: int8 x int8 -> int32 on the tensor cores (tcgen05 kind::i8), dequantised as
    (input_scale[m] * weight_scale[n]) * acc, rounded to bf16, then `+= bias` in bf16; the reference's test asks for
    a bitwise match (threshold 0, test/python/ag_gemm/test_ag_kernel.py:143-150,615)."""
    g = torch.Generator().manual_seed(m + n)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int32).to(torch.int8)
    b = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int32).to(torch.int8)
    sa = torch.rand(m, 1, generator=g) * 0.01 + 0.001
    sb = torch.rand(1, n, generator=g) * 0.01 + 0.001
    bias = (torch.randn(1, n, generator=g) * 0.5).to(torch.bfloat16)
    op = flux.GemmOnly(torch.int8)
    for with_bias in (False, True):
        out = op.forward(a.cuda(), b.cuda(), bias=bias.cuda() if with_bias else None, input_scale=sa.cuda(),
                         weight_scale=sb.cuda(), tuning={"cta_group": cta_group})
        torch.cuda.synchronize()
        op.comm.check_status()
        ref, _ = golden.ag_gemm_single([a], b, bias=bias if with_bias else None, input_scales=[sa], weight_scale=sb)
        assert out.dtype == torch.bfloat16
        assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16)), \
            f"not bit-identical (bias {with_bias}): max rel err {golden.max_rel_err(out, ref)}"


@pytest.mark.parametrize("block_n", [64, 128, 192, 256])
@pytest.mark.parametrize("group_m", [1, 3, 16])
def test_gemm_tile_configs(flux, block_n, group_m):
    m, n, k = 640, 1000, 768
    a, b = _mk(m, n, k, torch.bfloat16, seed=block_n + group_m)
    op = flux.AGKernel(None, 1, m, n, k, torch.bfloat16)
    out = op.gemm_only(a.cuda(), b.cuda(), tuning={"block_n": block_n, "group_m": group_m, "num_ctas": 37})
    torch.cuda.synchronize()
    op.comm.check_status()
    ref, _ = golden.ag_gemm_single([a], b)
    assert golden.max_rel_err(out, ref) <= BF16_TOL


def test_gemm_bias_and_world1_forward(flux):
    m, n, k = 300, 520, 256
    a, b = _mk(m, n, k, torch.bfloat16, seed=3)
    g = torch.Generator().manual_seed(4)
    bias_mn = (torch.randn(m, n, generator=g) * 0.1).to(torch.bfloat16)
    bias_1n = (torch.randn(1, n, generator=g) * 0.1).to(torch.bfloat16)
    op = flux.AGKernel(None, 1, m, n, k, torch.bfloat16)
    for bias in (bias_mn, bias_1n):
        gathered = torch.empty(m, k, dtype=torch.bfloat16, device="cuda")
        out = op.forward(a.cuda(), b.cuda(), bias=bias.cuda(), gathered_input=gathered)
        torch.cuda.synchronize()
        ref, ref_g = golden.ag_gemm_single([a], b, bias=bias)
        assert golden.max_rel_err(out, ref) <= BF16_TOL
        assert torch.equal(gathered.cpu(), ref_g)


def test_gemm_debug_known_answer(flux):
    """test/python/ag_gemm/test_ag_kernel.py:670-678 style: A zero except column 0 = 3, W = 1."""
    m, n, k = 256, 256, 512
    a = torch.zeros(m, k, dtype=torch.bfloat16)
    a[:, 0] = 3
    w = torch.ones(n, k, dtype=torch.bfloat16)
    op = flux.AGKernel(None, 1, m, n, k, torch.bfloat16)
    out = op.gemm_only(a.cuda(), w.cuda())
    assert torch.all(out.cpu() == 3)


def test_gemm_linearity_at_full_size(flux):
    """Size-independent property at the headline shape (M=4096, N=6144, K=12288): the kernel is linear
    in A, and a sampled set of output entries matches an fp64 dot product."""
    m, n, k = 4096, 6144, 12288
    g = torch.Generator(device="cuda").manual_seed(7)
    a1 = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    a2 = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    op = flux.AGKernel(None, 1, m, n, k, torch.bfloat16)
    o1 = op.gemm_only(a1, b).float()
    o2 = op.gemm_only(a2, b).float()
    # a1 + a2 rounded to bf16 is not exactly the sum; use the exactly representable 2*a1
    o3 = op.gemm_only((a1 * 2).to(torch.bfloat16), b).float()
    torch.cuda.synchronize()
    op.comm.check_status()
    assert golden.max_rel_err(o3, 2 * o1) <= 1e-2
    rows = torch.randint(0, m, (64,), generator=torch.Generator().manual_seed(1))
    cols = torch.randint(0, n, (64,), generator=torch.Generator().manual_seed(2))
    for o, a in ((o1, a1), (o2, a2)):
        exact = (a[rows.cuda()].double() * b[cols.cuda()].double()).sum(1)
        got = o[rows.cuda(), cols.cuda()].double()
        assert float((got - exact).abs().max() / exact.abs().max()) <= 1e-2


def test_argument_errors(flux):
    """Shape/dtype violations raise RuntimeError, as FLUX_CHECK does in the reference."""
    op = flux.AGKernel(None, 1, 256, 256, 256, torch.bfloat16)
    a, b = _mk(256, 256, 256, torch.bfloat16)
    with pytest.raises(RuntimeError):
        op.forward(a.cuda(), b.cuda()[:, :128])  # K mismatch
    with pytest.raises(RuntimeError):
        op.forward(a.cuda().float(), b.cuda())  # dtype mismatch
    a2, _ = _mk(512, 256, 256, torch.bfloat16)
    with pytest.raises(RuntimeError):
        op.forward(a2.cuda(), b.cuda())  # M > full_m
    rs = flux.GemmRS(None, 1, 256, 256, torch.bfloat16)
    with pytest.raises(RuntimeError):
        rs.forward(a2.cuda(), b.cuda())  # M > max_m


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 512, 1024), (200, 264, 144), (1024, 1536, 2048)])
@pytest.mark.parametrize("cta_group", [1, 2])
def test_fp8_gemm_with_row_and_channel_scales(flux, m, n, k, cta_group):
    """FP8 e4m3 operands, per-row input scale and per-output-channel weight scale applied in the epilogue,
    bf16 out; oracle = bf16 matmul of the e4m3 values times the scales (test_ag_kernel.py:119-124,143-147)."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g)
    b = torch.randn(n, k, generator=g) * 0.02
    qa, sa = golden.quantize_fp8_rows(a)
    qb, sb = golden.quantize_fp8_rows(b)
    op = flux.AGKernel(None, 1, m, n, k, torch.float8_e4m3fn)
    out = op.gemm_only(qa.cuda(), qb.cuda(), input_scale=sa.cuda(), weight_scale=sb.cuda(),
                       tuning={"cta_group": cta_group})
    torch.cuda.synchronize()
    op.comm.check_status()
    ref, _ = golden.ag_gemm_single([qa], qb, input_scales=[sa], weight_scale=sb)
    assert out.dtype == torch.bfloat16
    assert golden.max_rel_err(out, ref) <= FP8_TOL
    # scalar scales, the reference's own fp8 form (cpp_mod.pyi:439-440)
    one_a, one_b = torch.tensor([0.5]), torch.tensor([2.0])
    out2 = op.gemm_only(qa.cuda(), qb.cuda(), input_scale=one_a.cuda(), weight_scale=one_b.cuda())
    ref2, _ = golden.ag_gemm_single([qa], qb, input_scales=[one_a], weight_scale=one_b)
    assert golden.max_rel_err(out2, ref2) <= FP8_TOL


def test_fp8_rejects_transpose_weight(flux):
    op = flux.AGKernel(None, 1, 128, 128, 128, torch.float8_e4m3fn)
    q = torch.zeros(128, 128).to(torch.float8_e4m3fn).cuda()
    with pytest.raises(RuntimeError):
        op.forward(q, q, transpose_weight=True)


@pytest.mark.parametrize("m,n,k", [(256, 384, 512), (300, 264, 200), (1024, 2048, 1024), (128, 64, 64)])
@pytest.mark.parametrize("cta_group", [1, 2])
def test_transpose_weight(flux, m, n, k, cta_group):
    """transpose_weight=True: the weight arrives as [K, N] and is read in place (MN-major operand)."""
    a, b = _mk(m, n, k, torch.bfloat16, seed=9 + m)
    op = flux.AGKernel(None, 1, m, n, k, torch.bfloat16)
    w_kn = b.t().contiguous().cuda()
    out = op.forward(a.cuda(), w_kn, transpose_weight=True, tuning={"cta_group": cta_group})
    torch.cuda.synchronize()
    op.comm.check_status()
    ref, _ = golden.ag_gemm_single([a], b)
    assert golden.max_rel_err(out, ref) <= BF16_TOL
    rs = flux.GemmRS(None, 1, m, n, torch.bfloat16, transpose_weight=True)
    out2 = rs.forward(a.cuda(), w_kn)
    torch.cuda.synchronize()
    assert golden.max_rel_err(out2, ref) <= BF16_TOL


def _need(n):
    if gpu_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("with_bias", [False, True])
def test_ag_gemm_multi_rank(with_bias):
    _need(2)
    w = min(gpu_count(), 8)
    w = 1 << (w.bit_length() - 1)
    shapes = [(256, 512, 512), (128, 256, 512), (200, 264, 512), (1, 64, 512), (256, 512, 512)]
    run_distributed(dist_cases.ag_gemm_case, w, shapes, "bfloat16", with_bias, None)


@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_rs_multi_rank(with_bias):
    _need(2)
    w = min(gpu_count(), 8)
    w = 1 << (w.bit_length() - 1)
    shapes = [(512, 512, 512), (256, 512, 256), (8 * w, 512, 512), (200 * w, 512, 1024), (512, 512, 512)]
    run_distributed(dist_cases.gemm_rs_case, w, shapes, "bfloat16", with_bias, None)


def test_gemm_rs_fp32_wire_multi_rank():
    """Partials sent as fp32 (FLUXB_RS_FP32_WIRE) instead of the 16-bit output format, and fp16 outputs."""
    _need(2)
    w = min(gpu_count(), 8)
    w = 1 << (w.bit_length() - 1)
    shapes = [(512, 512, 512), (200 * w, 512, 1024), (8 * w, 512, 512)]
    run_distributed(dist_cases.gemm_rs_case, w, shapes, "bfloat16", False, None, True)
    run_distributed(dist_cases.gemm_rs_case, w, shapes, "float16", False, None, False)


def test_fp8_multi_rank():
    _need(2)
    w = min(gpu_count(), 8)
    w = 1 << (w.bit_length() - 1)
    run_distributed(dist_cases.fp8_case, w, [(256, 512, 512), (100, 264, 256)])


def test_stress_random_m_multi_rank():
    """Random local M per call on one op, as the reference's stress scripts do
    (test/python/stress/stress_ag_gemm.py:218-310): no hang, every call checked."""
    _need(2)
    w = min(gpu_count(), 8)
    w = 1 << (w.bit_length() - 1)
    g = torch.Generator().manual_seed(42)
    ms = [int(x) for x in torch.randint(1, 513, (10,), generator=g)]
    run_distributed(dist_cases.ag_gemm_case, w, [(m, 512, 512) for m in ms], "bfloat16", False, None)
    run_distributed(dist_cases.gemm_rs_case, w, [(m * w, 512, 256) for m in ms], "bfloat16", False, None)


def test_baseline_shapes_multi_rank():
    """D0, D1 and F of the benchmark at the box's GPU count, one process per GPU (fp64 samples)."""
    w = min(gpu_count(), 8)
    if w < 2:
        pytest.skip("needs >= 2 GPUs")
    w = 1 << (w.bit_length() - 1)
    run_distributed(dist_cases.baseline_shapes_case, w)
