"""CPU tests of the host-side mirror of the reference interface: option carriers, dtype rules, scale
normalisation, tuning marshalling, and the loud failure when no B200 is present (no CPU fallback)."""
import pytest
import torch

import flux_b200 as flux
from flux_b200 import _lib, ops


def test_output_dtype_rule():
    # fp8 inputs produce bf16 (src/ag_gemm/ths_op/gemm_with_barrier.cc:184-185); 16-bit keeps its type
    assert ops._out_dtype(torch.bfloat16, None) == torch.bfloat16
    assert ops._out_dtype(torch.float16, None) == torch.float16
    assert ops._out_dtype(torch.float8_e4m3fn, None) == torch.bfloat16
    assert ops._out_dtype(torch.bfloat16, torch.float32) == torch.float32
    assert flux.is_fp8_dtype(torch.float8_e5m2) and not flux.is_fp8_dtype(torch.bfloat16)


def test_scale_normalisation():
    # scalar [1] scales (the reference's fp8 form) and [n], [n,1], [1,n] vectors (its int8 form) all end as [n]
    s = ops._expand_scale(torch.tensor([0.5]), 4, "input_scale")
    assert s.shape == (4,) and torch.all(s == 0.5) and s.is_contiguous()
    v = torch.arange(4, dtype=torch.float32)
    for shaped in (v, v.reshape(4, 1), v.reshape(1, 4)):
        assert torch.equal(ops._expand_scale(shaped, 4, "weight_scale"), v)
    assert ops._expand_scale(None, 4, "x") is None
    with pytest.raises(RuntimeError):
        ops._expand_scale(torch.zeros(3), 4, "weight_scale")
    with pytest.raises(RuntimeError):
        ops._expand_scale(torch.zeros(4, dtype=torch.float16), 4, "weight_scale")


def test_tuning_marshalling():
    assert ops._tuning(None) is None
    t = _lib.Tuning(256, 8, 148, 2)
    assert (t.block_n, t.group_m, t.num_ctas, t.cta_group) == (256, 8, 148, 2)
    assert ops._tuning({"block_n": 128}) is not None


def test_option_carriers_default_to_unset():
    # every field optional, as in src/coll/ths_op/all_gather_types.h:35-43 and reduce_scatter_op.h:35-46
    ag = flux.AllGatherOption()
    assert [ag.input_buffer_copied, ag.use_cuda_core_local, ag.use_cuda_core_ag, ag.fuse_sync, ag.use_read, ag.mode] == [None] * 6
    ag.mode = flux.AGRingMode.Ring2D
    assert "Ring2D" in repr(ag)
    rs = flux.ReduceScatterOption()
    assert rs.n_split is None and rs.ring_mode is None
    m = flux.MoeArguments(8192, 4096, 14336, 8, 2, torch.bfloat16)
    assert m.output_dtype == torch.bfloat16 and m.topk == 2


def test_bitwise_check_on_cpu_tensors():
    a = torch.arange(16, dtype=torch.float32).reshape(4, 4)
    assert flux.bitwise_check(a, a.clone())
    b = a.clone()
    b[0, 0] = -0.0  # equal as numbers, different bits
    assert not flux.bitwise_check(a, b)
    assert not flux.bitwise_check(a, a.to(torch.float64))


def test_dtype_codes():
    from flux_b200.shm import fluxb_dtype

    assert fluxb_dtype(torch.bfloat16) == _lib.BF16 and fluxb_dtype(torch.float8_e4m3fn) == _lib.E4M3
    assert fluxb_dtype(torch.int8) == _lib.S8  # w8a8
    with pytest.raises(RuntimeError):
        fluxb_dtype(torch.int64)


def test_ops_fail_loudly_without_a_gpu():
    """No CUDA device (or not sm_100): constructing an op raises; nothing falls back to the CPU."""
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        flux.init_flux_shm(None)
    with pytest.raises(RuntimeError):
        flux.AGKernel(None, 1, 256, 256, 256, torch.bfloat16)
    with pytest.raises(RuntimeError):
        flux.GemmRS(None, 1, 256, 256, torch.bfloat16)


def test_build_recipe_lists_every_source():
    from flux_b200 import build

    names = {p.name for p in build.sources()}
    assert {"gemm_ops.cu", "moe_ops.cu", "moe_index.cu", "runtime.cu"} <= names
    assert "arch=compute_100a,code=sm_100a" in build.NVCC_FLAGS


def test_gemm_only_rejects_unsupported_modes():
    """Input types outside bf16 / fp16 / fp8 / int8 and 8-bit inputs with transposed weights are refused at
    construction, before any device is touched (python/flux/cpp_mod.pyi:215-253 lists the modes;
    src/ag_gemm/ths_op/gemm_with_barrier.cc:188 the fp8 rule)."""
    import pytest
    import torch

    import flux_b200 as flux

    with pytest.raises(RuntimeError, match="not supported"):
        flux.GemmOnly(torch.int32)
    with pytest.raises(RuntimeError, match="transpose_weight"):
        flux.GemmOnly(torch.float8_e4m3fn, transpose_weight=True)
    with pytest.raises(RuntimeError, match="transpose_weight"):
        flux.GemmOnly(torch.int8, transpose_weight=True)
