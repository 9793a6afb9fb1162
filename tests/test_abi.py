"""CPU tests of the drop-in boundary: the C ABI library builds/loads without a GPU, exports every
symbol `include/fluxb.h` declares, and its pure host helpers (sizes) answer. No compute calls."""
import ctypes as C
import os
import re

from flux_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fluxb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fluxb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    declared = _declared_symbols()
    assert len(declared) >= 30
    assert sorted(_lib.SIGNATURES) == declared


def test_library_loads_and_exports_every_symbol():
    lib = _lib.load()
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in fluxb.h but missing from libfluxb.so"
    assert lib.fluxb_version() >= 100
    assert isinstance(_lib.last_error(), str)


def test_size_helpers():
    lib = _lib.load()
    # two parities of [full_m + one tile, k] elements
    assert lib.fluxb_ag_gemm_gather_bytes(4096, 12288, _lib.BF16) == 2 * (4096 + 128) * 12288 * 2
    assert lib.fluxb_ag_gemm_gather_bytes(8192, 8192, _lib.E4M3) == 2 * (8192 + 128) * 8192
    # two parities x world x ceil(ceil(full_m/world)/128) chunks x 64 slice groups of counters
    assert lib.fluxb_ag_gemm_flag_bytes(4096, 8) == 2 * 8 * 4 * 64 * 4
    assert lib.fluxb_ag_gemm_flag_bytes(100, 8) == 2 * 8 * 1 * 64 * 4
    assert lib.fluxb_ag_gemm_scale_bytes(4096) == 2 * 4096 * 4
    # fp32 partial tiles, two parities
    assert lib.fluxb_gemm_rs_stage_bytes(4096, 12288, 8) == 2 * 4096 * 12288 * 4
    assert lib.fluxb_gemm_rs_cnt_bytes(4096, 12288, 8) == 2 * 3 * 4 * (12288 // 64) * 4  # early, ready, late


def test_no_gpu_means_loud_failure():
    """Without a usable device the library refuses to create a communicator (no CPU fallback)."""
    import torch

    if torch.cuda.is_available():
        return
    lib = _lib.load()
    h = C.c_void_p()
    rc = lib.fluxb_comm_create(0, 1, C.byref(h))
    assert rc != _lib.FLUXB_OK
    assert _lib.last_error() != ""
    assert lib.fluxb_device_supported() == 0


def test_python_api_surface():
    """Names a user of the reference's fused path imports (python/flux/cpp_mod.py:96-196)."""
    import flux_b200 as flux

    for name in ["AGKernel", "GemmRS", "GemmGroupedV3AGScatter", "GemmGroupedV3GatherRS", "AllGatherOption",
                 "ReduceScatterOption", "AGRingMode", "RingMode", "DistEnvTP", "DistEnvTPWithEP", "MoeArguments",
                 "init_flux_shm", "flux_create_tensor_list", "create_tensor_list", "GroupBarrier", "bitwise_check",
                 "uniform_initialize", "calc_scatter_index", "ProfilingContext", "bench_func", "torch_allclose",
                 "is_fp8_dtype", "get_arch", "group_profile"]:
        assert hasattr(flux, name), name
    opt = flux.AllGatherOption()
    assert opt.mode is None and opt.use_read is None
    assert flux.AGRingMode.All2All == 0 and flux.RingMode.Ring2D == 2
