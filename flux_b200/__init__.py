"""flux_b200 - B200-native (sm_100a) fused tensor-parallel GEMM ops behind the
API of bytedance/flux's fused path: `AGKernel`, `GemmRS` and the MoE grouped
ops, plus the runtime helpers their callers use. `import flux_b200 as flux`
is the intended drop-in spelling (names follow python/flux/cpp_mod.py:96-196).

The compute lives in `libfluxb.so` (hand-written CUDA behind the C ABI of
`include/fluxb.h`); there is no CPU or library fallback.
"""
from . import layers, tune, util
from ._lib import FluxbError, Tuning
from .ops import (
    AGKernel,
    AGRingMode,
    AllGatherOption,
    DistEnvTP,
    DistEnvTPWithEP,
    GemmOnly,
    GemmRS,
    MoeArguments,
    ProfilingContext,
    ReduceScatterOption,
    TuningRecord,
    load_tuning_record,
    RingMode,
    bitwise_check,
    is_fp8_dtype,
    uniform_initialize,
)
from .layers import ColumnParallelLinear, MoEMLP, RowParallelLinear, TensorParallelMLP
from .moe import GemmGroupedV3AGScatter, GemmGroupedV3GatherRS, calc_gather_index, calc_scatter_index
from .shm import GroupBarrier, default_comm, flux_create_tensor_list, get_comm, init_flux_shm
from .util import bench_func, get_arch, group_profile, torch_allclose, with_torch_deterministic

create_tensor_list = flux_create_tensor_list

__all__ = [
    "AGKernel", "AGRingMode", "AllGatherOption", "DistEnvTP", "DistEnvTPWithEP", "GemmOnly", "GemmRS", "MoeArguments",
    "ProfilingContext", "ReduceScatterOption", "RingMode", "bitwise_check", "is_fp8_dtype", "uniform_initialize",
    "GroupBarrier", "flux_create_tensor_list", "create_tensor_list", "get_comm", "init_flux_shm", "bench_func",
    "get_arch", "group_profile", "GemmGroupedV3AGScatter", "GemmGroupedV3GatherRS", "calc_scatter_index",
    "calc_gather_index", "default_comm", "torch_allclose", "with_torch_deterministic", "FluxbError", "Tuning", "util", "TuningRecord", "load_tuning_record",
    "layers", "tune", "ColumnParallelLinear", "RowParallelLinear", "TensorParallelMLP", "MoEMLP",
]
