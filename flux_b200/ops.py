"""Torch-facing ops with the reference's names, arguments and error behaviour.

Mirrors the pybind classes of the reference:
  AGKernel  - src/pybind/ag_gemm.cc:31-103  (AllGatherGemmOp, src/ag_gemm/ths_op/all_gather_gemm_op.cc)
  GemmRS    - src/pybind/gemm_rs.cc:30-102  (GemmRS, src/gemm_rs/ths_op/gemm_reduce_scatter.cc)
  option / env carriers - src/pybind/ths_op.cc:94-179
Each forward is one call into the C ABI (`include/fluxb.h`) on the current
CUDA stream; tensors are only used for their device pointers and shapes.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import List, Optional

import torch

from . import _lib
from . import tune as _tune
from .shm import Comm, SymmBuffer, default_comm, fluxb_dtype, get_comm


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def is_fp8_dtype(dt: torch.dtype) -> bool:
    return dt in (getattr(torch, "float8_e4m3fn", None), getattr(torch, "float8_e5m2", None))


def is_s8_dtype(dt: torch.dtype) -> bool:
    return dt == torch.int8


def _is_8bit(dt: torch.dtype) -> bool:
    return is_fp8_dtype(dt) or is_s8_dtype(dt)


def _cur_stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _tuning(t) -> Optional[C.Array]:
    if t is None:
        return None
    if isinstance(t, _lib.Tuning):
        return C.byref(t)
    return C.byref(_lib.make_tuning(t))


class AGRingMode(enum.IntEnum):
    """src/coll/ths_op/all_gather_types.h:26-30"""

    All2All = 0
    Ring1D = 1
    Ring2D = 2


class RingMode(enum.IntEnum):
    """src/coll/ths_op/reduce_scatter_op.h:26-30"""

    All2All = 0
    Ring1D = 1
    Ring2D = 2


class AllGatherOption:
    """All fields optional (src/coll/ths_op/all_gather_types.h:35-43). `use_cuda_core_ag` chooses the transport
    of the all-gather as in the reference: True = pushed by the communication warps of the fused kernel, False =
    copy engines on a side stream, None = the library's default. On an NVSwitch domain the transfer is always a
    direct all-to-all; the PCIe-oriented knobs (ring modes, `use_read`) are accepted and ignored."""

    def __init__(self):
        self.input_buffer_copied = None
        self.use_cuda_core_local = None
        self.use_cuda_core_ag = None
        self.fuse_sync = None
        self.use_read = None
        self.mode = None

    def __repr__(self):
        return (
            f"AllGatherOption(mode={self.mode!r}, fuse_sync={self.fuse_sync}, "
            f"use_cuda_core_local={self.use_cuda_core_local}, use_cuda_core_ag={self.use_cuda_core_ag}, "
            f"input_buffer_copied={self.input_buffer_copied}, use_read={self.use_read})"
        )


class ReduceScatterOption:
    """All fields optional (src/coll/ths_op/reduce_scatter_op.h:35-46); PCIe-oriented, ignored by
    the NVLink push epilogue, as they are by the reference's sm90 NVLink kernel."""

    def __init__(self):
        self.use_barrier_queue = None
        self.use_1d_ring = None
        self.use_p2p_read = None
        self.use_cudaMemcpyAsync = None
        self.use_gemmk = None
        self.per_tile_flags = None
        self.n_split = None
        self.num_blocks = None
        self.ring_mode = None


class DistEnvTP:
    """src/pybind/ths_op.cc:94-118 / include/flux/ths_op/ths_op.h:53-75"""

    def __init__(self, tp_group, nnodes: int = 1):
        comm = get_comm(tp_group)
        self.tp_group = tp_group
        self.nnodes = int(nnodes)
        self.rank = comm.rank
        self.world_size = comm.world
        _check(self.nnodes == 1, "only nnodes == 1 (one NVSwitch domain) is supported")
        self.local_world_size = self.world_size // self.nnodes
        self.local_rank = self.rank % self.local_world_size


class DistEnvTPWithEP(DistEnvTP):
    """src/ths_op/ths_op.cc:334-346"""

    def __init__(self, tp_group, nnodes: int = 1, ep_group=None):
        super().__init__(tp_group, nnodes)
        self.ep_group = ep_group
        if ep_group is None:
            self.ep_rank, self.ep_size = 0, 1
        else:
            import torch.distributed as dist

            self.ep_rank, self.ep_size = dist.get_rank(ep_group), dist.get_world_size(ep_group)
        _check(self.world_size % self.ep_size == 0, "DistEnvTPWithEP: the EP size must divide the world size")
        self.ffn_tp_size = self.world_size // self.ep_size
        self.ffn_tp_rank = self.rank % self.ffn_tp_size


class MoeArguments:
    """src/ths_op/ths_op.cc:348-375"""

    def __init__(self, max_ntokens, hidden, ffn_hidden, nexperts, topk, input_dtype, output_dtype=None):
        self.max_ntokens = int(max_ntokens)
        self.hidden = int(hidden)
        self.ffn_hidden = int(ffn_hidden)
        self.nexperts = int(nexperts)
        self.topk = int(topk)
        self.input_dtype = input_dtype
        self.output_dtype = output_dtype if output_dtype is not None else input_dtype


class TuningRecord:
    """One tuned launch configuration: the problem key (op, M, N, K, dtype, TP size - the reference's
    `UnifiedGemmMeta` + `RuntimeConfig`) and the winning `fluxb_tuning` fields (its `UnifiedGemmHParams`);
    src/ths_op/ths_op.cc:208-210 `PyTuningRecord`."""

    def __init__(self, key: str, tuning, ms: float = float("nan")):
        self.key = key
        self.tuning = dict(tuning) if tuning else None
        self.ms = float(ms)

    def __repr__(self):
        return _tune.record_line(self.key, {"tuning": self.tuning, "ms": self.ms})


def load_tuning_record(record: "TuningRecord") -> None:
    """`flux.load_tuning_record(record)` (src/ths_op/ths_op.cc:212-215): later forwards of the record's problem
    use its configuration."""
    _tune.TABLE.put(record.key, record.tuning, record.ms)


class ProfilingContext:
    """`flux.ProfilingContext(name)` (src/ths_op/ths_op.cc:217-318): collects what the `profiling()` methods
    measured. The reference records generated C++ registration code; here a record is the `fluxb_tuning` fields
    of the winner, printed as one line of text, and `get_all_records()` / `load_tuning_record` carry them into
    another process (or `flux_b200.tune.TABLE.save/load` as JSON)."""

    def __init__(self, name: str):
        self.name = name
        self.records: List[str] = []          # one line per profiled problem (the winner)
        self._results: List[tuple] = []       # (key, [(tuning, ms), ...] sorted by time)

    def add(self, key: str, table) -> "TuningRecord":
        ranked = sorted(table, key=lambda kv: kv[1])
        self._results.append((key, ranked))
        best, ms = ranked[0]
        self.records.append(_tune.record_line(key, {"tuning": best, "ms": ms}))
        return TuningRecord(key, best, ms)

    def get_code(self) -> str:
        return "\n".join(self.records)

    def get_all_record_codes(self) -> List[str]:
        return list(self.records)

    def get_all_prof_results(self, topk: int = 5) -> List[str]:
        out = []
        for key, ranked in self._results:
            lines = [key] + [f" * TopK={i + 1} ({ms:.3f} ms): {t}" for i, (t, ms) in enumerate(ranked[:topk])]
            out.append("\n".join(lines))
        return out

    def get_latest_prof_result(self) -> str:
        _check(bool(self._results), "no latest prof results found")
        return self.get_all_prof_results()[-1]

    def get_all_records(self) -> List["TuningRecord"]:
        return [TuningRecord(key, ranked[0][0], ranked[0][1]) for key, ranked in self._results]

    def get_latest_record(self):
        _check(bool(self._results), "no latest prof results found")
        return self.get_all_records()[-1]


def _profile(run, group, key: str, prof_ctx):
    """Shared body of the `profiling()` methods: sweep, remember the winner, report it, run it once more."""
    best, table = _tune.sweep(run, group)
    _tune.TABLE.put(key, best, min(ms for _, ms in table))
    if prof_ctx is not None:
        prof_ctx.add(key, table)
    return run(best)


def _out_dtype(input_dtype: torch.dtype, output_dtype: Optional[torch.dtype]) -> torch.dtype:
    # fp8 / int8 inputs produce bf16 (src/ag_gemm/ths_op/gemm_with_barrier.cc:184-185)
    if output_dtype is not None:
        return output_dtype
    return torch.bfloat16 if _is_8bit(input_dtype) else input_dtype


def _expand_scale(s: Optional[torch.Tensor], n: int, what: str) -> Optional[torch.Tensor]:
    """Scalar [1] scales (the reference's fp8 form) become a vector without a host sync; vectors
    [n], [n,1] or [1,n] (the reference's int8 form) are used as they are."""
    if s is None:
        return None
    _check(s.dtype == torch.float32, f"{what} must be float32")
    if s.numel() == 1:
        return s.reshape(1).expand(n).contiguous()
    _check(s.numel() == n, f"{what} has {s.numel()} elements, expected 1 or {n}")
    return s.reshape(n).contiguous()


class AGKernel:
    """`flux.AGKernel(tp_group, nnodes, full_m, n_dim, k_dim, input_dtype, output_dtype=None,
    use_pdl=False)` - all-gather fused into the GEMM (src/pybind/ag_gemm.cc:31-62)."""

    def __init__(self, tp_group, nnodes, full_m, n_dim, k_dim, input_dtype, output_dtype=None, use_pdl=False):
        _check(int(nnodes) == 1, "AGKernel: only nnodes == 1 is supported")
        self.comm: Comm = get_comm(tp_group)
        self.full_m, self.n_dim, self.k_dim = int(full_m), int(n_dim), int(k_dim)
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        lib = _lib.load()
        in_dt, out_dt = fluxb_dtype(input_dtype), fluxb_dtype(self.output_dtype)
        w = self.comm.world
        self._gather = SymmBuffer(self.comm, lib.fluxb_ag_gemm_gather_bytes(self.full_m, self.k_dim, in_dt))
        self._flags = SymmBuffer(self.comm, lib.fluxb_ag_gemm_flag_bytes(self.full_m, w))
        self._scales = SymmBuffer(self.comm, lib.fluxb_ag_gemm_scale_bytes(self.full_m))
        h = C.c_void_p()
        _lib.check(
            lib.fluxb_ag_gemm_create(
                self.comm.handle, self.full_m, self.n_dim, self.k_dim, in_dt, out_dt,
                self._gather.table(), self._flags.table(), self._scales.table(), C.byref(h),
            )
        )
        self._h = h
        self.comm.host_barrier()  # every rank's buffers are zeroed and mapped before the first push

    def __del__(self):
        try:
            _lib.load().fluxb_ag_gemm_destroy(self._h)
        except Exception:
            pass

    def reset(self):
        """Re-arm the op after a call that ended with a device status (a bounded wait expired): clears the
        arrival counters and restarts the buffer-parity sequence. Collective; ends with a host barrier."""
        _lib.check(_lib.load().fluxb_ag_gemm_reset(self._h, _cur_stream()))
        self.comm.host_barrier()

    def _prep(self, input, weight, bias, output, input_scale, weight_scale, output_scale, transpose_weight, world):
        _check(input.is_cuda and weight.is_cuda, "AGKernel: tensors must be CUDA tensors")
        _check(input.dim() == 2 and weight.dim() == 2, "AGKernel: input and weight must be 2-D")
        _check(input.dtype == self.input_dtype and weight.dtype == self.input_dtype, "AGKernel: dtype mismatch")
        _check(output_scale is None, "AGKernel: output_scale is not supported")
        flags = 0
        if transpose_weight:
            # weight arrives as [K, N] ("RRR"); fp8 forbids it (src/ag_gemm/ths_op/gemm_with_barrier.cc:188,196-197).
            # The kernel reads it in place as an MN-major operand: no transposing copy.
            _check(not _is_8bit(self.input_dtype), "AGKernel: 8-bit inputs do not support transpose_weight")
            flags |= _lib.WEIGHT_KN
        _check(input.is_contiguous(), "AGKernel: input must be contiguous")
        if not weight.is_contiguous():
            weight = weight.contiguous()
        m_local, k = input.shape
        n = weight.shape[1] if transpose_weight else weight.shape[0]
        wk = weight.shape[0] if transpose_weight else weight.shape[1]
        _check(wk == k, f"AGKernel: weight K {wk} != input K {k}")
        _check(k == self.k_dim, f"AGKernel: k={k} differs from k_dim={self.k_dim}")
        m = m_local * world
        _check(m <= self.full_m, f"AGKernel: M={m} exceeds full_m={self.full_m}")
        if output is None:
            output = torch.empty((m, n), dtype=self.output_dtype, device=input.device)
        else:
            _check(tuple(output.shape) == (m, n) and output.dtype == self.output_dtype and output.is_contiguous(),
                   "AGKernel: output has the wrong shape, dtype or layout")
        bias_mode = _lib.BIAS_NONE
        if bias is not None:
            _check(bias.dtype == self.output_dtype and bias.is_contiguous(), "AGKernel: bias dtype/layout")
            if tuple(bias.shape) == (m, n):
                bias_mode = _lib.BIAS_MN
            elif tuple(bias.shape) == (1, n) or tuple(bias.shape) == (n,):
                bias_mode = _lib.BIAS_1N
            else:
                raise RuntimeError(f"AGKernel: bias shape {tuple(bias.shape)} is neither [M,N] nor [1,N]")
        return input, weight, output, bias_mode, m_local, n, k, flags

    def forward(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None,
                output_scale=None, fast_accum=False, transpose_weight=False, all_gather_option=None,
                gathered_input=None, tuning=None):
        w = self.comm.world
        input, weight, output, bias_mode, m_local, n, k, flags = self._prep(
            input, weight, bias, output, input_scale, weight_scale, output_scale, transpose_weight, w)
        sa = _expand_scale(input_scale, m_local, "input_scale")
        sb = _expand_scale(weight_scale, n, "weight_scale")
        if gathered_input is not None:
            _check(tuple(gathered_input.shape) == (m_local * w, k) and gathered_input.dtype == self.input_dtype
                   and gathered_input.is_contiguous(), "AGKernel: gathered_input has the wrong shape, dtype or layout")
        if tuning is None and _tune.TABLE.records:
            tuning = _tune.TABLE.get(_tune.record_key("ag_gemm", m_local * w, n, k, self.input_dtype, w))
        if all_gather_option is not None and all_gather_option.use_cuda_core_ag is not None:
            tuning = dict(tuning) if isinstance(tuning, dict) else {}
            tuning["ag_mode"] = _lib.AG_MODE_KERNEL_PUSH if all_gather_option.use_cuda_core_ag else _lib.AG_MODE_COPY_ENGINE
        lib = _lib.load()
        _lib.check(
            lib.fluxb_ag_gemm_forward(
                self._h, input.data_ptr(), m_local, weight.data_ptr(), n, k, output.data_ptr(), _ptr(bias),
                bias_mode, _ptr(sa), _ptr(sb), 1.0, flags, _ptr(gathered_input), _tuning(tuning), _cur_stream(),
            )
        )
        return output

    def gemm_only(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None,
                  output_scale=None, fast_accum=False, transpose_weight=False, tuning=None):
        """Same kernel without communication: `input` is the full [M,K] matrix
        (src/ag_gemm/ths_op/all_gather_gemm_op.cc:166-194)."""
        input, weight, output, bias_mode, m, n, k, flags = self._prep(
            input, weight, bias, output, input_scale, weight_scale, output_scale, transpose_weight, 1)
        sa = _expand_scale(input_scale, m, "input_scale")
        sb = _expand_scale(weight_scale, n, "weight_scale")
        lib = _lib.load()
        _lib.check(
            lib.fluxb_gemm(
                self.comm.handle, input.data_ptr(), weight.data_ptr(), output.data_ptr(), m, n, k,
                fluxb_dtype(self.input_dtype), fluxb_dtype(self.output_dtype), _ptr(bias), bias_mode,
                _ptr(sa), _ptr(sb), 1.0, flags, _tuning(tuning), _cur_stream(),
            )
        )
        return output

    def profiling(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None,
                  output_scale=None, fast_accum=False, transpose_weight=False, all_gather_option=None,
                  gathered_input=None, prof_ctx=None):
        """Sweep the tile shapes for this problem (every rank times every candidate, the slowest rank
        decides), remember the winner for later `forward` calls of the same shape, add it to `prof_ctx`
        and return the output computed with it (src/ag_gemm/ths_op/all_gather_gemm_op.cc:361-474)."""
        w = self.comm.world
        n = weight.shape[1] if transpose_weight else weight.shape[0]
        key = _tune.record_key("ag_gemm", input.shape[0] * w, n, input.shape[1], self.input_dtype, w)

        def run(t):
            return self.forward(input, weight, bias, output, input_scale, weight_scale, output_scale, fast_accum,
                                transpose_weight, all_gather_option, gathered_input, tuning=t if t else {})

        return _profile(run, self.comm.group, key, prof_ctx)


class GemmRS:
    """`flux.GemmRS(tp_group, nnodes, max_m, n_dim, input_dtype, output_dtype=None,
    transpose_weight=False, fuse_reduction=False, ring_reduction=False)` - reduce-scatter fused into
    the GEMM epilogue (src/pybind/gemm_rs.cc:30-60).

    Partial products travel to the rank that owns their rows in the 16-bit output format (one rounding per
    partial, as in the reference, whose reduce buffer has the output dtype) and are summed there in fp32 in a
    fixed order (the peers that delivered early, summed by the communication warps; then the own fp32 partial;
    then the peers that deliver last, added by the epilogue of the own tiles) and rounded once.
    `ring_reduction=True` sums in the order rank+1, rank+2, ..., own partial last, and rounds the sum to the
    element type after every addition, which is what the reference's `ring_reduce` kernel computes
    (src/gemm_rs/ring_reduce.cu:54-80). `fuse_reduction` asks the reference for
    an in-kernel reduction; here the reduction is always inside the kernel, so the flag changes nothing.
    `fp32_wire = True` sends the partials as fp32 instead (no rounding before the sum, twice the NVLink bytes).
    Rounding points against the 1e-2 tolerance: one per partial + one at the end (default)."""

    def __init__(self, tp_group, nnodes, max_m, n_dim, input_dtype, output_dtype=None, transpose_weight=False,
                 fuse_reduction=False, ring_reduction=False):
        _check(int(nnodes) == 1, "GemmRS: only nnodes == 1 is supported")
        self.comm: Comm = get_comm(tp_group)
        self.max_m, self.n_dim = int(max_m), int(n_dim)
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        self.transpose_weight = bool(transpose_weight)
        self.ring_reduction = bool(ring_reduction)
        self.fuse_reduction = bool(fuse_reduction)
        self.fp32_wire = False
        lib = _lib.load()
        w = self.comm.world
        self._stage = SymmBuffer(self.comm, lib.fluxb_gemm_rs_stage_bytes(self.max_m, self.n_dim, w))
        self._cnt = SymmBuffer(self.comm, lib.fluxb_gemm_rs_cnt_bytes(self.max_m, self.n_dim, w))
        h = C.c_void_p()
        _lib.check(
            lib.fluxb_gemm_rs_create(
                self.comm.handle, self.max_m, self.n_dim, fluxb_dtype(input_dtype), fluxb_dtype(self.output_dtype),
                self._stage.table(), self._cnt.table(), C.byref(h),
            )
        )
        self._h = h
        self.comm.host_barrier()

    def __del__(self):
        try:
            _lib.load().fluxb_gemm_rs_destroy(self._h)
        except Exception:
            pass

    def forward(self, input, weight, bias=None, input_scale=None, weight_scale=None, output_scale=None,
                fast_accum=False, reduce_scatter_option=None, tuning=None, output=None):
        """`output` (not in the reference, which returns a tensor derived from its internal buffers): an optional
        [M/TP, N] tensor to write into, for callers that must not allocate inside a timed or captured region."""
        _check(input.is_cuda and weight.is_cuda, "GemmRS: tensors must be CUDA tensors")
        _check(input.dim() == 2 and weight.dim() == 2, "GemmRS: input and weight must be 2-D")
        _check(input.dtype == self.input_dtype and weight.dtype == self.input_dtype, "GemmRS: dtype mismatch")
        _check(output_scale is None, "GemmRS: output_scale is not supported")
        flags = 0
        if self.transpose_weight:
            _check(not _is_8bit(self.input_dtype), "GemmRS: 8-bit inputs do not support transpose_weight")
            flags |= _lib.WEIGHT_KN  # [K, N] weight read in place as an MN-major operand
        if self.fp32_wire:
            flags |= _lib.RS_FP32_WIRE
        if self.ring_reduction:
            flags |= _lib.RS_RING_ORDER
        if not weight.is_contiguous():
            weight = weight.contiguous()
        _check(input.is_contiguous(), "GemmRS: input must be contiguous")
        m, k = input.shape
        n = weight.shape[1] if self.transpose_weight else weight.shape[0]
        wk = weight.shape[0] if self.transpose_weight else weight.shape[1]
        w = self.comm.world
        _check(wk == k, f"GemmRS: weight K {wk} != input K {k}")
        # shape rules of src/gemm_rs/ths_op/gemm_reduce_scatter.cc:499-504
        _check(m <= self.max_m, f"GemmRS: M={m} exceeds max_m={self.max_m}")
        _check(n == self.n_dim, f"GemmRS: N={n} differs from n_dim={self.n_dim}")
        _check(m % w == 0, f"GemmRS: M={m} is not a multiple of the world size {w}")
        bias_mode = _lib.BIAS_NONE
        if bias is not None:
            # fp8 rejects bias (gemm_reduce_scatter.cc:601-603)
            _check(not is_fp8_dtype(self.input_dtype), "GemmRS: fp8 does not support bias")
            _check(bias.dtype == self.output_dtype and bias.is_contiguous(), "GemmRS: bias dtype/layout")
            if tuple(bias.shape) == (m, n):
                bias_mode = _lib.BIAS_MN
            elif tuple(bias.shape) in ((1, n), (n,)):
                # the int8 form: [1,N], applied by rank 0 only (gemm_reduce_scatter.cc:596-599)
                bias_mode = _lib.BIAS_1N
            else:
                raise RuntimeError(f"GemmRS: bias shape {tuple(bias.shape)} is neither [M,N] nor [1,N]")
        sa = _expand_scale(input_scale, m, "input_scale")
        sb = _expand_scale(weight_scale, n, "weight_scale")
        if output is None:
            out = torch.empty((m // w, n), dtype=self.output_dtype, device=input.device)
        else:
            _check(tuple(output.shape) == (m // w, n) and output.dtype == self.output_dtype and output.is_contiguous(),
                   "GemmRS: output has the wrong shape, dtype or layout")
            out = output
        if tuning is None and _tune.TABLE.records:
            tuning = _tune.TABLE.get(_tune.record_key("gemm_rs", m, n, k, self.input_dtype, w))
        lib = _lib.load()
        _lib.check(
            lib.fluxb_gemm_rs_forward(
                self._h, input.data_ptr(), weight.data_ptr(), m, n, k, out.data_ptr(), _ptr(bias), bias_mode,
                _ptr(sa), _ptr(sb), 1.0, flags, _tuning(tuning), _cur_stream(),
            )
        )
        return out

    def forward_barrier(self, *args, **kwargs):
        """`GemmRS.forward_barrier` (src/pybind/gemm_rs.cc:61-75) is the all-rank stream barrier the reference
        puts before its GEMM. The push epilogue needs none (counters are double-buffered by call parity), so
        this only issues the library's barrier on the current stream for callers that rely on the ordering."""
        self.comm.barrier_on_stream()

    def forward_reduce_scatter(self, *args, **kwargs):
        raise RuntimeError("GemmRS.forward_reduce_scatter: the reduction is fused; call forward()")

    def zero_buffers(self):
        """`GemmRS.zero_buffers` (gemm_reduce_scatter.cc:654-657): clears the arrival counters and ready flags
        of both buffer parities and restarts the parity sequence. In normal operation the counters clear
        themselves; this is the recovery call after a bounded wait expired. Collective; ends with a host barrier."""
        _lib.check(_lib.load().fluxb_gemm_rs_reset(self._h, _cur_stream()))
        self.comm.host_barrier()

    reset = zero_buffers

    def profiling(self, input, weight, bias=None, input_scale=None, weight_scale=None, output_scale=None,
                  fast_accum=False, prof_ctx=None, reduce_scatter_option=None):
        """Sweep the tile shapes for this problem; see `AGKernel.profiling`
        (src/gemm_rs/ths_op/gemm_reduce_scatter.cc:902-960)."""
        m, k = input.shape
        n = weight.shape[1] if self.transpose_weight else weight.shape[0]
        key = _tune.record_key("gemm_rs", m, n, k, self.input_dtype, self.comm.world)

        def run(t):
            return self.forward(input, weight, bias, input_scale, weight_scale, output_scale, fast_accum,
                                reduce_scatter_option, tuning=t if t else {})

        return _profile(run, self.comm.group, key, prof_ctx)


class GemmOnly:
    """`flux.GemmOnly(input_dtype, output_dtype=None, transpose_weight=False, use_fp8_gemm=False)`: the plain
    GEMM the reference uses as its unfused building block (src/pybind/gemm_only.cc; shapes and formulas in
    python/flux/cpp_mod.pyi:215-253): output = input[M,K] @ weight[N,K].T (weight [K,N] if transpose_weight),
    fp8 with scalar or per-row / per-channel scales, int8 (w8a8) with per-row x per-channel dequantisation, bias [M,N]
    (16-bit) or [1,N]. Same kernel as the fused ops, without communication."""

    def __init__(self, input_dtype, output_dtype=None, transpose_weight=False, use_fp8_gemm=False):
        _check(input_dtype in (torch.bfloat16, torch.float16) or _is_8bit(input_dtype),
               f"GemmOnly: input dtype {input_dtype} is not supported (bf16, fp16, fp8, int8)")
        _check(not (transpose_weight and _is_8bit(input_dtype)), "GemmOnly: 8-bit inputs do not support transpose_weight")
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        self.transpose_weight = bool(transpose_weight)
        try:
            self.comm: Comm = default_comm()
        except RuntimeError:
            self.comm = get_comm(None)

    def forward(self, input, weight, bias=None, output_buf=None, input_scale=None, weight_scale=None,
                output_scale=None, fast_accum=False, tuning=None):
        _check(input.is_cuda and weight.is_cuda, "GemmOnly: tensors must be CUDA tensors")
        _check(input.dim() == 2 and weight.dim() == 2, "GemmOnly: input and weight must be 2-D")
        _check(input.dtype == self.input_dtype and weight.dtype == self.input_dtype, "GemmOnly: dtype mismatch")
        _check(output_scale is None, "GemmOnly: output_scale is not supported")
        _check(input.is_contiguous(), "GemmOnly: input must be contiguous")
        if not weight.is_contiguous():
            weight = weight.contiguous()
        m, k = input.shape
        n = weight.shape[1] if self.transpose_weight else weight.shape[0]
        wk = weight.shape[0] if self.transpose_weight else weight.shape[1]
        _check(wk == k, f"GemmOnly: weight K {wk} != input K {k}")
        if output_buf is None:
            output_buf = torch.empty((m, n), dtype=self.output_dtype, device=input.device)
        else:
            _check(tuple(output_buf.shape) == (m, n) and output_buf.dtype == self.output_dtype
                   and output_buf.is_contiguous(), "GemmOnly: output_buf has the wrong shape, dtype or layout")
        bias_mode = _lib.BIAS_NONE
        if bias is not None:
            _check(bias.dtype == self.output_dtype and bias.is_contiguous(), "GemmOnly: bias dtype/layout")
            if tuple(bias.shape) == (m, n):
                bias_mode = _lib.BIAS_MN
            elif tuple(bias.shape) in ((1, n), (n,)):
                bias_mode = _lib.BIAS_1N
            else:
                raise RuntimeError(f"GemmOnly: bias shape {tuple(bias.shape)} is neither [M,N] nor [1,N]")
        sa = _expand_scale(input_scale, m, "input_scale")
        sb = _expand_scale(weight_scale, n, "weight_scale")
        _lib.check(
            _lib.load().fluxb_gemm(
                self.comm.handle, input.data_ptr(), weight.data_ptr(), output_buf.data_ptr(), m, n, k,
                fluxb_dtype(self.input_dtype), fluxb_dtype(self.output_dtype), _ptr(bias), bias_mode,
                _ptr(sa), _ptr(sb), 1.0, _lib.WEIGHT_KN if self.transpose_weight else 0, _tuning(tuning),
                _cur_stream(),
            )
        )
        return output_buf

    def profiling(self, input, weight, bias=None, output_buf=None, input_scale=None, weight_scale=None,
                  output_scale=None, fast_accum=False, prof_ctx=None):
        """Sweep the tile shapes for this problem and return the output of the fastest one."""
        m, k = input.shape
        n = weight.shape[1] if self.transpose_weight else weight.shape[0]
        key = _tune.record_key("gemm_only", m, n, k, self.input_dtype, 1)

        def run(t):
            return self.forward(input, weight, bias, output_buf, input_scale, weight_scale, output_scale, fast_accum,
                                tuning=t if t else {})

        return _profile(run, None, key, prof_ctx)


def bitwise_check(a: torch.Tensor, b: torch.Tensor) -> bool:
    """`flux.bitwise_check` (src/pybind/ths_op.cc:304-306): same shape, dtype and bits."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return bool(torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)))


def uniform_initialize(t: torch.Tensor, seed: int, lo: float, hi: float) -> None:
    """`flux.uniform_initialize` (src/pybind/ths_op.cc:307-315)."""
    g = torch.Generator(device=t.device).manual_seed(int(seed))
    tmp = torch.empty(t.shape, dtype=torch.float32, device=t.device).uniform_(lo, hi, generator=g)
    t.copy_(tmp.to(t.dtype))
