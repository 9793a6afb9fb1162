"""Symmetric memory, communicator and barrier for one process per GPU.

Host-side mirror of the reference's runtime (`src/ths_op/flux_shm.cc`):
`init_flux_shm` (:379-408), `flux_create_tensor_list` (:434-452, cudaIpc
variant :275-366) and `GroupBarrier` (:656-733). Allocation, IPC export and
mapping are done by the native library; the only cross-process step, the
exchange of the 64-byte handles, goes through the caller's process group
(`all_gather_object`, any backend), as `Group::all_gather_cpu` does in the
reference (`flux_shm.cc:161-168`). No NVSHMEM and no NCCL call is made here.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib

_TORCH_TO_FLUXB = {
    torch.bfloat16: _lib.BF16,
    torch.float16: _lib.F16,
    torch.float32: _lib.F32,
    torch.int8: _lib.S8,
}
if hasattr(torch, "float8_e4m3fn"):
    _TORCH_TO_FLUXB[torch.float8_e4m3fn] = _lib.E4M3
    _TORCH_TO_FLUXB[torch.float8_e5m2] = _lib.E5M2


def fluxb_dtype(dt: torch.dtype) -> int:
    try:
        return _TORCH_TO_FLUXB[dt]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {dt}") from None


class _CudaArray:
    """Exposes raw device memory to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }
        self._owner = owner


def tensor_from_ptr(ptr: int, shape: Sequence[int], dtype: torch.dtype, device, owner=None) -> torch.Tensor:
    nbytes = int(torch.empty((), dtype=dtype).element_size())
    for s in shape:
        nbytes *= int(s)
    if nbytes == 0:
        return torch.empty(tuple(shape), dtype=dtype, device=device)
    raw = torch.as_tensor(_CudaArray(ptr, nbytes, owner), device=device)
    return raw.view(dtype).view(*shape)


class SymmBuffer:
    """One symmetric allocation: the local block plus every peer's mapping."""

    def __init__(self, comm: "Comm", nbytes: int):
        lib = _lib.load()
        self.comm = comm
        self.nbytes = int(nbytes)
        local = C.c_void_p()
        handle = (C.c_ubyte * _lib.IPC_HANDLE_BYTES)()
        _lib.check(lib.fluxb_symm_alloc(self.nbytes, C.byref(local), handle if comm.world > 1 else None))
        self.local_ptr = int(local.value)
        self.ptrs: List[int] = [0] * comm.world
        self.ptrs[comm.rank] = self.local_ptr
        self._opened: List[int] = []
        if comm.world > 1:
            blobs: List[Optional[bytes]] = [None] * comm.world
            dist.all_gather_object(blobs, bytes(handle), group=comm.group)
            for r, blob in enumerate(blobs):
                if r == comm.rank:
                    continue
                buf = (C.c_ubyte * _lib.IPC_HANDLE_BYTES).from_buffer_copy(blob)
                peer = C.c_void_p()
                _lib.check(lib.fluxb_symm_open(buf, C.byref(peer)))
                self.ptrs[r] = int(peer.value)
                self._opened.append(int(peer.value))
        self._finalizer = weakref.finalize(self, SymmBuffer._release, self.local_ptr, list(self._opened))

    @staticmethod
    def _release(local_ptr: int, opened: List[int]) -> None:
        try:
            lib = _lib.load()
            for p in opened:
                lib.fluxb_symm_close(C.c_void_p(p))
            lib.fluxb_symm_free(C.c_void_p(local_ptr))
        except Exception:
            pass

    def table(self):
        return _lib.ptr_table(self.ptrs)

    def tensor(self, rank: int, shape, dtype) -> torch.Tensor:
        return tensor_from_ptr(self.ptrs[rank], shape, dtype, self.comm.device, owner=self)


class Comm:
    """Per-process-group state: native communicator, sync array, status word."""

    def __init__(self, group):
        lib = _lib.load()
        self.group = group
        if group is None or not dist.is_initialized():
            self.rank, self.world = 0, 1
        else:
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if not torch.cuda.is_available():
            raise RuntimeError("flux_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.device = torch.device("cuda", torch.cuda.current_device())
        h = C.c_void_p()
        _lib.check(lib.fluxb_comm_create(self.rank, self.world, C.byref(h)))
        self.handle = h
        self._finalizer = weakref.finalize(self, Comm._release, h)
        self.sync = SymmBuffer(self, 2 * _lib.MAX_WORLD * 4)
        self.host_barrier()

    @staticmethod
    def _release(h) -> None:
        try:
            _lib.load().fluxb_comm_destroy(h)
        except Exception:
            pass

    def host_barrier(self) -> None:
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)

    def barrier_on_stream(self, stream: Optional[int] = None) -> None:
        lib = _lib.load()
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        _lib.check(lib.fluxb_barrier_all(self.handle, self.sync.table(), C.c_void_p(st)))

    def set_timeout_ms(self, ms: int) -> None:
        _lib.check(_lib.load().fluxb_comm_set_timeout_ms(self.handle, int(ms)))

    def enable_trace(self, on: bool = True):
        """Per-CTA timeline of the fused kernel (see fluxb_comm_set_trace): returns the [SMs, 8] int64
        tensor later launches fill with %globaltimer stamps, or None when switched off."""
        if not on:
            _lib.check(_lib.load().fluxb_comm_set_trace(self.handle, None))
            self._trace = None
            return None
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._trace = torch.zeros((sms, 8), dtype=torch.int64, device=self.device)
        _lib.check(_lib.load().fluxb_comm_set_trace(self.handle, self._trace.data_ptr()))
        return self._trace

    def status(self) -> int:
        s = C.c_int(0)
        _lib.check(_lib.load().fluxb_status_peek(self.handle, C.byref(s)))
        return s.value

    def clear_status(self) -> None:
        _lib.check(_lib.load().fluxb_status_clear(self.handle))

    def check_status(self) -> None:
        """Raise if a bounded device wait expired (call after a synchronize)."""
        s = self.status()
        if s != 0:
            raise _lib.FluxbError(_lib.FLUXB_ERR_TIMEOUT, _lib.STATUS_NAMES.get(s, f"device status {s}"))


_COMMS: Dict[int, Comm] = {}
_LAST: List[Comm] = []


def get_comm(group) -> Comm:
    key = id(group) if group is not None else 0
    c = _COMMS.get(key)
    if c is None:
        c = Comm(group)
        _COMMS[key] = c
    _LAST[:] = [c]
    return c


def default_comm() -> Comm:
    """Communicator of the most recent `init_flux_shm` / `get_comm` call (ops whose constructor takes
    no process group bind to it, as the reference binds to its global NVSHMEM state)."""
    if not _LAST:
        raise RuntimeError("call flux.init_flux_shm(process_group) first")
    return _LAST[0]


def init_flux_shm(pg) -> None:
    """`flux.init_flux_shm(pg)` (src/pybind/ths_op.cc:209-211): set up the communicator of `pg`."""
    get_comm(pg)


def flux_create_tensor_list(shape, dtype, pg, ring_mode: bool = False, init_zero: bool = False) -> List[torch.Tensor]:
    """`flux.flux_create_tensor_list` (src/pybind/ths_op.cc:212-224): one tensor per rank, all on
    symmetric memory; entry `rank` is local, the others are the peers' blocks mapped here."""
    comm = get_comm(pg)
    nbytes = int(torch.empty((), dtype=dtype).element_size())
    for s in shape:
        nbytes *= int(s)
    buf = SymmBuffer(comm, max(nbytes, 16))
    return [buf.tensor(r, shape, dtype) for r in range(comm.world)]


class GroupBarrier:
    """`flux.GroupBarrier(process_group, ring_mode=False)` (src/ths_op/flux_shm.cc:656-733)."""

    def __init__(self, process_group, ring_mode: bool = False):
        self._comm = get_comm(process_group)

    def barrier_all(self, stream: Optional[int] = None) -> None:
        self._comm.barrier_on_stream(stream)
