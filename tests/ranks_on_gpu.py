"""Harness for running all ranks of a fused op on ONE GPU through the C ABI.

Each rank gets its own communicator (rank r of world n) and its own op handle; the "symmetric" buffers are n
local allocations whose pointers fill the per-rank tables exactly as mapped peer pointers would. The forward
calls queue their work (`fluxb_comm_set_ranks_on_gpu`) and `run()` issues all ranks' fused launches as one
cooperative launch (`fluxb_run_ranks`), so the pushes, arrival counters and owner-side sums run through the
same device code as on n GPUs."""
import ctypes as C

import torch

from flux_b200 import _lib
from flux_b200.shm import fluxb_dtype


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class Ranks:
    def __init__(self, n, timeout_ms=4000):
        self.n = n
        self.lib = _lib.load()
        self.comms = []
        for r in range(n):
            h = C.c_void_p()
            _lib.check(self.lib.fluxb_comm_create(r, n, C.byref(h)))
            _lib.check(self.lib.fluxb_comm_set_timeout_ms(h, timeout_ms))
            _lib.check(self.lib.fluxb_comm_set_ranks_on_gpu(h, n))
            self.comms.append(h)
        self._keep = []

    def close(self):
        for h in self.comms:
            self.lib.fluxb_comm_destroy(h)
        self.comms = []

    def symm(self, nbytes):
        """n zero-filled allocations and the pointer table every rank is given."""
        bufs = [torch.zeros(max(int(nbytes), 16), dtype=torch.uint8, device="cuda") for _ in range(self.n)]
        self._keep.append(bufs)
        return bufs, _lib.ptr_table([b.data_ptr() for b in bufs])

    def run(self):
        arr = (C.c_void_p * self.n)(*[h.value for h in self.comms])
        _lib.check(self.lib.fluxb_run_ranks(arr, self.n, _stream()))
        torch.cuda.synchronize()
        for r, h in enumerate(self.comms):
            s = C.c_int(0)
            _lib.check(self.lib.fluxb_status_peek(h, C.byref(s)))
            assert s.value == 0, f"rank {r}: device status {s.value} ({_lib.STATUS_NAMES.get(s.value)})"

    # ------------------------------------------------------------------ ops
    def ag_gemm_ops(self, full_m, n_dim, k_dim, in_dtype, out_dtype, with_scales=False):
        lib = self.lib
        in_dt, out_dt = fluxb_dtype(in_dtype), fluxb_dtype(out_dtype)
        _, gt = self.symm(lib.fluxb_ag_gemm_gather_bytes(full_m, k_dim, in_dt))
        _, ft = self.symm(lib.fluxb_ag_gemm_flag_bytes(full_m, self.n))
        st = self.symm(lib.fluxb_ag_gemm_scale_bytes(full_m))[1] if with_scales else None
        ops = []
        for r in range(self.n):
            h = C.c_void_p()
            _lib.check(lib.fluxb_ag_gemm_create(self.comms[r], full_m, n_dim, k_dim, in_dt, out_dt, gt, ft, st, C.byref(h)))
            ops.append(h)
        return ops

    def ag_gemm_forward(self, ops, shards, weights, outs, biases=None, bias_mode=0, scales_a=None, scales_b=None,
                        gathered=None, tuning=None, flags=0):
        m_local, k = shards[0].shape
        n = weights[0].shape[1] if flags & _lib.WEIGHT_KN else weights[0].shape[0]
        tun = C.byref(_lib.make_tuning(tuning)) if tuning else None
        for r in range(self.n):
            _lib.check(self.lib.fluxb_ag_gemm_forward(
                ops[r], _p(shards[r]), m_local, _p(weights[r]), n, k, _p(outs[r]),
                _p(biases[r]) if biases else None, bias_mode,
                _p(scales_a[r]) if scales_a else None, _p(scales_b[r]) if scales_b else None, 1.0, flags,
                _p(gathered[r]) if gathered else None, tun, _stream()))
        self.run()

    def gemm_rs_ops(self, max_m, n_dim, in_dtype, out_dtype):
        lib = self.lib
        _, st = self.symm(lib.fluxb_gemm_rs_stage_bytes(max_m, n_dim, self.n))
        _, ct = self.symm(lib.fluxb_gemm_rs_cnt_bytes(max_m, n_dim, self.n))
        ops = []
        for r in range(self.n):
            h = C.c_void_p()
            _lib.check(lib.fluxb_gemm_rs_create(self.comms[r], max_m, n_dim, fluxb_dtype(in_dtype), fluxb_dtype(out_dtype),
                                                st, ct, C.byref(h)))
            ops.append(h)
        return ops

    def gemm_rs_forward(self, ops, inputs, weights, outs, biases=None, scales_a=None, scales_b=None, flags=0, tuning=None):
        m, k_local = inputs[0].shape
        n = weights[0].shape[0]
        tun = C.byref(_lib.make_tuning(tuning)) if tuning else None
        for r in range(self.n):
            _lib.check(self.lib.fluxb_gemm_rs_forward(
                ops[r], _p(inputs[r]), _p(weights[r]), m, n, k_local, _p(outs[r]),
                _p(biases[r]) if biases else None, _lib.BIAS_MN if biases else _lib.BIAS_NONE,
                _p(scales_a[r]) if scales_a else None, _p(scales_b[r]) if scales_b else None, 1.0, flags, tun, _stream()))
        self.run()

    def moe_ops(self, max_ntokens, hidden, ffn_local, nexperts, topk, dtype, ep_size=1):
        """Layer-0 and layer-1 op handles of every rank; with ep_size > 1 rank r belongs to expert group
        r // (n / ep_size) and `ffn_local` is the ffn share inside a group."""
        lib = self.lib
        dt = fluxb_dtype(dtype)
        _, gt = self.symm(lib.fluxb_ag_gemm_gather_bytes(max_ntokens, hidden, dt))
        _, ft = self.symm(lib.fluxb_ag_gemm_flag_bytes(max_ntokens, self.n))
        max_m = max_ntokens * topk
        _, st = self.symm(lib.fluxb_moe_gather_rs_stage_bytes(max_m, hidden, topk, self.n))
        _, ct = self.symm(lib.fluxb_moe_gather_rs_cnt_bytes(max_m, hidden, topk, self.n))
        l0, l1 = [], []
        for r in range(self.n):
            ws0 = torch.zeros(lib.fluxb_moe_ag_scatter_workspace_bytes(max_ntokens, topk, nexperts, hidden, dt),
                              dtype=torch.uint8, device="cuda")
            ws1 = torch.zeros(lib.fluxb_moe_gather_rs_workspace_bytes(max_m, hidden, topk, nexperts),
                              dtype=torch.uint8, device="cuda")
            self._keep.append((ws0, ws1))
            h0, h1 = C.c_void_p(), C.c_void_p()
            _lib.check(lib.fluxb_moe_ag_scatter_create(self.comms[r], max_ntokens, hidden, ffn_local, nexperts, topk, dt, dt,
                                                       gt, ft, _p(ws0), C.byref(h0)))
            _lib.check(lib.fluxb_moe_gather_rs_create(self.comms[r], nexperts, max_m, hidden, topk, dt, dt, st, ct, _p(ws1),
                                                      C.byref(h1)))
            if ep_size > 1:
                _lib.check(lib.fluxb_moe_ag_scatter_set_ep(h0, r // (self.n // ep_size), ep_size))
                _lib.check(lib.fluxb_moe_gather_rs_set_ep(h1, r // (self.n // ep_size), ep_size))
            l0.append(h0)
            l1.append(h1)
        return l0, l1

    def moe_l0_forward(self, ops, tokens, weights, splits_dev, scatter_index, outs, out_scales=None, gathered=None,
                       tuning=None):
        nlocal = tokens[0].shape[0]
        tun = C.byref(_lib.make_tuning(tuning)) if tuning else None
        for r in range(self.n):
            _lib.check(self.lib.fluxb_moe_ag_scatter_forward(
                ops[r], _p(tokens[r]), nlocal, _p(weights[r]), _p(splits_dev), _p(scatter_index),
                _p(out_scales[r]) if out_scales else None, _p(outs[r]), _p(gathered[r]) if gathered else None, tun, _stream()))
        self.run()

    def moe_l1_forward(self, ops, xs, weights, splits_cpu, routing_idx, outs, vec_scale=None, vec_scales=None):
        """`vec_scale`: one row-scale vector for every rank; `vec_scales`: one per rank (expert parallelism: every
        rank holds different rows)."""
        topk = routing_idx.numel() // (outs[0].shape[0] * self.n)
        ntokens = routing_idx.numel() // topk
        for r in range(self.n):
            m, k_local = xs[r].shape
            vs = vec_scales[r] if vec_scales is not None else vec_scale
            _lib.check(self.lib.fluxb_moe_gather_rs_forward_ep(
                ops[r], _p(xs[r]), m, ntokens, k_local, _p(weights[r]), C.c_void_p(splits_cpu.data_ptr()), _p(routing_idx),
                None, None, _p(vs), _p(outs[r]), None, _stream()))
        self.run()
