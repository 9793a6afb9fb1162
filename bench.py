#!/usr/bin/env python
"""Headline benchmark: the dense tensor-parallel MLP of the reference's performance table
(docs/performance.md:13-20) - layer 0 = AG-GEMM (M=4096, N=49152, K=12288), layer 1 = GEMM-RS
(M=4096, N=12288, K=49152), bf16, TP = number of GPUs. One step = AGKernel.forward followed by
GemmRS.forward on its output. Global (M, N, K) are fixed, so N GPUs split the same work ("strong").

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...     # the reference's torch golden path on the host cores
    python bench.py --workload moe|fp8 ...   # the secondary workloads alone
    python bench.py --kernel-only --case d0|d1|fp8|moe   # one small single-GPU launch for profiler captures

Prints ONE JSON line on rank 0. `value` = aggregate TFLOP/s over all GPUs with inputs resident in HBM;
`e2e` = the same through host buffers (H2D of the activations and D2H of the result inside the timed
region); `roofline` = the fused kernel against the measured bf16 tensor peak, with the NVLink side taken from
the kernel's own timeline; `parity` = sampled fp64 dot products of both fused outputs, rows pushed by every
peer included; `unfused` = cuBLAS + NCCL on the same box; `cpu_baseline` = the oracle on the host cores (a
baseline, not the target); `fp8_ag_gemm` / `moe` = the two secondary configurations. A leg that fails records
`{"error": ...}` in its field; the line is printed all the same and the exit code is non-zero only when the
parity check of the headline workload fails.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
import traceback

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, N0, K0 = 4096, 49152, 12288  # layer 0: C0[M, N0/TP] = all_gather(A)[M, K0] . B0[N0/TP, K0]^T
N1, K1 = 12288, 49152           # layer 1: out[M/TP, N1] = reduce_scatter(C0[M, K1/TP] . B1[N1, K1/TP]^T)
FP8_M, FP8_N, FP8_K = 8192, 28672, 8192           # fp8 AG-GEMM configuration
MOE_T, MOE_H, MOE_E, MOE_FFN, MOE_TOPK = 8192, 4096, 8, 14336, 2   # MoE MLP configuration
SEED = 1234
FALLBACK_BF16_TFLOPS = 1590.0   # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent
NVLINK_GBS = 900.0              # nominal, per direction per GPU
CPU_SLICE = (512, 3072, 12288)  # (M, N, K) of the host-core sample, the same at every N
METRIC = "dense TP MLP (AG-GEMM + GEMM-RS) aggregate TFLOP/s"
AG_TOL, RS_TOL, FP8_TOL = 1e-2, 2e-2, 3e-2  # elementwise |x-y| <= tol + tol*|y| (the reference's own test bars)
REL_TOL = 1e-2                               # max|x-y| / max|y| for the bf16 ops


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), float(d["bf16_tflops"]), "measured"
    return FALLBACK_BF16_TFLOPS, FALLBACK_BF16_TFLOPS, "fallback"


def _env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def _err(exc):
    return {"error": f"{type(exc).__name__}: {exc}"[:400]}


def workload_name(world):
    return f"D0 AG-GEMM M={M} N={N0} K={K0} then D1 GEMM-RS M={M} N={N1} K={K1}, bf16, TP={world}"


# ----------------------------------------------------------------------------------------------
# the JSON line (pure: no GPU, no clock; tests/test_bench_line.py feeds it fake measurements)
# ----------------------------------------------------------------------------------------------
def make_line(meas):
    """Build the result line from a dict of measurements.

    Required keys: world, steps, warmup, ms_per_step, ag_ms, rs_ms, timed_region_s, peaks = (sustained, burst,
    source). Optional legs (each a dict, possibly {"error": ...}, or absent): unfused, e2e, parity, nvlink,
    cpu_baseline, clocks, fp8_ag_gemm, moe, fp8_peak_tflops, native_library, wall_ms_timed_region."""
    world = int(meas["world"])
    ms = float(meas["ms_per_step"])
    ag_ms, rs_ms = float(meas["ag_ms"]), float(meas["rs_ms"])
    sustained, burst, peak_src = meas["peaks"]
    ag_flops = 2.0 * M * (N0 // world) * K0
    rs_flops = 2.0 * M * N1 * (K1 // world)
    flops_gpu = ag_flops + rs_flops
    total_flops = flops_gpu * world
    ag_tflops = ag_flops / (ag_ms * 1e-3) / 1e12
    rs_tflops = rs_flops / (rs_ms * 1e-3) / 1e12
    # a kernel timed inside a region shorter than a second runs at burst clocks: compare it with the burst peak
    use_burst = float(meas["timed_region_s"]) < 1.0
    peak = burst if use_burst else sustained
    nvl = meas.get("nvlink")
    ag_link_s = ((world - 1) / world) * M * K0 * 2 / (NVLINK_GBS * 1e9)
    rs_link_s = ((world - 1) / world) * M * N1 * 2 / (NVLINK_GBS * 1e9)
    roofline = {
        "bound": "tensor", "achieved": ag_tflops, "peak": peak, "unit": "TFLOP/s", "frac": ag_tflops / peak,
        "frac_is": "of measured burst peak (timed region < 1 s)" if use_burst
                   else "of measured sustained peak (timed region >= 1 s)",
        "frac_of_burst_peak": ag_tflops / burst, "frac_of_sustained_peak": ag_tflops / sustained,
        "peak_burst": burst, "peak_sustained": sustained, "peak_source": f"{peak_src} cuBLAS bf16",
        "kernel": "fused_gemm_kernel (AG-GEMM launch)",
        # ncu (dram__bytes_read.sum + dram__bytes_write.sum) on the M=4096, N=6144, K=12288 launch: 712.7 MB;
        # DRAM traffic grows with the number of 6144-column blocks a launch covers
        "traffic": 712.7e6 * (N0 // world) / 6144.0,
        "traffic_source": "ncu capture of the N=6144 launch (profiles/), scaled by N/6144",
        "algorithmic_bytes": 2.0 * (M * K0 + (N0 // world) * K0 + M * (N0 // world)),
        "gemm_rs": {"achieved": rs_tflops, "frac": rs_tflops / peak},
        # the roofline time of a fused op is the slower of the tensor time and the NVLink time at 900 GB/s
        "roofline_ms": {"ag_gemm": max(ag_flops / (peak * 1e12), ag_link_s) * 1e3,
                        "gemm_rs": max(rs_flops / (peak * 1e12), rs_link_s) * 1e3},
        "nvlink": nvl,
    }
    unfused = meas.get("unfused")
    speedup = None
    if isinstance(unfused, dict) and "ms_per_step" in unfused:
        unfused = dict(unfused)
        unfused["tflops_per_gpu"] = flops_gpu / (unfused["ms_per_step"] * 1e-3) / 1e12
        speedup = unfused["ms_per_step"] / ms
    e2e = meas.get("e2e")
    if isinstance(e2e, dict) and "ms_per_step" in e2e:
        e2e = dict(e2e)
        e2e["value"] = total_flops / (e2e["ms_per_step"] * 1e-3) / 1e12
        e2e["unit"] = "TFLOP/s"
    e2e = e2e if e2e is not None else {"error": "not measured"}
    # bytes copied per step over all ranks, counted from the tensors the e2e leg copies
    e2e.setdefault("h2d_bytes_per_step", (M // world) * K0 * 2 * world)
    e2e.setdefault("d2h_bytes_per_step", (M // world) * N1 * 2 * world)
    line = {
        "metric": METRIC,
        "value": total_flops / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": int(meas["steps"]),
        "warmup": int(meas["warmup"]),
        "ms_per_step": ms,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (CPU-seeded N(0,1) activations, N(0,0.02) weights, seed = 1234 + rank; shapes of the "
                "reference's dense MLP test)",
        "config": {
            "workload": workload_name(world),
            "parallelism": f"tp{world}",
            "l2": "weights per rank (>= 302 MB) exceed the 126 MB L2 between iterations; no explicit flush",
            "settle": "every timed region (fused, unfused, end to end) is preceded by the same idle pause and 3 warm-up "
                      "steps, so no arm inherits the power-cap state of the arm before it",
        },
        "tflops_per_gpu": flops_gpu / (ms * 1e-3) / 1e12,
        "ag_gemm": {"ms": ag_ms, "tflops_per_gpu": ag_tflops},
        "gemm_rs": {"ms": rs_ms, "tflops_per_gpu": rs_tflops},
        "unfused": unfused,
        "speedup_vs_unfused": speedup,
        "e2e": e2e,
        "gpu_launches": int(meas["steps"]) * 2,
        "roofline": roofline,
        "parity": meas.get("parity"),
        "clocks": meas.get("clocks"),
        "cpu_baseline": meas.get("cpu_baseline"),
        "fp8_ag_gemm": meas.get("fp8_ag_gemm"),
        "moe": meas.get("moe"),
        "wall_ms_timed_region": meas.get("wall_ms_timed_region"),
        "native_library": meas.get("native_library"),
    }
    return line


def parity_ok(parity):
    """True unless the headline parity leg ran and found an output outside its tolerance."""
    if not isinstance(parity, dict) or "error" in parity:
        return True
    # GEMM-RS elementwise: the kernel accumulates a partial in fp32, the check in fp64, so a partial that sits on
    # a bf16 rounding boundary may round the other way (one ulp of a partial, up to 0.03 here, against a bar of
    # 0.02 for outputs near zero): isolated elements are tolerated, a pattern is not
    return bool(parity.get("ag_max_rel_err", 0.0) <= REL_TOL and parity.get("rs_max_rel_err", 0.0) <= REL_TOL
                and parity.get("ag_allclose_1e-2", True)
                and (parity.get("rs_allclose_2e-2", True) or parity.get("rs_outside_2e-2_frac", 1.0) <= 0.01))


# ----------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi in loop mode, started well before the timed region (it takes a while to come up on a
    multi-GPU box); samples are selected afterwards by their timestamps."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, t_begin, t_end):
        import datetime

        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.flush()
        rows = [l.strip().split(", ") for l in open(self.f.name) if l.strip()]
        os.unlink(self.f.name)
        sm, pw, reasons, mx = [], [], set(), None
        for r in rows:
            if len(r) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk, mxv, watts = float(r[1]), float(r[2]), float(r[3])
            except ValueError:
                continue
            if ts < t_begin - 0.02 or ts > t_end + 0.02:
                continue
            sm.append(clk)
            pw.append(watts)
            mx = mxv
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if val.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = mx
            out["power_w"] = statistics.median(pw)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def _max_over_ranks(x, world):
    if world == 1:
        return float(x)
    t = torch.tensor([x], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _randn_rows(g, rows, cols, scale, dtype, chunk=4096):
    """Seeded on the CPU in fp32 (so that every arm - CPU, unfused, fused - sees identical values), cast and
    moved to the GPU chunk by chunk to bound the host memory."""
    out = torch.empty((rows, cols), dtype=dtype, device="cuda")
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        x = torch.randn(r1 - r0, cols, generator=g)
        if scale != 1.0:
            x *= scale
        out[r0:r1].copy_(x.to(dtype))
    return out


def _make_inputs(rank, world):
    """Seeded synthetic tensors with the shapes and distributions of the reference's dense MLP test
    (A ~ N(0,1), weights ~ N(0,0.02), seed = base + rank), drawn from the CPU generator."""
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    g = torch.Generator().manual_seed(SEED + rank)
    a = _randn_rows(g, M // world, K0, 1.0, torch.bfloat16)
    b0 = _randn_rows(g, N0 // world, K0, 0.02, torch.bfloat16)
    b1 = _randn_rows(g, N1, K1 // world, 0.02, torch.bfloat16)
    return a, b0, b1


def _spread(n, count):
    """`count` indices spread over [0, n), first and last included."""
    count = min(count, n)
    if count <= 1:
        return torch.zeros(1, dtype=torch.long)
    return torch.tensor([round(i * (n - 1) / (count - 1)) for i in range(count)], dtype=torch.long)


def _cmp(got, exact, tol):
    """(max relative error, elementwise-allclose with atol = rtol = tol) of `got` against fp64 `exact`."""
    got, exact = got.double(), exact.double()
    rel = float((got - exact).abs().max() / exact.abs().max().clamp_min(1e-30))
    close = bool(((got - exact).abs() <= tol + tol * exact.abs()).all())
    return rel, close


def _all_max(vals, world):
    if world == 1:
        return [float(v) for v in vals]
    t = torch.tensor(vals, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def dense_parity(a, b0, b1, c0, out, rank, world):
    """Live parity of both fused outputs against fp64 dot products on the benchmark's own tensors.
    AG-GEMM: rows sampled from EVERY source shard (rows of peers reached this rank through the fused push).
    GEMM-RS: entries of every rank's output; each rank contributes the fp64 dot over its K slice, the sum over
    the ranks is the exact value. Two measures, as in the test suite: max|x-y| / max|y| and the reference
    tests' elementwise |x-y| <= tol + tol*|y| (1e-2 for AG, 2e-2 for RS)."""
    m_local, n_local = M // world, N0 // world
    rows_l = _spread(m_local, 8).cuda()
    cols0 = _spread(n_local, 16).cuda()
    mine = a[rows_l].contiguous()
    if world > 1:
        allrows = torch.empty((world * rows_l.numel(), K0), dtype=a.dtype, device="cuda")
        dist.all_gather_into_tensor(allrows, mine)
    else:
        allrows = mine
    exact0 = allrows.double() @ b0[cols0].double().t()
    grows = (torch.arange(world, device="cuda")[:, None] * m_local + rows_l[None, :]).reshape(-1)
    ag_rel, ag_close = _cmp(c0[grows][:, cols0], exact0, AG_TOL)
    # rows of peers only (the part that crossed NVLink)
    peer = torch.ones(world * rows_l.numel(), dtype=torch.bool, device="cuda")
    peer[rank * rows_l.numel():(rank + 1) * rows_l.numel()] = False
    ag_rel_peer = _cmp(c0[grows][peer][:, cols0], exact0[peer], AG_TOL)[0] if world > 1 else None
    cols1 = _spread(N1, 16).cuda()
    part = c0[grows].double() @ b1[cols1].double().t()   # [world*8, 16] over this rank's K slice
    # the reference's golden path rounds each rank's partial product to bf16 (torch.matmul in bf16) before the
    # reduce-scatter: the elementwise bar of its test is meant against that, the max-rel figure against fp64
    gold = part.to(torch.bfloat16).double()
    if world > 1:
        dist.all_reduce(part)
        dist.all_reduce(gold)
    lo = rank * rows_l.numel()
    got1 = out[rows_l][:, cols1]
    rs_rel, rs_close_exact = _cmp(got1, part[lo:lo + rows_l.numel()], RS_TOL)
    gold_mine = gold[lo:lo + rows_l.numel()].to(torch.bfloat16).double()
    _, rs_close = _cmp(got1, gold_mine, RS_TOL)
    rs_outside = float(((got1.double() - gold_mine).abs() > RS_TOL + RS_TOL * gold_mine.abs()).double().mean())
    ag_rel, rs_rel, ag_bad, rs_bad, rs_bad_exact, rs_outside = _all_max(
        [ag_rel, rs_rel, 0.0 if ag_close else 1.0, 0.0 if rs_close else 1.0, 0.0 if rs_close_exact else 1.0,
         rs_outside], world)
    res = {"ag_max_rel_err": ag_rel, "rs_max_rel_err": rs_rel, "ag_allclose_1e-2": ag_bad == 0.0,
           "rs_allclose_2e-2": rs_bad == 0.0, "rs_outside_2e-2_frac": rs_outside,
           "rs_allclose_2e-2_vs_fp64": rs_bad_exact == 0.0,
           "tolerance_max_rel": REL_TOL,
           "what": f"fp64 dots: AG {world * 8} rows (8 from every source shard) x 16 cols per rank; RS 8 rows x 16 "
                   f"cols of every rank's output, K slices summed over the ranks; max over ranks. max_rel_err = "
                   f"max|x-y|/max|y| against fp64; allclose = |x-y| <= t + t*|y| (AG against fp64; RS against the "
                   f"reference's golden path, which rounds every rank's partial to bf16 before the reduce-scatter)"}
    if ag_rel_peer is not None:
        res["ag_max_rel_err_peer_rows"] = _all_max([ag_rel_peer], world)[0]
    return res


def _nvlink_from_trace(comm, fn, col, nbytes, world, barrier):
    """Run `fn` once with the kernel's timeline on and derive the NVLink rate from it: bytes that crossed the
    links of this GPU divided by the time from the first CTA's start to the last CTA's stamp `col` (4 = comm
    warps done: the all-gather push is out; 3 = epilogue done: the reduce-scatter pushes are out)."""
    tr = comm.enable_trace(True)
    try:
        barrier()
        fn()
        torch.cuda.synchronize()
        t = tr.cpu().double()
    finally:
        comm.enable_trace(False)
    x = t[:, col]
    x = x[x > 0]
    if x.numel() == 0 or nbytes == 0:
        return None
    secs = float(x.max() - t[:, 0][t[:, 0] > 0].min()) * 1e-9
    secs = _max_over_ranks(secs, world)
    return {"bytes": nbytes, "seconds": secs, "gbs": nbytes / secs / 1e9, "frac_of_900": nbytes / secs / 1e9 / NVLINK_GBS}


def measure_fp8_peak():
    """fp8 tensor peak measured the way MEASURED_PEAKS.json's bf16 figure was: cuBLAS (torch._scaled_mm) on
    8192^3, best of 10, CUDA events."""
    n = 8192
    a = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
    one = torch.ones((), device="cuda")
    for _ in range(3):
        torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return 2.0 * n ** 3 / (best * 1e-3) / 1e12


def _time_loop(fn, steps, warmup, world):
    for _ in range(max(warmup, 3)):
        r = fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        r = fn()
    e1.record()
    torch.cuda.synchronize()
    return _max_over_ranks(e0.elapsed_time(e1) / steps, world), r


# ----------------------------------------------------------------------------------------------
# secondary workloads
# ----------------------------------------------------------------------------------------------
def fp8_leg(flux, comm, group, rank, world, steps, warmup):
    """FP8 e4m3 AG-GEMM (M=8192, N=28672, K=8192, TP = world) with per-row input scales (which travel with the
    shard) and per-channel weight scales applied in the epilogue; parity against fp64 dots of the dequantised
    operands, rows from every source shard; fraction of the fp8 tensor peak measured here."""
    f8 = torch.float8_e4m3fn
    m_local, n_local = FP8_M // world, FP8_N // world
    g = torch.Generator().manual_seed(SEED + 100 + rank)
    a = torch.randn(m_local, FP8_K, generator=g).cuda()
    b = (torch.randn(n_local, FP8_K, generator=g) * 0.02).cuda()
    sa = (a.abs().amax(dim=1).clamp_min(1e-12) / 448.0).float()
    sb = (b.abs().amax(dim=1).clamp_min(1e-12) / 448.0).float()
    qa = (a / sa[:, None]).to(f8)
    qb = (b / sb[:, None]).to(f8)
    del a, b
    op = flux.AGKernel(group, 1, FP8_M, n_local, FP8_K, f8)
    out = torch.empty((FP8_M, n_local), dtype=torch.bfloat16, device="cuda")
    ms, _ = _time_loop(lambda: op.forward(qa, qb, output=out, input_scale=sa, weight_scale=sb), steps, warmup, world)
    comm.check_status()
    rows_l = _spread(m_local, 8).cuda()
    cols = _spread(n_local, 16).cuda()
    mine = (qa[rows_l].double() * sa[rows_l].double()[:, None]).contiguous()
    if world > 1:
        allrows = torch.empty((world * rows_l.numel(), FP8_K), dtype=torch.float64, device="cuda")
        dist.all_gather_into_tensor(allrows, mine)
    else:
        allrows = mine
    exact = allrows @ (qb[cols].double() * sb[cols].double()[:, None]).t()
    grows = (torch.arange(world, device="cuda")[:, None] * m_local + rows_l[None, :]).reshape(-1)
    rel, close = _cmp(out[grows][:, cols], exact, FP8_TOL)
    rel, bad = _all_max([rel, 0.0 if close else 1.0], world)
    peak = measure_fp8_peak() if rank == 0 else 0.0
    flops = 2.0 * FP8_M * n_local * FP8_K
    tf = flops / (ms * 1e-3) / 1e12
    res = {"workload": f"FP8 e4m3 AG-GEMM M={FP8_M} N={FP8_N} K={FP8_K}, per-row x per-channel scales, bf16 out, TP={world}",
           "ms": ms, "tflops_per_gpu": tf, "max_rel_err": rel, "allclose_3e-2": bad == 0.0,
           "tolerance_max_rel": FP8_TOL}
    if rank == 0:
        res["fp8_peak_tflops"] = peak
        res["frac_of_fp8_peak"] = tf / peak
        res["fp8_peak_source"] = "measured here: torch._scaled_mm 8192^3, best of 10 (burst)"
    return res


def moe_leg(flux, comm, group, rank, world, steps, warmup, with_unfused=True):
    """MoE MLP of the reference's examples (8192 tokens, hidden 4096, 8 experts, ffn 14336 sharded over TP,
    top-2): layer 0 = GemmGroupedV3AGScatter, layer 1 = GemmGroupedV3GatherRS, beside the torch sequence
    (all_gather + index_select + per-expert matmul; per-expert matmul + top-k sum + reduce_scatter) on the same
    GPUs, with fp64 parity samples of both layers (layer 0 rows of tokens from every source rank)."""
    T, H, E, FFN, TOPK = MOE_T, MOE_H, MOE_E, MOE_FFN, MOE_TOPK
    ffn_l = FFN // world
    g = torch.Generator().manual_seed(SEED)  # routing is global: same seed on every rank
    logits = torch.randn(T, E, generator=g).cuda()
    w, chosen = torch.topk(torch.softmax(logits, -1), TOPK, dim=-1)
    chosen = chosen.to(torch.int32)
    si, splits = flux.calc_scatter_index(chosen, torch.empty(E), return_splits=True)
    gi, ti = flux.calc_gather_index(si)
    vec = w.reshape(-1)[(gi.long() * TOPK + ti.long())].contiguous().float()
    splits_cpu = splits.cpu()
    gr = torch.Generator().manual_seed(SEED + 1 + rank)
    tok = _randn_rows(gr, T // world, H, 1.0, torch.bfloat16)
    w0 = _randn_rows(gr, E * ffn_l, H, 0.02, torch.bfloat16).view(E, ffn_l, H)
    w1 = _randn_rows(gr, E * H, ffn_l, 0.02, torch.bfloat16).view(E, H, ffn_l)
    env = flux.DistEnvTPWithEP(group, 1, None)
    l0 = flux.GemmGroupedV3AGScatter(env, flux.MoeArguments(T, H, FFN, E, TOPK, torch.bfloat16))
    l1 = flux.GemmGroupedV3GatherRS(E, T * TOPK, H, TOPK, rank, world, world, 1)
    act = torch.empty((T * TOPK, ffn_l), dtype=torch.bfloat16, device="cuda")

    def fused():
        l0.forward(tok, w0, splits, si, outputs_buf=act)
        return l1.forward_gather_rs(act, w1, splits_cpu, si.view(-1), output_vec_scale=vec)

    full_tok = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    offs = [0] + torch.cumsum(splits_cpu, 0).tolist()
    rs_out = torch.empty((T // world, H), dtype=torch.bfloat16, device="cuda")

    def unfused():
        if world > 1:
            dist.all_gather_into_tensor(full_tok, tok)
            x = full_tok
        else:
            x = tok
        scat = x.index_select(0, gi.long())
        h = torch.empty((T * TOPK, ffn_l), dtype=torch.bfloat16, device="cuda")
        for e in range(E):
            if offs[e + 1] > offs[e]:
                torch.matmul(scat[offs[e]:offs[e + 1]], w0[e].t(), out=h[offs[e]:offs[e + 1]])
        o = torch.empty((T * TOPK, H), dtype=torch.bfloat16, device="cuda")
        for e in range(E):
            if offs[e + 1] > offs[e]:
                torch.matmul(h[offs[e]:offs[e + 1]], w1[e].t(), out=o[offs[e]:offs[e + 1]])
        o = (o.float() * vec[:, None]).to(torch.bfloat16)
        red = o[si.view(-1).long()].view(T, TOPK, H).sum(1)
        if world > 1:
            dist.reduce_scatter_tensor(rs_out, red)
            return rs_out
        return red

    ms_l0, _ = _time_loop(lambda: l0.forward(tok, w0, splits, si, outputs_buf=act), steps, warmup, world)
    ms_l1, _ = _time_loop(lambda: l1.forward_gather_rs(act, w1, splits_cpu, si.view(-1), output_vec_scale=vec),
                          steps, warmup, world)
    ms_f, rf = _time_loop(fused, steps, warmup, world)
    comm.check_status()
    flops_layer = 2.0 * T * TOPK * ffn_l * H
    res = {"workload": f"MoE T={T} H={H} E={E} ffn={FFN} top{TOPK}, bf16, TP={world}",
           "ms_per_step": ms_f, "tflops_per_gpu": 2 * flops_layer / (ms_f * 1e-3) / 1e12,
           "layer0": {"ms": ms_l0, "tflops_per_gpu": flops_layer / (ms_l0 * 1e-3) / 1e12},
           "layer1": {"ms": ms_l1, "tflops_per_gpu": flops_layer / (ms_l1 * 1e-3) / 1e12}}
    # ---- parity against fp64 on sampled entries
    if world > 1:
        dist.all_gather_into_tensor(full_tok, tok)
        x_all = full_tok
    else:
        x_all = tok
    tokens_s = (torch.arange(world)[:, None] * (T // world) + _spread(T // world, 4)[None, :]).reshape(-1).cuda()
    rows0 = si[tokens_s].reshape(-1).long()                        # sorted rows of the sampled tokens (all k)
    tok_of_row = tokens_s.repeat_interleave(TOPK)
    exp_of_row = chosen[tokens_s].reshape(-1).long()
    cols0 = _spread(ffn_l, 16).cuda()
    exact0 = torch.einsum("rh,rch->rc", x_all[tok_of_row].double(), w0[exp_of_row[:, None], cols0[None, :]].double())
    l0_rel, l0_close = _cmp(act[rows0][:, cols0], exact0, AG_TOL)
    cols1 = _spread(H, 16).cuda()
    rows_all = si[tokens_s].long()                                 # [S, topk]
    part = torch.zeros((tokens_s.numel(), cols1.numel()), dtype=torch.float64, device="cuda")
    tk = torch.zeros_like(part)
    for k in range(TOPK):
        r = rows_all[:, k]
        e = chosen[tokens_s][:, k].long()
        d = torch.einsum("rf,rcf->rc", act[r].double(), w1[e[:, None], cols1[None, :]].double())
        part += vec[r].double()[:, None] * d
        # golden path: matmul rounded to bf16, times the row scale, rounded; the top-k sum is rounded again
        tk += (d.to(torch.bfloat16).float() * vec[r][:, None]).to(torch.bfloat16).double()
    gold = tk.to(torch.bfloat16).double()
    if world > 1:
        dist.all_reduce(part)
        dist.all_reduce(gold)
    per = tokens_s.numel() // world
    mine = slice(rank * per, (rank + 1) * per)
    got1 = rf[_spread(T // world, 4).cuda()][:, cols1]
    l1_rel, _ = _cmp(got1, part[mine], RS_TOL)
    _, l1_close = _cmp(got1, gold[mine].to(torch.bfloat16), RS_TOL)
    l0_rel, l1_rel, b0_, b1_ = _all_max([l0_rel, l1_rel, 0.0 if l0_close else 1.0, 0.0 if l1_close else 1.0], world)
    res["parity"] = {"layer0_max_rel_err": l0_rel, "layer1_max_rel_err": l1_rel, "layer0_allclose_1e-2": b0_ == 0.0,
                     "layer1_allclose_2e-2": b1_ == 0.0,
                     "what": "fp64 dots: 4 tokens of every source rank, all top-k rows x 16 cols (layer 0); the same "
                             "tokens' output rows x 16 cols, ffn slices summed over the ranks (layer 1; its elementwise "
                             "bar is taken against the golden path's bf16 rounding points)"}
    if with_unfused:
        ms_u, ru = _time_loop(unfused, steps, warmup, world)
        res["unfused"] = {"what": "torch: all_gather + index_select + per-expert matmul; per-expert matmul + top-k sum + "
                                  "reduce_scatter", "ms_per_step": ms_u,
                          "max_rel_diff_vs_fused": float((rf.float() - ru.float()).abs().max() /
                                                         ru.float().abs().max().clamp_min(1e-30))}
        res["speedup_vs_unfused"] = ms_u / ms_f
    return res


# ----------------------------------------------------------------------------------------------
# headline arm
# ----------------------------------------------------------------------------------------------
def run_ours(args):
    rank, world, local = _env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
        group = dist.group.WORLD
    import flux_b200 as flux
    from flux_b200 import _lib

    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(3000)  # a device wait that runs out ends its call after 3 s (default 10 s)
    a, b0, b1 = _make_inputs(rank, world)
    ag = flux.AGKernel(group, 1, M, N0 // world, K0, torch.bfloat16)
    rs = flux.GemmRS(group, 1, M, N1, torch.bfloat16)
    c0 = torch.empty((M, N0 // world), dtype=torch.bfloat16, device="cuda")
    steps, warmup = args.steps, max(args.warmup, 3)
    meas = {"world": world, "steps": steps, "warmup": warmup, "peaks": _peaks(), "native_library": str(_lib.lib_path())}

    def step():
        ag.forward(a, b0, output=c0)
        return rs.forward(c0, b1)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def settle():
        # Every timed region (unfused before, fused, unfused after, end to end) starts from the same state: an
        # idle pause first, so that no arm inherits the power-cap state the previous arm drove the GPU into.
        barrier()
        time.sleep(args.settle_ms * 1e-3)
        barrier()

    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(warmup):
        out = step()
    barrier()
    comm.check_status()
    try:
        meas["parity"] = dense_parity(a, b0, b1, c0, out, rank, world)
    except Exception as exc:
        traceback.print_exc()
        meas["parity"] = _err(exc)

    # ---- unfused sequence on the same box: NCCL all_gather + cuBLAS, cuBLAS + NCCL reduce_scatter.
    # Timed once before and once after the fused region, so that neither arm is favoured by the
    # power / thermal state it inherits.
    full_a = torch.empty((M, K0), dtype=torch.bfloat16, device="cuda")
    rs_out = torch.empty((M // world, N1), dtype=torch.bfloat16, device="cuda")

    def unfused_step():
        if world > 1:
            dist.all_gather_into_tensor(full_a, a)
            x = full_a
        else:
            x = a
        h = torch.matmul(x, b0.t())
        full = torch.matmul(h, b1.t())
        if world > 1:
            dist.reduce_scatter_tensor(rs_out, full)
            return rs_out
        return full

    def time_unfused():
        settle()
        for _ in range(3):
            unfused_step()
        barrier()
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        u0.record()
        for _ in range(steps):
            uo_ = unfused_step()
        u1.record()
        barrier()
        return _max_over_ranks(u0.elapsed_time(u1) / steps, world), uo_

    unfused_before = None
    try:
        unfused_before, _ = time_unfused()
    except Exception as exc:
        traceback.print_exc()
        meas["unfused"] = _err(exc)
    settle()
    for _ in range(3):
        out = step()

    # ---- timed region: K steps, per-op split from extra events on the same stream
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    barrier()
    t_begin = time.time()
    t_wall = time.perf_counter()
    for i in range(steps):
        ev[i][0].record()
        ag.forward(a, b0, output=c0)
        ev[i][1].record()
        out = rs.forward(c0, b1)
        ev[i][2].record()
    end = torch.cuda.Event(enable_timing=True)
    end.record()
    barrier()
    meas["wall_ms_timed_region"] = (time.perf_counter() - t_wall) * 1e3
    t_end = time.time()
    comm.check_status()
    total_ms = ev[0][0].elapsed_time(end)
    meas["timed_region_s"] = total_ms * 1e-3
    meas["ms_per_step"] = _max_over_ranks(total_ms / steps, world)
    meas["ag_ms"] = _max_over_ranks(statistics.mean(e[0].elapsed_time(e[1]) for e in ev), world)
    meas["rs_ms"] = _max_over_ranks(statistics.mean(e[1].elapsed_time(e[2]) for e in ev), world)

    if unfused_before is not None:
        try:
            unfused_after, uo = time_unfused()
            meas["unfused"] = {
                "what": "NCCL all_gather + cuBLAS matmul, cuBLAS matmul + NCCL reduce_scatter (torch)",
                "ms_per_step": 0.5 * (unfused_before + unfused_after), "ms_before_fused_region": unfused_before,
                "ms_after_fused_region": unfused_after,
                "max_rel_diff_vs_fused": float((uo.float() - out.float()).abs().max() /
                                               uo.float().abs().max().clamp_min(1e-30))}
        except Exception as exc:
            traceback.print_exc()
            meas["unfused"] = _err(exc)
    meas["clocks"] = sampler.stop(t_begin, t_end) if sampler else None

    # ---- NVLink side of the roofline, from the kernel's own timeline (one traced call per op)
    try:
        if world > 1:
            meas["nvlink"] = {
                "ag_gemm": _nvlink_from_trace(comm, lambda: ag.forward(a, b0, output=c0, tuning={"ag_mode": 1}), 4,
                                              (world - 1) * (M // world) * K0 * 2, world, barrier),
                "gemm_rs": _nvlink_from_trace(comm, lambda: rs.forward(c0, b1), 3,
                                              (world - 1) * (M // world) * N1 * 2, world, barrier),
                "what": "bytes this GPU sends (AG: its shard to every peer, pushed by the kernel's comm warps; RS: bf16 "
                        "partials to every owner, spread over the whole kernel by design) / time from the first CTA's "
                        "start to the last push (per-CTA %globaltimer stamps), max over ranks"}
        else:
            meas["nvlink"] = {"note": "TP=1: nothing crosses NVLink"}
    except Exception as exc:
        traceback.print_exc()
        meas["nvlink"] = _err(exc)

    # ---- end to end through host buffers: H2D of this rank's activations, both ops, D2H of the result.
    # Every step copies its own input from pinned host memory and its own result back; the copies run on two
    # copy streams with double-buffered device inputs / host outputs, so that step i's copies overlap the
    # kernels of steps i-1 / i+1 (what a serving loop does): a throughput figure, not a latency.
    try:
        settle()
        meas["e2e"] = e2e_leg(ag, rs, a, b0, b1, c0, steps, world, barrier)
        comm.check_status()
    except Exception as exc:
        traceback.print_exc()
        meas["e2e"] = _err(exc)

    if not args.no_secondary:
        del full_a, rs_out
        try:
            meas["fp8_ag_gemm"] = fp8_leg(flux, comm, group, rank, world, max(5, steps // 2), 3)
        except Exception as exc:
            traceback.print_exc()
            meas["fp8_ag_gemm"] = _err(exc)
        try:
            meas["moe"] = moe_leg(flux, comm, group, rank, world, max(5, steps // 2), 3)
        except Exception as exc:
            traceback.print_exc()
            meas["moe"] = _err(exc)

    ok = True
    if rank == 0:
        if not args.no_cpu_baseline:
            try:
                meas["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_seconds)
            except Exception as exc:
                traceback.print_exc()
                meas["cpu_baseline"] = _err(exc)
        line = make_line(meas)
        print(json.dumps(line), flush=True)
        ok = parity_ok(meas.get("parity"))
        if not ok:
            print("parity check of the headline workload FAILED (see `parity` in the line)", file=sys.stderr)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        sys.exit(3)


def e2e_leg(ag, rs, a, b0, b1, c0, steps, world, barrier):
    a_host = a.cpu().pin_memory()
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    a_dev = [torch.empty_like(a) for _ in range(2)]
    out_dev = [torch.empty((M // world, N1), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    out_host = [torch.empty((M // world, N1), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)]

    def step(i):
        # nothing is allocated inside a step: device inputs, device outputs and host outputs are double-buffered
        j = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[j])  # the all-gather GEMM that read this buffer two steps ago is done
            a_dev[j].copy_(a_host, non_blocking=True)
            in_ready[j].record(s_in)
        main.wait_event(in_ready[j])
        ag.forward(a_dev[j], b0, output=c0)
        in_free[j].record(main)
        main.wait_event(out_done[j])     # the copy-out of the result written two steps ago is done
        rs.forward(c0, b1, output=out_dev[j])
        done[j].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done[j])
            out_host[j].copy_(out_dev[j], non_blocking=True)
            out_done[j].record(s_out)

    for e in in_free + out_done:
        e.record(main)
    for i in range(4):
        step(i)
    main.wait_stream(s_in)
    main.wait_stream(s_out)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    s_in.wait_stream(main)    # copies of the timed region start after its first event
    s_out.wait_stream(main)
    for i in range(steps):
        step(i)
    main.wait_stream(s_in)    # ... and its last event waits for the last copies
    main.wait_stream(s_out)
    s1.record()
    barrier()
    ms = _max_over_ranks(s0.elapsed_time(s1) / steps, world)
    # the copies alone, for reading the figure: when the host link is slower than the kernels (a shared host),
    # the end-to-end step is copy-bound however well the copies overlap
    o_last = rs.forward(c0, b1, output=out_dev[0])
    torch.cuda.synchronize()
    c0_, c1_, c2_ = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    c0_.record()
    a_dev[0].copy_(a_host, non_blocking=True)
    c1_.record()
    out_host[0].copy_(o_last, non_blocking=True)
    c2_.record()
    torch.cuda.synchronize()
    h2d_ms, d2h_ms = c0_.elapsed_time(c1_), c1_.elapsed_time(c2_)
    return {"ms_per_step": ms, "h2d_ms_alone": h2d_ms, "d2h_ms_alone": d2h_ms, "mode": "pipelined: H2D / D2H on two copy streams, double-buffered, overlapping the "
                                       "neighbouring steps' kernels (throughput, not latency)",
            "h2d_bytes_per_step": a_host.numel() * 2 * world, "d2h_bytes_per_step": out_host[0].numel() * 2 * world}


# ----------------------------------------------------------------------------------------------
# single-launch cases for profiler captures
# ----------------------------------------------------------------------------------------------
def run_kernel_only(args):
    """Small single-GPU cases for profiler captures: the fused kernel alone at a per-rank shape of TP=8
    (operands of a few hundred MB: larger than L2, far below the capture size limit).
      d0  : M=4096, N=6144,  K=12288 bf16 (AG-GEMM launch shape)
      d1  : M=4096, N=12288, K=6144  bf16 (GEMM-RS launch shape)
      fp8 : M=8192, N=3584,  K=8192  e4m3 with per-row x per-channel scales
      moe : grouped mode, 16384 routed rows, 8 experts, N=1792, K=4096 (MoE layer 0 per-rank shape)"""
    torch.cuda.set_device(0)
    import flux_b200 as flux

    flux.init_flux_shm(None)
    comm = flux.get_comm(None)
    tuning = {"block_n": args.block_n, "group_m": args.group_m, "cta_group": args.cta_group}
    g = torch.Generator(device="cuda").manual_seed(SEED)
    case = args.case
    if case in ("d0", "d1"):
        m, n, k = (M, N0 // 8, K0) if case == "d0" else (M, N1, K1 // 8)
        a = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
        b = (torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        op = flux.AGKernel(None, 1, m, n, k, torch.bfloat16)
        c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        fn = lambda: op.gemm_only(a, b, output=c, tuning=tuning)  # noqa: E731
        flops = 2.0 * m * n * k
    elif case == "fp8":
        m, n, k = FP8_M, FP8_N // 8, FP8_K
        a = torch.randn(m, k, generator=g, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(n, k, generator=g, device="cuda").to(torch.float8_e4m3fn)
        sa = torch.rand(m, generator=g, device="cuda") + 0.5
        sb = torch.rand(n, generator=g, device="cuda") + 0.5
        op = flux.AGKernel(None, 1, m, n, k, torch.float8_e4m3fn)
        c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        fn = lambda: op.gemm_only(a, b, output=c, input_scale=sa, weight_scale=sb, tuning=tuning)  # noqa: E731
        flops = 2.0 * m * n * k
    else:
        T, H, E, ffn_l, TOPK = MOE_T, MOE_H, MOE_E, MOE_FFN // 8, MOE_TOPK
        logits = torch.randn(T, E, generator=g, device="cuda")
        _, chosen = torch.topk(torch.softmax(logits, -1), TOPK, dim=-1)
        si, splits = flux.calc_scatter_index(chosen.to(torch.int32), torch.empty(E), return_splits=True)
        tok = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
        w0 = (torch.randn(E, ffn_l, H, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        l0 = flux.GemmGroupedV3AGScatter(flux.DistEnvTPWithEP(None, 1, None),
                                         flux.MoeArguments(T, H, ffn_l, E, TOPK, torch.bfloat16))
        act = torch.empty((T * TOPK, ffn_l), dtype=torch.bfloat16, device="cuda")
        m, n, k = T * TOPK, ffn_l, H
        fn = lambda: l0.forward(tok, w0, splits, si, outputs_buf=act, tuning=tuning)  # noqa: E731
        flops = 2.0 * m * n * k
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    comm.check_status()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"case": f"kernel-only {case}", "m": m, "n": n, "k": k, "tuning": tuning, "ms": ms,
                      "tflops": flops / (ms * 1e-3) / 1e12}), flush=True)


def run_secondary(args):
    """`--workload moe` / `--workload fp8`: one secondary workload alone, one JSON line on rank 0."""
    rank, world, local = _env()
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
        group = dist.group.WORLD
    import flux_b200 as flux

    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(3000)
    if args.workload == "moe":
        res = moe_leg(flux, comm, group, rank, world, args.steps, args.warmup)
        metric = "MoE MLP (AG+scatter grouped GEMM, grouped GEMM+gather-RS) aggregate TFLOP/s"
        value = res["tflops_per_gpu"] * world
    else:
        res = fp8_leg(flux, comm, group, rank, world, args.steps, args.warmup)
        metric = "FP8 AG-GEMM aggregate TFLOP/s"
        value = res["tflops_per_gpu"] * world
    if rank == 0:
        line = {"metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "strong",
                "dtype": "bf16" if args.workload == "moe" else "e4m3", "data": "synthetic (CPU-seeded)",
                "config": {"workload": res["workload"]}}
        line.update(res)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# host-core arm
# ----------------------------------------------------------------------------------------------
def _cpu_sample_run(m_s, n_s, k_s, iters=1):
    """The oracle's AG-GEMM + GEMM-RS sequence on the host cores for a slice of the workload."""
    from oracle import golden

    g = torch.Generator().manual_seed(SEED)
    a = torch.randn(m_s, k_s, generator=g).to(torch.bfloat16)
    b0 = (torch.randn(n_s, k_s, generator=g) * 0.02).to(torch.bfloat16)
    b1 = (torch.randn(k_s, n_s, generator=g) * 0.02).to(torch.bfloat16)
    t0 = time.perf_counter()
    for _ in range(iters):
        h, _ = golden.ag_gemm_single([a], b0)
        golden.gemm_rs_single([h], [b1])
    dt = (time.perf_counter() - t0) / iters
    return dt, 2.0 * m_s * n_s * k_s * 2


def _cpu_sample_text(iters=None, secs=None):
    m_s, n_s, k_s = CPU_SLICE
    s = f"oracle AG-GEMM + GEMM-RS on a slice M={m_s} N={n_s} K={k_s} of the workload (bf16, torch CPU, all host threads)"
    if iters is not None:
        s += f", {iters} passes, {secs:.1f} s"
    return s


def cpu_baseline(budget_s=15.0):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m_s, n_s, k_s = CPU_SLICE
    dt1, fl = _cpu_sample_run(m_s, n_s, k_s)
    iters = max(1, min(2000, int(budget_s / max(dt1, 1e-3))))
    dt, fl = _cpu_sample_run(m_s, n_s, k_s, iters=iters)
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": _cpu_sample_text(iters, dt * iters)}


def run_reference(args):
    """The reference's torch golden path (all_gather + matmul, matmul + reduce_scatter) on the host
    cores: the oracle restatement, single process with every host thread; rank 0 only. The slice is the
    same at every N; each step is one pass over it."""
    rank, world, _ = _env()
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)   # a launcher may have exported OMP_NUM_THREADS=1: this arm owns the host
    m_s, n_s, k_s = CPU_SLICE
    # inputs are generated once, outside the timed region (as the GPU arm's are resident before its timed region)
    _cpu_sample_run(m_s, n_s, k_s, iters=max(1, args.warmup))
    dt, fl = _cpu_sample_run(m_s, n_s, k_s, iters=max(1, args.steps))
    val = fl / dt / 1e12
    sample = _cpu_sample_text() + ", one pass per step"
    print(json.dumps({
        "impl": "reference",
        "metric": METRIC,
        "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args.gpus) + " (bounded sample per step)", "parallelism": "host cores"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the fp8 and MoE legs of the headline run")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--settle-ms", type=float, default=500.0,
                    help="idle pause before every timed region, so that all arms start from the same power state")
    ap.add_argument("--kernel-only", action="store_true", help="small single-GPU case for profiler captures")
    ap.add_argument("--case", default="d0", choices=["d0", "d1", "fp8", "moe"], help="kernel-only: which launch")
    ap.add_argument("--workload", default="dense", choices=["dense", "moe", "fp8"],
                    help="dense MLP (headline), or one secondary workload alone")
    ap.add_argument("--block-n", type=int, default=0, help="kernel-only: output tile width (0 = library default)")
    ap.add_argument("--group-m", type=int, default=0, help="kernel-only: rasterisation band height (0 = default)")
    ap.add_argument("--cta-group", type=int, default=0, help="kernel-only: 1 or 2 CTAs per tile (0 = default)")
    args = ap.parse_args()
    if args.kernel_only:
        run_kernel_only(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload != "dense":
        run_secondary(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
