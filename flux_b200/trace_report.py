"""Per-CTA timeline of the fused kernels on the dense benchmark shapes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m flux_b200.trace_report [--m 4096 --hidden 12288 --ffn 49152]

For the plain GEMM of each per-rank shape, the all-gather GEMM (both transports of the all-gather), the GEMM
reduce-scatter and, with --moe, the two MoE layers, it times 10 calls with CUDA events and then switches the
kernel's timeline stamps on (`Comm.enable_trace`), runs one call between barriers and prints, over the CTAs of
rank 0: when the first operands landed, when the last UMMA was issued, when the epilogue and the communication
warps finished (microseconds after the earliest CTA start; min / median / max), and the time lane 0 of the
producer / epilogue spent waiting for arrival flags and for the owner-side sum. It stands in for the reference's
host-side profiling hooks (python/flux/util.py:111-172, src/ag_gemm/ths_op/all_gather_gemm_op.cc:426-447).
The CUDA-event time of the same call is printed beside it. Also usable on one GPU (plain `python -m ...`).
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist


def _fmt(x: torch.Tensor) -> str:
    if x.numel() == 0:
        return "      -/      -/      -"
    return f"{x.min():7.1f}/{x.median():7.1f}/{x.max():7.1f}"


def _show(name: str, event_ms: float, tr: torch.Tensor) -> None:
    t = tr.cpu().double()
    t0 = t[:, 0].min()

    def rel(col):
        # CTAs that never reached a stage leave 0 in its stamp: keep only real stamps
        x = t[:, col]
        return (x[x > 0] - t0) / 1e3

    print(f"{name:40s} event {event_ms:.4f} ms | us after first CTA start (min/med/max): first-operands {_fmt(rel(1))}"
          f" | last-UMMA {_fmt(rel(2))} | epilogue-end {_fmt(rel(3))} | comm-end {_fmt(rel(4))}"
          f" | drain {_fmt((t[:, 3] - t[:, 2])[(t[:, 2] > 0) & (t[:, 3] > 0)] / 1e3)}"
          f" | flag-wait {_fmt(t[:, 5] / 1e3)} | ready-wait {_fmt(t[:, 6] / 1e3)}"
          f" | work items per CTA {int(t[:, 7].min())}-{int(t[:, 7].max())}", flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=12288)
    ap.add_argument("--ffn", type=int, default=49152)
    ap.add_argument("--reps", type=int, default=2)
    ap.add_argument("--push-units", action="store_true", help="also the kernel push in units of 64 and 128 rows")
    ap.add_argument("--moe", action="store_true", help="also the MoE layers at 8192 tokens, hidden 4096, 8 experts, top-2")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    import flux_b200 as flux

    group = dist.group.WORLD if world > 1 else None
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(2000)  # a wait that runs out ends the call after 2 s instead of the default 10
    m, k0, n0, n1, k1 = args.m, args.hidden, args.ffn, args.hidden, args.ffn
    gen = torch.Generator(device="cuda").manual_seed(rank)
    a = torch.randn(m // world, k0, generator=gen, device="cuda").bfloat16()
    a_full = torch.randn(m, k0, generator=gen, device="cuda").bfloat16()
    b0 = (torch.randn(n0 // world, k0, generator=gen, device="cuda") * 0.02).bfloat16()
    c0 = torch.randn(m, k1 // world, generator=gen, device="cuda").bfloat16()
    b1 = (torch.randn(n1, k1 // world, generator=gen, device="cuda") * 0.02).bfloat16()
    out = torch.empty(m, n0 // world, dtype=torch.bfloat16, device="cuda")
    ag = flux.AGKernel(group, 1, m, n0 // world, k0, torch.bfloat16)
    plain1 = flux.AGKernel(group, 1, m, n1, k1 // world, torch.bfloat16)
    rs = flux.GemmRS(group, 1, m, n1, torch.bfloat16)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def run(name, fn):
        # every measurement starts from the same idle state: without the pause the later ones inherit the
        # power-cap state of the earlier ones and look slower than they are
        barrier()
        time.sleep(0.5)
        barrier()
        for _ in range(3):
            fn()
        barrier()
        # event time without the timeline stamps: mean of 10 calls, maximum over the ranks
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / 10], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        barrier()
        tr = comm.enable_trace(True)
        for _ in range(args.reps):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            t0.record()
            fn()
            t1.record()
            torch.cuda.synchronize()
            if rank == 0:
                _show(f"{name} [{float(ms):.4f} ms untraced]", t0.elapsed_time(t1), tr)
        comm.enable_trace(False)

    kernel_push, copy_engines = {"ag_mode": 1}, {"ag_mode": 2}
    run("gemm D0", lambda: ag.gemm_only(a_full, b0, output=out))
    if world > 1:
        run("ag-gemm, kernel push", lambda: ag.forward(a, b0, output=out, tuning=kernel_push))
        if args.push_units:
            run("ag-gemm, push 64-row units", lambda: ag.forward(a, b0, output=out, tuning={"ag_mode": 3}))
            run("ag-gemm, push 128-row units", lambda: ag.forward(a, b0, output=out, tuning={"ag_mode": 4}))
        run("ag-gemm, copy engines", lambda: ag.forward(a, b0, output=out, tuning=copy_engines))
    run("gemm D1", lambda: plain1.gemm_only(c0, b1))
    if world > 1:
        run("gemm-rs", lambda: rs.forward(c0, b1))
    if args.moe:
        T, H, E, FFN, TOPK = 8192, 4096, 8, 14336, 2
        ffn_l = FFN // world
        g0 = torch.Generator(device="cuda").manual_seed(1234)
        logits = torch.randn(T, E, generator=g0, device="cuda")
        w, chosen = torch.topk(torch.softmax(logits, -1), TOPK, dim=-1)
        si, splits = flux.calc_scatter_index(chosen.to(torch.int32), torch.empty(E), return_splits=True)
        gi, ti = flux.calc_gather_index(si)
        vec = w.reshape(-1)[(gi.long() * TOPK + ti.long())].contiguous().float()
        tok = torch.randn(T // world, H, generator=gen, device="cuda").bfloat16()
        w0 = (torch.randn(E, ffn_l, H, generator=gen, device="cuda") * 0.02).bfloat16()
        w1 = (torch.randn(E, H, ffn_l, generator=gen, device="cuda") * 0.02).bfloat16()
        l0 = flux.GemmGroupedV3AGScatter(flux.DistEnvTPWithEP(group, 1, None), flux.MoeArguments(T, H, FFN, E, TOPK, torch.bfloat16))
        l1 = flux.GemmGroupedV3GatherRS(E, T * TOPK, H, TOPK, rank, world, world, 1)
        act = torch.empty((T * TOPK, ffn_l), dtype=torch.bfloat16, device="cuda")
        splits_cpu = splits.cpu()
        run("moe-l0, kernel push", lambda: l0.forward(tok, w0, splits, si, outputs_buf=act, tuning=kernel_push))
        if world > 1:
            run("moe-l0, copy engines", lambda: l0.forward(tok, w0, splits, si, outputs_buf=act, tuning=copy_engines))
        run("moe-l1", lambda: l1.forward_gather_rs(act, w1, splits_cpu, si.view(-1), output_vec_scale=vec))
    comm.check_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
