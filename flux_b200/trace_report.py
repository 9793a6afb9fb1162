"""Per-CTA timeline of the fused kernels on the dense benchmark shapes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m flux_b200.trace_report [--m 4096 --hidden 12288 --ffn 49152]

For the plain GEMM of each per-rank shape, the all-gather GEMM and the GEMM reduce-scatter it switches the
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

    print(f"{name:10s} event {event_ms:.4f} ms | us after first CTA start (min/med/max): first-operands {_fmt(rel(1))}"
          f" | last-UMMA {_fmt(rel(2))} | epilogue-end {_fmt(rel(3))} | comm-end {_fmt(rel(4))}"
          f" | flag-wait {_fmt(t[:, 5] / 1e3)} | ready-wait {_fmt(t[:, 6] / 1e3)}"
          f" | work items per CTA {int(t[:, 7].min())}-{int(t[:, 7].max())}", flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=12288)
    ap.add_argument("--ffn", type=int, default=49152)
    ap.add_argument("--reps", type=int, default=2)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    import flux_b200 as flux

    group = dist.group.WORLD if world > 1 else None
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
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
        for _ in range(3):
            fn()
        barrier()
        tr = comm.enable_trace(True)
        for _ in range(args.reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if rank == 0:
                _show(name, e0.elapsed_time(e1), tr)
        comm.enable_trace(False)

    run("gemm D0", lambda: ag.gemm_only(a_full, b0, output=out))
    run("ag-gemm", lambda: ag.forward(a, b0, output=out))
    run("gemm D1", lambda: plain1.gemm_only(c0, b1))
    run("gemm-rs", lambda: rs.forward(c0, b1))
    comm.check_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
