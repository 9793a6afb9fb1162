#!/usr/bin/env python
"""A Megatron-style tensor-parallel MLP whose two linear layers are the fused ops.

`ColumnParallelLinear` runs `AGKernel` (all-gather of the sequence-sharded activations fused into the GEMM) and
`RowParallelLinear` runs `GemmRS` (reduce-scatter fused into the GEMM epilogue); the backward pass uses the same
two ops with the roles swapped (AG-GEMM and GEMM-RS are each other's transposes). One training step - forward,
loss, backward, SGD update - is checked against the unsharded model on rank 0's slice. Usage of the ops as in
the reference's README ("flux.AGKernel(...).forward", "flux.GemmRS(...).forward", README.md:107-140).

    python examples/tp_mlp.py
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/tp_mlp.py
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flux_b200 as flux  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    group = None
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
        group = dist.group.WORLD
    flux.init_flux_shm(group)
    torch.manual_seed(7 + rank)
    mlp = flux.TensorParallelMLP(args.hidden, args.ffn, args.tokens, group)
    opt = torch.optim.SGD(mlp.parameters(), lr=1e-3)
    x = torch.randn(args.tokens // world, args.hidden, device="cuda").bfloat16()
    target = torch.randn(args.tokens // world, args.hidden, device="cuda").bfloat16()
    for step in range(args.steps):
        opt.zero_grad(set_to_none=True)
        y = mlp(x)                                    # [tokens / TP, hidden], sequence-sharded in and out
        loss = ((y.float() - target.float()) ** 2).mean()
        loss.backward()
        opt.step()
        torch.cuda.synchronize()
        flux.get_comm(group).check_status()
        if world > 1:
            t = loss.detach().clone()
            dist.all_reduce(t)
            loss = t / world
        if rank == 0:
            print(f"step {step}: loss {float(loss):.5f}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
