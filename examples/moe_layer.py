#!/usr/bin/env python
"""A tensor-parallel MoE MLP on the fused ops, beside the same layer in plain torch collectives.

Counterpart of the reference's usage examples (examples/moe.py:141-211, examples/moe_flux_only.py:85-131): the
two fused calls a Megatron-style MoE layer makes - `GemmGroupedV3AGScatter.forward` (all-gather of the token
shards + scatter to expert order + grouped GEMM) and `GemmGroupedV3GatherRS.forward_gather_rs` (grouped GEMM +
top-k combine + reduce-scatter) - with an activation in between, checked against and timed beside the torch
sequence (all_gather, index_select, per-expert matmul, top-k sum, reduce_scatter).

    python examples/moe_layer.py                                   # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/moe_layer.py --tokens 8192 --hidden 4096 --ffn 14336 --experts 8 --topk 2
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flux_b200 as flux  # noqa: E402  (`import flux_b200 as flux` is the drop-in spelling)


class MoELayerFlux(torch.nn.Module):
    """Layer 0 (dispatch + GEMM), GELU, layer 1 (GEMM + combine), all on the fused ops."""

    def __init__(self, group, rank, world, tokens, hidden, ffn, experts, topk, dtype, w0, w1):
        super().__init__()
        env = flux.DistEnvTPWithEP(tp_group=group, nnodes=1, ep_group=None)
        args = flux.MoeArguments(max_ntokens=tokens, hidden=hidden, ffn_hidden=ffn, nexperts=experts, topk=topk,
                                 input_dtype=dtype, output_dtype=dtype)
        self.ag_op = flux.GemmGroupedV3AGScatter(tp_env=env, moe_args=args)
        self.rs_op = flux.GemmGroupedV3GatherRS(experts, tokens * topk, hidden, topk, rank, world, world, 1, 1,
                                                input_dtype=dtype)
        self.w0, self.w1 = w0, w1
        self.inter = torch.empty((tokens * topk, ffn // world), dtype=dtype, device="cuda")

    def forward(self, tokens_shard, splits_gpu, splits_cpu, scatter_index, row_weights):
        self.ag_op.forward(inputs_shard=tokens_shard, weights=self.w0, splits_gpu=splits_gpu,
                           scatter_index=scatter_index, outputs_buf=self.inter)
        act = torch.nn.functional.gelu(self.inter)
        return self.rs_op.forward_gather_rs(input=act, weight=self.w1, splits_cpu=splits_cpu,
                                            scatter_idx=scatter_index.view(-1), output_vec_scale=row_weights)


def moe_layer_torch(group, world, tokens_shard, w0, w1, splits_cpu, scatter_index, gather_index, row_weights, topk):
    """The same layer from torch collectives and per-expert matmuls."""
    if world > 1:
        full = torch.empty((tokens_shard.shape[0] * world, tokens_shard.shape[1]), dtype=tokens_shard.dtype, device="cuda")
        dist.all_gather_into_tensor(full, tokens_shard, group=group)
    else:
        full = tokens_shard
    scat = full.index_select(0, gather_index.long())
    offs = [0] + torch.cumsum(splits_cpu, 0).tolist()
    inter = torch.cat([scat[offs[e]:offs[e + 1]] @ w0[e].t() for e in range(w0.shape[0])])
    act = torch.nn.functional.gelu(inter)
    out = torch.cat([act[offs[e]:offs[e + 1]] @ w1[e].t() for e in range(w1.shape[0])])
    out = (out.float() * row_weights[:, None]).to(out.dtype)
    red = out[scatter_index.view(-1).long()].view(-1, topk, out.shape[1]).sum(1)
    if world == 1:
        return red
    mine = torch.empty((red.shape[0] // world, red.shape[1]), dtype=red.dtype, device="cuda")
    dist.reduce_scatter_tensor(mine, red, group=group)
    return mine


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    group = None
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
        group = dist.group.WORLD
    flux.init_flux_shm(group)
    dtype = torch.bfloat16
    T, H, F, E, K = args.tokens, args.hidden, args.ffn, args.experts, args.topk
    # token routing (global: the same on every rank), then the indices the fused ops take
    g = torch.Generator(device="cuda").manual_seed(0)
    gate, chosen = torch.topk(torch.softmax(torch.randn(T, E, generator=g, device="cuda"), -1), K, dim=-1)
    scatter_index, splits_gpu = flux.calc_scatter_index(chosen.to(torch.int32), torch.empty(E), return_splits=True)
    gather_index, topk_index = flux.calc_gather_index(scatter_index)
    row_weights = gate.reshape(-1)[gather_index.long() * K + topk_index.long()].contiguous().float()
    splits_cpu = splits_gpu.cpu()
    gr = torch.Generator(device="cuda").manual_seed(1 + rank)
    tokens_shard = torch.randn(T // world, H, generator=gr, device="cuda").to(dtype)
    w0 = (torch.randn(E, F // world, H, generator=gr, device="cuda") * 0.02).to(dtype)
    w1 = (torch.randn(E, H, F // world, generator=gr, device="cuda") * 0.02).to(dtype)

    layer = MoELayerFlux(group, rank, world, T, H, F, E, K, dtype, w0, w1)
    out_flux, ms_flux = flux.bench_func(
        lambda: layer(tokens_shard, splits_gpu, splits_cpu, scatter_index, row_weights), args.iters, 3)
    out_torch, ms_torch = flux.bench_func(
        lambda: moe_layer_torch(group, world, tokens_shard, w0, w1, splits_cpu, scatter_index, gather_index,
                                row_weights, K), args.iters, 3)
    flux.get_comm(group).check_status()
    flux.torch_allclose(out_flux.float(), out_torch.float(), rtol=2e-2, atol=2e-2, verbose=False)
    if rank == 0:
        print(f"MoE layer, {T} tokens, hidden {H}, ffn {F}, {E} experts, top-{K}, TP={world}: "
              f"fused {ms_flux:.3f} ms, torch {ms_torch:.3f} ms ({ms_torch / ms_flux:.2f}x); outputs agree within 2e-2")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
