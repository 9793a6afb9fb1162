"""CPU oracle: restatement of the reference's torch golden paths.

TEST INFRASTRUCTURE ONLY. Nothing in the product (`flux_b200/`) imports this
file; it is used by `tests/`, by `__graft_entry__.smoke()` and by the
`cpu_baseline` / `--impl reference` legs of `bench.py`, always as the checker
or the timed CPU baseline, never as the thing shipped.

The reference validates its fused kernels against plain torch sequences that
live in its test scripts and `flux.testing` helpers. Those files cannot be
imported as they are (they import the compiled `flux` extension), so each
function below restates one of them and cites it by the file's path inside
bytedance/flux. Pinning: `tests/golden/` holds vectors produced by running the
reference's own pure-torch helpers (loaded from its source files with a stub
for the compiled module; `tests/golden/make_golden.py`), by running the dense
golden functions of its test scripts (`perf_torch`, compiled unmodified from
their source and run on 2 gloo ranks) and the hand-computable `--debug` cases
of its tests; `tests/test_oracle.py` checks this file against
both. The arithmetic itself is PyTorch's matmul and gloo/NCCL reductions on
either side, so float parity is by tolerance (as in the reference's tests) and
only routing/indexing is bit-exact.

Two forms of every path:
  *_dist   : one rank of a torch.distributed job (gloo on CPU, NCCL on GPU) -
             the literal sequence the reference times and compares with.
  *_single : the same mathematics in one process from the list of all ranks'
             inputs (all_gather = concatenation, reduce_scatter = sum + slice).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

FP8_DTYPES = tuple(
    d for d in (getattr(torch, "float8_e4m3fn", None), getattr(torch, "float8_e5m2", None)) if d is not None
)


def is_fp8(dt: torch.dtype) -> bool:
    return dt in FP8_DTYPES


# --------------------------------------------------------------------------- data
def init_seed(seed: int = 0) -> None:
    """python/flux/testing/utils.py:49-62 (seed = 3 + rank, deterministic settings, TF32 off)."""
    torch.use_deterministic_algorithms(True, warn_only=True)
    torch.manual_seed(3 + seed)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


def make_tensor(shape, dtype: torch.dtype, scale: float, bias: float, generator: torch.Generator) -> torch.Tensor:
    """python/flux/testing/utils.py:132-164 `_make_tensor` for float types:
    (rand * 2 - 1) * scale + bias, drawn on the CPU in fp32 so that CPU and GPU runs share values."""
    out = (torch.rand(shape, dtype=torch.float32, generator=generator) * 2 - 1) * scale + bias
    return out.to(dtype)


def quantize_fp8_rows(x: torch.Tensor, dtype=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric quantisation used by the fp8 configuration: scale = amax(row)/448,
    q = (x / scale) cast to e4m3. Returns (q, scale[rows] fp32)."""
    dtype = dtype or torch.float8_e4m3fn
    amax = x.float().abs().amax(dim=1).clamp_min(1e-12)
    scale = (amax / 448.0).float()
    q = (x.float() / scale[:, None]).to(dtype)
    return q, scale


# --------------------------------------------------------------------------- dense AG-GEMM
def _ag_gemm_math(full_input, weight, bias, full_input_scale, weight_scale, out_dtype):
    """test/python/ag_gemm/test_ag_kernel.py:139-153: matmul with weight.t(), scales, cast, `+= bias`.
    fp8: operands are cast to bf16 and the product is multiplied by the scales (:119-124,:147);
    per-row x per-channel scales follow the int8 rule `full_input_scale * weight_scale * accum` (:143-145)."""
    if full_input.dtype == torch.int8:
        # w8a8 (:143-150): `accum = matmul_int8(full_input, weight.t()).to(float32)`,
        # `output = full_input_scale * weight_scale * accum`, cast to bf16; the tests ask for a bitwise match
        accum = torch.matmul(full_input.to(torch.int32), weight.to(torch.int32).t()).to(torch.float32)
        out = full_input_scale.reshape(-1, 1).float() * weight_scale.reshape(1, -1).float() * accum
        out = out.to(torch.bfloat16)
    elif is_fp8(full_input.dtype):
        a = full_input.to(torch.bfloat16)
        w = weight.to(torch.bfloat16)
        out = torch.matmul(a, w.t()).float()
        if full_input_scale is not None:
            out = out * full_input_scale.reshape(-1, 1).float() if full_input_scale.numel() > 1 else out * full_input_scale.float()
        if weight_scale is not None:
            out = out * weight_scale.reshape(1, -1).float() if weight_scale.numel() > 1 else out * weight_scale.float()
        out = out.to(torch.bfloat16)
    else:
        out = torch.matmul(full_input, weight.t())
        out = out.to(out_dtype)
    if bias is not None:
        out = out + bias
    return out


def ag_gemm_dist(group, input, weight, bias=None, input_scale=None, weight_scale=None, out_dtype=None):
    """One rank of the golden AG-GEMM (test_ag_kernel.py:88-176 `perf_torch`):
    all_gather_into_tensor(input) -> matmul. Returns (output, gathered_input)."""
    world = dist.get_world_size(group)
    m_local, k = input.shape
    raw = input.view(torch.uint8) if is_fp8(input.dtype) else input
    full_raw = torch.zeros((m_local * world, raw.shape[1]), dtype=raw.dtype, device=input.device)
    dist.all_gather_into_tensor(full_raw, raw.contiguous(), group=group)
    full_input = full_raw.view(input.dtype) if is_fp8(input.dtype) else full_raw
    full_scale = None
    if input_scale is not None:
        if input_scale.numel() > 1:
            full_scale = torch.zeros((m_local * world,), dtype=input_scale.dtype, device=input.device)
            dist.all_gather_into_tensor(full_scale, input_scale.reshape(-1).contiguous(), group=group)
        else:
            full_scale = input_scale
    od = out_dtype or (torch.bfloat16 if is_fp8(input.dtype) else input.dtype)
    return _ag_gemm_math(full_input, weight, bias, full_scale, weight_scale, od), full_input


def ag_gemm_single(inputs: Sequence[torch.Tensor], weight, bias=None, input_scales=None, weight_scale=None,
                   out_dtype=None):
    """All ranks' shards in one process: all_gather == torch.cat along rows. Returns (output of the rank that
    holds `weight`, gathered input)."""
    raw = [x.view(torch.uint8) if is_fp8(x.dtype) else x for x in inputs]
    full = torch.cat(raw, dim=0)
    full_input = full.view(inputs[0].dtype) if is_fp8(inputs[0].dtype) else full
    full_scale = None
    if input_scales is not None:
        full_scale = torch.cat([s.reshape(-1) for s in input_scales]) if input_scales[0].numel() > 1 else input_scales[0]
    od = out_dtype or (torch.bfloat16 if is_fp8(inputs[0].dtype) else inputs[0].dtype)
    return _ag_gemm_math(full_input, weight, bias, full_scale, weight_scale, od), full_input


# --------------------------------------------------------------------------- dense GEMM-RS
def _rs_partial(input, weight, bias, input_scale, weight_scale):
    """test/python/gemm_rs/test_gemm_rs.py:113-135: matmul (fp8: scaled, bf16 out), `+= bias` on every rank."""
    if input.dtype == torch.int8:
        # :127-135: dequantised int8 product in the output dtype; the caller passes the bias on rank 0 only
        accum = torch.matmul(input.to(torch.int32), weight.to(torch.int32).t()).to(torch.float32)
        out = (input_scale.reshape(-1, 1).float() * weight_scale.reshape(1, -1).float() * accum).to(torch.bfloat16)
    elif is_fp8(input.dtype):
        out = torch.matmul(input.to(torch.bfloat16), weight.to(torch.bfloat16).t()).float()
        if input_scale is not None:
            out = out * (input_scale.reshape(-1, 1).float() if input_scale.numel() > 1 else input_scale.float())
        if weight_scale is not None:
            out = out * (weight_scale.reshape(1, -1).float() if weight_scale.numel() > 1 else weight_scale.float())
        out = out.to(torch.bfloat16)
    else:
        out = torch.matmul(input, weight.t())
    if bias is not None:
        out = out + bias
    return out


def gemm_rs_dist(group, input, weight, bias=None, input_scale=None, weight_scale=None):
    """One rank of the golden GEMM-RS (test_gemm_rs.py:57-157 `perf_torch`): matmul -> reduce_scatter_tensor."""
    world = dist.get_world_size(group)
    full = _rs_partial(input, weight, bias, input_scale, weight_scale).contiguous()
    out = torch.zeros((full.shape[0] // world, full.shape[1]), dtype=full.dtype, device=full.device)
    try:
        dist.reduce_scatter_tensor(out, full, group=group)
    except (RuntimeError, NotImplementedError):
        # backends without reduce_scatter (gloo on some builds): all_reduce and slice, same sum
        tmp = full.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out = tmp[r * out.shape[0]:(r + 1) * out.shape[0]].clone()
    return out


def gemm_rs_single(inputs, weights, biases=None, input_scales=None, weight_scales=None) -> List[torch.Tensor]:
    """All ranks in one process: partials are summed in fp32 in rank order, rounded once to the
    partial dtype, and sliced by rows. Returns the list of per-rank outputs."""
    world = len(inputs)
    parts = []
    for r in range(world):
        parts.append(
            _rs_partial(inputs[r], weights[r], None if biases is None else biases[r],
                        None if input_scales is None else input_scales[r],
                        None if weight_scales is None else weight_scales[r])
        )
    total = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        total += p.float()
    total = total.to(parts[0].dtype)
    mpr = total.shape[0] // world
    return [total[r * mpr:(r + 1) * mpr].contiguous() for r in range(world)]


def ring_reduce_single(parts: Sequence[torch.Tensor], rank: int) -> torch.Tensor:
    """src/gemm_rs/ring_reduce.cu:54-80 (`packed_ring_reduction`) for the rows of `rank`: a running sum in the
    element dtype that starts at zero and adds the partials of rank+1, rank+2, ..., rank (own last), rounding
    after every addition."""
    world = len(parts)
    mpr = parts[0].shape[0] // world
    acc = torch.zeros_like(parts[0][:mpr])
    for i in range(rank + 1, rank + 1 + world):
        acc = acc + parts[i % world][rank * mpr:(rank + 1) * mpr]
    return acc


# --------------------------------------------------------------------------- MoE routing (integer, bit-exact)
def calc_scatter_index_stable(chosen_experts: torch.Tensor) -> torch.Tensor:
    """python/flux/testing/moe_utils.py:141-144."""
    return chosen_experts.flatten().argsort(stable=True).argsort().int().view(chosen_experts.shape)


def calc_splits(chosen_experts: torch.Tensor, nexperts: int) -> torch.Tensor:
    """python/flux/testing/moe_utils.py:212-214: bincount of the chosen experts."""
    return torch.bincount(chosen_experts.view(-1).long(), minlength=nexperts).to(torch.int32)


def calc_gather_index(scatter_index: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse permutation (python/flux/testing/moe_utils.py:100-136, device kernel
    src/moe_ag_scatter/sort_util.cu:39-92): gather_index[scatter_index[t,k]] = t, topk_index[...] = k."""
    ntokens, topk = scatter_index.shape
    flat = scatter_index.reshape(-1).long()
    gather_index = torch.zeros(ntokens * topk, dtype=torch.int32)
    topk_index = torch.zeros(ntokens * topk, dtype=torch.int32)
    ids = torch.arange(ntokens * topk, dtype=torch.int64)
    gather_index[flat] = (ids // topk).int()
    topk_index[flat] = (ids % topk).int()
    return gather_index, topk_index


def topk_routing(logits: torch.Tensor, topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax gate then top-k (examples/moe.py:60-75 style): returns (chosen experts int32 [T,topk],
    routing weights fp32 [T,topk])."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, topk, dim=-1)
    return idx.to(torch.int32), w.float()


# --------------------------------------------------------------------------- MoE layer 0
def moe_ag_scatter_single(token_shards, weights, splits, scatter_index, output_scale=None, out_dtype=None,
                          ep_rank: int = 0, ep_size: int = 1):
    """python/flux/testing/moe_ag_scatter_utils.py:195-262 (`comm_impl`, `scatter_impl`, `gemm_impl`):
    all_gather tokens -> index_select(gather_index) -> per-expert matmul with W[e].t() -> `mul_(output_scale[e])`.
    `weights` is this rank's [E / ep_size, ffn_local, hidden]; with expert parallelism only the experts
    [ep_rank, ep_rank + 1) * E / ep_size are computed, from the rows `input_offset = sum(splits[:first expert])`
    onwards (:228-236), and the output holds just those rows. Returns (out, gathered tokens)."""
    full = torch.cat(list(token_shards), dim=0)
    gather_index, _ = calc_gather_index(scatter_index.cpu())
    scat = torch.index_select(full, 0, gather_index.long().to(full.device))
    od = out_dtype or full.dtype
    e_local = weights.shape[0]
    e_first = e_local * ep_rank
    assert e_local * ep_size == len(splits)
    input_offset = int(sum(int(x) for x in splits[:e_first]))
    nrows = int(sum(int(x) for x in splits[e_first:e_first + e_local]))
    out = torch.zeros((nrows, weights.shape[1]), dtype=od, device=full.device)
    off = 0
    for e in range(e_local):
        nxt = off + int(splits[e + e_first])
        if nxt > off:
            o = torch.matmul(scat[off + input_offset:nxt + input_offset], weights[e].t())
            if output_scale is not None:
                o = o * output_scale[e]
            out[off:nxt] = o.to(od)
        off = nxt
    return out, full


# --------------------------------------------------------------------------- MoE layer 1
def moe_gather_rs_partial(x, weights, splits, scatter_index, topk, input_scale=None, weight_scale=None,
                          output_vec_scale=None, ep_rank: int = 0, ep_size: int = 1):
    """One rank's contribution before the reduce-scatter
    (python/flux/testing/moe_gather_rs_utils.py:26-101): per-expert matmul * (weight_scale[e] * input_scale),
    `* output_vec_scale`, cast, rows placed at `topk * token + k`, `.view(T, topk, N).sum(1)`. With expert
    parallelism `x` / `weights` hold this rank's experts only (`eid_start`, `ep_rank_m_start:ep_rank_m_end`,
    :70,:102-105) and the rows of other ranks' experts stay zero."""
    n = weights.shape[1]
    e_first = weights.shape[0] * ep_rank
    assert weights.shape[0] * ep_size == len(splits)
    m_start = int(sum(int(v) for v in splits[:e_first]))
    total_rows = int(sum(int(v) for v in splits))
    out_list = []
    acc = 0
    for e in range(weights.shape[0]):
        mi = int(splits[e + e_first])
        xe = x[acc:acc + mi]
        acc += mi
        sv = 1.0
        if weight_scale is not None and input_scale is not None:
            sv = float(weight_scale[e]) * float(input_scale.reshape(-1)[0])
        out_list.append(sv * torch.matmul(xe, weights[e].t()))
    output = torch.cat(out_list)
    if output_vec_scale is not None:
        output = output * output_vec_scale.unsqueeze(1)
    output = output.to(x.dtype)
    gather_index, topk_index = calc_gather_index(scatter_index.cpu())
    new_index = (topk * gather_index.long() + topk_index.long())[m_start:m_start + x.shape[0]].to(x.device)
    full = torch.zeros((total_rows, n), dtype=x.dtype, device=x.device)
    full[new_index] = output
    return full.view(full.shape[0] // topk, topk, n).sum(1)


def moe_gather_rs_single(xs, weights_per_rank, splits, scatter_index, topk, input_scales=None, weight_scales=None,
                         output_vec_scales=None, ep_size: int = 1) -> List[torch.Tensor]:
    """All ranks in one process; reduce_scatter_tensor (moe_gather_rs_utils.py:111-119) = fp32 sum of the
    per-rank partials in rank order, one rounding, row slice. With expert parallelism rank r belongs to expert
    group r // (world / ep_size)."""
    world = len(xs)
    parts = [
        moe_gather_rs_partial(
            xs[r], weights_per_rank[r], splits, scatter_index, topk,
            None if input_scales is None else input_scales[r],
            None if weight_scales is None else weight_scales[r],
            None if output_vec_scales is None else output_vec_scales[r],
            ep_rank=r // (world // ep_size), ep_size=ep_size,
        )
        for r in range(world)
    ]
    total = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        total += p.float()
    total = total.to(parts[0].dtype)
    tpr = total.shape[0] // world
    return [total[r * tpr:(r + 1) * tpr].contiguous() for r in range(world)]


def moe_gather_rs_dist(group, x, weights, splits, scatter_index, topk, input_scale=None, weight_scale=None,
                       output_vec_scale=None):
    """One rank of the golden MoE layer 1 over a process group."""
    part = moe_gather_rs_partial(x, weights, splits, scatter_index, topk, input_scale, weight_scale,
                                 output_vec_scale).contiguous()
    world = dist.get_world_size(group)
    out = torch.zeros((part.shape[0] // world, part.shape[1]), dtype=part.dtype, device=part.device)
    try:
        dist.reduce_scatter_tensor(out, part, group=group)
    except (RuntimeError, NotImplementedError):
        tmp = part.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out = tmp[r * out.shape[0]:(r + 1) * out.shape[0]].clone()
    return out


# --------------------------------------------------------------------------- comparison
def max_rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max |x - ref| / max |ref| - the relative error the parity bar is written in."""
    x = x.float().cpu()
    ref = ref.float().cpu()
    denom = ref.abs().max().item()
    return (x - ref).abs().max().item() / (denom if denom > 0 else 1.0)


def torch_allclose(x, y, rtol, atol) -> bool:
    """python/flux/util.py `torch_allclose`: elementwise |x-y| <= atol + rtol*|y|."""
    x = x.float().cpu()
    y = y.float().cpu()
    return bool(((x - y).abs() <= atol + rtol * y.abs()).all())
