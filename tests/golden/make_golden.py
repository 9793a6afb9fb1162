"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run where a checkout of the reference (bytedance/flux) is available:

    python tests/golden/make_golden.py --reference /path/to/flux

The reference's pure-torch golden helpers live in `python/flux/testing/*.py`,
which `import flux` (the compiled extension, not buildable here). This script
registers a stub module named `flux` that only supplies `is_fp8_dtype` and
placeholder attributes, loads the helper files from the reference tree as they
are, and runs them on seeded CPU inputs (2 gloo ranks where a collective is
involved). Inputs and outputs are written to `tests/golden/*.pt`; the tests
then check `oracle/golden.py` against them without needing the reference.
Nothing from the reference is copied: only its outputs are stored.
"""
import argparse
import ast
import contextlib
import importlib.util
import os
import socket
import sys
import types
from pathlib import Path
from unittest import mock

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent


def _install_stub():
    flux = types.ModuleType("flux")
    util = types.ModuleType("flux.util")

    def is_fp8_dtype(dt):
        return dt in (torch.float8_e4m3fn, torch.float8_e5m2)

    util.is_fp8_dtype = is_fp8_dtype
    flux.is_fp8_dtype = is_fp8_dtype
    flux.util = util
    # anything else the helper modules touch at import time is a placeholder
    flux.__getattr__ = lambda name: mock.MagicMock(name=f"flux.{name}")
    testing = types.ModuleType("flux.testing")
    testing.__path__ = []
    flux.testing = testing
    sys.modules["flux"] = flux
    sys.modules["flux.util"] = util
    sys.modules["flux.testing"] = testing
    return flux, testing


def _load(ref_root: Path, name: str, testing_mod):
    path = ref_root / "python" / "flux" / "testing" / f"{name}.py"
    spec = importlib.util.spec_from_file_location(f"flux.testing.{name}", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[f"flux.testing.{name}"] = mod
    spec.loader.exec_module(mod)
    for k, v in vars(mod).items():
        if not k.startswith("_"):
            setattr(testing_mod, k, v)
    return mod


def load_reference_helpers(ref_root: Path):
    _, testing = _install_stub()
    utils = _load(ref_root, "utils", testing)
    moe_utils = _load(ref_root, "moe_utils", testing)
    ag = _load(ref_root, "moe_ag_scatter_utils", testing)
    rs = _load(ref_root, "moe_gather_rs_utils", testing)
    return utils, moe_utils, ag, rs


# ----------------------------------------------------------------------------- routing (integer)
def gen_routing(moe_utils):
    cases = []
    for seed, (ntokens, topk, nexperts) in enumerate([(16, 2, 4), (64, 2, 8), (37, 3, 5), (128, 4, 32), (8, 1, 8)]):
        g = torch.Generator().manual_seed(100 + seed)
        scores = torch.rand(ntokens, nexperts, generator=g)
        chosen = torch.topk(scores, topk, dim=-1).indices.to(torch.int32)
        scatter = moe_utils.calc_scatter_index_stable(chosen)  # reference function
        splits = torch.bincount(chosen.view(-1), minlength=nexperts).to(torch.int32)  # moe_utils.py:212-214
        cases.append({"chosen": chosen, "nexperts": nexperts, "scatter_index": scatter, "splits": splits})
    torch.save(cases, HERE / "routing.pt")
    print("routing.pt:", len(cases), "cases")


# ----------------------------------------------------------------------------- MoE layer 0 (scatter + grouped GEMM)
def gen_moe_l0(ag, moe_utils):
    cases = []
    for seed, (ntokens, topk, nexperts, hidden, ffn, dtype) in enumerate(
        [(32, 2, 4, 64, 48, torch.float32), (64, 2, 8, 128, 96, torch.bfloat16)]
    ):
        g = torch.Generator().manual_seed(200 + seed)
        scores = torch.rand(ntokens, nexperts, generator=g)
        chosen = torch.topk(scores, topk, dim=-1).indices.to(torch.int32)
        scatter = moe_utils.calc_scatter_index_stable(chosen)
        splits = torch.bincount(chosen.view(-1), minlength=nexperts).to(torch.int32)
        inv = torch.empty(ntokens * topk, dtype=torch.int64)
        inv[scatter.view(-1).long()] = torch.arange(ntokens * topk) // topk
        tokens = torch.randn(ntokens, hidden, generator=g).to(dtype)
        weights = (torch.randn(nexperts, ffn, hidden, generator=g) * 0.05).to(dtype)
        out_scale = torch.rand(nexperts, generator=g) + 0.5
        ctx = types.SimpleNamespace(
            inputs=tokens, scatter_inputs=torch.zeros(ntokens * topk, hidden, dtype=dtype), gather_index=inv,
            is_s8=False, input_scale=None, weight_groups=1, nexperts_ep=nexperts, ep_rank=0,
            splits_cpu=splits, outputs=[torch.zeros(ntokens * topk, ffn, dtype=dtype)], weights=[weights],
            fast_accum=False, bias=None, output_scale=[out_scale],
        )
        ag.MoeAgScatterWithTorch.scatter_impl(ctx)  # reference functions
        ag.MoeAgScatterWithTorch.gemm_impl(ctx, None)
        cases.append({"tokens": tokens, "weights": weights, "splits": splits, "scatter_index": scatter,
                      "output_scale": out_scale, "out": ctx.outputs[0].clone()})
    torch.save(cases, HERE / "moe_l0.pt")
    print("moe_l0.pt:", len(cases), "cases")


def gen_moe_l0_ep(ag, moe_utils):
    """Layer 0 with expert parallelism: the reference's gemm_impl for every ep_rank of ep_size = 2 (each rank holds
    half of the experts and produces only their rows)."""
    cases = []
    ntokens, topk, nexperts, hidden, ffn, dtype, ep_size = 48, 2, 8, 64, 40, torch.bfloat16, 2
    g = torch.Generator().manual_seed(230)
    scores = torch.rand(ntokens, nexperts, generator=g)
    chosen = torch.topk(scores, topk, dim=-1).indices.to(torch.int32)
    scatter = moe_utils.calc_scatter_index_stable(chosen)
    splits = torch.bincount(chosen.view(-1), minlength=nexperts).to(torch.int32)
    inv = torch.empty(ntokens * topk, dtype=torch.int64)
    inv[scatter.view(-1).long()] = torch.arange(ntokens * topk) // topk
    tokens = torch.randn(ntokens, hidden, generator=g).to(dtype)
    e_local = nexperts // ep_size
    for ep_rank in range(ep_size):
        weights = (torch.randn(e_local, ffn, hidden, generator=g) * 0.05).to(dtype)
        out_scale = torch.rand(e_local, generator=g) + 0.5
        nrows = int(splits[ep_rank * e_local:(ep_rank + 1) * e_local].sum())
        ctx = types.SimpleNamespace(
            inputs=tokens, scatter_inputs=torch.zeros(ntokens * topk, hidden, dtype=dtype), gather_index=inv,
            is_s8=False, input_scale=None, weight_groups=1, nexperts_ep=e_local, ep_rank=ep_rank,
            splits_cpu=splits, outputs=[torch.zeros(nrows, ffn, dtype=dtype)], weights=[weights],
            fast_accum=False, bias=None, output_scale=[out_scale],
        )
        ag.MoeAgScatterWithTorch.scatter_impl(ctx)
        ag.MoeAgScatterWithTorch.gemm_impl(ctx, None)
        cases.append({"tokens": tokens, "weights": weights, "splits": splits, "scatter_index": scatter,
                      "output_scale": out_scale, "ep_rank": ep_rank, "ep_size": ep_size, "out": ctx.outputs[0].clone()})
    torch.save(cases, HERE / "moe_l0_ep.pt")
    print("moe_l0_ep.pt:", len(cases), "cases")


def _l1_ep_worker(rank, world, port, ref_root, out_path):
    """Layer 1 with expert parallelism on 2 gloo ranks: ffn TP size 1, EP size 2 (rank = ep_rank)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _, moe_utils, _, rs = load_reference_helpers(Path(ref_root))
    ntokens, topk, nexperts, kloc, n, dtype = 32, 2, 8, 48, 40, torch.bfloat16
    g = torch.Generator().manual_seed(330)
    chosen = torch.topk(torch.rand(ntokens, nexperts, generator=g), topk, dim=-1).indices.to(torch.int32)
    scatter = moe_utils.calc_scatter_index_stable(chosen)
    splits = torch.bincount(chosen.view(-1), minlength=nexperts).to(torch.int32)
    order = chosen.flatten().sort(stable=True).indices
    token_index = (order // topk).to(torch.int32)
    topk_index = torch.arange(topk, dtype=torch.int32).repeat(ntokens)[order]
    e_local = nexperts // world
    eid_start = rank * e_local
    m_start = int(splits[:eid_start].sum())
    m_end = m_start + int(splits[eid_start:eid_start + e_local].sum())
    gr = torch.Generator().manual_seed(340 + rank)
    x = torch.randn(m_end - m_start, kloc, generator=gr).to(dtype)
    w = (torch.randn(e_local, n, kloc, generator=gr) * 0.05).to(dtype)
    vec = torch.rand(m_end - m_start, generator=gr) + 0.25
    full = rs.moe_gather_rs_forward_torch(
        dist.group.WORLD, ntokens * topk, eid_start, m_start, m_end, x, w, splits, token_index, topk_index, topk,
        torch.ones(1), torch.ones(e_local), vec, do_all_reduce=True,
    )
    tpr = ntokens // world
    mine = {"x": x, "w": w, "vec": vec, "out": full[rank * tpr:(rank + 1) * tpr].clone()}
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        torch.save({"topk": topk, "scatter_index": scatter, "splits": splits, "ep_size": world, "ranks": gathered}, out_path)
    dist.destroy_process_group()


def gen_moe_l1_ep(ref_root):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_l1_ep_worker, args=(2, port, str(ref_root), str(HERE / "moe_l1_ep.pt")), nprocs=2, join=True)
    print("moe_l1_ep.pt: 1 case")


# ----------------------------------------------------------------------------- MoE layer 1 (2 gloo ranks)
def _l1_inputs(rank, case):
    ntokens, topk, nexperts, kloc, n, dtype = case
    g = torch.Generator().manual_seed(300)  # routing is global: same on every rank
    scores = torch.rand(ntokens, nexperts, generator=g)
    chosen = torch.topk(scores, topk, dim=-1).indices.to(torch.int32)
    gr = torch.Generator().manual_seed(310 + rank)
    x = torch.randn(ntokens * topk, kloc, generator=gr).to(dtype)
    w = (torch.randn(nexperts, n, kloc, generator=gr) * 0.05).to(dtype)
    vec = torch.rand(ntokens * topk, generator=gr) + 0.25
    return chosen, x, w, vec


def _l1_worker(rank, world, port, ref_root, case, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _, moe_utils, _, rs = load_reference_helpers(Path(ref_root))
    ntokens, topk, nexperts, kloc, n, dtype = case
    chosen, x, w, vec = _l1_inputs(rank, case)
    scatter = moe_utils.calc_scatter_index_stable(chosen)
    splits = torch.bincount(chosen.view(-1), minlength=nexperts).to(torch.int32)
    order = chosen.flatten().sort(stable=True).indices  # calc_gather_index_stable (moe_utils.py:87-93) on CPU
    token_index = (order // topk).to(torch.int32)
    topk_index = torch.arange(topk, dtype=torch.int32).repeat(ntokens)[order]
    # reference golden; do_all_reduce=True keeps every tensor on the CPU (the reduce-scatter branch
    # allocates on CUDA); the reduce-scattered result is the row slice of the all-reduced one.
    full = rs.moe_gather_rs_forward_torch(
        dist.group.WORLD, ntokens * topk, 0, 0, ntokens * topk, x, w, splits, token_index, topk_index, topk,
        torch.ones(1), torch.ones(nexperts), vec, do_all_reduce=True,
    )
    tpr = ntokens // world
    mine = {"x": x, "w": w, "vec": vec, "out": full[rank * tpr:(rank + 1) * tpr].clone()}
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        torch.save({"case": case, "chosen": chosen, "scatter_index": scatter, "splits": splits, "ranks": gathered},
                   out_path)
    dist.destroy_process_group()


def gen_moe_l1(ref_root):
    outs = []
    for i, case in enumerate([(16, 2, 4, 32, 24, torch.float32), (32, 2, 8, 64, 48, torch.bfloat16)]):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        tmp = HERE / f"_l1_{i}.pt"
        mp.spawn(_l1_worker, args=(2, port, str(ref_root), case, str(tmp)), nprocs=2, join=True)
        outs.append(torch.load(tmp, weights_only=False))
        tmp.unlink()
    torch.save(outs, HERE / "moe_l1.pt")
    print("moe_l1.pt:", len(outs), "cases")


# ----------------------------------------------------------------------------- dense AG-GEMM / GEMM-RS (2 gloo ranks)
class _NoCudaEvent:
    """Timing events of the reference's golden functions; the timings are not used."""

    def __init__(self, *a, **k):
        pass

    def record(self, *a, **k):
        pass

    def synchronize(self):
        pass

    def elapsed_time(self, other):
        return 0.0


class _TorchOnCpu:
    """`torch` as the extracted functions see it: everything is the real module except `torch.cuda`, whose
    events do nothing and whose current device is the CPU (the functions allocate on `current_device()`)."""

    cuda = types.SimpleNamespace(Event=_NoCudaEvent, current_device=lambda: "cpu")

    def __getattr__(self, name):
        return getattr(torch, name)


def _extract(ref_root: Path, rel: str, names):
    """Compile the named top-level functions / classes of a reference script, unmodified, without running
    the script (it parses arguments and needs the compiled extension at import)."""
    path = ref_root / rel
    tree = ast.parse(path.read_text(), filename=str(path))
    keep = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    assert len(keep) == len(names), f"{rel}: expected {names}"
    return compile(ast.Module(body=keep, type_ignores=[]), str(path), "exec")


def dense_inputs(case, rank, world):
    """Seeded inputs of one rank for a dense case (m, n, k, dtype, with_bias); shared with tests/test_oracle.py."""
    m, n, k, dtype, with_bias = case
    g = torch.Generator().manual_seed(400 + rank)
    out = {"ag_input": torch.randn(m // world, k, generator=g).to(dtype),
           "ag_weight": (torch.randn(n // world, k, generator=g) * 0.05).to(dtype),
           "ag_bias": (torch.randn(m, n // world, generator=g) * 0.1).to(dtype) if with_bias else None,
           "rs_input": torch.randn(m, k // world, generator=g).to(dtype),
           "rs_weight": (torch.randn(n, k // world, generator=g) * 0.05).to(dtype),
           "rs_bias": (torch.randn(m, n, generator=g) * 0.1).to(dtype) if with_bias else None,
           "input_scale": None, "weight_scale": None}
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        # the reference's fp8 golden takes one scalar scale per operand, the same on every rank
        gs = torch.Generator().manual_seed(499)
        out["input_scale"] = torch.rand(1, generator=gs) + 0.5
        out["weight_scale"] = torch.rand(1, generator=gs) + 0.5
    return out


def _dense_worker(rank, world, port, ref_root, case, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    flux_stub, _ = _install_stub()
    flux_stub.util.with_torch_deterministic = lambda mode, warn_only=True: contextlib.nullcontext()
    from typing import Optional

    base = {"torch": _TorchOnCpu(), "flux": flux_stub, "TP_GROUP": dist.group.WORLD, "WORLD_SIZE": world,
            "RANK": rank, "Optional": Optional,
            "zeros_with_fp8": lambda *a, **kw: torch.zeros(*a, **kw)}
    d = dense_inputs(case, rank, world)
    # AG-GEMM: test/python/ag_gemm/test_ag_kernel.py `perf_torch`
    ns_ag = dict(base)
    exec(_extract(Path(ref_root), "test/python/ag_gemm/test_ag_kernel.py", ["PerfResult", "perf_torch"]), ns_ag)
    is_fp8 = d["input_scale"] is not None
    r_ag = ns_ag["perf_torch"](d["ag_input"], d["ag_weight"], d["ag_bias"], d["input_scale"], d["weight_scale"],
                               is_fp8, False, 0, 1)
    # GEMM-RS: test/python/gemm_rs/test_gemm_rs.py `perf_torch`
    ns_rs = dict(base)
    exec(_extract(Path(ref_root), "test/python/gemm_rs/test_gemm_rs.py", ["PerfResult", "perf_torch"]), ns_rs)
    # (its fp8 branch calls the compiled GemmOnly op, so fp8 cases stop at the AG-GEMM)
    r_rs = None if is_fp8 else ns_rs["perf_torch"](d["rs_input"], d["rs_weight"], d["rs_bias"], 0, 1)
    # only the outputs are stored; the test regenerates the seeded inputs with `dense_inputs`
    mine = {"ag_out": r_ag.output.clone(), "ag_gathered_sum": r_ag.gathered_output.double().sum().item(),
            "rs_out": None if r_rs is None else r_rs.output.clone()}
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        torch.save({"case": case, "ranks": gathered}, out_path)
    dist.destroy_process_group()


def gen_dense(ref_root):
    outs = []
    cases = [(256, 512, 512, torch.float32, False),   # the reference's CPU-runnable smoke shape
             (64, 96, 128, torch.bfloat16, True), (48, 64, 64, torch.float16, True),
             (64, 96, 128, torch.float8_e4m3fn, False)]
    for i, case in enumerate(cases):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        tmp = HERE / f"_dense_{i}.pt"
        mp.spawn(_dense_worker, args=(2, port, str(ref_root), case, str(tmp)), nprocs=2, join=True)
        outs.append(torch.load(tmp, weights_only=False))
        tmp.unlink()
    torch.save(outs, HERE / "dense.pt")
    print("dense.pt:", len(outs), "cases")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference")
    ap.add_argument("--only-ep", action="store_true", help="only the expert-parallel MoE vectors")
    args = ap.parse_args()
    ref_root = Path(args.reference)
    _, moe_utils, ag, _ = load_reference_helpers(ref_root)
    gen_moe_l0_ep(ag, moe_utils)
    gen_moe_l1_ep(ref_root)
    if args.only_ep:
        return
    gen_routing(moe_utils)
    gen_moe_l0(ag, moe_utils)
    gen_moe_l1(ref_root)
    gen_dense(ref_root)


if __name__ == "__main__":
    main()
