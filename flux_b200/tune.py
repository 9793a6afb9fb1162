"""Run-time tuning of the fused ops: sweep tile shapes per problem shape, keep the best, persist it.

Stands in for the reference's `profiling()` methods and tuning records (`ProfilingContext`,
src/ths_op/ths_op.cc:217-318; `tools/tune_ag_gemm_kernel.py`, `tools/tune_gemm_rs.py`): the reference sweeps
its generated kernel configurations, max-reduces each time over the ranks and records the winner as code; here
the kernel is one template, so a record is the `fluxb_tuning` fields (tile width, band height, CTA-pair mode)
for one (op, M, N, K, dtype, world) key. Records are plain dicts and are saved as JSON.

Every rank times every candidate and the maximum over the ranks decides, so all ranks choose the same record
(the reduce-scatter counters are indexed by tile width: ranks must agree).
"""
from __future__ import annotations

import json
import math
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

Tuning = Optional[Dict[str, int]]

# `None` (the library's own choice) comes first so that it wins ties.
DEFAULT_CANDIDATES: Tuple[Tuning, ...] = (
    None,
    {"block_n": 256, "cta_group": 2},
    {"block_n": 256, "cta_group": 2, "group_m": 4},
    {"block_n": 256, "cta_group": 2, "group_m": 8},
    {"block_n": 256, "cta_group": 2, "group_m": 16},
    {"block_n": 128, "cta_group": 2},
    {"block_n": 256, "cta_group": 1},
    {"block_n": 192, "cta_group": 1},
    {"block_n": 128, "cta_group": 1},
    # transport of the all-gather (ignored by ops without one): kernel push / copy engines
    {"ag_mode": 1},
    {"ag_mode": 2},
)


def record_key(op: str, m: int, n: int, k: int, dtype: torch.dtype, world: int) -> str:
    return f"{op}|m={int(m)}|n={int(n)}|k={int(k)}|{str(dtype).replace('torch.', '')}|tp={int(world)}"


def cuda_event_timer(fn: Callable[[], object], iters: int, warmup: int) -> float:
    """Milliseconds per call, CUDA events on the current stream, synchronised on both sides."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _max_over_ranks(ms: float, group) -> float:
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ms
    # inf marks a candidate this rank could not run; the maximum keeps it inf for everyone
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sweep(run: Callable[[Tuning], object], group=None, candidates: Iterable[Tuning] = DEFAULT_CANDIDATES,
          iters: int = 5, warmup: int = 2, timer: Callable[[Callable[[], object], int, int], float] = cuda_event_timer
          ) -> Tuple[Tuning, List[Tuple[Tuning, float]]]:
    """Time `run(tuning)` for every candidate; returns (best tuning, [(tuning, ms max over ranks), ...]).

    A candidate the library rejects (RuntimeError from argument checks: the same on every rank, because the
    checks depend only on the shapes) counts as infinitely slow. Ties go to the earlier candidate.
    """
    table: List[Tuple[Tuning, float]] = []
    best: Tuning = None
    best_ms = math.inf
    for cand in candidates:
        try:
            ms = timer(lambda: run(cand), iters, warmup)
        except RuntimeError:
            ms = math.inf
        ms = _max_over_ranks(ms, group)
        table.append((cand, ms))
        if ms < best_ms:
            best, best_ms = cand, ms
    return best, table


class TuningTable:
    """Best-known tuning per problem key; consulted by the ops when the caller passes no tuning."""

    def __init__(self):
        self.records: Dict[str, Dict] = {}

    def put(self, key: str, tuning: Tuning, ms: float) -> Dict:
        rec = {"tuning": dict(tuning) if tuning else None, "ms": ms}
        self.records[key] = rec
        return rec

    def get(self, key: str) -> Tuning:
        rec = self.records.get(key)
        return rec["tuning"] if rec else None

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.records, f, indent=1, sort_keys=True)

    def load(self, path: str) -> None:
        with open(path) as f:
            loaded = json.load(f)
        for key, rec in loaded.items():
            if not isinstance(rec, dict) or "tuning" not in rec:
                raise RuntimeError(f"tuning file {path}: malformed record for {key!r}")
            self.records[key] = {"tuning": rec["tuning"], "ms": float(rec.get("ms", math.nan))}


#: process-wide table (one per process = one per GPU)
TABLE = TuningTable()


def record_line(key: str, rec: Dict) -> str:
    """One record as a line of text for `ProfilingContext` (the reference records generated code there)."""
    return f"fluxb_tuning[{key}] = {json.dumps(rec['tuning'], sort_keys=True)}  # {rec['ms']:.4f} ms"
