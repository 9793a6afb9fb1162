"""Python-level helpers with the reference's names (python/flux/util.py)."""
from __future__ import annotations

import json
import pathlib
import sys
from contextlib import contextmanager, nullcontext
from typing import List

import torch

from .ops import is_fp8_dtype  # noqa: F401  (python/flux/util.py:175-177)


def get_arch() -> int:
    """python/flux/util.py:31-35: compute capability as major*10 + minor."""
    p = torch.cuda.get_device_properties(torch.cuda.current_device())
    return p.major * 10 + p.minor


def torch_allclose(x, y, rtol, atol, verbose=True):
    """python/flux/util.py:38-69: raise RuntimeError with a mismatch report unless allclose."""
    if not torch.allclose(x, y, rtol=rtol, atol=atol):
        diff_loc = ~torch.isclose(x, y, rtol=rtol, atol=atol)
        num = int(diff_loc.sum())
        print(f"diff count: {num} of {y.numel()}, max diff {float((x - y).abs().max())}, atol {atol}, rtol {rtol}",
              file=sys.stderr)
        print(f"diff locations:\n{diff_loc.nonzero(as_tuple=False)[:16]}", file=sys.stderr)
        raise RuntimeError("torch_allclose failed")
    if verbose:
        print("all close!")


@contextmanager
def with_torch_deterministic(mode: bool, warn_only: bool = True):
    """python/flux/util.py:180-186."""
    old_mode = torch.are_deterministic_algorithms_enabled()
    old_warn = torch.is_deterministic_algorithms_warn_only_enabled()
    torch.use_deterministic_algorithms(mode, warn_only=warn_only)
    try:
        yield
    finally:
        torch.use_deterministic_algorithms(old_mode, warn_only=old_warn)


def bench_func(func, iters, warmup_iters):
    """python/flux/util.py:189-203: CUDA-event timing; returns (last output, ms per iteration)."""
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    out = None
    for n in range(iters + warmup_iters):
        if n == warmup_iters:
            start.record()
        out = func()
    stop.record()
    start.wait()
    stop.wait()
    torch.cuda.current_stream().synchronize()
    return out, start.elapsed_time(stop) / iters


class group_profile:
    """python/flux/util.py:111-172: torch.profiler around a block, one chrome trace per rank,
    merged on rank 0 of `group`."""

    def __init__(self, name: str = None, do_prof: bool = True, merge_group=None, keep_merged_only: bool = True):
        self.name, self.do_prof, self.group = name, do_prof, merge_group
        self.keep_merged_only = keep_merged_only
        self.prof = None

    def __enter__(self):
        if self.do_prof:
            self.prof = torch.profiler.profile(
                activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA],
                record_shapes=True, with_stack=False)
            self.prof.__enter__()
        return self

    def __exit__(self, *exc):
        if self.prof is None:
            return False
        self.prof.__exit__(*exc)
        import torch.distributed as dist

        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        outdir = pathlib.Path("prof") / (self.name or "trace")
        outdir.mkdir(parents=True, exist_ok=True)
        mine = outdir / f"rank{rank}.json"
        self.prof.export_chrome_trace(str(mine))
        if world > 1:
            dist.barrier(group=self.group)
        if rank == 0:
            events: List[dict] = []
            for r in range(world):
                f = outdir / f"rank{r}.json"
                if not f.exists():
                    continue
                data = json.loads(f.read_text())
                for ev in data.get("traceEvents", []):
                    if isinstance(ev.get("pid"), int):
                        ev["pid"] = ev["pid"] + r * 1000000
                    events.append(ev)
                if self.keep_merged_only:
                    f.unlink()
            (outdir / "merged.json").write_text(json.dumps({"traceEvents": events}))
        return False
