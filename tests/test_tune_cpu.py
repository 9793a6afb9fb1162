"""Tuning sweep and records (flux_b200/tune.py) with an injected timer: no GPU needed."""
import math

import pytest
import torch
import torch.distributed as dist

from _dist import run_distributed


def test_sweep_picks_fastest_and_skips_rejected():
    from flux_b200 import tune

    cost = {None: 3.0, 256: 2.0, 128: 1.0, 64: 1.0}
    calls = []

    def run(t):
        bn = t["block_n"] if t else None
        if bn == 192:
            raise RuntimeError("rejected by the library")
        calls.append(bn)
        return bn

    def timer(fn, iters, warmup):
        return cost[fn()]

    cands = (None, {"block_n": 256}, {"block_n": 192}, {"block_n": 128}, {"block_n": 64})
    best, table = tune.sweep(run, None, cands, timer=timer)
    assert best == {"block_n": 128}  # the earlier of the two fastest
    assert [ms for _, ms in table] == [3.0, 2.0, math.inf, 1.0, 1.0]


def test_table_roundtrip(tmp_path):
    from flux_b200 import tune

    t = tune.TuningTable()
    key = tune.record_key("gemm_rs", 4096, 12288, 6144, torch.bfloat16, 8)
    assert key == "gemm_rs|m=4096|n=12288|k=6144|bfloat16|tp=8"
    rec = t.put(key, {"block_n": 256, "cta_group": 2}, 0.5)
    t.put(tune.record_key("ag_gemm", 1, 8, 8, torch.float16, 1), None, 0.01)
    assert "block_n" in tune.record_line(key, rec)
    path = tmp_path / "tuning.json"
    t.save(str(path))
    u = tune.TuningTable()
    u.load(str(path))
    assert u.get(key) == {"block_n": 256, "cta_group": 2}
    assert u.get("ag_gemm|m=1|n=8|k=8|float16|tp=1") is None and len(u.records) == 2
    assert u.get("unknown") is None
    path.write_text('{"x": 3}')
    with pytest.raises(RuntimeError):
        u.load(str(path))


def _agree_case(rank, world):
    from flux_b200 import tune

    # rank 0 finds candidate A faster, rank 1 candidate B; the slowest rank decides for both
    times = [{"a": 1.0, "b": 2.0}, {"a": 5.0, "b": 2.5}][rank]
    cands = ({"block_n": 64}, {"block_n": 128})
    names = {64: "a", 128: "b"}
    best, table = tune.sweep(lambda t: names[t["block_n"]], dist.group.WORLD, cands,
                             timer=lambda fn, i, w: times[fn()])
    assert best == {"block_n": 128}
    assert [ms for _, ms in table] == [5.0, 2.5]


def test_sweep_ranks_agree_world2():
    run_distributed(_agree_case, 2, use_cuda=False)


def test_profiling_context_and_load_tuning_record():
    """`ProfilingContext` keeps every candidate's time per problem, reports the top ones as text and hands out
    records that `load_tuning_record` installs (src/ths_op/ths_op.cc:208-318)."""
    from flux_b200 import ops, tune

    ctx = ops.ProfilingContext("x")
    with pytest.raises(RuntimeError):
        ctx.get_latest_record()
    table = [(None, 0.50), ({"block_n": 128, "cta_group": 2}, 0.42), ({"ag_mode": 2}, 0.47)]
    rec = ctx.add("ag_gemm|m=8|n=8|k=8|bfloat16|tp=2", table)
    assert rec.tuning == {"block_n": 128, "cta_group": 2} and rec.ms == 0.42
    text = ctx.get_latest_prof_result()
    assert text.splitlines()[0] == rec.key and "TopK=1 (0.420 ms)" in text and "TopK=3 (0.500 ms)" in text
    assert ctx.get_code() == repr(rec) and len(ctx.get_all_records()) == 1
    try:
        ops.load_tuning_record(rec)
        assert tune.TABLE.get(rec.key) == rec.tuning
    finally:
        tune.TABLE.records.clear()
