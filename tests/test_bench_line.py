"""CPU checks of bench.py: the JSON line is built by a pure function from a dict of measurements, so the keys the
harness reads can be checked without a GPU; and a static pass over the scripts that only ever run on a GPU box
finds names that are used but defined nowhere (a typo there would otherwise surface after the timing has run)."""
import builtins
import importlib.util
import json
import os
import symtable
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _fake_meas(world, with_optional=True):
    meas = {"world": world, "steps": 20, "warmup": 5, "ms_per_step": 8.0 / world, "ag_ms": 3.9 / world,
            "rs_ms": 4.0 / world, "timed_region_s": 0.16 / world, "peaks": (1418.9, 1647.8, "measured"),
            "wall_ms_timed_region": 170.0 / world, "native_library": "/x/libfluxb.so"}
    if with_optional:
        meas.update({
            "unfused": {"what": "x", "ms_per_step": 7.5 / world, "ms_before_fused_region": 7.4, "ms_after_fused_region": 7.6,
                        "max_rel_diff_vs_fused": 1e-3},
            "e2e": {"ms_per_step": 9.0 / world, "mode": "pipelined", "h2d_bytes_per_step": 100663296,
                    "d2h_bytes_per_step": 100663296},
            "parity": {"ag_max_rel_err": 2e-3, "rs_max_rel_err": 3e-3, "ag_allclose_1e-2": True, "rs_allclose_2e-2": True},
            "nvlink": {"ag_gemm": {"bytes": 88e6, "seconds": 2e-4, "gbs": 440.0, "frac_of_900": 0.49}},
            "cpu_baseline": {"value": 0.2, "unit": "TFLOP/s", "cores": 16, "kind": "port", "sample": "s"},
            "clocks": {"sm_mhz": 1400.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"]},
            "fp8_ag_gemm": {"ms": 0.4}, "moe": {"ms_per_step": 0.9},
        })
    return meas


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_line_has_every_key_the_harness_reads(world):
    bench = _load_bench()
    line = bench.make_line(_fake_meas(world))
    json.loads(json.dumps(line))  # serialisable
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "roofline", "cpu_baseline", "clocks",
                "parity", "unfused", "speedup_vs_unfused"):
        assert key in line, key
    assert line["n_gpus"] == world and line["config"]["workload"].endswith(f"TP={world}")
    assert "model" not in line["config"]
    for key in ("bound", "achieved", "peak", "unit", "frac", "traffic", "algorithmic_bytes", "nvlink"):
        assert key in line["roofline"], key
    for key in ("value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"):
        assert key in line["e2e"], key
    # whole-job throughput: 2 GEMMs of 2*M*N*K flops over all ranks
    flops = 2 * 2.0 * bench.M * bench.N0 * bench.K0
    assert line["value"] == pytest.approx(flops / (line["ms_per_step"] * 1e-3) / 1e12)
    assert line["e2e"]["value"] == pytest.approx(flops / (9.0 / world * 1e-3) / 1e12)
    assert line["e2e"]["value"] != line["value"]
    assert line["gpu_launches"] == 40
    # a timed region shorter than a second is compared with the burst peak
    assert line["roofline"]["peak"] == 1647.8
    assert line["roofline"]["frac"] == pytest.approx(line["roofline"]["achieved"] / 1647.8)
    assert line["speedup_vs_unfused"] == pytest.approx(7.5 / 8.0)


def test_line_survives_failed_optional_legs():
    bench = _load_bench()
    meas = _fake_meas(8, with_optional=False)
    meas["timed_region_s"] = 2.5
    meas["e2e"] = {"error": "RuntimeError: boom"}
    meas["unfused"] = {"error": "RuntimeError: boom"}
    line = bench.make_line(meas)
    json.dumps(line)
    assert line["roofline"]["peak"] == 1418.9  # a long region is compared with the sustained peak
    assert line["speedup_vs_unfused"] is None
    assert "error" in line["e2e"] and "h2d_bytes_per_step" in line["e2e"]
    assert line["cpu_baseline"] is None and line["parity"] is None


def test_parity_gate():
    bench = _load_bench()
    assert bench.parity_ok(None) and bench.parity_ok({"error": "x"})
    good = {"ag_max_rel_err": 1e-3, "rs_max_rel_err": 9e-3, "ag_allclose_1e-2": True, "rs_allclose_2e-2": True}
    assert bench.parity_ok(good)
    assert not bench.parity_ok(dict(good, rs_max_rel_err=2e-2))
    assert not bench.parity_ok(dict(good, **{"ag_allclose_1e-2": False}))
    # GEMM-RS elementwise bar: an isolated rounding flip is tolerated, a pattern is not
    assert bench.parity_ok(dict(good, **{"rs_allclose_2e-2": False, "rs_outside_2e-2_frac": 1 / 128}))
    assert not bench.parity_ok(dict(good, **{"rs_allclose_2e-2": False, "rs_outside_2e-2_frac": 0.05}))
    assert not bench.parity_ok(dict(good, **{"rs_allclose_2e-2": False}))


# ------------------------------------------------------------------------------------------------
def _undefined_globals(path):
    """Names a function reads as globals although neither the module nor builtins define them."""
    src = open(path).read()
    top = symtable.symtable(src, path, "exec")
    module_names = {s.get_name() for s in top.get_symbols() if s.is_assigned() or s.is_imported() or s.is_namespace()}
    known = module_names | set(dir(builtins)) | {"__file__", "__name__", "__doc__"}
    bad = []

    def walk(tab):
        for child in tab.get_children():
            if child.get_type() in ("function", "class"):
                for s in child.get_symbols():
                    if s.is_global() and s.is_referenced() and not s.is_assigned() and s.get_name() not in known:
                        bad.append(f"{os.path.basename(path)}:{child.get_name()}:{s.get_name()}")
            walk(child)

    walk(top)
    return bad


def _gpu_side_sources():
    files = [os.path.join(ROOT, "bench.py"), os.path.join(ROOT, "__graft_entry__.py")]
    for d in ("flux_b200", "tests", "examples"):
        full = os.path.join(ROOT, d)
        if os.path.isdir(full):
            files += [os.path.join(full, f) for f in sorted(os.listdir(full)) if f.endswith(".py")]
    return files


def test_no_undefined_names_in_gpu_side_scripts():
    bad = []
    for f in _gpu_side_sources():
        bad += _undefined_globals(f)
    assert not bad, bad


def test_static_pass_catches_a_closure_variable_used_outside():
    src = "def f():\n    def g():\n        inner = 1\n    return inner\n"
    path = os.path.join(ROOT, "tests", "_build", "undef_probe.py")
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as fh:
        fh.write(src)
    try:
        assert _undefined_globals(path) == ["undef_probe.py:f:inner"]
    finally:
        os.unlink(path)
