"""Invariants of the kernel's tile schedule, checked on the host.

`tests/csrc/schedule_probe.cu` compiles the product's own `decode_tile` / `make_bands`
(flux_b200/csrc/gemm_kernel.cuh) for the host with nvcc and walks every work item of a segmented launch.
As the reference does for its MoE problem schedule (src/moe_ag_scatter/test/test_sort_utils.cc:20-46,210-227:
fixed cases plus random ones, every tile covered exactly once), the tests check that each (segment, 128-row
chunk, column tile) is visited exactly once for every tile width, both tile shapes, ragged segments, uniform
and variable bands, and that the bands keep the visiting order the protocols rely on: all-gather starts with
this rank's own shard and walks the segments in arrival order, reduce-scatter ends with this rank's own rows.
"""
import ctypes as C
import os
import random
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
KBM = 128


@pytest.fixture(scope="module")
def probe():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is needed to compile the host-side schedule probe")
    out_dir = os.path.join(HERE, "_build")
    os.makedirs(out_dir, exist_ok=True)
    so = os.path.join(out_dir, "libschedule_probe.so")
    src = os.path.join(HERE, "csrc", "schedule_probe.cu")
    libdir = os.path.join(ROOT, "flux_b200")
    if not os.path.exists(os.path.join(libdir, "libfluxb.so")):
        pytest.skip("libfluxb.so has not been built")
    deps = [src, os.path.join(libdir, "libfluxb.so")] + [os.path.join(libdir, "csrc", f) for f in
                                                          ("gemm_kernel.cuh", "ptx.cuh", "internal.h")]
    if not os.path.exists(so) or any(os.path.getmtime(d) > os.path.getmtime(so) for d in deps):
        subprocess.run([nvcc, "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler",
                        "-fPIC", "-I" + os.path.join(ROOT, "include"), "-o", so, src, "-L" + libdir, "-lfluxb",
                        "-Xlinker", "-rpath=" + libdir], check=True)
    lib = C.CDLL(so)
    lib.probe_dense_schedule.restype = C.c_int
    lib.probe_dense_schedule.argtypes = [C.c_int] * 8 + [C.POINTER(C.c_int)] * 3 + [C.c_int]
    for fn in (lib.probe_splitk_owner, lib.probe_splitk_owners):
        fn.restype = C.c_int
    lib.probe_splitk_owner.argtypes = [C.c_int] * 4
    lib.probe_splitk_owners.argtypes = [C.c_int] * 3
    lib.probe_rs_late_peers.restype = C.c_int
    lib.probe_rs_late_peers.argtypes = [C.c_int] * 3
    lib.probe_resolve.restype = None
    lib.probe_resolve.argtypes = [C.c_int] * 8 + [C.POINTER(C.c_int)] * 2
    return lib


def walk(lib, nseg, seg_rows, n, block_n, cta_group, seg_first, group_m, bands):
    chunks = (seg_rows + KBM - 1) // KBM
    n_tiles = (n + block_n - 1) // block_n
    tile_m = 256 if cta_group == 2 else 128
    total = nseg * ((seg_rows + tile_m - 1) // tile_m) * n_tiles
    visits = (C.c_int * (nseg * chunks * n_tiles))()
    item_seg = (C.c_int * total)()
    item_m = (C.c_int * total)()
    rc = lib.probe_dense_schedule(nseg, seg_rows, n, block_n, cta_group, seg_first, group_m, bands, visits, item_seg,
                                  item_m, total)
    assert rc == total, f"probe returned {rc} for {(nseg, seg_rows, n, block_n, cta_group, seg_first, group_m, bands)}"
    assert all(v == 1 for v in visits), "a tile is visited twice or never"
    return list(item_seg)


def check_order(segs, nseg, seg_first, bands):
    """Segments appear band by band; the order of first appearance is seg_first, seg_first+1, ... (mod nseg)."""
    first_seen = []
    for s in segs:
        if s not in first_seen:
            first_seen.append(s)
    assert first_seen == [(seg_first + i) % nseg for i in range(nseg)]
    if nseg == 1:
        return
    if bands == 1:  # all-gather: the own shard (= seg_first) is in the first band only
        last_own = max(i for i, s in enumerate(segs) if s == seg_first)
        early = set(segs[:last_own + 1])
        assert early <= {(seg_first + i) % nseg for i in range(4)}, "the first band holds at most four segments"
        k = next((i for i, s in enumerate(segs) if s not in early), len(segs))
        assert all(s not in early for s in segs[k:]), "a later band returns to a segment of the first band"
    if bands == 2:  # reduce-scatter: the own rows (= the last segment of the rotation) are a band of their own at the end
        own = (seg_first + nseg - 1) % nseg
        k = next(i for i, s in enumerate(segs) if s == own)
        assert all(s == own for s in segs[k:])


FIXED = [
    # nseg, seg_rows, n, block_n, cta_group
    (8, 512, 6144, 256, 2),    # D0 per-rank shape at TP=8
    (8, 512, 12288, 256, 2),   # D1 at TP=8
    (4, 1024, 12288, 256, 2),  # TP=4
    (2, 2048, 24576, 256, 2),  # TP=2
    (1, 4096, 49152, 256, 2),  # TP=1
    (8, 200, 520, 64, 1),      # ragged rows and columns
    (8, 1, 8, 64, 1),          # one row per rank
    (3, 300, 1000, 192, 2),    # pair tiles with a ragged second half
]


@pytest.mark.parametrize("case", FIXED)
@pytest.mark.parametrize("bands", [0, 1, 2])
def test_fixed_cases(probe, case, bands):
    nseg, seg_rows, n, bn, cg = case
    for seg_first in {0, nseg - 1, nseg // 2}:
        for gm in ([1, 3, 8, 16] if bands == 0 else [0]):
            segs = walk(probe, nseg, seg_rows, n, bn, cg, seg_first, gm, bands)
            if bands:
                check_order(segs, nseg, seg_first, bands)


def test_random_cases(probe):
    rng = random.Random(1234)
    for _ in range(3000):
        nseg = rng.choice([1, 2, 3, 4, 8])
        seg_rows = rng.choice([rng.randint(1, 2200), 128 * rng.randint(1, 16)])
        n = 8 * rng.randint(1, 400)
        bn = rng.choice([64, 128, 192, 256])
        cg = rng.choice([1, 2])
        bands = rng.choice([0, 1, 2])
        gm = rng.randint(1, 20) if bands == 0 else 0
        seg_first = rng.randrange(nseg)
        segs = walk(probe, nseg, seg_rows, n, bn, cg, seg_first, gm, bands)
        if bands:
            check_order(segs, nseg, seg_first, bands)


def resolve(lib, nseg, seg_rows, n, sms=148, kn=0, bn=0, cg=0, ctas=0):
    out_bn, out_cg = C.c_int(), C.c_int()
    lib.probe_resolve(nseg, seg_rows, n, sms, kn, bn, cg, ctas, C.byref(out_bn), C.byref(out_cg))
    return out_bn.value, out_cg.value


def test_tile_shape_choice(probe):
    """The library's own choice of tile shape for the benchmark shapes (the measured fast configuration is a
    CTA pair on 256 x 256 tiles) and the rules around it."""
    for nseg, seg_rows, n in [(8, 512, 6144), (8, 512, 12288), (4, 1024, 12288), (2, 2048, 24576), (1, 4096, 49152),
                              (1, 4096, 12288)]:
        assert resolve(probe, nseg, seg_rows, n) == (256, 2)
    # segments shorter than a pair tile: one CTA per tile
    assert resolve(probe, 8, 200, 4096)[1] == 1
    # narrow outputs never get a tile more than twice their width
    assert resolve(probe, 1, 128, 64)[0] == 64 and resolve(probe, 1, 128, 8)[0] == 64
    # a [K,N] weight needs whole 64-column boxes per CTA: 128 or 256 for a pair, never 192 (96 per CTA) or 64 (32)
    rng = random.Random(7)
    for _ in range(500):
        nseg, seg_rows, n = rng.choice([1, 2, 8]), rng.randint(1, 3000), 8 * rng.randint(8, 3000)
        bn, cg = resolve(probe, nseg, seg_rows, n, kn=1)
        assert bn in (64, 128, 192, 256) and (bn // cg) % 64 == 0
        bn, cg = resolve(probe, nseg, seg_rows, n)
        assert bn in (64, 128, 192, 256) and cg == (2 if seg_rows >= 256 else 1)
    # the caller's tuning wins
    assert resolve(probe, 8, 512, 6144, bn=128, cg=1) == (128, 1)
    assert resolve(probe, 8, 512, 6144, cg=1)[1] == 1


def _band_segments(segs, nseg):
    """Segments grouped by band, from the visiting order: a band ends where a segment that was already left
    is never returned to; inside a band the walk interleaves the band's segments column by column."""
    last_seen = {s: max(i for i, x in enumerate(segs) if x == s) for s in set(segs)}
    bands, cur, end = [], [], -1
    for i, s in enumerate(segs):
        if s not in cur:
            cur.append(s)
        end = max(end, last_seen[s])
        if i == end:
            bands.append(cur)
            cur = []
    return bands


def test_band_sizes_of_the_benchmark_shapes(probe):
    """The bands the two protocols rely on, at the per-rank shapes of the dense benchmark."""
    # all-gather (bands = 1), rank 3 of 8: own shard + the first arrival, two more, then the remaining four
    segs = walk(probe, 8, 512, 6144, 256, 2, 3, 0, 1)
    assert _band_segments(segs, 8) == [[3, 4], [5, 6], [7, 0, 1, 2]]
    # TP=4: own, next, last two; TP=2: one shard per band
    assert _band_segments(walk(probe, 4, 1024, 12288, 256, 2, 1, 0, 1), 4) == [[1], [2], [3, 0]]
    assert _band_segments(walk(probe, 2, 2048, 24576, 256, 2, 1, 0, 1), 2) == [[1], [0]]
    # reduce-scatter (bands = 2), rank 2 of 8 (seg_first = 3): the owner that starts its own rows next (rank 1)
    # is a band of its own before this rank's own rows, so every owner has exactly one late peer
    segs = walk(probe, 8, 512, 12288, 256, 2, 3, 0, 2)
    assert _band_segments(segs, 8) == [[3, 4, 5, 6], [7, 0], [1], [2]]
    assert _band_segments(walk(probe, 4, 1024, 12288, 256, 2, 3, 0, 2), 4) == [[3, 0], [1], [2]]
    assert _band_segments(walk(probe, 2, 2048, 12288, 256, 2, 1, 0, 2), 2) == [[1], [0]]


def test_late_peers_match_the_last_peer_band(probe):
    """Reduce-scatter: the owner side's count of late peers equals the number of segments in the band whose tiles
    the pushing side publishes at once (the band before this rank's own rows), for any shape: a mismatch would
    leave an owner waiting for arrivals on the wrong counter."""
    rng = random.Random(99)
    cases = [(8, 512, 2), (4, 1024, 2), (2, 2048, 2), (8, 512, 1), (8, 37, 1), (3, 300, 2)]
    cases += [(rng.choice([2, 3, 4, 8]), rng.choice([rng.randint(1, 2200), 128 * rng.randint(1, 16)]), rng.choice([1, 2]))
              for _ in range(300)]
    for nseg, seg_rows, cg in cases:
        segs = walk(probe, nseg, seg_rows, 512, 256, cg, 1 % nseg, 0, 2)
        bands = _band_segments(segs, nseg)
        assert len(bands) >= 2 and len(bands[-1]) == 1
        assert probe.probe_rs_late_peers(nseg, seg_rows, cg) == len(bands[-2]), (nseg, seg_rows, cg, bands)
        if nseg >= 3:
            assert len(bands[-2]) == 1, "every owner has exactly one late peer"


def test_split_tail_box_ownership(probe):
    """Split-K tail: every 32-column step of a tail tile is finished by exactly one part below `owners`, the two
    steps of a 64-column box (one staged store) by the same part, every owning part has work, and a tile that is
    pushed to another rank is finished by part 0 alone (its owner counts the publishes of one CTA per tile)."""
    for bn in (64, 128, 192, 256):
        steps = bn // 32
        for split in range(2, 9):
            owners = probe.probe_splitk_owners(split, bn, 0)
            assert owners == min(split, max(1, bn // 64))
            own = [probe.probe_splitk_owner(c, split, bn, 0) for c in range(steps)]
            assert all(0 <= o < owners for o in own) and sorted(set(own)) == list(range(owners))
            assert own == sorted(own)
            if bn >= 64:
                assert all(own[c] == own[c ^ 1] for c in range(steps))
            assert probe.probe_splitk_owners(split, bn, 1) == 1
            assert all(probe.probe_splitk_owner(c, split, bn, 1) == 0 for c in range(steps))
