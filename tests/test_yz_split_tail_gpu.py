"""Reduce-scatter launches whose split last wave reaches into rows owned by another rank (one GPU, both ranks in
one cooperative launch).

With 256-column tiles, 1024 output columns, 256 rows per rank and K = 1024 per rank, each rank has 8 tiles for 37
CTA pairs: every tile belongs to the last, partial wave and is cut four ways along K. The four tiles of the
peer's rows are pushed to it: they must be finished - and published to the owner's arrival counter - by one
part only, whereas the four tiles of the rank's own rows are finished box by box by all four parts, each adding
the peer's 16-bit partial to its boxes. Checked against the CPU oracle with the tolerances of the other bf16
reduce-scatter tests (max relative error 1e-2, elementwise 2e-2)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from ranks_on_gpu import Ranks  # noqa: E402

from oracle import golden  # noqa: E402

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.mark.parametrize("block_n", [256, 128])
def test_split_tail_with_pushed_and_own_tiles(block_n):
    world, m, n, k_local = 2, 512, 1024, 1024
    rk = Ranks(world)
    try:
        ops = rk.gemm_rs_ops(m, n, BF16, BF16)
        for call in range(2):  # both buffer parities
            ab = []
            for r in range(world):
                g = torch.Generator().manual_seed(777 + 31 * call + r)
                ab.append((torch.randn(m, k_local, generator=g).to(BF16),
                           (torch.randn(n, k_local, generator=g) * 0.02).to(BF16)))
            outs = [torch.full((m // world, n), float("nan"), dtype=BF16, device="cuda") for _ in range(world)]
            rk.gemm_rs_forward(ops, [a.cuda() for a, _ in ab], [b.cuda() for _, b in ab], outs,
                               tuning={"block_n": block_n, "cta_group": 2})
            refs = golden.gemm_rs_single([a for a, _ in ab], [b for _, b in ab], None)
            for r in range(world):
                assert not torch.isnan(outs[r].float()).any(), f"call {call} rank {r}: rows were left unwritten"
                err = golden.max_rel_err(outs[r], refs[r])
                assert err <= 1e-2, f"call {call} rank {r}: max rel err {err}"
                assert golden.torch_allclose(outs[r], refs[r], rtol=2e-2, atol=2e-2), f"call {call} rank {r}: elementwise"
    finally:
        rk.close()
