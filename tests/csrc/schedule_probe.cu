// Host-side probe of the kernel's tile schedule for the CPU tests: walks every work item of a dense
// (segmented) launch through the product's own decode_tile / make_bands, compiled for the host, and reports
// what each item covers. Mirrors what the reference checks for its MoE schedule in
// src/moe_ag_scatter/test/test_sort_utils.cc:20-46 (every tile covered exactly once).
#include <cstring>

#include "../../flux_b200/csrc/gemm_kernel.cuh"
#include "../../flux_b200/csrc/internal.h"

using namespace fluxb;

template <int BN, int TILE_M>
static int walk(const GemmParams& p, int* visits, int* item_seg, int* item_m, int max_items) {
  const int n_tiles = (p.N + BN - 1) / BN;
  const int tps = (p.seg_rows + TILE_M - 1) / TILE_M;
  const int m_tiles = p.nseg * tps;
  const int chunks = (p.seg_rows + kBM - 1) / kBM;
  const int total = m_tiles * n_tiles;
  if (total > max_items) return -1;
  int bad = 0;
  for (int t = 0; t < total; ++t) {
    for (int half = 0; half < TILE_M / kBM; ++half) {
      TileCoord tc;
      decode_tile<BN, TILE_M>(p, t, m_tiles, n_tiles, tps, half, tc);
      if (half == 0) {
        item_seg[t] = tc.seg;
        item_m[t] = tc.row0;
      }
      if (tc.n_idx < 0 || tc.n_idx >= n_tiles || tc.seg < 0 || tc.seg >= p.nseg) {
        ++bad;
        continue;
      }
      if (tc.rows <= 0) continue;  // second half of a pair past the segment's end
      if (tc.chunk < 0 || tc.chunk >= chunks || tc.row0 != tc.seg * p.seg_rows + tc.chunk * kBM ||
          tc.rows != imin(kBM, p.seg_rows - tc.chunk * kBM) || tc.n0 != tc.n_idx * BN || tc.b_row0 != tc.n0) {
        ++bad;
        continue;
      }
      visits[(tc.seg * chunks + tc.chunk) * n_tiles + tc.n_idx] += 1;
    }
  }
  return bad == 0 ? total : -2 - bad;
}

// bands: 0 = uniform bands of group_m tiles, 1 = all-gather bands (own shard first, doubling),
// 2 = reduce-scatter bands (peers' rows in tall bands, own rows last). Returns the number of work items
// (>= 0) or a negative error. visits: [nseg][chunks][n_tiles] counts, item_seg / item_m: per work item.
extern "C" int probe_dense_schedule(int nseg, int seg_rows, int n, int block_n, int cta_group, int seg_first,
                                    int group_m, int bands, int* visits, int* item_seg, int* item_m,
                                    int max_items) {
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.nseg = nseg;
  p.seg_rows = seg_rows;
  p.seg_first = seg_first;
  p.N = n;
  p.group_m = group_m > 0 ? group_m : 1;
  const int tile_m = cta_group == 2 ? 2 * kBM : kBM;
  const int tps = (seg_rows + tile_m - 1) / tile_m;
  if (bands == 1) make_bands(p, nseg, tps, true, false);
  if (bands == 2) make_bands(p, nseg, tps, false, true);
#define WALK(BN_)                                                                                      \
  if (block_n == BN_)                                                                                  \
    return cta_group == 2 ? walk<BN_, 2 * kBM>(p, visits, item_seg, item_m, max_items)                 \
                          : walk<BN_, kBM>(p, visits, item_seg, item_m, max_items);
  WALK(64) WALK(128) WALK(192) WALK(256)
#undef WALK
  return -1;
}

// Tile shape the library would choose for a segmented launch (resolve_cta_group / resolve_block_n of
// flux_b200/csrc/gemm_ops.cu, linked from libfluxb.so). tun_* = 0 leaves the choice to the library.
extern "C" void probe_resolve(int nseg, int seg_rows, int n, int sm_count, int b_mn_major, int tun_bn, int tun_cg,
                              int tun_ctas, int* bn, int* cg) {
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.nseg = nseg;
  p.seg_rows = seg_rows;
  p.N = n;
  p.b_mn_major = b_mn_major;
  fluxb_comm comm;
  comm.sm_count = sm_count;
  fluxb_tuning t{tun_bn, 0, tun_ctas, tun_cg};
  const fluxb_tuning* tp = (tun_bn || tun_cg || tun_ctas) ? &t : nullptr;
  *cg = resolve_cta_group(p, tp);
  *bn = resolve_block_n(&comm, p, tp, 0);
}

// Late peers per owner of a reduce-scatter launch with the library's own bands (rs_late_peers of gemm_kernel.cuh).
extern "C" int probe_rs_late_peers(int nseg, int seg_rows, int cta_group) {
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int tile_m = cta_group == 2 ? 2 * kBM : kBM;
  const int tps = (seg_rows + tile_m - 1) / tile_m;
  make_bands(p, nseg, tps, false, true);
  return rs_late_peers(p, nseg, tps);
}

// Owner part of column step c of a split tail tile (splitk_owner_of / splitk_owners of gemm_kernel.cuh).
extern "C" int probe_splitk_owner(int c, int split, int bn, int pushed) { return splitk_owner_of(c, split, bn, pushed != 0); }
extern "C" int probe_splitk_owners(int split, int bn, int pushed) { return splitk_owners(split, bn, pushed != 0); }
