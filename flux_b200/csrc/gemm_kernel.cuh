// The one tensor-core kernel of the library: a persistent, warp-specialised
// sm_100a GEMM  D[M,N] = A[M,K] * B[N,K]^T  (both operands K-major, fp32
// accumulation in tensor memory) whose prologue and epilogue carry the
// tensor-parallel collectives:
//
//   * all-gather prologue  - four "comm" warps in every CTA push this rank's
//     activation shard into every peer's gather buffer over NVLink (plain
//     16-byte stores to peer memory) and bump per-chunk arrival counters; the
//     TMA warp waits (bounded) on the counter of the chunk a tile reads before
//     it issues the loads, and tiles are visited own-shard-first.
//     Replaces the reference's copy-engine all-gather + per-rank flags
//     (src/coll/ths_op/all_gather_op.cc:529-574) and the flag waits inside its
//     sm90 kernel (src/ag_gemm/sm90_all_gather_gemm_tma_warpspecialized_cooperative.hpp:512-586).
//   * reduce-scatter epilogue - the epilogue warps store partial tiles (in the
//     16-bit output format, or fp32 on request) straight into the staging slot
//     of the rank that owns those rows and bump that rank's per-tile counter;
//     rows owned by peers are computed first, the owner's comm warps sum the
//     peers' partials in fp32 and its own tiles add that sum in their epilogue.
//     Replaces the reference's store-then-pull design
//     (src/gemm_rs/sm90_epilogue_evt.hpp:231-242, sm90_reduce_scatter_utils.hpp:212-262).
//   * grouped (MoE) mode - M tiles come from a device-side table, A rows come
//     from an expert-sorted buffer the comm warps fill as tokens arrive (or are
//     fetched by index with TMA gather4), B is the expert's weight slab.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 UMMA issuer + TMEM
// owner, warps 2-5 epilogue (one TMEM lane quadrant each), warps 6-9 comm.
//
// Two tile shapes: one CTA per 128 x BN tile (cta_group::1), or a CTA pair
// (cluster of 2) per 256 x BN tile (cta_group::2): each CTA of the pair loads
// its own 128 rows of A and half of the B tile, the even CTA issues the UMMAs
// for both, each CTA drains its own 128 accumulator rows. The pair form needs
// a third less operand traffic per flop and buys two more pipeline stages.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "ptx.cuh"

namespace fluxb {

constexpr int kBM = 128;          // rows per tile (= TMEM lanes)
constexpr int kRowBytes = 128;    // bytes of K per smem row (one swizzle span)
constexpr int kThreads = 320;
constexpr int kMaxWorld = 8;
constexpr int kCommSliceBytes = 2048;  // bytes of one row handled by one comm unit
constexpr int kPermUnitRows = 32;      // rows of one permute unit of MoE layer 0 (32 rows x 2 KB by the 128 comm threads)
constexpr int kPermUnitsPerSlice = kBM / kPermUnitRows;
constexpr int kGrTokBlock = 32;        // tokens per combine / reduce work item of MoE layer 1
constexpr int kAgMaxGroups = 64;       // arrival counters per (source rank, chunk): one per group of 2 KB slices

enum EpiMode : int {
  kEpiStore = 0,    // write D (out dtype) to p.out
  kEpiRsPush = 1,   // write partials (16-bit or fp32) into the owner's staging slot + counter
};
enum OutType : int { kOutBf16 = 0, kOutF16 = 1, kOutF32 = 2 };
enum BiasMode : int { kBiasNone = 0, kBiasFull = 1, kBiasRow = 2 };

// One M tile of a grouped problem (MoE). `a_row0` indexes the sorted row space.
struct GroupTile {
  int a_row0;      // first sorted row of the tile
  int rows;        // valid rows (1..128)
  int expert;      // which weight slab
  int need_mask;   // bit (r * g_nvr + j) set = tile reads tokens of block j of source rank r
};

struct GemmParams {
  CUtensorMap tmap_a;
  CUtensorMap tmap_b;
  CUtensorMap tmap_a_own;  // all-gather: this rank's own shard, read in place (valid if a_own_valid)
  CUtensorMap tmap_out;    // 16-bit output [rows, N] as 32-row x 64-column boxes (valid if tmap_out_valid): full
                           // 32-row groups of a tile leave through shared memory and one tiled store per box
  int tmap_out_valid;
  int a_own_valid;
  int b_mn_major;  // 1: B is stored [K, N] (N contiguous), loaded as 64-column boxes (16-bit inputs only)
  int acc_int;     // 1: 8-bit operands are signed integers and the accumulator is int32 (w8a8 with dequantisation)
  int M, N, K;
  // M segmentation: nseg segments of seg_rows rows; tiles never straddle a
  // segment; segments are visited (seg_first + i) % nseg.
  int nseg, seg_rows, seg_first;
  int group_m;  // rasterisation band height in M tiles (uniform bands, used when n_bands == 0)
  int n_group;  // > 0: tile columns are visited in groups of this many (all M tiles of a group before the next group)
  int rs_wire16;  // reduce-scatter partials cross NVLink in the 16-bit output format instead of fp32
  int rs_ring;    // with rs_wire16: every addition of the reduction is rounded to the 16-bit type, own partial last
  // The peers that compute this rank's rows in their last band of peer rows (rank+1 .. rank+rs_n_late) deliver
  // just before the own tiles start: their 16-bit partials are added by the own tiles' epilogue itself, straight
  // from the staging slots (arrivals counted at rs_late_off ints behind the ordinary counters); only the other
  // peers' partials go through the comm warps' fp32 sum. 0 = every peer goes through the comm warps.
  int rs_n_late;
  int rs_late_off;
  int n_bands;  // > 0: explicit bands, band b covers M tiles [band_end[b-1], band_end[b])
  int band_end[8];
  // epilogue
  int epi_mode, out_type, bias_mode;
  void* out;
  long long ldo;  // elements
  const void* bias;  // same dtype as out
  long long ldbias;
  const float* scale_a;  // per output row (may be null)
  const float* scale_b;  // per output column (may be null)
  float alpha;
  const float* alpha_ptr;  // optional device scalar multiplied into alpha
  // all-gather: consumer side
  // Arrival counters [source rank][128-row chunk][slice group]: a group is `ag_spf` consecutive 2 KB slices
  // of the rows (1 unless a row has more than kAgMaxGroups slices); every push unit of ag_unit_rows rows x 2 KB
  // adds 1, so a complete group counts (128 / ag_unit_rows) x (slices in the group). The GEMM waits group by group as
  // it walks along K, so a tile starts as soon as the first 2 KB of its rows are in.
  const int* ag_flags;  // null = no waits
  int ag_flag_stride;   // counters per source rank (= chunks of the buffer x ag_groups)
  int ag_groups;        // counters per chunk
  int ag_spf;           // 2 KB slices per counter
  int ag_unit_rows;     // rows of one push unit: 32, 64 or 128 (one release per unit)
  // all-gather: producer side (comm warps)
  const uint8_t* ag_src;          // this rank's shard, row-major, row_bytes per row
  uint8_t* ag_dst[kMaxWorld];     // gather buffer of every rank (own included)
  int* ag_dst_flags[kMaxWorld];   // flag array of every rank
  const float* ag_src_scale;      // optional per-row scales of the shard
  float* ag_dst_scale[kMaxWorld];
  long long ag_row_bytes;
  int rank, world;
  // reduce-scatter push
  CUtensorMap tmap_rs[kMaxWorld];  // [rows_per_owner, N] view of this rank's slot at owner o: 16-bit 32x64 boxes, or fp32 32x32
  float* rs_stage[kMaxWorld];  // rs_stage[o] = slot of this rank inside owner o's staging
  int* rs_cnt[kMaxWorld];      // per-tile counters at owner o: [tiles_per_seg][n_tiles]
  // reduce-scatter: owner side. The comm warps sum the partial tiles the peers pushed for this
  // rank's rows into this rank's own (otherwise unused) slot and raise a per-tile ready flag; the
  // epilogue of this rank's own tiles adds that sum to its accumulator and writes the result.
  const float* rs_local_stage;  // [world] slots of seg_rows x N floats: partials received by this rank (16-bit ones fill half a slot)
  int* rs_local_cnt;            // this rank's arrival counters, [tiles]
  int* rs_local_ready;          // this rank's "remote partials summed" flags, [tiles]
  void* rs_out;                 // [seg_rows, N] result, type rs_out_type
  int rs_out_type;
  // grouped mode
  const GroupTile* g_tiles;  // null = dense
  const int* g_order;        // optional visiting order of the M tiles (null = table order)
  const int* g_num_tiles;    // device scalar
  const int* g_gather;       // sorted row -> source row of A (null: A rows are already sorted)
  int g_rows_per_expert_b;   // rows of B per expert (= N)
  const float* g_expert_scale;  // optional per-expert alpha
  const int* g_scatter_rows;    // optional: sorted row -> output row (null = identity)
  int g_rows_per_rank;          // tokens per source rank (for need_mask -> flags)
  int g_ntokens;                // rows of the gathered A matrix
  // grouped mode, permute form: the comm warps copy every gathered token row to its top-k places in
  // an expert-sorted buffer (which tmap_a then describes) and count finished work items per source rank
  uint8_t* g_sorted;              // [rows, K] sorted activations, null = gather4 form
  int* g_perm_done;               // [world * g_nvr] finished permute units per source block (local, zeroed per call)
  int g_vblk, g_nvr;              // tokens per source block (a multiple of 128) and blocks per rank (world * g_nvr <= 32)
  const int* g_scatter_index;     // [tokens, topk]
  const int* g_row_range;         // device [2]: rows [lo, hi) of the sorted order that this rank computes (expert
                                  // parallelism: the rows of its experts); null = all rows. Row lo is row 0 of g_sorted.
  const uint8_t* g_tokens;        // gathered tokens [tokens, K] (this rank's gather buffer, or the input at world 1)
  const uint8_t* g_tokens_own;    // this rank's own token shard, read in place (no copy to itself, no wait); null = in g_tokens
  int g_topk;
  // MoE layer 1: the comm warps combine every token's top-k rows of D column slab by column slab (a slab =
  // one tile column, BN wide) as soon as all tiles of the slab are stored, push the combined rows (16-bit) to
  // the token's owner and, on the owner, sum the per-source partials: grouped GEMM, gather and reduce-scatter
  // in one launch. Tiles are walked slab by slab (one rasterisation band over all M tiles).
  int* gr_slab_done;             // [n_tiles] one arrival per epilogue warp per tile (local, zeroed per call); null = off
  int gr_slab_expected;          // arrivals of a complete slab
  const int* gr_scatter_index;   // [tokens * topk]: row of the expert-sorted order that holds (token, k)
  int gr_row_lo, gr_rows;        // D holds rows [gr_row_lo, gr_row_lo + gr_rows) of that order (expert parallelism:
                                 // this rank's experts; the other rows are other ranks' and contribute nothing here)
  int gr_topk;
  int gr_tokens_per_rank;
  void* gr_stage[kMaxWorld];     // owner o's staging slot of THIS rank: [tokens_per_rank][N], 16-bit
  int* gr_cnt[kMaxWorld];        // owner o's arrival counters [n_tiles][token blocks]
  const void* gr_local_stage;    // this rank's staging: [world][tokens_per_rank][N]
  int* gr_local_cnt;
  void* gr_out;                  // [tokens_per_rank][N]
  // split-K tail: the tiles of the last, partial wave are split along K over the otherwise idle
  // workers; every part parks here its fp32 accumulators of the 64-column boxes that another part finishes
  float* splitk_scratch;  // [tail tile][split - 1 other parts][tile rows][BN]; null = never split
  int* splitk_cnt;        // [tail tile][half][epilogue warp] parts that have parked, self-clearing
  int* splitk_done;       // same shape: parts that have seen all others parked (the last one clears both)
  // optional timeline: 8 x u64 per CTA (globaltimer ns): 0 kernel start, 1 first operands landed,
  // 2 last UMMA issued, 3 epilogue done, 4 comm warps done, 5 ns spent waiting on arrival flags,
  // 6 ns the epilogue waited for "peers summed" flags, 7 work items of this CTA
  unsigned long long* trace;
  // status / bounded waits
  int* status;
  unsigned long long timeout_ns;
};

template <int BN, int STAGES, bool CTA2>
struct SmemLayout {
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBRows = CTA2 ? BN / 2 : BN;
  static constexpr int kBBytes = kBRows * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // epilogue staging: per epilogue warp 4 KB blocks (32 x 32 fp32 or 32 x 64 16-bit), 128-byte rows, 128-byte swizzle; two
  // blocks per warp where shared memory allows, so that two pushes per warp can be in flight
  static constexpr int kEpiPitch = 128;
  static constexpr int kEpiBlockBytes = 32 * kEpiPitch;
  static constexpr int kEpiOffset = STAGES * kStageBytes;
  static constexpr int kNumBars = 2 * STAGES + 5;  // full/empty per stage, 2 x accumulator full/empty, 1 x "UMMAs retired" (abort path)
  static constexpr int kEpiBufs = (kEpiOffset + 8 * kEpiBlockBytes + kNumBars * 8 + 64 + 1024 <= 232448) ? 2 : 1;
  static constexpr int kEpiWarpBytes = kEpiBufs * kEpiBlockBytes;
  static constexpr int kBarOffset = kEpiOffset + 4 * kEpiWarpBytes;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  static constexpr int kTotal = kMiscOffset + 64 + 1024;  // + slack for 1024-byte alignment
};

struct TileCoord {
  int row0;        // first A row of THIS CTA (global row, or sorted row in grouped mode)
  int rows;        // valid rows of this CTA (0..128)
  int n0;          // first output column
  int seg, chunk;  // segment and 128-row chunk inside it (dense)
  int b_row0;      // first B row of the tile
  int n_idx;
  int need_mask;
  int expert;
  int band;        // rasterisation band of the tile (explicit bands only, else 0)
};

__host__ __device__ __forceinline__ int imin(int a, int b) { return a < b ? a : b; }
__host__ __device__ __forceinline__ int imax(int a, int b) { return a > b ? a : b; }

// Rasterisation bands for the segmented ops, in units of segments (= shards / owners) of `tps` M tiles.
// Bands are at most 8 M tiles tall (taller bands re-stream B less often and draw less power; measured on the
// plain GEMM: a band of 2 M tiles costs 8 % of its tiles' time, one of 4 costs 2 %).
// first_single (all-gather): the first band starts with this rank's own shard, available at once, and is filled
// up to 4 M tiles with the shards that arrive first (the push is slice-major: their first 2 KB slices are in
// after a few microseconds). The second band has the same size and the sizes double from the third on: a
// shard crosses NVLink in about 40 % of the time its tiles take to compute, so when band k starts, at
// (segments before it) x (compute time of a segment), its last shard has been in for a while.
// last_single (reduce-scatter): this rank's own rows are the last band, and the segment before them - the
// owner that is about to start its own rows and waits for exactly these partials - is a band of its own, so
// that every owner has one late peer only.
inline void make_bands(GemmParams& p, int nseg, int tps, bool first_single, bool last_single) {
  int max_seg = tps > 0 ? 8 / tps : 1;
  if (max_seg < 1) max_seg = 1;
  int done = 0, nb = 0, next = tps > 0 && 4 / tps > 1 ? 4 / tps : 1;
  const int tail_single = last_single ? (nseg >= 3 ? 2 : 1) : 0;
  const int body_end = nseg - tail_single;
  while (done < body_end && nb < 8 - 1 - tail_single) {
    int take = first_single ? next : max_seg;
    if (take > max_seg) take = max_seg;
    if (take > body_end - done) take = body_end - done;
    done += take;
    p.band_end[nb++] = done * tps;
    if (nb >= 2) next *= 2;
  }
  if (done < body_end) {
    if (nb > 0) p.band_end[nb - 1] = body_end * tps; else p.band_end[nb++] = body_end * tps;
    done = body_end;
  }
  while (done < nseg && nb < 8) {
    done += 1;
    p.band_end[nb++] = done * tps;
  }
  p.band_end[nb - 1] = nseg * tps;
  p.n_bands = nb;
}

// Split-K tail: which part finishes the 32-column step `c` of a tail tile that is BN columns wide and cut into
// `split` parts. Steps are owned in pairs (one 64-column box = one staged store), box b by part
// b * owners / boxes with owners = min(split, boxes); parts >= owners only park. A tile that is pushed to
// another owner (`pushed`) is finished by part 0 alone.
__host__ __device__ __forceinline__ int splitk_owners(int split, int bn, bool pushed) {
  const int boxes = bn / 64 > 0 ? bn / 64 : 1;
  return pushed ? 1 : (split < boxes ? split : boxes);
}
__host__ __device__ __forceinline__ int splitk_owner_of(int c, int split, int bn, bool pushed) {
  const int boxes = bn / 64 > 0 ? bn / 64 : 1;
  return ((bn >= 64 ? c >> 1 : 0) * splitk_owners(split, bn, pushed)) / boxes;
}

// Reduce-scatter: how many peers deliver their partials of an owner's rows late, i.e. compute them in their
// last band of peer rows (the band whose tiles the pushing side publishes at once). By symmetry it is the number
// of segments in that band: with explicit bands the band before the last, otherwise (uniform bands) the rows of
// the previous rank only. The kernel's pushing side and the owner side must agree on this number.
inline int rs_late_peers(const GemmParams& p, int world, int tps) {
  if (p.n_bands >= 2 && tps > 0) {
    const int first_seg = p.n_bands >= 3 ? p.band_end[p.n_bands - 3] / tps : 0;
    return (world - 1) - first_seg;
  }
  return 1;
}

// TILE_M = 128 (one CTA) or 256 (CTA pair, `half` = rank of this CTA inside the pair).
// Also compiled for the host: the CPU tests walk the schedule to check that every tile is visited once.
template <int BN, int TILE_M>
__host__ __device__ __forceinline__ void decode_tile(const GemmParams& p, int t, int m_tiles, int n_tiles,
                                            int tps, int half, TileCoord& tc) {
  // Rasterisation: M tiles are grouped into bands; inside a band consecutive work items walk down the
  // band's M tiles first, then move to the next column block (A band stays in L2, B streams once per band).
  int m_idx, n_idx;
  tc.band = 0;
  // Column groups (n_group > 0): all tiles of the first n_group tile columns come first, then the next group ...;
  // inside a group the bands below apply. The output is then complete group by group.
  int n_base = 0;
  if (p.n_group > 0 && p.n_group < n_tiles) {
    const int per_group = m_tiles * p.n_group;
    const int g = t / per_group;
    t -= g * per_group;
    n_base = g * p.n_group;
    n_tiles = imin(p.n_group, n_tiles - n_base);
  }
  if (p.n_bands > 0) {
    int b = 0;
    while (b + 1 < p.n_bands && t >= p.band_end[b] * n_tiles) ++b;
    tc.band = b;
    const int m_lo = b > 0 ? p.band_end[b - 1] : 0;
    const int h = p.band_end[b] - m_lo;
    const int r = t - m_lo * n_tiles;
    m_idx = m_lo + r % h;
    n_idx = r / h;
  } else {
    const int gmn = p.group_m * n_tiles;
    const int band = t / gmn;
    const int r = t - band * gmn;
    const int gm_eff = imin(p.group_m, m_tiles - band * p.group_m);
    m_idx = band * p.group_m + r % gm_eff;
    n_idx = r / gm_eff;
  }
  n_idx += n_base;
  tc.n_idx = n_idx;
  tc.n0 = n_idx * BN;
  if (p.g_tiles == nullptr) {
    const int sp = m_idx / tps;
    const int c = m_idx - sp * tps;
    int seg = p.seg_first + sp;
    if (seg >= p.nseg) seg -= p.nseg;
    const int off = c * TILE_M + half * kBM;  // row offset inside the segment
    tc.seg = seg;
    tc.chunk = off / kBM;
    tc.row0 = seg * p.seg_rows + off;
    tc.rows = imax(0, imin(kBM, p.seg_rows - off));
    tc.b_row0 = tc.n0;
    tc.need_mask = 0;
    tc.expert = 0;
  } else {
    const int mi = p.g_order != nullptr ? p.g_order[m_idx] : m_idx;
    const GroupTile g = p.g_tiles[mi];
    tc.seg = 0;
    tc.chunk = mi;
    tc.row0 = g.a_row0 + half * kBM;
    tc.rows = imax(0, imin(kBM, g.rows - half * kBM));
    tc.expert = g.expert;
    tc.b_row0 = g.expert * p.g_rows_per_expert_b + tc.n0;
    tc.need_mask = g.need_mask;
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// KIND: 0 = 16-bit inputs (bf16/f16 chosen by the instruction descriptor), 1 = fp8
// CTA2: false = one CTA per 128-row tile, true = CTA pair per 256-row tile (launch with cluster 2x1x1)
// `cta_id` / `num_ctas`: this CTA's index and the number of CTAs that work on problem `p` (the whole grid for
// an ordinary launch; a slice of it when one launch runs several ranks' problems side by side).
template <int BN, int STAGES, int KIND, bool CTA2>
__device__ __forceinline__ void fused_gemm_body(const GemmParams& p, const uint32_t idesc, const int cta_id,
                                                const int num_ctas) {
  using L = SmemLayout<BN, STAGES, CTA2>;
  constexpr int ELT = (KIND == 0) ? 2 : 1;
  constexpr int BKE = kRowBytes / ELT;  // K elements per stage
  constexpr int TILE_M = CTA2 ? 2 * kBM : kBM;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                 : (2 * BN <= 256) ? 256 : 512;
  static_assert(2 * BN <= 512, "two accumulators must fit in tensor memory");
  static_assert(BN % 32 == 0, "epilogue reads 32 columns at a time");
  static_assert(L::kTotal <= 232448, "shared memory budget exceeded");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 8);

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto bar_full = [&](int s) { return bar_base + 8u * s; };
  auto bar_empty = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto bar_tfull = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto bar_tempty = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t bar_retired = bar_base + 8u * (2 * STAGES + 4);
  auto smem_a = [&](int s) { return smem_base + s * L::kStageBytes; };
  auto smem_b = [&](int s) { return smem_base + s * L::kStageBytes + L::kABytes; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t budget = p.timeout_ns;
  const int half = CTA2 ? static_cast<int>(cluster_ctarank()) : 0;  // rank inside the CTA pair
  const bool leader = half == 0;
  const int tile_first = CTA2 ? (cta_id >> 1) : cta_id;
  const int tile_step = CTA2 ? (num_ctas >> 1) : num_ctas;
  // raised by any role that gives up; in a CTA pair the partner's word is raised too
  const AbortWord ab{s_abort, CTA2 ? mapa_u32(smem_u32(const_cast<int*>(s_abort)), static_cast<uint32_t>(half ^ 1)) : 0u};

  unsigned long long* tr = p.trace != nullptr ? p.trace + static_cast<size_t>(cta_id) * 8 : nullptr;
  if (threadIdx.x == 0) {
    if (tr != nullptr) {
      tr[0] = globaltimer_ns();
      tr[5] = 0;
      tr[6] = 0;
    }
    *s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull(a), 1);
      mbar_init(bar_tempty(a), CTA2 ? 8 : 4);  // one arrival per epilogue warp (of both CTAs)
    }
    mbar_init(bar_retired, 1);
    mbar_init_fence();
    tma_prefetch_desc(&p.tmap_a);
    tma_prefetch_desc(&p.tmap_b);
    if (p.a_own_valid) tma_prefetch_desc(&p.tmap_a_own);
  }
  if (warp == 1) {
    if (CTA2) {
      tmem_alloc_2cta(smem_u32(tmem_holder), TMEM_COLS);
      tmem_relinquish_2cta();
    } else {
      tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (CTA2) cluster_sync_all(); else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int n_tiles = (p.N + BN - 1) / BN;
  int tps = 1, m_tiles;
  if (p.g_tiles == nullptr) {
    tps = (p.seg_rows + TILE_M - 1) / TILE_M;
    m_tiles = p.nseg * tps;
  } else {
    m_tiles = *p.g_num_tiles;
  }
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + BKE - 1) / BKE;
  // all-gather bookkeeping: a K block is 128 bytes of a row, a push slice 2 KB, a counter covers ag_spf slices
  const int ag_nslices = static_cast<int>((p.ag_row_bytes + kCommSliceBytes - 1) / kCommSliceBytes);
  const int kb_per_group = (kCommSliceBytes / kRowBytes) * (p.ag_spf > 0 ? p.ag_spf : 1);
  const int ag_ups = kBM / (p.ag_unit_rows > 0 ? p.ag_unit_rows : 32);  // push units per (chunk, slice)

  // Work schedule, identical in every role: worker w (a CTA, or a CTA pair) takes tiles w, w+P, ...
  // of the full waves; if the last wave is at most half full, each of its tiles is cut along K into
  // `split` parts and worker w takes part w % split of tail tile w / split.
  const int full_waves = total_tiles / tile_step;
  const int full_tiles = full_waves * tile_step;
  const int tail_tiles = total_tiles - full_tiles;
  int split = 1;
  if (p.splitk_scratch != nullptr && p.g_tiles == nullptr && tail_tiles > 0 && 2 * tail_tiles <= tile_step) {
    int sp = tile_step / tail_tiles;
    if (sp > 8) sp = 8;
    if (sp > num_kb / 4) sp = num_kb / 4;
    if (sp >= 2) split = sp;
  }
  auto get_item = [&](int i, int& t, int& kb0, int& kb1, int& part) -> bool {
    part = 0;
    kb0 = 0;
    kb1 = num_kb;
    if (split <= 1) {
      t = tile_first + i * tile_step;
      return t < total_tiles;
    }
    if (i < full_waves) {
      t = tile_first + i * tile_step;
      return true;
    }
    if (i > full_waves || tile_first >= tail_tiles * split) return false;
    t = full_tiles + tile_first / split;
    part = tile_first % split;
    kb0 = static_cast<int>(static_cast<long long>(part) * num_kb / split);
    kb1 = static_cast<int>(static_cast<long long>(part + 1) * num_kb / split);
    return true;
  };

  // MoE layer 0, permute form. One unit = 32 token rows x one 2 KB slice of source rank `src_rank`: copy every
  // row to its top-k rows of the expert-sorted buffer (one load, top-k stores per 16-byte piece) and count the
  // unit as done for its source block; a tile waits until every source block it reads is complete. Units of a
  // source run block-major (block j: its slices, chunks, 32-row quarters), so that the source's blocks complete
  // one after the other. Called by 128 threads (`tid` 0..127) that own named barrier BAR.
  const int perm_nvr = p.g_nvr > 0 ? p.g_nvr : 1;
  const int perm_cpv = (p.g_vblk > 0 ? p.g_vblk : p.g_rows_per_rank + kBM - 1) / kBM;  // chunks per block
  const int perm_slots = ag_nslices * perm_cpv * kPermUnitsPerSlice;
  const int perm_units = perm_nvr * perm_slots;
  // step 0 (this rank's own tokens, nothing to wait for) gates the first tiles: the epilogue warps, idle until
  // the first accumulator is complete, permute every second unit of it
  const bool perm_helped = p.g_sorted != nullptr && (p.ag_flags == nullptr || p.g_tokens_own != nullptr);
  auto permute_unit = [&](auto bar_tag, int u, int src_rank, int tid, bool may_wait) -> bool {
    constexpr int BAR = decltype(bar_tag)::value;
    const long long tok0 = static_cast<long long>(src_rank) * p.g_rows_per_rank;
    const int perm_lo = p.g_row_range != nullptr ? p.g_row_range[0] : 0;
    const int perm_rows = p.g_row_range != nullptr ? p.g_row_range[1] - perm_lo : p.M;
    const int perm_chunks = (p.g_rows_per_rank + kBM - 1) / kBM;
    const int vb = u / perm_slots;
    const int ub = u - vb * perm_slots;
    const int ks = ub / (perm_cpv * kPermUnitsPerSlice);
    const int rem = ub - ks * (perm_cpv * kPermUnitsPerSlice);
    const int chunk = vb * perm_cpv + rem / kPermUnitsPerSlice;
    if (chunk >= perm_chunks) return true;  // the last block of a rank may hold fewer chunks
    const int r0 = imin(chunk * kBM + (rem % kPermUnitsPerSlice) * kPermUnitRows, p.g_rows_per_rank);
    const int nrows = imin(kPermUnitRows, p.g_rows_per_rank - r0);
    const bool own_src = p.g_tokens_own != nullptr && src_rank == p.rank;
    if (may_wait && p.ag_flags != nullptr && !own_src) {
      volatile int* s_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 16);
      if (tid == 0) {
        const int grp = ks / p.ag_spf;
        const int in_group = imin(p.ag_spf, ag_nslices - grp * p.ag_spf);
        *s_flag = flag_wait_eq(p.ag_flags + src_rank * p.ag_flag_stride + chunk * p.ag_groups + grp,
                               ag_ups * in_group, ab, kStatusTimeoutFlag, budget) ? 1 : 0;
      }
      asm volatile("bar.sync %0, 128;" ::"n"(BAR) : "memory");
      const int okp = *s_flag;
      asm volatile("bar.sync %0, 128;" ::"n"(BAR) : "memory");
      if (!okp) return false;
    }
    const long long b0 = static_cast<long long>(ks) * kCommSliceBytes;
    const int slice_bytes = static_cast<int>((b0 + kCommSliceBytes < p.ag_row_bytes ? b0 + kCommSliceBytes : p.ag_row_bytes) - b0);
    {
      const bool active = tid * 16 < slice_bytes;
      const uint8_t* s0 = (own_src ? p.g_tokens_own + static_cast<long long>(r0) * p.ag_row_bytes
                                   : p.g_tokens + (tok0 + r0) * p.ag_row_bytes) + b0 + tid * 16;
      uint8_t* d0 = p.g_sorted + b0 + tid * 16;
      const int* si = p.g_scatter_index + (tok0 + r0) * p.g_topk;
      // The unit's destination rows (rows x top-k entries of the scatter index) are fetched up front, spread
      // over the lanes of each warp, and handed out by shuffles: a load of the index between two stores cannot
      // be moved ahead of the store by the compiler, and one dependent load per stored row made a unit
      // take ~23 us.
      const int nidx = nrows * p.g_topk;
      const bool in_regs = nidx <= 128;
      int sreg[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) sreg[q] = (in_regs && q * 32 + lane < nidx) ? si[q * 32 + lane] : -1;
#pragma unroll 1
      for (int rr = 0; rr < nrows; rr += 8) {
        uint4 val[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (active && rr + j < nrows) val[j] = *reinterpret_cast<const uint4*>(s0 + (rr + j) * p.ag_row_bytes);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (rr + j < nrows)
            for (int k = 0; k < p.g_topk; ++k) {
              const int idx = (rr + j) * p.g_topk + k;
              int entry;
              if (in_regs) {
                const int q = idx >> 5;
                const int mine = q == 0 ? sreg[0] : q == 1 ? sreg[1] : q == 2 ? sreg[2] : sreg[3];
                entry = __shfl_sync(0xffffffffu, mine, idx & 31);
              } else {
                entry = si[idx];
              }
              const long long drow = static_cast<long long>(entry) - perm_lo;
              if (active && drow >= 0 && drow < perm_rows)  // rows of other ranks' experts; a corrupt entry must not become a wild store
                *reinterpret_cast<uint4*>(d0 + drow * p.ag_row_bytes) = val[j];
            }
      }
    }
    // the release by one thread covers every thread's stores (ordered before it by the barrier); the counter
    // and the sorted buffer are local, so device scope is enough
    asm volatile("bar.sync %0, 128;" ::"n"(BAR) : "memory");
    if (tid == 0) red_add_release_gpu(p.g_perm_done + src_rank * perm_nvr + vb, 1);
    return true;
  };

  // Abort path of the producer: every stage it armed still has copies in flight or has been filled; wait
  // (1 ms per stage at most) until each armed phase completes, so that no copy outlives the CTA's shared
  // memory. Stages [0, stage) were last armed in phase `phase`, the others one round earlier. In a CTA pair
  // the leader's barriers count both CTAs' bytes, and the final cluster barrier keeps the partner alive
  // until the leader is through here.
  auto drain_loads = [&](int stage, uint32_t phase) {
    if (!leader) return;
    const AbortWord none{nullptr, 0u};
    for (int s2 = 0; s2 < STAGES; ++s2)
      mbar_wait(bar_full(s2), s2 < stage ? phase : (phase ^ 1u), none, 0, 1000000ull);
  };

  if (warp == 0 && p.g_gather != nullptr) {
    // ------------------------------------------------- TMA, row-gather form (MoE layer 0)
    // All 32 lanes work: lane l keeps the four source rows of rows 4l..4l+3 of the tile in registers
    // for the whole tile and issues its own gather4 per stage; lane 0 also arms the barrier and loads B.
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = tile_first; ok && t < total_tiles; t += tile_step) {
      TileCoord tc;
      decode_tile<BN, TILE_M>(p, t, m_tiles, n_tiles, tps, half, tc);
      // rows past the tile end re-read a valid row (their results are never stored)
      const int* gi = p.g_gather + (tc.rows > 0 ? tc.row0 : 0);
      const int nr = tc.rows > 0 ? tc.rows : 1;
      const int r0 = lane * 4;
      const int i0 = gi[r0 < nr ? r0 : 0];
      const int i1 = gi[r0 + 1 < nr ? r0 + 1 : 0];
      const int i2 = gi[r0 + 2 < nr ? r0 + 2 : 0];
      const int i3 = gi[r0 + 3 < nr ? r0 + 3 : 0];
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(bar_empty(stage), phase ^ 1u, ab, kStatusTimeoutSmemEmpty, budget, 40)) {
          ok = false;
          break;
        }
        uint32_t fb = bar_full(stage);
        if (CTA2) {
          if (leader && lane == 0) mbar_arrive_expect_tx(fb, 2 * L::kStageBytes);
          fb = mapa_u32(fb, 0);
        } else if (lane == 0) {
          mbar_arrive_expect_tx(fb, L::kStageBytes);
        }
        if (CTA2) tma_gather4_2d_2cta(smem_a(stage) + lane * 4 * kRowBytes, &p.tmap_a, fb, kb * BKE, i0, i1, i2, i3);
        else tma_gather4_2d(smem_a(stage) + lane * 4 * kRowBytes, &p.tmap_a, fb, kb * BKE, i0, i1, i2, i3);
        if (lane == 0) {
          if (CTA2) tma_load_2d_2cta(smem_b(stage), &p.tmap_b, fb, kb * BKE, tc.b_row0 + half * (BN / 2));
          else tma_load_2d(smem_b(stage), &p.tmap_b, fb, kb * BKE, tc.b_row0);
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && ok;
    }
    if (lane == 0 && *s_abort != 0) drain_loads(stage, phase);
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t, kb0, kb1, part;
      for (int wi = 0; ok && get_item(wi, t, kb0, kb1, part); ++wi) {
        TileCoord tc;
        decode_tile<BN, TILE_M>(p, t, m_tiles, n_tiles, tps, half, tc);
        // all-gather: the rows of this tile arrive slice group by slice group along K
        const int* tile_flags = nullptr;
        if (p.ag_flags != nullptr && p.g_tiles == nullptr && tc.rows > 0 && !(p.a_own_valid && tc.seg == p.rank))
          tile_flags = p.ag_flags + tc.seg * p.ag_flag_stride + tc.chunk * p.ag_groups;
        if (p.g_perm_done != nullptr) {
          // grouped, permute form: every source block the tile reads must be fully permuted
          const int nvr = p.g_nvr > 0 ? p.g_nvr : 1;
          const int cpv = (p.g_vblk > 0 ? p.g_vblk : p.g_rows_per_rank + kBM - 1) / kBM;  // chunks per block
          const int all_chunks = (p.g_rows_per_rank + kBM - 1) / kBM;
          const uint64_t w0 = tr != nullptr ? globaltimer_ns() : 0;
          for (int b = 0; ok && b < p.world * nvr; ++b)
            if ((tc.need_mask >> b) & 1) {
              const int j = b % nvr;
              const int expected = imin(cpv, all_chunks - j * cpv) * kPermUnitsPerSlice * ag_nslices;
              ok = flag_wait_eq(p.g_perm_done + b, expected, ab, kStatusTimeoutFlag, budget);
            }
          if (tr != nullptr) tr[5] += globaltimer_ns() - w0;
          if (!ok) break;
          fence_proxy_async();
        }
        // K block at which the next slice group of the rows begins (never, if there is nothing to wait for):
        // one compare per K block on the producer's critical path, the arithmetic only when a group begins
        int next_group_kb = tile_flags != nullptr ? kb0 : 0x7fffffff;
        if (tile_flags != nullptr) {
          // Look ahead: read the counters of all slice groups of the rows in one sweep (relaxed loads issued
          // together, 16 counters at a time) and make the leading complete ones visible with ONE acquire fence.
          // In the steady state every group has arrived and the tile costs one load latency instead of one
          // acquire per group; the groups still missing are waited for one by one below.
          const int ngroups = (ag_nslices + p.ag_spf - 1) / p.ag_spf;
          int lead = 0;
          bool scanning = true;
          for (int g0 = 0; scanning && g0 < ngroups; g0 += 16) {
            uint4 v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              v[q] = g0 + 4 * q < ngroups ? ld_relaxed_sys_v4(tile_flags + g0 + 4 * q) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              const uint4 w = v[q >> 2];
              const int val = static_cast<int>((q & 3) == 0 ? w.x : (q & 3) == 1 ? w.y : (q & 3) == 2 ? w.z : w.w);
              const int gi = g0 + q;
              if (scanning && gi < ngroups) {
                if (val == ag_ups * imin(p.ag_spf, ag_nslices - gi * p.ag_spf)) lead = gi + 1;
                else scanning = false;
              }
            }
          }
          if (lead > 0) {
            fence_acq_rel_sys();
            fence_proxy_async();
            if (lead * kb_per_group > kb0) next_group_kb = lead >= ngroups ? 0x7fffffff : lead * kb_per_group;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (kb == next_group_kb) {
            // entering a new slice group of the rows: wait (bounded) until all of its push units are in
            const int grp = kb / kb_per_group;
            next_group_kb = (grp + 1) * kb_per_group;
            const int in_group = imin(p.ag_spf, ag_nslices - grp * p.ag_spf);
            const uint64_t w0 = tr != nullptr ? globaltimer_ns() : 0;
            ok = flag_wait_eq(tile_flags + grp, ag_ups * in_group, ab, kStatusTimeoutFlag, budget);
            if (tr != nullptr) tr[5] += globaltimer_ns() - w0;
            if (!ok) break;
            fence_proxy_async();
          }
          if (!mbar_wait(bar_empty(stage), phase ^ 1u, ab, kStatusTimeoutSmemEmpty, budget, 40)) {
            ok = false;
            break;
          }
          // Pair mode: both CTAs' copies are credited to the leader's barrier, which the leader
          // arms for the bytes of both.
          uint32_t fb = bar_full(stage);
          if (CTA2) {
            if (leader) mbar_arrive_expect_tx(fb, 2 * L::kStageBytes);
            fb = mapa_u32(fb, 0);
          } else {
            mbar_arrive_expect_tx(fb, L::kStageBytes);
          }
          if (p.g_gather == nullptr) {
            // tiles of this rank's own shard read the caller's tensor in place
            const bool own_a = p.a_own_valid && p.g_tiles == nullptr && tc.seg == p.rank;
            const void* ta = own_a ? &p.tmap_a_own : &p.tmap_a;
            const int arow = own_a ? tc.row0 - p.rank * p.seg_rows : tc.row0;
            if (CTA2) tma_load_2d_2cta(smem_a(stage), ta, fb, kb * BKE, arow);
            else tma_load_2d(smem_a(stage), ta, fb, kb * BKE, arow);
          } else {
            // 32 gather4 copies of 4 rows each; rows past the tile end re-read a valid row
            const int* gi = p.g_gather + (tc.rows > 0 ? tc.row0 : 0);
            const int nr = tc.rows > 0 ? tc.rows : 1;
            for (int q = 0; q < kBM / 4; ++q) {
              const int r0 = q * 4;
              const int i0 = gi[r0 < nr ? r0 : 0];
              const int i1 = gi[r0 + 1 < nr ? r0 + 1 : 0];
              const int i2 = gi[r0 + 2 < nr ? r0 + 2 : 0];
              const int i3 = gi[r0 + 3 < nr ? r0 + 3 : 0];
              if (CTA2)
                tma_gather4_2d_2cta(smem_a(stage) + q * 4 * kRowBytes, &p.tmap_a, fb, kb * BKE, i0, i1, i2, i3);
              else
                tma_gather4_2d(smem_a(stage) + q * 4 * kRowBytes, &p.tmap_a, fb, kb * BKE, i0, i1, i2, i3);
            }
          }
          if (p.b_mn_major) {
            // B is [K, N]: one box of 64 columns x BKE rows per 64 output columns
            constexpr int kBoxes = L::kBRows / 64;
            const int ncol0 = tc.b_row0 + (CTA2 ? half * (BN / 2) : 0);
#pragma unroll
            for (int j = 0; j < kBoxes; ++j) {
              if (CTA2) tma_load_2d_2cta(smem_b(stage) + j * (BKE * kRowBytes), &p.tmap_b, fb, ncol0 + j * 64, kb * BKE);
              else tma_load_2d(smem_b(stage) + j * (BKE * kRowBytes), &p.tmap_b, fb, ncol0 + j * 64, kb * BKE);
            }
          } else if (CTA2) {
            tma_load_2d_2cta(smem_b(stage), &p.tmap_b, fb, kb * BKE, tc.b_row0 + half * (BN / 2));
          } else {
            tma_load_2d(smem_b(stage), &p.tmap_b, fb, kb * BKE, tc.b_row0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*s_abort != 0) drain_loads(stage, phase);
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------- UMMA
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      int t, kb0, kb1, part;
      for (; ok && get_item(it, t, kb0, kb1, part); ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(bar_tempty(acc), acc_phase ^ 1u, ab, kStatusTimeoutTmemEmpty, budget))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_full(stage), phase, ab, kStatusTimeoutSmemFull, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (tr != nullptr && it == 0 && kb == kb0) tr[1] = globaltimer_ns();
          const uint64_t a_desc = make_kmajor_sw128_desc(smem_a(stage));
          const uint64_t b_desc = p.b_mn_major ? make_mnmajor_sw128_desc(smem_b(stage), BKE * kRowBytes)
                                               : make_kmajor_sw128_desc(smem_b(stage));
          // each UMMA consumes 32 bytes of K of a K-major operand: advance the start address by 32 B
          // (>>4 = 2); of an MN-major operand it consumes 16 K rows of 128 B: 2048 B (>>4 = 128)
          const uint32_t b_step = p.b_mn_major ? 128u : 2u;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            if (CTA2) {
              if (KIND == 0) umma_f16_2cta(d_tmem, a_desc + 2u * k, b_desc + b_step * k, idesc, accum);
              else if (p.acc_int) umma_i8_2cta(d_tmem, a_desc + 2u * k, b_desc + b_step * k, idesc, accum);
              else umma_f8_2cta(d_tmem, a_desc + 2u * k, b_desc + b_step * k, idesc, accum);
            } else {
              if (KIND == 0) umma_f16(d_tmem, a_desc + 2u * k, b_desc + b_step * k, idesc, accum);
              else if (p.acc_int) umma_i8(d_tmem, a_desc + 2u * k, b_desc + b_step * k, idesc, accum);
              else umma_f8(d_tmem, a_desc + 2u * k, b_desc + b_step * k, idesc, accum);
            }
          }
          if (CTA2) umma_commit_2cta(bar_empty(stage), 3); else umma_commit(bar_empty(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          if (CTA2) umma_commit_2cta(bar_tfull(acc), 3); else umma_commit(bar_tfull(acc));
        }
      }
      if (tr != nullptr) {
        tr[2] = globaltimer_ns();
        tr[7] = static_cast<unsigned long long>(it);
      }
      if (*s_abort != 0) {
        // abort path: the UMMAs issued so far still read shared memory and write tensor memory; let them
        // retire (bounded) before the CTA tears both down
        if (CTA2) umma_commit_2cta(bar_retired, 1); else umma_commit(bar_retired);
        mbar_wait(bar_retired, 0, AbortWord{nullptr, 0u}, 0, 2000000ull);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------- epilogue
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t stage_blk0 = smem_base + L::kEpiOffset + (warp - 2) * L::kEpiWarpBytes;
    int* pending_cnt = nullptr;  // reduce-scatter: counter of the previous pushed tile, published one tile late
    if (perm_helped) {
      // MoE layer 0: nothing to drain until this rank's own tokens are permuted; take every second unit of them
      for (int u = cta_id + num_ctas; u < perm_units; u += 2 * num_ctas)
        permute_unit(std::integral_constant<int, 2>{}, u, p.rank, static_cast<int>(threadIdx.x) - 2 * 32, false);
    }
    int it = 0;
    int t, kb0, kb1, part;
    for (; get_item(it, t, kb0, kb1, part); ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      TileCoord tc;
      decode_tile<BN, TILE_M>(p, t, m_tiles, n_tiles, tps, half, tc);
      if (!mbar_wait(bar_tfull(acc), acc_phase, ab, kStatusTimeoutTmemFull, budget, 300)) break;
      tc_fence_after();
      // split-K tail: where this warp's 32 rows of a tail tile's partial accumulators live
      const bool is_tail = split > 1 && it == full_waves;
      float* sk_rows = nullptr;
      int* sk_cnt = nullptr;
      int* sk_done = nullptr;
      if (is_tail) {
        const int tt = t - full_tiles;
        sk_rows = p.splitk_scratch + (static_cast<long long>(tt) * (split - 1) * TILE_M + half * kBM + quad * 32 + lane) * BN;
        sk_cnt = p.splitk_cnt + (tt * 2 + half) * 4 + quad;
        sk_done = p.splitk_done + (tt * 2 + half) * 4 + quad;
      }
      // Every part of a split tail tile finishes a share of the tile's 64-column boxes (box b belongs to part
      // b * owners / boxes, owners = min(split, boxes)): it parks its raw fp32 accumulators of the other boxes
      // for their owners, waits until all parts have parked, and runs the ordinary epilogue on its own boxes
      // with the other parts' partials added. The tail's epilogue work - bound by load latency - is thereby
      // spread over all the CTAs that worked on the tile instead of falling on one.
      // A tile whose result is pushed to its owner (reduce-scatter, another rank's rows) is finished by part 0
      // alone: the owner counts one publish per epilogue warp of ONE CTA (pair half) per tile.
      const bool sk_pushed = p.epi_mode == kEpiRsPush && tc.seg != p.rank;
      const int sk_owners = splitk_owners(split, BN, sk_pushed);
      auto sk_owner_of = [&](int c) { return splitk_owner_of(c, split, BN, sk_pushed); };
      if (is_tail) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int oc = sk_owner_of(c);
          if (oc == part) continue;
          float* dst = sk_rows + static_cast<long long>(part < oc ? part : part - 1) * TILE_M * BN;
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN + c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 4) = make_uint4(r[q * 4], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]);
        }
        __threadfence();
        __syncwarp();
        int okw = 1;
        if (lane == 0) {
          red_add_release_sys(sk_cnt, 1);
          if (part < sk_owners) okw = flag_wait_eq(sk_cnt, split, ab, kStatusTimeoutTmemFull, budget) ? 1 : 0;
          // the last part through clears both counters for the next launch
          if (okw && atomicAdd(sk_done, 1) == split - 1) {
            *sk_cnt = 0;
            *sk_done = 0;
          }
        }
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) break;
        if (part >= sk_owners) {
          // more parts than boxes: this one only parked
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CTA2) mbar_arrive_cluster(mapa_u32(bar_tempty(acc), 0));
            else mbar_arrive(bar_tempty(acc));
          }
          continue;
        }
      }
      const bool row_ok = row_in_tile < tc.rows;
      const int grow = tc.row0 + row_in_tile;  // global / sorted row
      float row_scale = p.alpha;
      if (p.alpha_ptr != nullptr) row_scale *= *p.alpha_ptr;
      if (p.scale_a != nullptr && row_ok) row_scale *= p.scale_a[grow];
      if (p.g_expert_scale != nullptr) row_scale *= p.g_expert_scale[tc.expert];

      // Reduce-scatter, tiles of this rank's own rows: the peers' partials have been summed by the comm
      // warps; wait (bounded) for that, then add the sum to the accumulator and write the final rows.
      const bool own = p.epi_mode == kEpiRsPush && tc.seg == p.rank;
      const float* sum_row = nullptr;
      if (own && lane == 0 && pending_cnt != nullptr) {
        // Never hold back a publish while waiting on the peers: they may be waiting for exactly this one.
        bulk_wait_all();
        fence_acq_rel_sys();
        red_add_release_sys(pending_cnt, 1);
        pending_cnt = nullptr;
      }
      if (own && tc.rows > 0) {  // a pair's second half may lie entirely past the segment: nothing to wait for
        int okw = 1;
        if (lane == 0) {
          const uint64_t w0 = (tr != nullptr && warp == 2) ? globaltimer_ns() : 0;
          const int tix = tc.chunk * n_tiles + tc.n_idx;
          if (p.rs_n_late < p.world - 1)  // the comm warps' sum of the early peers' partials
            okw = flag_wait_eq(p.rs_local_ready + tix, 4, ab, kStatusTimeoutReduce, budget) ? 1 : 0;
          if (okw && p.rs_n_late > 0)  // the late peers' partials themselves (4 arrivals each)
            okw = flag_wait_eq(p.rs_local_cnt + p.rs_late_off + tix, 4 * p.rs_n_late, ab, kStatusTimeoutReduce,
                               budget) ? 1 : 0;
          if (tr != nullptr && warp == 2) tr[6] += globaltimer_ns() - w0;
        }
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) break;
      }
      const int otype = own ? p.rs_out_type : p.out_type;

      // destination row pointer
      uint8_t* dst_row = nullptr;
      const uint8_t* bias_row = nullptr;
      if (own) {
        const long long lrow = static_cast<long long>(tc.chunk) * kBM + row_in_tile;
        const int osz = (otype == kOutF32) ? 4 : 2;
        dst_row = static_cast<uint8_t*>(p.rs_out) + lrow * p.N * osz;
        sum_row = p.rs_local_stage + static_cast<long long>(p.rank) * p.seg_rows * p.N + lrow * p.N;
        if (p.bias_mode == kBiasFull)
          bias_row = static_cast<const uint8_t*>(p.bias) + static_cast<long long>(grow) * p.ldbias * 2;
        else if (p.bias_mode == kBiasRow)
          bias_row = static_cast<const uint8_t*>(p.bias);
      } else if (p.epi_mode == kEpiStore) {
        long long orow = grow;
        if (p.g_scatter_rows != nullptr && row_ok) orow = p.g_scatter_rows[grow];
        const int osz = (p.out_type == kOutF32) ? 4 : 2;
        dst_row = static_cast<uint8_t*>(p.out) + orow * p.ldo * osz;
        if (p.bias_mode == kBiasFull)
          bias_row = static_cast<const uint8_t*>(p.bias) + orow * p.ldbias * osz;
        else if (p.bias_mode == kBiasRow)
          bias_row = static_cast<const uint8_t*>(p.bias);
      } else {
        // reduce-scatter: the segment is the owner, the row inside it is the owner's local row
        const long long lrow = static_cast<long long>(tc.chunk) * kBM + row_in_tile;
        dst_row = reinterpret_cast<uint8_t*>(p.rs_stage[tc.seg] + lrow * p.N);
        if (p.bias_mode == kBiasFull)
          bias_row = static_cast<const uint8_t*>(p.bias) + static_cast<long long>(grow) * p.ldbias * 2;
        else if (p.bias_mode == kBiasRow)
          bias_row = static_cast<const uint8_t*>(p.bias);
      }

      // Plain output whose 32 rows of this warp are all valid: staged in shared memory and written with tiled
      // stores (full 128-byte rows, one instruction per 32 x 64 box) instead of 16 bytes per lane per row.
      const bool tma_out = p.tmap_out_valid && p.epi_mode == kEpiStore && otype != kOutF32 &&
                           p.g_scatter_rows == nullptr && quad * 32 + 32 <= tc.rows;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        if (is_tail && sk_owner_of(c) != part) continue;  // another part finishes this box
        uint32_t r[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                               static_cast<uint32_t>(acc * BN + c * 32);
        tmem_ld_32x32(taddr, r);
        tmem_ld_wait();
        const int col0 = tc.n0 + c * 32;
        const bool active = row_ok && col0 < p.N;
        if (is_tail) {
          // add the parked partial accumulators of the other K parts, two parts' loads in flight at a time
          for (int sp = 0; sp < split - 1; sp += 2) {
            float4 pv[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u)
              if (sp + u < split - 1) {
                const float* src = sk_rows + static_cast<long long>(sp + u) * TILE_M * BN + c * 32;
#pragma unroll
                for (int q = 0; q < 8; ++q) pv[u][q] = *reinterpret_cast<const float4*>(src + q * 4);
              }
#pragma unroll
            for (int u = 0; u < 2; ++u)
              if (sp + u < split - 1) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  r[q * 4] = __float_as_uint(__uint_as_float(r[q * 4]) + pv[u][q].x);
                  r[q * 4 + 1] = __float_as_uint(__uint_as_float(r[q * 4 + 1]) + pv[u][q].y);
                  r[q * 4 + 2] = __float_as_uint(__uint_as_float(r[q * 4 + 2]) + pv[u][q].z);
                  r[q * 4 + 3] = __float_as_uint(__uint_as_float(r[q * 4 + 3]) + pv[u][q].w);
                }
              }
          }
        }
        float v[32];
        if (KIND == 1 && p.acc_int) {
          // int8 operands, int32 accumulator. Dequantisation in the reference's order, so that the result is
          // bit-identical to its golden path (test/python/ag_gemm/test_ag_kernel.py:143-150, threshold 0):
          // (input_scale[row] * weight_scale[col]) * float(acc), rounded to the 16-bit output; a bias is then
          // added in 16-bit arithmetic (`output += bias` on the rounded tensor).
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float sb = (active && p.scale_b != nullptr && col0 + j < p.N) ? p.scale_b[col0 + j] : 1.0f;
            v[j] = (row_scale * sb) * __int2float_rn(static_cast<int>(r[j]));
            if (bias_row != nullptr)
              v[j] = ((p.epi_mode == kEpiRsPush ? p.rs_out_type : p.out_type) == kOutF16)
                         ? __half2float(__float2half_rn(v[j])) : __bfloat162float(__float2bfloat16_rn(v[j]));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * row_scale;
          if (active && p.scale_b != nullptr) {
            if (col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(p.scale_b) & 15) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {  // 8 x 16-byte loads instead of 32 scalar ones
                const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.scale_b + col0) + q);
                v[q * 4] *= s4.x;
                v[q * 4 + 1] *= s4.y;
                v[q * 4 + 2] *= s4.z;
                v[q * 4 + 3] *= s4.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] *= p.scale_b[col0 + j];
            }
          }
        }
        if (active && bias_row != nullptr) {
          // bias has the output dtype in store mode, bf16 in reduce-scatter mode
          const int bt = (p.epi_mode == kEpiStore) ? p.out_type : kOutBf16;  // own tiles included
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + j < p.N) {
              float b;
              if (bt == kOutBf16)
                b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias_row)[col0 + j]);
              else if (bt == kOutF16)
                b = __half2float(reinterpret_cast<const __half*>(bias_row)[col0 + j]);
              else
                b = reinterpret_cast<const float*>(bias_row)[col0 + j];
              v[j] += b;
            }
          }
        }
        if (own && active && (p.rs_ring || (KIND == 1 && p.acc_int))) {
          // ring order: the own partial joins last, as a 16-bit value like the peers'; w8a8: every rank's
          // dequantised partial is a 16-bit tensor in the reference (test/python/gemm_rs/test_gemm_rs.py:127-135)
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = (p.rs_out_type == kOutF16) ? __half2float(__float2half_rn(v[j])) : __bfloat162float(__float2bfloat16_rn(v[j]));
        }
        if (own && active && p.rs_n_late < p.world - 1) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (col0 + q * 4 + 4 <= p.N) {
              const float4 sv = *reinterpret_cast<const float4*>(sum_row + col0 + q * 4);
              v[q * 4] += sv.x;
              v[q * 4 + 1] += sv.y;
              v[q * 4 + 2] += sv.z;
              v[q * 4 + 3] += sv.w;
            }
          }
        }
        if (own && active && p.rs_n_late > 0) {
          // late peers (rank+1, rank+2, ...): their 16-bit partials straight from the staging slots
          const long long slot = static_cast<long long>(p.seg_rows) * p.N;
          const long long eoff = (static_cast<long long>(tc.chunk) * kBM + row_in_tile) * p.N + col0;
#pragma unroll 1
          for (int i = 0; i < p.rs_n_late; ++i) {
            int sr = p.rank + 1 + i;
            if (sr >= p.world) sr -= p.world;
            const uint16_t* lp = reinterpret_cast<const uint16_t*>(p.rs_local_stage + sr * slot) + eoff;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col0 + q * 8 + 8 <= p.N) {
                const uint4 lv = __ldcg(reinterpret_cast<const uint4*>(lp + q * 8));
                const uint32_t w[4] = {lv.x, lv.y, lv.z, lv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (p.rs_out_type == kOutBf16) {
                    v[q * 8 + 2 * j] += __uint_as_float(w[j] << 16);
                    v[q * 8 + 2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
                  } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                    v[q * 8 + 2 * j] += f.x;
                    v[q * 8 + 2 * j + 1] += f.y;
                  }
                }
              }
            }
          }
        }
        // keeps the number of store groups per tile uniform (one per staged box)
        if (own && lane == 0 && (!p.rs_wire16 || (c & 1))) bulk_commit();
        if (p.epi_mode == kEpiRsPush && !own && p.rs_wire16) {
          // 16-bit wire format: two 32-column steps fill one 32 x 64 box (128-byte rows, 16-byte pieces
          // XOR-swizzled by row like the tensor map's 128-byte swizzle); the box is pushed to the owner
          // with one tiled store after the second step. Rows and columns outside the owner's slot are
          // clipped by the tensor map.
          const int box = c >> 1, h = c & 1;
          const uint32_t stage_blk = stage_blk0 + (L::kEpiBufs == 2 ? (box & 1) * L::kEpiBlockBytes : 0);
          const uint32_t stage_row = stage_blk + lane * L::kEpiPitch;
          if (h == 0) {
            if (lane == 0) {  // the previous store out of this block has been read
              if (L::kEpiBufs == 2) bulk_wait_read_keep1(); else bulk_wait_read();
            }
            __syncwarp();
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w[j] = (p.rs_out_type == kOutBf16) ? pack_bf16(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1])
                                                  : pack_f16(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_row + (((h * 4 + q) ^ (lane & 7)) << 4)),
                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
          if (h == 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (tc.rows > quad * 32 && col0 - 32 < p.N)
                tma_store_2d(&p.tmap_rs[tc.seg], stage_blk, col0 - 32, tc.chunk * kBM + quad * 32);
              bulk_commit();
            }
          }
        } else if (tma_out) {
          // same staging as the 16-bit reduce-scatter push, into the output tensor itself
          const int box = c >> 1, h = c & 1;
          const uint32_t stage_blk = stage_blk0 + (L::kEpiBufs == 2 ? (box & 1) * L::kEpiBlockBytes : 0);
          const uint32_t stage_row = stage_blk + lane * L::kEpiPitch;
          if (h == 0) {
            if (lane == 0) {  // the previous store out of this block has been read
              if (L::kEpiBufs == 2) bulk_wait_read_keep1(); else bulk_wait_read();
            }
            __syncwarp();
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w[j] = (otype == kOutBf16) ? pack_bf16(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1])
                                         : pack_f16(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_row + (((h * 4 + q) ^ (lane & 7)) << 4)),
                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
          if (h == 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (col0 - 32 < p.N) tma_store_2d(&p.tmap_out, stage_blk, col0 - 32, tc.row0 + quad * 32);
              bulk_commit();
            }
          }
        } else if (p.epi_mode == kEpiRsPush && !own) {
          // fp32 wire format. Park the warp's 32 x 32 fp32 block in shared memory (lane = row, 16-byte pieces XOR-swizzled
          // by row so that the writes spread over all banks and match the tensor map's 128-byte swizzle),
          // then push it to the owner with one tiled store: 4 KB per operation over NVLink, rows and
          // columns outside the owner's slot are clipped by the tensor map.
          const uint32_t stage_blk = stage_blk0 + (L::kEpiBufs == 2 ? (c & 1) * L::kEpiBlockBytes : 0);
          const uint32_t stage_row = stage_blk + lane * L::kEpiPitch;
          if (lane == 0) {  // the previous store out of this block has been read
            if (L::kEpiBufs == 2) bulk_wait_read_keep1(); else bulk_wait_read();
          }
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage_row + ((q ^ (lane & 7)) << 4)),
                         "f"(v[q * 4]), "f"(v[q * 4 + 1]), "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3])
                         : "memory");
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (tc.rows > quad * 32 && col0 < p.N)
              tma_store_2d(&p.tmap_rs[tc.seg], stage_blk, col0, tc.chunk * kBM + quad * 32);
            bulk_commit();
          }
        } else if (active) {
          if (otype == kOutF32) {
            float* d = reinterpret_cast<float*>(dst_row) + col0;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              if (col0 + q * 4 + 4 <= p.N) {
                *reinterpret_cast<float4*>(d + q * 4) =
                    make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  if (col0 + q * 4 + j < p.N) d[q * 4 + j] = v[q * 4 + j];
              }
            }
          } else {
            uint16_t* d = reinterpret_cast<uint16_t*>(dst_row) + col0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                w[j] = (otype == kOutBf16) ? pack_bf16(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1])
                                                : pack_f16(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
              if (col0 + q * 8 + 8 <= p.N) {
                *reinterpret_cast<uint4*>(d + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (col0 + q * 8 + j < p.N)
                    d[q * 8 + j] = static_cast<uint16_t>((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xFFFFu));
              }
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTA2) mbar_arrive_cluster(mapa_u32(bar_tempty(acc), 0));
        else mbar_arrive(bar_tempty(acc));
        // MoE layer 1: this warp's rows of the tile are stored (tiled stores complete, and the release covers
        // the whole warp's plain stores)
        if (p.gr_slab_done != nullptr) {
          if (tma_out) {
            bulk_wait_all();
            fence_proxy_async();
          }
          red_add_release_gpu(p.gr_slab_done + tc.n_idx, 1);
        }
      }
      if (p.epi_mode == kEpiRsPush) {
        // Publish the PREVIOUS pushed tile of this warp: its stores were issued a whole tile ago, so
        // waiting for all groups but this tile's BN/32 costs nothing, whereas waiting for the stores
        // just issued (one group per staged box) would put NVLink round trips on the epilogue's critical path. Each epilogue warp
        // adds 1, so a complete 128-row tile counts 4 per source rank. (No CTA-wide barrier here: a
        // role that gave up must never strand the others.)
        if (lane == 0) {
          if (pending_cnt != nullptr) {
            // (a split tail tile issues fewer store groups than a whole tile: wait for everything there)
            if (is_tail) bulk_wait_all();
            else if (p.rs_wire16) bulk_wait_all_but<BN / 64>();
            else bulk_wait_all_but<BN / 32>();
            fence_acq_rel_sys();
            red_add_release_sys(pending_cnt, 1);
          }
          const int prev_rank = p.rank == 0 ? p.nseg - 1 : p.rank - 1;
          const bool urgent = p.n_bands >= 2 ? tc.band == p.n_bands - 2 : tc.seg == prev_rank;
          pending_cnt = (!own && tc.rows > 0) ? p.rs_cnt[tc.seg] + ((urgent && p.rs_n_late > 0) ? p.rs_late_off : 0) +
                                                    tc.chunk * n_tiles + tc.n_idx
                                              : nullptr;
          // Exception: the tiles of the last band of peer-owned rows are the ones their owners are waiting
          // for when they reach their own rows (every rank computes its own rows last), so their publish is
          // latency-critical: with the late publish, the owners' last epilogues waited about one tile time for
          // them (seen in the kernel's timeline on 8 GPUs). The accumulator has been released already, so waiting for these
          // stores holds up nothing but this warp. (Without explicit bands: the rows of the previous rank.)
          if (pending_cnt != nullptr && urgent) {
            bulk_wait_all();
            fence_acq_rel_sys();
            red_add_release_sys(pending_cnt, 1);
            pending_cnt = nullptr;
          }
        }
      }
    }
    if (tr != nullptr && warp == 2 && lane == 0) tr[3] = globaltimer_ns();
    if (p.epi_mode == kEpiStore && p.tmap_out_valid && lane == 0) bulk_wait_all();  // tiled stores must not outlive the CTA
    if (p.epi_mode == kEpiRsPush && lane == 0) {
      // also on the way out after a failed wait: the stores must not outlive the CTA
      bulk_wait_all();
      if (pending_cnt != nullptr) {
        fence_acq_rel_sys();
        red_add_release_sys(pending_cnt, 1);
      }
    }
  } else {
    // ----------------------------------------------------------------- comm
    // All-gather push and (MoE layer 0) permute by the 128 comm threads of the CTA. A push unit is
    // ag_unit_rows (32, 64 or 128) rows x 2 KB: one 16-byte column per thread, 8 rows in flight, then ONE
    // system-scope release per unit (measured on 8 GPUs: the release waits for the unit's stores to be
    // acknowledged over NVLink, so a release per 8 rows per warp halved the push rate).
    // Steps d = 0 .. world-1 interleave the two jobs: permute the tokens of source rank+d (own tokens first,
    // read in place; the others were pushed by their source during its step d-1), then push this rank's shard
    // to the rank that needs it d-th soonest (rank-1, rank-2, ...; one destination at a time, so every link
    // carries one stream at full rate and shards land in the order they are consumed).
    // The push is skipped when the copy engines carry the all-gather (p.ag_src == nullptr).
    if (p.ag_src != nullptr || p.g_sorted != nullptr) {
      const int ctid = threadIdx.x - 6 * 32;  // 0..127
      // own rows are read from the caller's tensor (dense: by the own tiles; MoE: by the permute): no copy to itself
      const int d_first = (p.ag_src != nullptr && (p.a_own_valid || p.g_tokens_own != nullptr)) ? 1 : 0;
      const int push_chunks = (p.seg_rows + kBM - 1) / kBM;
      const int units_per_dest = ag_nslices * push_chunks * ag_ups;
      const int unit_rows = kBM / ag_ups;
      bool comm_ok = true;
      for (int d = 0; comm_ok && d < p.world; ++d) {
        if (p.g_sorted != nullptr) {
          // MoE layer 0, permute form: copy every token row of source rank+d to its top-k rows of the
          // expert-sorted buffer (one load, top-k stores per 16-byte piece) and count the unit as done
          // for that source; a tile waits until every source rank it reads is complete.
          int src_rank = p.rank + d;
          if (src_rank >= p.world) src_rank -= p.world;
          // units of this CTA: u = cta_id, cta_id + num_ctas, ...; while the epilogue warps help (step 0, see
          // there) they take every second one
          const int stride = perm_helped && d == 0 ? 2 * num_ctas : num_ctas;
          int pu_first = cta_id - static_cast<int>((static_cast<long long>(d) * perm_units) % num_ctas);
          if (pu_first < 0) pu_first += num_ctas;  // as for the push below: rotate the CTA that takes unit 0
          for (int u = pu_first; comm_ok && u < perm_units; u += stride)
            comm_ok = permute_unit(std::integral_constant<int, 1>{}, u, src_rank, ctid, true);
        }
        if (p.ag_src != nullptr && d + d_first < p.world) {
          int dest = p.rank - (d + d_first);
          if (dest < 0) dest += p.world;
          // units of one destination in slice-major order: the first 2 KB of every row go out first, so
          // that the consumer's walk along K can begin after a fraction of the shard has crossed
          // (the CTA that takes unit 0 rotates from destination to destination, so that all CTAs push even
          // when a destination has fewer units than there are CTAs: 96 units per destination at TP=8)
          int u_first = cta_id - static_cast<int>((static_cast<long long>(d) * units_per_dest) % num_ctas);
          if (u_first < 0) u_first += num_ctas;
          for (int u = u_first; u < units_per_dest; u += num_ctas) {
            const int ks = u / (push_chunks * ag_ups);
            const int rem = u - ks * (push_chunks * ag_ups);
            const int chunk = rem / ag_ups;
            const int r0 = imin(chunk * kBM + (rem - chunk * ag_ups) * unit_rows, p.seg_rows);
            const int nrows = imin(unit_rows, p.seg_rows - r0);  // 0 for a unit past the shard's last row: it still signals
            const long long b0 = static_cast<long long>(ks) * kCommSliceBytes;
            const int slice_bytes = static_cast<int>((b0 + kCommSliceBytes < p.ag_row_bytes ? b0 + kCommSliceBytes : p.ag_row_bytes) - b0);
            if (ctid * 16 < slice_bytes) {
              const uint8_t* src = p.ag_src + static_cast<long long>(r0) * p.ag_row_bytes + b0 + ctid * 16;
              uint8_t* dst = p.ag_dst[dest] + (static_cast<long long>(p.rank) * p.seg_rows + r0) * p.ag_row_bytes + b0 + ctid * 16;
#pragma unroll 1
              for (int rr = 0; rr < nrows; rr += 8) {
                uint4 val[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (rr + j < nrows) val[j] = __ldg(reinterpret_cast<const uint4*>(src + (rr + j) * p.ag_row_bytes));
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (rr + j < nrows) *reinterpret_cast<uint4*>(dst + (rr + j) * p.ag_row_bytes) = val[j];
              }
            }
            if (ks == 0 && p.ag_src_scale != nullptr && ctid < nrows)
              p.ag_dst_scale[dest][static_cast<long long>(p.rank) * p.seg_rows + r0 + ctid] = p.ag_src_scale[r0 + ctid];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            // the release covers every thread's stores (ordered before it by the barrier)
            if (ctid == 0)
              red_add_release_sys(p.ag_dst_flags[dest] + p.rank * p.ag_flag_stride + chunk * p.ag_groups + ks / p.ag_spf, 1);
          }
        }
      }
    }
    if (p.gr_slab_done != nullptr) {
      // MoE layer 1, combine + reduce-scatter. For slab s (in the order the GEMM produces them): wait until
      // every tile of the slab is stored, then item = (owner, block of 32 of its tokens): sum each token's
      // top-k rows of the slab in fp32, round, store into the owner's staging slot of this rank and add 1 to
      // the owner's counter of (slab, block). One slab behind, the owner side: item = (block of this rank's
      // tokens): wait (bounded) for `world` arrivals, sum the per-source partials in fp32, write the result.
      // A warp handles 8 tokens of an item, four at a time, one 16-byte column piece per lane.
      const int ctid = threadIdx.x - 6 * 32;
      const int cw = ctid >> 5;
      const int tpr = p.gr_tokens_per_rank;
      const int bpo = (tpr + kGrTokBlock - 1) / kGrTokBlock;  // token blocks per owner
      const int osz = 2;                                       // 16-bit staging and output
      const bool out_bf16 = p.out_type == kOutBf16;
      volatile int* s_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 16);
      bool gr_ok = true;
      for (int slab = 0; gr_ok && slab <= n_tiles; ++slab) {
        if (slab < n_tiles) {
          if (ctid == 0)
            *s_flag = flag_wait_eq(p.gr_slab_done + slab, p.gr_slab_expected, ab, kStatusTimeoutReduce, budget) ? 1 : 0;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int oks = *s_flag;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (!oks) break;
          const int col0 = slab * BN;
          const int cols = imin(BN, p.N - col0);
          const bool lane_on = lane * 8 < cols;
          const int first = (cta_id + slab * 61) % num_ctas;  // rotate, so that slabs do not load the same CTAs
          for (int item = first; item < p.world * bpo; item += num_ctas) {
            const int oi = item / bpo;
            const int blk = item - oi * bpo;
            int owner = p.rank + 1 + oi;
            while (owner >= p.world) owner -= p.world;
            uint16_t* dst = static_cast<uint16_t*>(p.gr_stage[owner]);
#pragma unroll 1
            for (int b4 = 0; b4 < 8; b4 += 4) {
              float acc4[4][8];
              int tl[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                tl[j] = blk * kGrTokBlock + cw * 8 + b4 + j;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc4[j][e] = 0.f;
              }
              // The rows of the 4 tokens' top-k entries: lane (j * topk + k) fetches one entry of the scatter index
              // and shuffles hand them out (a load of the index in front of every data load doubled the length
              // of the dependent chain); the data loads of two k are in flight together.
              int my_row = -1;
              {
                const int jj = lane / p.gr_topk, kk = lane - jj * p.gr_topk;
                const int tok = blk * kGrTokBlock + cw * 8 + b4 + jj;
                if (jj < 4 && tok < tpr)
                  my_row = p.gr_scatter_index[(static_cast<long long>(owner) * tpr + tok) * p.gr_topk + kk] - p.gr_row_lo;
                if (my_row < 0 || my_row >= p.gr_rows) my_row = -1;  // rows of other ranks' experts; a corrupt entry must not become a wild load
              }
              const bool idx_in_regs = 4 * p.gr_topk <= 32;
              for (int k0 = 0; k0 < p.gr_topk; k0 += 2) {
                uint4 raw2[2][4];
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    raw2[u][j] = make_uint4(0u, 0u, 0u, 0u);
                    const int k = k0 + u;
                    int row = -1;
                    if (k < p.gr_topk) {
                      if (idx_in_regs) {
                        row = __shfl_sync(0xffffffffu, my_row, j * p.gr_topk + k);
                      } else if (tl[j] < tpr) {
                        row = p.gr_scatter_index[(static_cast<long long>(owner) * tpr + tl[j]) * p.gr_topk + k] - p.gr_row_lo;
                        if (row >= p.gr_rows) row = -1;
                      }
                    }
                    if (row >= 0 && tl[j] < tpr && lane_on)
                      raw2[u][j] = ld_relaxed_gpu_v4(static_cast<const uint16_t*>(p.out) + static_cast<long long>(row) * p.ldo + col0 + lane * 8);
                  }
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4* raw = raw2[u];
                  const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (out_bf16) {
                      acc4[j][2 * e] += __uint_as_float(w[e] << 16);
                      acc4[j][2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
                    } else {
                      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                      acc4[j][2 * e] += f.x;
                      acc4[j][2 * e + 1] += f.y;
                    }
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (tl[j] < tpr && lane_on) {
                  uint4 o;
                  if (out_bf16) {
                    o = make_uint4(pack_bf16(acc4[j][0], acc4[j][1]), pack_bf16(acc4[j][2], acc4[j][3]),
                                   pack_bf16(acc4[j][4], acc4[j][5]), pack_bf16(acc4[j][6], acc4[j][7]));
                  } else {
                    o = make_uint4(pack_f16(acc4[j][0], acc4[j][1]), pack_f16(acc4[j][2], acc4[j][3]),
                                   pack_f16(acc4[j][4], acc4[j][5]), pack_f16(acc4[j][6], acc4[j][7]));
                  }
                  *reinterpret_cast<uint4*>(dst + static_cast<long long>(tl[j]) * p.N + col0 + lane * 8) = o;
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (ctid == 0) red_add_release_sys(p.gr_cnt[owner] + slab * bpo + blk, 1);
          }
        }
        if (slab >= 1) {
          const int rs = slab - 1;
          const int col0 = rs * BN;
          const int cols = imin(BN, p.N - col0);
          const bool lane_on = lane * 8 < cols;
          const long long slot = static_cast<long long>(tpr) * p.N;
          const int first = (cta_id + rs * 61) % num_ctas;
          for (int blk = first; gr_ok && blk < bpo; blk += num_ctas) {
            if (ctid == 0)
              *s_flag = flag_wait_eq(p.gr_local_cnt + rs * bpo + blk, p.world, ab, kStatusTimeoutReduce, budget) ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int okr = *s_flag;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!okr) {
              gr_ok = false;
              break;
            }
#pragma unroll 1
            for (int b4 = 0; b4 < 8; b4 += 4) {
              float acc4[4][8];
              int tl[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                tl[j] = blk * kGrTokBlock + cw * 8 + b4 + j;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc4[j][e] = 0.f;
              }
              for (int sr0 = 0; sr0 < p.world; sr0 += 2) {  // two sources' loads in flight together
                uint4 raw2[2][4];
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    raw2[u][j] = make_uint4(0u, 0u, 0u, 0u);
                    if (sr0 + u < p.world && tl[j] < tpr && lane_on)
                      raw2[u][j] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.gr_local_stage) +
                                                                   (sr0 + u) * slot + static_cast<long long>(tl[j]) * p.N +
                                                                   col0 + lane * 8);
                  }
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4* raw = raw2[u];
                  const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (out_bf16) {
                      acc4[j][2 * e] += __uint_as_float(w[e] << 16);
                      acc4[j][2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
                    } else {
                      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                      acc4[j][2 * e] += f.x;
                      acc4[j][2 * e + 1] += f.y;
                    }
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (tl[j] < tpr && lane_on) {
                  uint4 o;
                  if (out_bf16) {
                    o = make_uint4(pack_bf16(acc4[j][0], acc4[j][1]), pack_bf16(acc4[j][2], acc4[j][3]),
                                   pack_bf16(acc4[j][4], acc4[j][5]), pack_bf16(acc4[j][6], acc4[j][7]));
                  } else {
                    o = make_uint4(pack_f16(acc4[j][0], acc4[j][1]), pack_f16(acc4[j][2], acc4[j][3]),
                                   pack_f16(acc4[j][4], acc4[j][5]), pack_f16(acc4[j][6], acc4[j][7]));
                  }
                  *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.gr_out) + static_cast<long long>(tl[j]) * p.N + col0 +
                                            lane * 8) = o;
                }
            }
          }
        }
      }
      (void)osz;
    }
      if (p.epi_mode == kEpiRsPush) {
      // Owner side of the reduce-scatter. Work item = 32 rows of one 128 x BN tile of this rank's rows:
      // wait (bounded) until every early peer has published the tile (4 arrivals per peer: one per epilogue
      // warp), sum their partials in fp32 in rank order into this rank's own slot, and add 1 to the
      // tile's ready count (the epilogue of the own tile waits for 4; the late peers' partials it adds itself). Items are spread over all CTAs and
      // every source's loads are in flight together. The peers compute this rank's rows before their own,
      // so this work is spread over the kernel and finished before the own tiles are.
      const int ctid = threadIdx.x - 6 * 32;  // 0..127
      const int m_chunks = (p.seg_rows + kBM - 1) / kBM;
      const int n_early = p.world - 1 - p.rs_n_late;            // peers whose partials are summed here
      const int total_items = n_early > 0 ? m_chunks * n_tiles * 4 : 0;
      constexpr int kVecPerRow = BN / 4;                 // float4 per tile row
      constexpr int kVecPerItem = 32 * kVecPerRow;       // float4 per work item
      const long long slot = static_cast<long long>(p.seg_rows) * p.N;
      float* sum_base = p.rs_stage[p.rank];  // this rank's slot in its own staging
      volatile int* s_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 16);
      for (int item = cta_id; item < total_items; item += num_ctas) {
        const int quarter = item & 3;
        const int rt = item >> 2;
        const int c = rt % m_chunks;
        const int nt = rt / m_chunks;
        const int tix = c * n_tiles + nt;
        if (ctid == 0)
          *s_flag = flag_wait_eq(p.rs_local_cnt + tix, 4 * n_early, ab, kStatusTimeoutReduce, budget) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int okr = *s_flag;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!okr) break;
        const int row_base = c * kBM + quarter * 32;
        const int rows = imax(0, imin(32, p.seg_rows - row_base));
        const int n0 = nt * BN;
        if (p.rs_wire16) {
          // peers' partials are 16-bit (8 values per 16-byte load); the sum stays fp32
          constexpr int kVec16PerRow = BN / 8;
          constexpr int kVec16PerItem = 32 * kVec16PerRow;
          for (int i0 = ctid; i0 < kVec16PerItem; i0 += 2 * 128) {
            long long off[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int i = i0 + u * 128;
              const int r = i / kVec16PerRow;
              const int col = n0 + (i - r * kVec16PerRow) * 8;
              off[u] = (i < kVec16PerItem && r < rows && col < p.N) ? static_cast<long long>(row_base + r) * p.N + col : -1;
            }
            // peers in ring order (rank+1, rank+2, ...): the order of the reference's ring_reduce
            // (src/gemm_rs/ring_reduce.cu:54-80); with rs_ring the running sum is also rounded to the
            // 16-bit element type after every addition, as that kernel does
            uint4 v[kMaxWorld][2];
#pragma unroll
            for (int i = 0; i < kMaxWorld - 1; ++i)
#pragma unroll
              for (int u = 0; u < 2; ++u)
                if (i >= p.rs_n_late && i + 1 < p.world && off[u] >= 0) {
                  int sr = p.rank + 1 + i;
                  if (sr >= p.world) sr -= p.world;
                  v[i][u] = *reinterpret_cast<const uint4*>(
                      reinterpret_cast<const uint16_t*>(p.rs_local_stage + sr * slot) + off[u]);
                }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              if (off[u] < 0) continue;
              float acc[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
              for (int i = 0; i < kMaxWorld - 1; ++i)
                if (i >= p.rs_n_late && i + 1 < p.world) {
                  const uint32_t w[4] = {v[i][u].x, v[i][u].y, v[i][u].z, v[i][u].w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (p.rs_out_type == kOutBf16) {
                      acc[2 * j] += __uint_as_float(w[j] << 16);
                      acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
                      if (p.rs_ring) {
                        acc[2 * j] = __bfloat162float(__float2bfloat16_rn(acc[2 * j]));
                        acc[2 * j + 1] = __bfloat162float(__float2bfloat16_rn(acc[2 * j + 1]));
                      }
                    } else {
                      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                      acc[2 * j] += f.x;
                      acc[2 * j + 1] += f.y;
                      if (p.rs_ring) {
                        acc[2 * j] = __half2float(__float2half_rn(acc[2 * j]));
                        acc[2 * j + 1] = __half2float(__float2half_rn(acc[2 * j + 1]));
                      }
                    }
                  }
                }
              *reinterpret_cast<float4*>(sum_base + off[u]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
              *reinterpret_cast<float4*>(sum_base + off[u] + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
          }
        } else
        for (int i0 = ctid; i0 < kVecPerItem; i0 += 2 * 128) {
          long long off[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int i = i0 + u * 128;
            const int r = i / kVecPerRow;
            const int col = n0 + (i - r * kVecPerRow) * 4;
            off[u] = (i < kVecPerItem && r < rows && col < p.N) ? static_cast<long long>(row_base + r) * p.N + col : -1;
          }
          float4 v[kMaxWorld][2];
#pragma unroll
          for (int sr = 0; sr < kMaxWorld; ++sr)
#pragma unroll
            for (int u = 0; u < 2; ++u)
              if (sr < p.world && sr != p.rank && off[u] >= 0)
                v[sr][u] = *reinterpret_cast<const float4*>(p.rs_local_stage + sr * slot + off[u]);
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (off[u] < 0) continue;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sr = 0; sr < kMaxWorld; ++sr)
              if (sr < p.world && sr != p.rank) {
                acc.x += v[sr][u].x;
                acc.y += v[sr][u].y;
                acc.z += v[sr][u].z;
                acc.w += v[sr][u].w;
              }
            *reinterpret_cast<float4*>(sum_base + off[u]) = acc;
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ctid == 0) {
          __threadfence();
          red_add_release_sys(p.rs_local_ready + tix, 1);
        }
      }
    }
  }

  if (tr != nullptr && threadIdx.x == 6 * 32) tr[4] = globaltimer_ns();
  // ------------------------------------------------------------------ teardown
  if (CTA2) cluster_sync_all(); else __syncthreads();
  const int err = *s_abort;
  if (err != 0) {
    // (copies and UMMAs that were in flight have been waited for by the roles that issued them)
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile int*>(p.status) = err;
      __threadfence_system();
    }
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (CTA2) tmem_dealloc_2cta(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, int KIND, bool CTA2>
__global__ void __launch_bounds__(kThreads, 1)
fused_gemm_kernel(const __grid_constant__ GemmParams p, const uint32_t idesc) {
  fused_gemm_body<BN, STAGES, KIND, CTA2>(p, idesc, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}

// Several ranks' problems in ONE launch on one GPU: CTAs [r * ctas_per_rank, (r + 1) * ctas_per_rank) work on
// problem `ps[r]` exactly as a launch of their own would. Kernels of different ranks wait on one another's
// flags, so they can only share a GPU inside a single (cooperative) launch whose CTAs are all resident; this
// is how a single-GPU machine exercises the multi-rank protocol (pushes, counters, owner-side sums).
// `ps` lives in global memory (64-byte aligned: it holds tensor maps).
template <int BN, int STAGES, int KIND, bool CTA2>
__global__ void __launch_bounds__(kThreads, 1)
fused_gemm_ranks_kernel(const GemmParams* __restrict__ ps, const int ctas_per_rank, const uint32_t idesc) {
  const int r = static_cast<int>(blockIdx.x) / ctas_per_rank;
  fused_gemm_body<BN, STAGES, KIND, CTA2>(ps[r], idesc, static_cast<int>(blockIdx.x) - r * ctas_per_rank, ctas_per_rank);
}

}  // namespace fluxb
