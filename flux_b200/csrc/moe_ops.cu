// MoE grouped ops on top of the fused kernel's grouped mode.
//
// Layer 0 (all-gather + scatter + grouped GEMM) replaces
// src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc:227-447: the token
// shard is pushed to every peer by the kernel's comm warps, the routing tables
// (inverse permutation, per-expert M tiles, which source ranks a tile reads)
// are built on the device - no device-to-host copy or host scheduling per call
// (the reference does both, :323-363) - and the comm warps copy arriving tokens
// into an expert-sorted activation buffer that the GEMM reads with plain tiled
// loads. (The entry point without a workspace, at the end of this file, has no
// room for that buffer and fetches A rows by token index with TMA gather4.)
//
// Layer 1 (grouped GEMM + top-k gather + reduce-scatter) replaces
// src/moe_gather_rs/ths_op/gemm_grouped_v3_gather_rs.cc:595-820 in ONE launch,
// like the reference's threadblock-specialised kernel
// (src/moe_gather_rs/sm90_gemm_array_threadblock_specialized.hpp:1315-1514):
// the grouped GEMM writes a local [rows, N] buffer with the per-row /
// per-expert scales applied in the epilogue, column slab by column slab; as
// soon as a slab is complete the kernel's comm warps sum every token's top-k
// rows of it in fp32, push the rounded rows to the token's owner, and the
// owner's comm warps sum the per-source partials in fp32.
#include <string.h>

#include <mutex>
#include <vector>

#include "internal.h"

namespace fluxb {

struct MoeTables {
  GroupTile* tiles;
  int* num_tiles;
  int* expert_off;  // [E+1]
  int* tile_base;   // [E+1]
  int* gather;      // [max_rows]
  int* order;       // [max tiles] visiting order of the tiles
};

static constexpr size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// bytes of the tables carve_tables() lays out (the two must change together)
static constexpr size_t tables_bytes(long long max_rows, int nexperts) {
  size_t b = 0;
  b += align_up((max_rows / kBM + nexperts + 1) * sizeof(GroupTile), 256);
  b += 256;                                                 // num_tiles
  b += align_up((nexperts + 1) * sizeof(int), 256) * 2;     // expert_off, tile_base
  b += align_up(static_cast<size_t>(max_rows) * sizeof(int), 256);  // gather
  b += align_up((max_rows / kBM + nexperts + 1) * sizeof(int), 256);  // order
  return b;
}

static MoeTables carve_tables(void* ws, long long max_rows, int nexperts) {
  uint8_t* p = static_cast<uint8_t*>(ws);
  MoeTables t;
  t.tiles = reinterpret_cast<GroupTile*>(p);
  p += align_up((max_rows / kBM + nexperts + 1) * sizeof(GroupTile), 256);
  t.num_tiles = reinterpret_cast<int*>(p);
  p += 256;
  t.expert_off = reinterpret_cast<int*>(p);
  p += align_up((nexperts + 1) * sizeof(int), 256);
  t.tile_base = reinterpret_cast<int*>(p);
  p += align_up((nexperts + 1) * sizeof(int), 256);
  t.gather = reinterpret_cast<int*>(p);
  p += align_up(static_cast<size_t>(max_rows) * sizeof(int), 256);
  t.order = reinterpret_cast<int*>(p);
  return t;
}

// One block. Prefix sums over the experts, then each expert writes its tiles.
__global__ void __launch_bounds__(1024)
moe_build_tiles_kernel(const int* __restrict__ splits, int nexperts, int e_first, int e_count, int total_rows,
                       int max_tiles, int tile_m, MoeTables t, int* status) {
  // Experts [e_first, e_first + e_count) live on this rank (expert parallelism; all of them without it): only
  // they get tiles, and rows are numbered from the first row of that range (t.num_tiles[1], [2] = the range).
  __shared__ int ok;
  if (threadIdx.x == 0) {
    int off = 0, tb = 0;
    for (int e = 0; e < nexperts; ++e) {
      t.expert_off[e] = off;
      t.tile_base[e] = tb;
      const int n = splits[e] < 0 ? 0 : splits[e];
      off += n;
      if (e >= e_first && e < e_first + e_count) tb += (n + tile_m - 1) / tile_m;
    }
    t.expert_off[nexperts] = off;
    t.tile_base[nexperts] = tb;
    t.num_tiles[1] = t.expert_off[e_first];
    t.num_tiles[2] = t.expert_off[e_first + e_count];
    ok = (off == total_rows && tb <= max_tiles) ? 1 : 0;
    *t.num_tiles = ok ? tb : 0;
    if (!ok) {
      *reinterpret_cast<volatile int*>(status) = kStatusBadTable;
      __threadfence_system();
    }
  }
  __syncthreads();
  if (!ok) return;
  const int row_lo = t.num_tiles[1];
  for (int e = e_first + threadIdx.x; e < e_first + e_count; e += blockDim.x) {
    const int off = t.expert_off[e];
    const int n = t.expert_off[e + 1] - off;
    const int tb = t.tile_base[e];
    for (int c = 0; c * tile_m < n; ++c) {
      GroupTile g;
      g.a_row0 = off - row_lo + c * tile_m;
      g.rows = imin(tile_m, n - c * tile_m);
      g.expert = e - e_first;
      g.need_mask = 0;
      t.tiles[tb + c] = g;
    }
  }
}

// One thread per (token, k): inverse permutation and the source-rank mask of the row's tile.
// A "source block" is a run of `vblk` consecutive tokens of one rank (nvr blocks per rank): the unit in which the
// comm warps report tokens as permuted and in which a tile states what it reads (bit src_rank * nvr + block).
__global__ void moe_route_rows_kernel(const int* __restrict__ scatter_index, int total, int topk,
                                      int tokens_per_rank, int vblk, int nvr, int nexperts, int tile_m, MoeTables t) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total || *t.num_tiles == 0) return;
  const int row = scatter_index[i];
  if (row < t.num_tiles[1] || row >= t.num_tiles[2]) return;  // not a row of this rank's experts (or corrupt)
  const int token = i / topk;
  t.gather[row - t.num_tiles[1]] = token;
  int lo = 0, hi = nexperts;  // largest e with expert_off[e] <= row
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (t.expert_off[mid] <= row) lo = mid; else hi = mid;
  }
  const int tile = t.tile_base[lo] + (row - t.expert_off[lo]) / tile_m;
  const int src = token / tokens_per_rank;
  atomicOr(&t.tiles[tile].need_mask, 1 << (src * nvr + (token - src * tokens_per_rank) / vblk));
}

// Visiting order of the tiles: stable counting sort by how late the tile's last source block is permuted
// (this rank's own blocks first, then rank+1's, ...), so that early tiles need early data.
__global__ void moe_order_tiles_kernel(MoeTables t, int rank, int world, int nvr) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int n = *t.num_tiles;
  int count[33];
  for (int i = 0; i <= 32; ++i) count[i] = 0;
  auto key_of = [&](int mask) {
    int key = 0;
    for (int b = 0; b < world * nvr; ++b)
      if ((mask >> b) & 1) {
        int d = b / nvr - rank;
        if (d < 0) d += world;
        const int k = d * nvr + b % nvr;
        if (k > key) key = k;
      }
    return key;
  };
  for (int i = 0; i < n; ++i) count[key_of(t.tiles[i].need_mask) + 1] += 1;
  for (int i = 1; i <= 32; ++i) count[i] += count[i - 1];
  for (int i = 0; i < n; ++i) t.order[count[key_of(t.tiles[i].need_mask)]++] = i;
}

}  // namespace fluxb

using namespace fluxb;


// CTA pairs work on 256-row tiles of one expert: worth it once experts are tall on average.
static int grouped_cta_group(const fluxb_tuning* tuning, long long rows, int nexperts) {
  if (tuning != nullptr && (tuning->cta_group == 1 || tuning->cta_group == 2)) return tuning->cta_group;
  return rows / (nexperts > 0 ? nexperts : 1) >= 512 ? 2 : 1;
}

struct fluxb_moe_ag_scatter {
  fluxb_comm* comm;
  int max_ntokens, hidden, ffn_local, nexperts, topk, in_dtype, out_dtype;
  int flag_stride;
  uint8_t* gather[kMaxWorld];
  int* flags[kMaxWorld];
  void* workspace;
  unsigned long long calls;
  int last_parity;      // parity of the buffers the last push filled
  int last_ntokens;     // tokens gathered by the last push
  int ep_rank = 0, ep_size = 1;  // expert parallelism: this rank holds experts [ep_rank, ep_rank + 1) * nexperts / ep_size
  AgDma dma;
};

struct fluxb_moe_gather_rs {
  fluxb_comm* comm;
  int nexperts, max_m, n_dim, topk, in_dtype, out_dtype;
  void* stage[kMaxWorld];
  int* cnt[kMaxWorld];
  void* workspace;
  long long cnt_cap;
  unsigned long long calls;
  int ep_rank = 0, ep_size = 1;
};

static int flag_stride_of(int full_m, int world) {
  const int per_rank = (full_m + world - 1) / world;
  return ((per_rank + kBM - 1) / kBM) * kAgMaxGroups;  // same layout as the dense all-gather counters
}

extern "C" {

// ------------------------------------------------------------------ layer 0
// [routing tables][permute counters][expert-sorted activations: max_ntokens*topk rows of `hidden` elements]
size_t fluxb_moe_ag_scatter_workspace_bytes(int max_ntokens, int topk, int nexperts, int hidden, int in_dtype) {
  const long long rows = static_cast<long long>(max_ntokens) * topk;
  return tables_bytes(rows, nexperts) + 256 +
         align_up(static_cast<size_t>(rows + kBM) * hidden * dtype_bytes(in_dtype), 256);
}

int fluxb_moe_ag_scatter_create(fluxb_comm_t comm, int max_ntokens, int hidden, int ffn_local,
                                int nexperts, int topk, int in_dtype, int out_dtype,
                                void* const* gather_bufs, int* const* flag_bufs, void* workspace,
                                fluxb_moe_ag_scatter_t* out) {
  FLUXB_REQUIRE(comm != nullptr && out != nullptr && workspace != nullptr, "moe_ag_scatter_create: NULL argument");
  FLUXB_REQUIRE(gather_bufs != nullptr && flag_bufs != nullptr, "moe_ag_scatter_create: NULL buffer table");
  FLUXB_REQUIRE(is_16bit(in_dtype) || is_fp8(in_dtype), "moe_ag_scatter_create: input dtype %d unsupported", in_dtype);
  FLUXB_REQUIRE(out_dtype == FLUXB_BF16 || out_dtype == FLUXB_F16, "moe_ag_scatter_create: output dtype %d unsupported", out_dtype);
  FLUXB_REQUIRE(max_ntokens >= comm->world && max_ntokens % comm->world == 0,
                "moe_ag_scatter_create: max_ntokens=%d must be a positive multiple of world=%d", max_ntokens, comm->world);
  FLUXB_REQUIRE(nexperts >= 1 && nexperts <= 1024 && topk >= 1, "moe_ag_scatter_create: nexperts=%d topk=%d invalid", nexperts, topk);
  FLUXB_REQUIRE(ffn_local % 8 == 0 && ffn_local >= 8, "moe_ag_scatter_create: ffn_local=%d must be a multiple of 8", ffn_local);
  FLUXB_REQUIRE((static_cast<long long>(hidden) * dtype_bytes(in_dtype)) % 16 == 0,
                "moe_ag_scatter_create: hidden=%d gives a row pitch that is not a multiple of 16 bytes", hidden);
  fluxb_moe_ag_scatter* op = new fluxb_moe_ag_scatter();
  op->calls = 0;
  op->comm = comm;
  op->max_ntokens = max_ntokens;
  op->hidden = hidden;
  op->ffn_local = ffn_local;
  op->nexperts = nexperts;
  op->topk = topk;
  op->in_dtype = in_dtype;
  op->out_dtype = out_dtype;
  op->flag_stride = flag_stride_of(max_ntokens, comm->world);
  op->workspace = workspace;
  op->last_parity = -1;
  for (int r = 0; r < comm->world; ++r) {
    if (gather_bufs[r] == nullptr || flag_bufs[r] == nullptr) {
      delete op;
      FLUXB_FAIL(FLUXB_ERR_INVALID, "moe_ag_scatter_create: buffer of rank %d is NULL", r);
    }
    op->gather[r] = static_cast<uint8_t*>(gather_bufs[r]);
    op->flags[r] = flag_bufs[r];
  }
  if (comm->world > 1) {
    int rc = ag_dma_create(&op->dma, op->flag_stride);
    if (rc != FLUXB_OK) {
      ag_dma_destroy(&op->dma);
      delete op;
      return rc;
    }
  }
  *out = op;
  return FLUXB_OK;
}

int fluxb_moe_ag_scatter_destroy(fluxb_moe_ag_scatter_t op) {
  if (op != nullptr) ag_dma_destroy(&op->dma);
  delete op;
  return FLUXB_OK;
}

int fluxb_moe_ag_scatter_set_ep(fluxb_moe_ag_scatter_t op, int ep_rank, int ep_size) {
  FLUXB_REQUIRE(op != nullptr, "moe_ag_scatter_set_ep: op is NULL");
  FLUXB_REQUIRE(ep_size >= 1 && ep_rank >= 0 && ep_rank < ep_size && op->nexperts % ep_size == 0 &&
                    op->comm->world % ep_size == 0,
                "moe_ag_scatter_set_ep: ep_rank=%d ep_size=%d must divide nexperts=%d and world=%d", ep_rank, ep_size,
                op->nexperts, op->comm->world);
  op->ep_rank = ep_rank;
  op->ep_size = ep_size;
  return FLUXB_OK;
}

int fluxb_moe_ag_scatter_reset(fluxb_moe_ag_scatter_t op, fluxb_stream_t stream) {
  FLUXB_REQUIRE(op != nullptr, "moe_ag_scatter_reset: op is NULL");
  FLUXB_CUDA(cudaMemsetAsync(op->flags[op->comm->rank], 0, fluxb_ag_gemm_flag_bytes(op->max_ntokens, op->comm->world),
                             static_cast<cudaStream_t>(stream)));
  op->calls = 0;
  op->last_parity = -1;
  return FLUXB_OK;
}

// tokens_shard == NULL: reuse the tokens gathered by the previous call (further weight groups
// of the same layer, forward_multiple_weights in the reference).
int fluxb_moe_ag_scatter_forward(fluxb_moe_ag_scatter_t op, const void* tokens_shard,
                                 int ntokens_local, const void* weights, const int* splits_dev,
                                 const int* scatter_index_dev, const float* out_scale, void* out,
                                 void* gathered_out, const fluxb_tuning* tuning,
                                 fluxb_stream_t stream_) {
  FLUXB_REQUIRE(op != nullptr && weights != nullptr && splits_dev != nullptr && scatter_index_dev != nullptr &&
                    out != nullptr, "moe_ag_scatter_forward: NULL argument");
  fluxb_comm* comm = op->comm;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int world = comm->world;
  const long long ntokens = static_cast<long long>(ntokens_local) * world;
  FLUXB_REQUIRE(ntokens_local >= 1 && ntokens <= op->max_ntokens,
                "moe_ag_scatter_forward: ntokens_local=%d * world=%d exceeds max_ntokens=%d", ntokens_local, world, op->max_ntokens);
  const bool reuse = tokens_shard == nullptr;
  FLUXB_REQUIRE(!reuse || (op->last_parity >= 0 && op->last_ntokens == ntokens_local),
                "moe_ag_scatter_forward: no gathered tokens of this size to reuse");
  const int eb = dtype_bytes(op->in_dtype);
  const long long row_bytes = static_cast<long long>(op->hidden) * eb;
  const long long rows = ntokens * op->topk;
  const long long max_rows = static_cast<long long>(op->max_ntokens) * op->topk;
  const int max_tiles = static_cast<int>(max_rows / kBM + op->nexperts + 1);

  MoeTables tb = carve_tables(op->workspace, max_rows, op->nexperts);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.g_tiles = tb.tiles;
  const int cg = grouped_cta_group(tuning, rows, op->nexperts);
  const int tile_m = cg == 2 ? 2 * kBM : kBM;
  const int e_count = op->nexperts / op->ep_size, e_first = op->ep_rank * e_count;
  moe_build_tiles_kernel<<<1, 1024, 0, stream>>>(splits_dev, op->nexperts, e_first, e_count, static_cast<int>(rows),
                                                max_tiles, tile_m, tb, comm->status_dev);
  FLUXB_CUDA(cudaGetLastError());
  // source blocks of about 1024 tokens (whole 128-token chunks), at most 32 over all ranks: a 256-row tile of an
  // expert spans about that many tokens, so it can start when a fraction of a rank's tokens is in place
  // (only while all experts' weights fit in L2: visiting tiles block by block instead of expert by expert
  // re-streams every expert's weights once per block - measured at TP=1, 940 MB of weights: 1.85 ms against 1.58)
  int nvr = ntokens_local / 1024;
  if (nvr > 32 / world) nvr = 32 / world;
  if (static_cast<double>(e_count) * op->ffn_local * row_bytes > 64.0 * 1024 * 1024) nvr = 1;
  if (nvr < 1) nvr = 1;
  const int vblk = ((ntokens_local + nvr - 1) / nvr + kBM - 1) / kBM * kBM;
  nvr = (ntokens_local + vblk - 1) / vblk;
  moe_route_rows_kernel<<<static_cast<int>((rows + 255) / 256), 256, 0, stream>>>(
      scatter_index_dev, static_cast<int>(rows), op->topk, ntokens_local, vblk, nvr, op->nexperts, tile_m, tb);
  FLUXB_CUDA(cudaGetLastError());
  if (world * nvr > 1) {
    moe_order_tiles_kernel<<<1, 32, 0, stream>>>(tb, comm->rank, world, nvr);
    FLUXB_CUDA(cudaGetLastError());
    p.g_order = tb.order;
  }
  p.g_vblk = vblk;
  p.g_nvr = nvr;

  const size_t half_gather = (static_cast<size_t>(op->max_ntokens) + kBM) * op->hidden * eb;
  const size_t half_flags = static_cast<size_t>(world) * op->flag_stride;
  bool dma = false;
  int parity;
  if (reuse) {
    parity = op->last_parity;
  } else {
    parity = static_cast<int>(op->calls & 1ull);
    if (world > 1)
      FLUXB_CUDA(cudaMemsetAsync(op->flags[comm->rank] + (parity ^ 1) * half_flags, 0, half_flags * sizeof(int), stream));
  }

  p.out_type = op->out_dtype == FLUXB_BF16 ? kOutBf16 : kOutF16;
  p.M = static_cast<int>(rows);
  p.N = op->ffn_local;
  p.K = op->hidden;
  p.nseg = world;
  p.seg_rows = ntokens_local;
  p.seg_first = comm->rank;
  p.epi_mode = kEpiStore;
  p.out = out;
  p.ldo = op->ffn_local;
  p.alpha = 1.0f;
  p.g_tiles = tb.tiles;
  p.g_num_tiles = tb.num_tiles;
  p.g_gather = nullptr;  // permute form: A comes from the expert-sorted buffer with plain tiled loads
  p.g_rows_per_expert_b = op->ffn_local;
  p.g_expert_scale = out_scale;
  p.g_rows_per_rank = ntokens_local;
  p.g_ntokens = static_cast<int>(ntokens);
  p.g_topk = op->topk;
  p.g_scatter_index = scatter_index_dev;
  p.g_row_range = tb.num_tiles + 1;  // rows of this rank's experts (all rows without expert parallelism)
  p.ag_row_bytes = row_bytes;
  uint8_t* ws = static_cast<uint8_t*>(op->workspace);
  int* perm_done = reinterpret_cast<int*>(ws + tables_bytes(max_rows, op->nexperts));
  p.g_perm_done = perm_done;
  p.g_sorted = ws + tables_bytes(max_rows, op->nexperts) + 256;
  FLUXB_CUDA(cudaMemsetAsync(perm_done, 0, 256, stream));
  uint8_t* local_gather = op->gather[comm->rank] + parity * half_gather;
  if (world == 1 && !reuse) {
    p.g_tokens = static_cast<const uint8_t*>(tokens_shard);  // nothing to gather: permute straight from the caller's tokens
  } else {
    p.g_tokens = local_gather;
    // this rank's own tokens are permuted straight from the caller's tensor: no copy to itself on the critical path
    if (!reuse) p.g_tokens_own = static_cast<const uint8_t*>(tokens_shard);
  }
  if (world > 1 && !reuse) {
    p.ag_flags = op->flags[comm->rank] + parity * half_flags;
    p.ag_flag_stride = op->flag_stride;
    p.ag_groups = kAgMaxGroups;
    p.ag_spf = ag_slices_per_flag(row_bytes);
    p.ag_unit_rows = resolve_ag_unit_rows(tuning);
    p.ag_src = static_cast<const uint8_t*>(tokens_shard);
    for (int r = 0; r < world; ++r) {
      p.ag_dst[r] = op->gather[r] + parity * half_gather;
      p.ag_dst_flags[r] = op->flags[r] + parity * half_flags;
    }
    if (resolve_ag_mode(tuning) == kAgModeCopyEngine) {
      // the copy engines carry the tokens to the peers; the comm warps only permute what arrives
      dma = true;
      int rc2 = ag_dma_push(comm, &op->dma, tokens_shard, ntokens_local, row_bytes, p.ag_dst, p.ag_dst_flags, nullptr, nullptr,
                            false, stream);
      if (rc2 != FLUXB_OK) return rc2;
      p.ag_src = nullptr;
    }
  }
  const int bn = resolve_block_n(comm, p, tuning, max_tiles);
  int rc = encode_tmap_2d(&p.tmap_a, p.g_sorted, op->in_dtype, rows, op->hidden, row_bytes, kBM);
  if (rc != FLUXB_OK) return rc;
  rc = encode_tmap_2d(&p.tmap_b, weights, op->in_dtype, static_cast<long long>(e_count) * op->ffn_local,
                      op->hidden, row_bytes, cg == 2 ? bn / 2 : bn);
  if (rc != FLUXB_OK) return rc;
  // (with expert parallelism the caller's buffer may hold fewer rows than `rows`: no tiled stores then, since
  // the map's row bound is what clips a store)
  if (op->ep_size == 1) encode_out_map(p, out, rows, op->ffn_local, p.out_type);
  fluxb_tuning t = tuning != nullptr ? *tuning : fluxb_tuning{0, 0, 0, 0, 0};
  t.block_n = bn;
  t.cta_group = cg;
  rc = launch_fused_gemm(comm, p, op->in_dtype, &t, stream);
  if (rc != FLUXB_OK) return rc;
  if (dma) FLUXB_CUDA(cudaStreamWaitEvent(stream, op->dma.ev_done, 0));
  if (!reuse) {
    // keep a copy of the own tokens in the gather buffer (after the launch, off its critical path) so that
    // further weight groups and `gathered_out` find every rank's tokens there
    uint8_t* own_dst = op->gather[comm->rank] + parity * half_gather + static_cast<size_t>(comm->rank) * ntokens_local * row_bytes;
    const size_t own_bytes = static_cast<size_t>(ntokens_local) * row_bytes;
    rc = enqueue_or_defer(comm, stream, [=](cudaStream_t st) -> int {
      FLUXB_CUDA(cudaMemcpyAsync(own_dst, tokens_shard, own_bytes, cudaMemcpyDeviceToDevice, st));
      return FLUXB_OK;
    });
    if (rc != FLUXB_OK) return rc;
    op->last_parity = parity;
    op->last_ntokens = ntokens_local;
    op->calls += 1;
  }
  if (gathered_out != nullptr) {
    const uint8_t* src = op->gather[comm->rank] + parity * half_gather;
    const size_t bytes = static_cast<size_t>(ntokens) * row_bytes;
    return enqueue_or_defer(comm, stream, [=](cudaStream_t st) -> int {
      FLUXB_CUDA(cudaMemcpyAsync(gathered_out, src, bytes, cudaMemcpyDeviceToDevice, st));
      return FLUXB_OK;
    });
  }
  return FLUXB_OK;
}

// ------------------------------------------------------------------ layer 1
// [grouped GEMM output: max_m x n_dim, 16-bit][tile table][slab counters: one per 64 columns]
size_t fluxb_moe_gather_rs_workspace_bytes(int max_m, int n_dim, int topk, int nexperts) {
  (void)topk;
  return align_up(static_cast<size_t>(max_m) * n_dim * 2, 256) + tables_bytes(max_m, nexperts) +
         align_up(static_cast<size_t>((n_dim + 63) / 64) * sizeof(int), 256);
}
size_t fluxb_moe_gather_rs_stage_bytes(int max_m, int n_dim, int topk, int world) {
  (void)world;
  return 2ull * (static_cast<size_t>(max_m) / topk) * n_dim * 2;
}
// two parities x (column slabs of 64) x (blocks of 32 tokens per rank)
size_t fluxb_moe_gather_rs_cnt_bytes(int max_m, int n_dim, int topk, int world) {
  const long long tpr = (static_cast<long long>(max_m) / topk + world - 1) / world;
  return 2ull * ((n_dim + 63) / 64) * ((tpr + kGrTokBlock - 1) / kGrTokBlock) * sizeof(int);
}

int fluxb_moe_gather_rs_create(fluxb_comm_t comm, int nexperts, int max_m, int n_dim, int topk,
                               int in_dtype, int out_dtype, float* const* stage_bufs,
                               int* const* cnt_bufs, void* workspace, fluxb_moe_gather_rs_t* out) {
  FLUXB_REQUIRE(comm != nullptr && out != nullptr && workspace != nullptr, "moe_gather_rs_create: NULL argument");
  FLUXB_REQUIRE(stage_bufs != nullptr && cnt_bufs != nullptr, "moe_gather_rs_create: NULL buffer table");
  FLUXB_REQUIRE(is_16bit(in_dtype) || is_fp8(in_dtype), "moe_gather_rs_create: input dtype %d unsupported", in_dtype);
  FLUXB_REQUIRE(out_dtype == FLUXB_BF16 || out_dtype == FLUXB_F16, "moe_gather_rs_create: output dtype %d unsupported", out_dtype);
  FLUXB_REQUIRE(nexperts >= 1 && nexperts <= 1024 && topk >= 1, "moe_gather_rs_create: nexperts=%d topk=%d invalid", nexperts, topk);
  // max_m % (topk * world) == 0 (src/moe_gather_rs/ths_op/gemm_grouped_v3_gather_rs.cc:580-581)
  FLUXB_REQUIRE(max_m >= topk * comm->world && max_m % (topk * comm->world) == 0,
                "moe_gather_rs_create: max_m=%d must be a positive multiple of topk*world=%d", max_m, topk * comm->world);
  FLUXB_REQUIRE(n_dim >= 8 && n_dim % 8 == 0, "moe_gather_rs_create: n_dim=%d must be a multiple of 8", n_dim);
  fluxb_moe_gather_rs* op = new fluxb_moe_gather_rs();
  op->calls = 0;
  op->comm = comm;
  op->nexperts = nexperts;
  op->max_m = max_m;
  op->n_dim = n_dim;
  op->topk = topk;
  op->in_dtype = in_dtype;
  op->out_dtype = out_dtype;
  op->workspace = workspace;
  op->cnt_cap = static_cast<long long>(fluxb_moe_gather_rs_cnt_bytes(max_m, n_dim, topk, comm->world) / (2 * sizeof(int)));
  for (int r = 0; r < comm->world; ++r) {
    if (stage_bufs[r] == nullptr || cnt_bufs[r] == nullptr) {
      delete op;
      FLUXB_FAIL(FLUXB_ERR_INVALID, "moe_gather_rs_create: buffer of rank %d is NULL", r);
    }
    op->stage[r] = stage_bufs[r];
    op->cnt[r] = cnt_bufs[r];
  }
  *out = op;
  return FLUXB_OK;
}

int fluxb_moe_gather_rs_destroy(fluxb_moe_gather_rs_t op) {
  delete op;
  return FLUXB_OK;
}

int fluxb_moe_gather_rs_set_ep(fluxb_moe_gather_rs_t op, int ep_rank, int ep_size) {
  FLUXB_REQUIRE(op != nullptr, "moe_gather_rs_set_ep: op is NULL");
  FLUXB_REQUIRE(ep_size >= 1 && ep_rank >= 0 && ep_rank < ep_size && op->nexperts % ep_size == 0 &&
                    op->comm->world % ep_size == 0,
                "moe_gather_rs_set_ep: ep_rank=%d ep_size=%d must divide nexperts=%d and world=%d", ep_rank, ep_size,
                op->nexperts, op->comm->world);
  op->ep_rank = ep_rank;
  op->ep_size = ep_size;
  return FLUXB_OK;
}

int fluxb_moe_gather_rs_reset(fluxb_moe_gather_rs_t op, fluxb_stream_t stream) {
  FLUXB_REQUIRE(op != nullptr, "moe_gather_rs_reset: op is NULL");
  FLUXB_CUDA(cudaMemsetAsync(op->cnt[op->comm->rank], 0, fluxb_moe_gather_rs_cnt_bytes(op->max_m, op->n_dim, op->topk, op->comm->world),
                             static_cast<cudaStream_t>(stream)));
  op->calls = 0;
  return FLUXB_OK;
}

int fluxb_moe_gather_rs_forward(fluxb_moe_gather_rs_t op, const void* x, int m, int k_local,
                                const void* weights, const int* splits_host,
                                const int* routing_idx_dev, const float* in_scale,
                                const float* w_scale, const float* vec_scale, void* out,
                                const fluxb_tuning* tuning, fluxb_stream_t stream_) {
  FLUXB_REQUIRE(op != nullptr, "moe_gather_rs_forward: NULL argument");
  FLUXB_REQUIRE(op->ep_size == 1, "moe_gather_rs_forward: with expert parallelism call fluxb_moe_gather_rs_forward_ep");
  return fluxb_moe_gather_rs_forward_ep(op, x, m, m / op->topk, k_local, weights, splits_host, routing_idx_dev, in_scale,
                                        w_scale, vec_scale, out, tuning, stream_);
}

int fluxb_moe_gather_rs_forward_ep(fluxb_moe_gather_rs_t op, const void* x, int m, int ntokens, int k_local,
                                   const void* weights, const int* splits_host,
                                   const int* routing_idx_dev, const float* in_scale,
                                   const float* w_scale, const float* vec_scale, void* out,
                                   const fluxb_tuning* tuning, fluxb_stream_t stream_) {
  FLUXB_REQUIRE(op != nullptr && x != nullptr && weights != nullptr && splits_host != nullptr &&
                    routing_idx_dev != nullptr && out != nullptr, "moe_gather_rs_forward: NULL argument");
  fluxb_comm* comm = op->comm;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int world = comm->world;
  const int topk = op->topk;
  const int n = op->n_dim;
  const long long rows_all = static_cast<long long>(ntokens) * topk;
  FLUXB_REQUIRE(ntokens >= world && rows_all <= op->max_m && ntokens % world == 0,
                "moe_gather_rs_forward: ntokens=%d must be a multiple of world=%d with ntokens*topk within max_m=%d",
                ntokens, world, op->max_m);
  FLUXB_REQUIRE(m >= 0 && m <= rows_all && (op->ep_size > 1 || m == rows_all),
                "moe_gather_rs_forward: m=%d rows for %d tokens x top-%d", m, ntokens, topk);
  const int eb = dtype_bytes(op->in_dtype);
  FLUXB_REQUIRE(k_local >= 8 && (static_cast<long long>(k_local) * eb) % 16 == 0,
                "moe_gather_rs_forward: k_local=%d gives a row pitch that is not a multiple of 16 bytes", k_local);
  const int tpr = ntokens / world;
  // expert parallelism: this rank computes the rows of experts [e_first, e_first + e_count), which are rows
  // [row_lo, row_lo + m) of the expert-sorted order; `x`, the row scales and the tiles count from row_lo
  const int e_count = op->nexperts / op->ep_size, e_first = op->ep_rank * e_count;

  // tile table from the host-side splits (the reference also packs its problem list on the host
  // and uploads it, gemm_grouped_v3_gather_rs.cc:245-416)
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int cg = grouped_cta_group(tuning, m, e_count);
  const int tile_m = cg == 2 ? 2 * kBM : kBM;
  std::vector<GroupTile> tiles;
  long long off = 0, row_lo = 0;
  for (int e = 0; e < op->nexperts; ++e) {
    const int cnt = splits_host[e];
    FLUXB_REQUIRE(cnt >= 0, "moe_gather_rs_forward: splits[%d]=%d is negative", e, cnt);
    if (e == e_first) row_lo = off;
    if (e >= e_first && e < e_first + e_count)
      for (int c = 0; c * tile_m < cnt; ++c) {
        GroupTile g;
        g.a_row0 = static_cast<int>(off - row_lo) + c * tile_m;
        g.rows = cnt - c * tile_m < tile_m ? cnt - c * tile_m : tile_m;
        g.expert = e - e_first;
        g.need_mask = 0;
        tiles.push_back(g);
      }
    off += cnt;
    if (e == e_first + e_count - 1)
      FLUXB_REQUIRE(off - row_lo == m, "moe_gather_rs_forward: the splits of this rank's experts sum to %lld, expected m=%d",
                    off - row_lo, m);
  }
  FLUXB_REQUIRE(off == rows_all, "moe_gather_rs_forward: splits sum to %lld, expected ntokens*topk=%lld", off, rows_all);
  uint8_t* ws = static_cast<uint8_t*>(op->workspace);
  void* inter = ws;
  MoeTables tb = carve_tables(ws + align_up(static_cast<size_t>(op->max_m) * n * 2, 256), op->max_m, op->nexperts);
  const int num_tiles = static_cast<int>(tiles.size());
  FLUXB_CUDA(cudaMemcpyAsync(tb.tiles, tiles.data(), tiles.size() * sizeof(GroupTile), cudaMemcpyHostToDevice, stream));
  FLUXB_CUDA(cudaMemcpyAsync(tb.num_tiles, &num_tiles, sizeof(int), cudaMemcpyHostToDevice, stream));

  p.out_type = op->out_dtype == FLUXB_BF16 ? kOutBf16 : kOutF16;
  p.M = m > 0 ? m : 1;
  p.N = n;
  p.K = k_local;
  p.nseg = 1;
  p.seg_rows = p.M;
  p.epi_mode = kEpiStore;
  p.out = inter;
  p.ldo = n;
  p.alpha = 1.0f;
  // scales follow python/flux/testing/moe_gather_rs_utils.py:76-79,99: weight_scale[e] * input_scale, then the row vector
  // (each scale applies on its own; a missing one counts as 1)
  p.alpha_ptr = in_scale;
  p.g_expert_scale = w_scale;
  p.scale_a = vec_scale;
  p.g_tiles = tb.tiles;
  p.g_num_tiles = tb.num_tiles;
  p.g_gather = nullptr;
  p.g_rows_per_expert_b = n;
  const long long row_bytes = static_cast<long long>(k_local) * eb;
  const int bn = resolve_block_n(comm, p, tuning, num_tiles > 0 ? num_tiles : 1);
  int rc = encode_tmap_2d(&p.tmap_a, x, op->in_dtype, p.M, k_local, row_bytes, kBM);
  if (rc != FLUXB_OK) return rc;
  rc = encode_tmap_2d(&p.tmap_b, weights, op->in_dtype, static_cast<long long>(e_count) * n, k_local, row_bytes,
                      cg == 2 ? bn / 2 : bn);
  if (rc != FLUXB_OK) return rc;
  encode_out_map(p, inter, p.M, n, p.out_type);
  // combine + reduce-scatter run inside the same launch (comm warps), column slab by column slab
  const int parity = static_cast<int>(op->calls & 1ull);
  const size_t half_stage_elems = (static_cast<size_t>(op->max_m) / topk) * n;
  const int n_tiles = (n + bn - 1) / bn;
  const int bpo = (tpr + kGrTokBlock - 1) / kGrTokBlock;
  FLUXB_REQUIRE(static_cast<long long>(n_tiles) * bpo <= op->cnt_cap, "moe_gather_rs_forward: counter buffer too small");
  int* slab_done = reinterpret_cast<int*>(ws + align_up(static_cast<size_t>(op->max_m) * n * 2, 256) +
                                          tables_bytes(op->max_m, op->nexperts));
  FLUXB_CUDA(cudaMemsetAsync(slab_done, 0, static_cast<size_t>(n_tiles) * sizeof(int), stream));
  // The other parity's counters were consumed by the previous call and are next written by peers only after
  // they have seen this call's pushes: clear them now.
  FLUXB_CUDA(cudaMemsetAsync(op->cnt[comm->rank] + (parity ^ 1) * op->cnt_cap, 0, op->cnt_cap * sizeof(int), stream));
  p.gr_slab_done = slab_done;
  p.gr_slab_expected = num_tiles * (cg == 2 ? 2 : 1) * 4;
  p.gr_scatter_index = routing_idx_dev;
  p.gr_row_lo = static_cast<int>(row_lo);
  p.gr_rows = m;
  p.gr_topk = topk;
  p.gr_tokens_per_rank = tpr;
  for (int r = 0; r < world; ++r) {
    p.gr_stage[r] = static_cast<uint8_t*>(op->stage[r]) +
                    (parity * half_stage_elems + static_cast<size_t>(comm->rank) * tpr * n) * 2;
    p.gr_cnt[r] = op->cnt[r] + parity * op->cnt_cap;
  }
  p.gr_local_stage = static_cast<uint8_t*>(op->stage[comm->rank]) + parity * half_stage_elems * 2;
  p.gr_local_cnt = op->cnt[comm->rank] + parity * op->cnt_cap;
  p.gr_out = out;
  // Tile order. If the activations fit in L2 with room to spare, one rasterisation band over all M tiles:
  // the output is produced slab by slab and the combine + reduce-scatter of slab s overlaps the GEMM of slab
  // s+1 (A is re-read once per slab, from L2). Otherwise the usual bands of 8 M tiles (A streams from HBM
  // once); the slabs then complete together at the end and the combine follows the GEMM inside the launch.
  const bool slab_order = static_cast<double>(p.M) * k_local * eb <= 64.0 * 1024 * 1024;
  fluxb_tuning t = tuning != nullptr ? *tuning : fluxb_tuning{0, 0, 0, 0, 0};
  t.block_n = bn;
  t.cta_group = cg;
  if (slab_order) {
    p.group_m = 1 << 20;
    t.group_m = p.group_m;
  } else {
    // Column groups: A streams once per group (there is bandwidth to spare next to a tensor-bound GEMM) and the
    // combine of a group overlaps the GEMM of the next one; only the last group's combine is exposed. Measured
    // at config X: with A = 117 MB (TP=4) eight groups beat four (0.516 vs 0.537 ms; 2 and 16: 0.587, 0.55); with
    // A = 470 MB (TP=1) four beat eight (1.68 vs 1.75 ms).
    const int groups = static_cast<double>(p.M) * k_local * eb <= 128.0 * 1024 * 1024 ? 8 : 4;
    p.n_group = (n_tiles + groups - 1) / groups;
  }
  rc = launch_fused_gemm(comm, p, op->in_dtype, &t, stream);
  if (rc != FLUXB_OK) return rc;
  op->calls += 1;
  return FLUXB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Scatter + grouped GEMM without any allocation: the routing tables live in a
// fixed device array of this translation unit instead of a caller workspace.
// ---------------------------------------------------------------------------
namespace fluxb {

// table bytes for FLUXB_STATIC_MAX_ROWS routed rows and FLUXB_STATIC_MAX_EXPERTS experts, from the same
// function that sizes the caller-provided workspace
constexpr size_t kStaticTableBytes = tables_bytes(FLUXB_STATIC_MAX_ROWS, FLUXB_STATIC_MAX_EXPERTS);
static_assert(kStaticTableBytes < (1u << 20), "the built-in routing tables are meant to stay modest");

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_tables[kStaticTableBytes];

// Device address of the array on the current device, looked up once per device.
static int static_tables_ptr(int device, void** out) {
  static void* ptrs[64] = {};
  static std::mutex mu;  // first calls on a device may come from several host threads
  FLUXB_REQUIRE(device >= 0 && device < 64, "device index %d not supported", device);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[device] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_tables);
    if (e != cudaSuccess || ptr == nullptr)
      FLUXB_FAIL(FLUXB_ERR_CUDA, "cudaGetSymbolAddress(routing tables) failed: %s", cudaGetErrorString(e));
    ptrs[device] = ptr;
  }
  *out = ptrs[device];
  return FLUXB_OK;
}

}  // namespace fluxb

extern "C" int fluxb_moe_scatter_gemm_static(fluxb_comm_t comm, const void* tokens, int ntokens, int hidden,
                                             const void* weights, int nexperts, int ffn, int topk,
                                             const int* splits_dev, const int* scatter_index_dev,
                                             const float* out_scale, void* out, int in_dtype, int out_dtype,
                                             const fluxb_tuning* tuning, fluxb_stream_t stream_) {
  FLUXB_REQUIRE(comm != nullptr && tokens != nullptr && weights != nullptr && splits_dev != nullptr &&
                    scatter_index_dev != nullptr && out != nullptr, "moe_scatter_gemm_static: NULL argument");
  FLUXB_REQUIRE(comm->world == 1, "moe_scatter_gemm_static: needs a world-1 communicator (got world=%d)", comm->world);
  FLUXB_REQUIRE(is_16bit(in_dtype) || is_fp8(in_dtype), "moe_scatter_gemm_static: input dtype %d unsupported", in_dtype);
  FLUXB_REQUIRE(out_dtype == FLUXB_BF16 || out_dtype == FLUXB_F16, "moe_scatter_gemm_static: output dtype %d unsupported", out_dtype);
  FLUXB_REQUIRE(ntokens >= 1 && topk >= 1 && nexperts >= 1, "moe_scatter_gemm_static: ntokens=%d topk=%d nexperts=%d invalid",
                ntokens, topk, nexperts);
  const long long rows = static_cast<long long>(ntokens) * topk;
  FLUXB_REQUIRE(rows <= FLUXB_STATIC_MAX_ROWS,
                "moe_scatter_gemm_static: ntokens*topk = %lld exceeds the built-in table capacity of %d rows; "
                "use fluxb_moe_ag_scatter_forward with a workspace", rows, FLUXB_STATIC_MAX_ROWS);
  FLUXB_REQUIRE(nexperts <= FLUXB_STATIC_MAX_EXPERTS,
                "moe_scatter_gemm_static: nexperts = %d exceeds the built-in table capacity of %d experts", nexperts,
                FLUXB_STATIC_MAX_EXPERTS);
  FLUXB_REQUIRE(ffn >= 8 && ffn % 8 == 0, "moe_scatter_gemm_static: ffn=%d must be a multiple of 8", ffn);
  const int eb = dtype_bytes(in_dtype);
  const long long row_bytes = static_cast<long long>(hidden) * eb;
  FLUXB_REQUIRE(hidden >= 1 && row_bytes % 16 == 0,
                "moe_scatter_gemm_static: hidden=%d gives a row pitch that is not a multiple of 16 bytes", hidden);
  int dev = -1;
  FLUXB_CUDA(cudaGetDevice(&dev));
  FLUXB_REQUIRE(dev == comm->device, "moe_scatter_gemm_static: device %d is current, the communicator lives on %d", dev,
                comm->device);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  void* tables = nullptr;
  int rc = static_tables_ptr(dev, &tables);
  if (rc != FLUXB_OK) return rc;

  // same table layout as the workspace form, sized for the built-in capacity
  MoeTables tb = carve_tables(tables, FLUXB_STATIC_MAX_ROWS, FLUXB_STATIC_MAX_EXPERTS);
  const int max_tiles = FLUXB_STATIC_MAX_ROWS / kBM + FLUXB_STATIC_MAX_EXPERTS + 1;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.g_tiles = tb.tiles;
  const int cg = resolve_cta_group(p, tuning);
  const int tile_m = cg == 2 ? 2 * kBM : kBM;
  // every table entry a later stage reads is written here first: tile list, tile count, offsets and
  // the source-rank masks by the first kernel, the gather index of all `rows` rows by the second
  moe_build_tiles_kernel<<<1, 1024, 0, stream>>>(splits_dev, nexperts, 0, nexperts, static_cast<int>(rows), max_tiles,
                                                tile_m, tb, comm->status_dev);
  FLUXB_CUDA(cudaGetLastError());
  moe_route_rows_kernel<<<static_cast<int>((rows + 255) / 256), 256, 0, stream>>>(
      scatter_index_dev, static_cast<int>(rows), topk, ntokens, ntokens, 1, nexperts, tile_m, tb);
  FLUXB_CUDA(cudaGetLastError());

  p.out_type = out_dtype == FLUXB_BF16 ? kOutBf16 : kOutF16;
  p.M = static_cast<int>(rows);
  p.N = ffn;
  p.K = hidden;
  p.nseg = 1;
  p.seg_rows = ntokens;
  p.epi_mode = kEpiStore;
  p.out = out;
  p.ldo = ffn;
  p.alpha = 1.0f;
  p.g_num_tiles = tb.num_tiles;
  p.g_gather = tb.gather;
  p.g_rows_per_expert_b = ffn;
  p.g_expert_scale = out_scale;
  p.g_rows_per_rank = ntokens;
  p.g_ntokens = ntokens;
  const int bn = resolve_block_n(comm, p, tuning, max_tiles);
  rc = encode_tmap_2d(&p.tmap_a, tokens, in_dtype, ntokens, hidden, row_bytes, 1);
  if (rc != FLUXB_OK) return rc;
  rc = encode_tmap_2d(&p.tmap_b, weights, in_dtype, static_cast<long long>(nexperts) * ffn, hidden, row_bytes,
                      cg == 2 ? bn / 2 : bn);
  if (rc != FLUXB_OK) return rc;
  fluxb_tuning t = tuning != nullptr ? *tuning : fluxb_tuning{0, 0, 0, 0, 0};
  t.block_n = bn;
  t.cta_group = cg;
  return launch_fused_gemm(comm, p, in_dtype, &t, stream);
}
