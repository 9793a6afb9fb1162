// Host side of the dense ops: the launcher of the fused kernel, the plain
// GEMM entry point, AG-GEMM and GEMM-RS (with the owner-side fp32 reduction).
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "internal.h"

namespace fluxb {

// ---------------------------------------------------------------------------
// launcher
// ---------------------------------------------------------------------------
template <int BN, int STAGES, int KIND, bool CTA2>
static int launch_inst(const fluxb_comm* comm, const GemmParams& p, uint32_t idesc, int grid, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES, CTA2>;
  auto kern = fused_gemm_kernel<BN, STAGES, KIND, CTA2>;
  static bool configured[64] = {};
  static int max_clusters[64] = {};
  int dev = 0;
  FLUXB_CUDA(cudaGetDevice(&dev));
  FLUXB_REQUIRE(dev < 64, "device index %d not supported", dev);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTA2 ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!configured[dev]) {
    FLUXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    if (CTA2) {
      // how many CTA pairs can be resident at once: the persistent grid must not exceed it
      cfg.gridDim = dim3(comm->sm_count & ~1, 1, 1);
      int n = 0;
      FLUXB_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
      FLUXB_REQUIRE(n >= 1, "no CTA pair of the fused kernel fits on this device");
      max_clusters[dev] = n;
    }
    configured[dev] = true;
  }
  if (CTA2) {
    grid &= ~1;
    if (grid > 2 * max_clusters[dev]) grid = 2 * max_clusters[dev];
    if (grid < 2) grid = 2;
  }
  cfg.gridDim = dim3(grid, 1, 1);
  FLUXB_CUDA(cudaLaunchKernelEx(&cfg, kern, p, idesc));
  return FLUXB_OK;
}

static int pick_block_n(long long m_tiles, int n, int ctas, int per_cta_div, bool need_box64) {
  // cost = waves * tile width, with a small penalty for narrow tiles (more
  // operand traffic per flop); the candidate with the lowest cost wins.
  const int cand[4] = {256, 192, 128, 64};
  const double pen[4] = {1.00, 1.15, 1.12, 1.30};  // measured: 192-wide tiles run ~12 % below 256-wide ones
  int best = 256;
  double best_cost = 1e30;
  for (int i = 0; i < 4; ++i) {
    const int bn = cand[i];
    if (bn > 64 && n <= bn / 2) continue;
    // a [K,N] weight is loaded in 64-column boxes: each CTA's share of the tile must be whole boxes
    if (need_box64 && ((bn / per_cta_div) % 64 != 0)) continue;
    const long long tiles = m_tiles * ((n + bn - 1) / bn);
    const long long waves = (tiles + ctas - 1) / ctas;
    const double cost = static_cast<double>(waves) * bn * pen[i];
    if (cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

int ag_slices_per_flag(long long row_bytes) {
  const long long nslices = (row_bytes + kCommSliceBytes - 1) / kCommSliceBytes;
  const long long spf = (nslices + kAgMaxGroups - 1) / kAgMaxGroups;
  return spf < 1 ? 1 : static_cast<int>(spf);
}

// Transport when the caller's tuning names none: the environment variable FLUXB_AG_MODE (1 or 2), else the
// kernel's own push.
static int default_ag_mode() {
  const char* e = getenv("FLUXB_AG_MODE");
  return (e != nullptr && atoi(e) == kAgModeCopyEngine) ? kAgModeCopyEngine : kAgModeKernelPush;
}

int resolve_ag_mode(const fluxb_tuning* tuning) {
  if (tuning != nullptr && tuning->ag_mode == kAgModeCopyEngine) return kAgModeCopyEngine;
  if (tuning != nullptr && tuning->ag_mode != 0) return kAgModeKernelPush;
  return default_ag_mode();
}

int resolve_ag_unit_rows(const fluxb_tuning* tuning) {
  if (resolve_ag_mode(tuning) == kAgModeCopyEngine) return kBM;  // a copied piece arrives whole
  if (tuning != nullptr && tuning->ag_mode == 3) return 64;
  if (tuning != nullptr && tuning->ag_mode == 4) return 128;
  return 32;
}

int ag_dma_create(AgDma* d, int flag_stride) {
  int lo = 0, hi = 0;
  FLUXB_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  FLUXB_CUDA(cudaStreamCreateWithPriority(&d->side, cudaStreamNonBlocking, hi));
  FLUXB_CUDA(cudaEventCreateWithFlags(&d->ev_start, cudaEventDisableTiming));
  FLUXB_CUDA(cudaEventCreateWithFlags(&d->ev_done, cudaEventDisableTiming));
  FLUXB_CUDA(cudaMalloc(reinterpret_cast<void**>(&d->expected_dev), static_cast<size_t>(flag_stride) * sizeof(int)));
  d->flag_stride = flag_stride;
  d->expected_row_bytes = -1;
  return FLUXB_OK;
}

void ag_dma_destroy(AgDma* d) {
  if (d->side != nullptr) cudaStreamDestroy(d->side);
  if (d->ev_start != nullptr) cudaEventDestroy(d->ev_start);
  if (d->ev_done != nullptr) cudaEventDestroy(d->ev_done);
  if (d->expected_dev != nullptr) cudaFree(d->expected_dev);
  *d = AgDma();
}

int ag_dma_push(const fluxb_comm* comm, AgDma* d, const void* src, int m_local, long long row_bytes,
                uint8_t* const* gather, int* const* flags, const float* src_scale, float* const* dst_scale,
                bool include_self, cudaStream_t main) {
  const int world = comm->world, rank = comm->rank;
  constexpr int kUnitsPerSlice = 1;  // counter value of a complete (chunk, slice): the consumer is told 128-row units
  if (d->expected_row_bytes != row_bytes) {
    // counter values of a complete shard: every used slice group of every chunk holds its unit count
    const int nslices = static_cast<int>((row_bytes + kCommSliceBytes - 1) / kCommSliceBytes);
    const int spf = ag_slices_per_flag(row_bytes);
    std::vector<int> v(static_cast<size_t>(d->flag_stride), 0);
    for (int i = 0; i < d->flag_stride; ++i) {
      const int g = i % kAgMaxGroups;
      const int left = nslices - g * spf;
      if (left > 0) v[i] = kUnitsPerSlice * (left < spf ? left : spf);
    }
    FLUXB_CUDA(cudaMemcpy(d->expected_dev, v.data(), v.size() * sizeof(int), cudaMemcpyHostToDevice));
    d->expected_row_bytes = row_bytes;
  }
  FLUXB_CUDA(cudaEventRecord(d->ev_start, main));
  FLUXB_CUDA(cudaStreamWaitEvent(d->side, d->ev_start, 0));
  // One copy per 1024 rows: a peer-to-peer cudaMemcpyAsync costs the host ~20 us, so pieces of 256 rows made a
  // launch at TP=8 host-bound (28 copies: ten launches in a row took 0.6 ms each, a single one 0.47 ms), and the
  // tiles of a peer's shard are not due before this rank's own shard is worked off anyway.
  const int piece = 8 * kBM;
  for (int dd = include_self ? 0 : 1; dd < world; ++dd) {
    const int dest = (rank - dd + world) % world;
    for (int r0 = 0; r0 < m_local; r0 += piece) {
      const int rows = m_local - r0 < piece ? m_local - r0 : piece;
      const size_t row_off = static_cast<size_t>(rank) * m_local + r0;
      FLUXB_CUDA(cudaMemcpyAsync(gather[dest] + row_off * row_bytes, static_cast<const uint8_t*>(src) + static_cast<size_t>(r0) * row_bytes,
                                 static_cast<size_t>(rows) * row_bytes, cudaMemcpyDeviceToDevice, d->side));
      if (src_scale != nullptr)
        FLUXB_CUDA(cudaMemcpyAsync(dst_scale[dest] + row_off, src_scale + r0, static_cast<size_t>(rows) * sizeof(float),
                                   cudaMemcpyDeviceToDevice, d->side));
      // the piece's chunks are complete: publish their counters (stream order puts this after the data)
      const int c0 = r0 / kBM, c1 = (r0 + rows + kBM - 1) / kBM;
      FLUXB_CUDA(cudaMemcpyAsync(flags[dest] + static_cast<size_t>(rank) * d->flag_stride + static_cast<size_t>(c0) * kAgMaxGroups,
                                 d->expected_dev + static_cast<size_t>(c0) * kAgMaxGroups,
                                 static_cast<size_t>(c1 - c0) * kAgMaxGroups * sizeof(int), cudaMemcpyDeviceToDevice, d->side));
    }
  }
  FLUXB_CUDA(cudaEventRecord(d->ev_done, d->side));
  return FLUXB_OK;
}

int resolve_cta_group(const GemmParams& p, const fluxb_tuning* tuning) {
  if (tuning != nullptr && (tuning->cta_group == 1 || tuning->cta_group == 2)) return tuning->cta_group;
  if (p.g_tiles != nullptr) return 1;
  // a CTA pair works on 256 rows of one segment: worth it once segments are at least that tall
  return p.seg_rows >= 256 ? 2 : 1;
}

int resolve_block_n(const fluxb_comm* comm, const GemmParams& p, const fluxb_tuning* tuning,
                    long long m_tiles_hint) {
  int bn = (tuning != nullptr) ? tuning->block_n : 0;
  if (bn == 0) {
    const int cg = resolve_cta_group(p, tuning);
    const int tile_m = cg == 2 ? 2 * kBM : kBM;
    long long m_tiles = m_tiles_hint;
    if (m_tiles <= 0) m_tiles = static_cast<long long>(p.nseg) * ((p.seg_rows + tile_m - 1) / tile_m);
    int share = comm->ranks_on_gpu > 1 ? ((comm->sm_count / comm->ranks_on_gpu) & ~1) : comm->sm_count;
    int ctas = (tuning != nullptr && tuning->num_ctas > 0 && tuning->num_ctas < share) ? tuning->num_ctas : share;
    bn = pick_block_n(m_tiles, p.N, cg == 2 ? ctas / 2 : ctas, cg == 2 ? 2 : 1, p.b_mn_major != 0);
  }
  return bn;
}

int enqueue_or_defer(fluxb_comm* comm, cudaStream_t stream, std::function<int(cudaStream_t)> fn) {
  if (comm->ranks_on_gpu <= 1) return fn(stream);
  DeferredItem it;
  it.fused = false;
  it.plain = std::move(fn);
  comm->deferred.push_back(std::move(it));
  return FLUXB_OK;
}

int launch_fused_gemm(fluxb_comm* comm, GemmParams& p, int in_dtype,
                      const fluxb_tuning* tuning, cudaStream_t stream) {
  const int cg = resolve_cta_group(p, tuning);
  const int bn = resolve_block_n(comm, p, tuning, p.g_tiles != nullptr ? 1024 : 0);
  FLUXB_REQUIRE(bn == 64 || bn == 128 || bn == 192 || bn == 256, "block_n=%d not in {64,128,192,256}", bn);
  FLUXB_REQUIRE(!p.b_mn_major || (bn / (cg == 2 ? 2 : 1)) % 64 == 0,
                "a [K,N] weight needs a tile width whose per-CTA share is a multiple of 64 (block_n=%d, cta_group=%d)", bn, cg);
  int grid = comm->sm_count;
  if (comm->ranks_on_gpu > 1) grid = (grid / comm->ranks_on_gpu) & ~1;  // this rank's share of the GPU
  if (tuning != nullptr && tuning->num_ctas > 0) grid = tuning->num_ctas < grid ? tuning->num_ctas : grid;
  if (p.g_tiles == nullptr) {
    const int tile_m = cg == 2 ? 2 * kBM : kBM;
    const long long tiles = static_cast<long long>(p.nseg) * ((p.seg_rows + tile_m - 1) / tile_m) *
                            ((p.N + bn - 1) / bn) * (cg == 2 ? 2 : 1);
    // the all-gather push is spread over every CTA's comm warps, so keep the full grid there
    if (p.ag_src == nullptr && tiles < grid) grid = static_cast<int>(tiles);
  }
  if (grid < 1) grid = 1;
  if (p.group_m <= 0) p.group_m = (tuning != nullptr && tuning->group_m > 0) ? tuning->group_m : 8;
  if (p.ag_spf <= 0) p.ag_spf = 1;
  if (p.ag_groups <= 0) p.ag_groups = kAgMaxGroups;
  p.status = comm->status_dev;
  p.timeout_ns = comm->timeout_ns;
  p.trace = comm->trace;
  p.splitk_scratch = comm->splitk_scratch;
  p.splitk_cnt = comm->splitk_cnt;
  p.splitk_done = comm->splitk_cnt + comm->sm_count * 8;
  p.rank = comm->rank;
  p.world = comm->world;
  const int kind = is_8bit(in_dtype) ? 1 : 0;
  uint32_t fmt;
  switch (in_dtype) {
    case FLUXB_BF16: fmt = 1; break;
    case FLUXB_F16: fmt = 0; break;
    case FLUXB_E4M3: fmt = 0; break;
    case FLUXB_E5M2: fmt = 1; break;
    case FLUXB_S8: fmt = 1; break;
    default: FLUXB_FAIL(FLUXB_ERR_INVALID, "input dtype %d is not bf16/f16/e4m3/e5m2/s8", in_dtype);
  }
  p.acc_int = is_int8(in_dtype) ? 1 : 0;
  if (p.acc_int) {
    FLUXB_REQUIRE(p.out_type != kOutF32 || p.epi_mode == kEpiRsPush, "int8 inputs produce a 16-bit output");
    p.splitk_scratch = nullptr;  // the split-K tail adds parked accumulators as fp32: not for int32 accumulators
  }
  const uint32_t idesc = make_idesc(fmt, cg == 2 ? 2 * kBM : kBM, static_cast<uint32_t>(bn), p.b_mn_major ? 1u : 0u,
                                    p.acc_int ? 2u : 1u);
  if (comm->ranks_on_gpu > 1) {
    DeferredItem it;
    it.fused = true;
    it.p = p;
    it.idesc = idesc;
    it.bn = bn;
    it.kind = kind;
    it.cta_group = cg;
    it.grid = cg == 2 ? (grid & ~1) : grid;
    comm->deferred.push_back(std::move(it));
    return FLUXB_OK;
  }
#define FLUXB_LAUNCH(BN_, ST1_, ST2_)                                                              \
  (cg == 2 ? (kind == 0 ? launch_inst<BN_, ST2_, 0, true>(comm, p, idesc, grid, stream)            \
                        : launch_inst<BN_, ST2_, 1, true>(comm, p, idesc, grid, stream))           \
           : (kind == 0 ? launch_inst<BN_, ST1_, 0, false>(comm, p, idesc, grid, stream)           \
                        : launch_inst<BN_, ST1_, 1, false>(comm, p, idesc, grid, stream)))
  switch (bn) {
    case 256: return FLUXB_LAUNCH(256, stages_for(256, false), stages_for(256, true));
    case 192: return FLUXB_LAUNCH(192, stages_for(192, false), stages_for(192, true));
    case 128: return FLUXB_LAUNCH(128, stages_for(128, false), stages_for(128, true));
    default: return FLUXB_LAUNCH(64, stages_for(64, false), stages_for(64, true));
  }
#undef FLUXB_LAUNCH
}

static int out_type_of(int out_dtype, int* ot) {
  switch (out_dtype) {
    case FLUXB_BF16: *ot = kOutBf16; return FLUXB_OK;
    case FLUXB_F16: *ot = kOutF16; return FLUXB_OK;
    case FLUXB_F32: *ot = kOutF32; return FLUXB_OK;
    default: FLUXB_FAIL(FLUXB_ERR_INVALID, "output dtype %d is not bf16/f16/f32", out_dtype);
  }
}

static int check_gemm_shapes(const char* who, int m, int n, int k, int in_dtype, int out_dtype) {
  const int eb = dtype_bytes(in_dtype);
  FLUXB_REQUIRE(is_16bit(in_dtype) || is_8bit(in_dtype), "%s: input dtype %d unsupported", who, in_dtype);
  FLUXB_REQUIRE(m >= 1 && n >= 1 && k >= 1, "%s: empty problem m=%d n=%d k=%d", who, m, n, k);
  FLUXB_REQUIRE((static_cast<long long>(k) * eb) % 16 == 0,
                "%s: k=%d gives a row pitch of %lld bytes; it must be a multiple of 16", who, k,
                static_cast<long long>(k) * eb);
  FLUXB_REQUIRE(n % 8 == 0, "%s: n=%d must be a multiple of 8", who, n);
  (void)out_dtype;
  return FLUXB_OK;
}

static void zero_params(GemmParams& p) { memset(&p, 0, sizeof(p)); }
}  // namespace fluxb

namespace fluxb {
// Tiled-store map over a plain 16-bit output [rows, n] (row pitch n); left invalid where the map's alignment
// rules do not hold, in which case the epilogue uses per-lane stores.
void encode_out_map(GemmParams& p, void* out, long long rows, long long n, int out_type) {
  p.tmap_out_valid = 0;
  if (out_type == kOutF32 || out == nullptr || rows <= 0) return;
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0 || (n * 2) % 16 != 0) return;
  if (encode_tmap_b16_store(&p.tmap_out, out, rows, n) == FLUXB_OK) p.tmap_out_valid = 1;
}

// B operand: [n, k] (k contiguous) as one box of `box_rows` rows, or, with the FLUXB_WEIGHT_KN flag,
// [k, n] (n contiguous) as 64-column boxes feeding an MN-major UMMA operand.
static int encode_b(GemmParams& p, const void* b, int in_dtype, int n, int k, int box_rows, int flags) {
  const long long eb = dtype_bytes(in_dtype);
  if (flags & FLUXB_WEIGHT_KN) {
    FLUXB_REQUIRE(is_16bit(in_dtype), "a [K,N] weight needs 16-bit inputs (fp8 forbids transpose_weight)");
    p.b_mn_major = 1;
    return encode_tmap_kn(&p.tmap_b, b, in_dtype, k, n, static_cast<long long>(n) * eb, kRowBytes / static_cast<int>(eb));
  }
  return encode_tmap_2d(&p.tmap_b, b, in_dtype, n, k, static_cast<long long>(k) * eb, box_rows);
}

}  // namespace fluxb

using namespace fluxb;

struct fluxb_ag_gemm {
  fluxb_comm* comm;
  int full_m, n_dim, k_dim, in_dtype, out_dtype;
  int flag_stride;
  uint8_t* gather[kMaxWorld];
  int* flags[kMaxWorld];
  float* scales[kMaxWorld];
  bool has_scales;
  unsigned long long calls;
  AgDma dma;
};

struct fluxb_gemm_rs {
  fluxb_comm* comm;
  int max_m, n_dim, in_dtype, out_dtype;
  float* stage[kMaxWorld];
  int* cnt[kMaxWorld];
  long long cnt_cap;
  unsigned long long calls;
};

// arrival counters per source rank: one per (128-row chunk, slice group)
static int ag_flag_stride(int full_m, int world) {
  const int per_rank = (full_m + world - 1) / world;
  return ((per_rank + kBM - 1) / kBM) * kAgMaxGroups;
}

extern "C" {

int fluxb_gemm(fluxb_comm_t comm, const void* a, const void* b, void* c, int m, int n, int k,
               int in_dtype, int out_dtype, const void* bias, int bias_mode, const float* scale_a,
               const float* scale_b, float alpha, int flags, const fluxb_tuning* tuning, fluxb_stream_t stream) {
  FLUXB_REQUIRE(comm != nullptr && a != nullptr && b != nullptr && c != nullptr, "gemm: NULL argument");
  int rc = check_gemm_shapes("gemm", m, n, k, in_dtype, out_dtype);
  if (rc != FLUXB_OK) return rc;
  FLUXB_REQUIRE(bias_mode == FLUXB_BIAS_NONE || bias != nullptr, "gemm: bias_mode set but bias is NULL");
  GemmParams p;
  zero_params(p);
  const int eb = dtype_bytes(in_dtype);
  rc = out_type_of(out_dtype, &p.out_type);
  if (rc != FLUXB_OK) return rc;
  p.M = m;
  p.N = n;
  p.K = k;
  p.nseg = 1;
  p.seg_rows = m;
  p.seg_first = 0;
  p.epi_mode = kEpiStore;
  p.bias_mode = bias_mode;
  p.out = c;
  p.ldo = n;
  p.bias = bias;
  p.ldbias = n;
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  p.alpha = alpha;
  p.b_mn_major = (flags & FLUXB_WEIGHT_KN) ? 1 : 0;
  const int bn = resolve_block_n(comm, p, tuning, 0);
  rc = encode_tmap_2d(&p.tmap_a, a, in_dtype, m, k, static_cast<long long>(k) * eb, kBM);
  if (rc != FLUXB_OK) return rc;
  encode_out_map(p, c, m, n, p.out_type);
  rc = encode_b(p, b, in_dtype, n, k, resolve_cta_group(p, tuning) == 2 ? bn / 2 : bn, flags);
  if (rc != FLUXB_OK) return rc;
  fluxb_tuning t = tuning != nullptr ? *tuning : fluxb_tuning{0, 0, 0, 0, 0};
  t.block_n = bn;
  return launch_fused_gemm(comm, p, in_dtype, &t, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------ AG-GEMM
size_t fluxb_ag_gemm_gather_bytes(int full_m, int k_dim, int in_dtype) {
  // two parities; one extra tile of rows so that a 128-row box never leaves the allocation
  return 2ull * (static_cast<size_t>(full_m) + kBM) * k_dim * dtype_bytes(in_dtype);
}
size_t fluxb_ag_gemm_flag_bytes(int full_m, int world) {
  return 2ull * world * ag_flag_stride(full_m, world) * sizeof(int);
}
size_t fluxb_ag_gemm_scale_bytes(int full_m) { return 2ull * full_m * sizeof(float); }

int fluxb_ag_gemm_create(fluxb_comm_t comm, int full_m, int n_dim, int k_dim, int in_dtype,
                         int out_dtype, void* const* gather_bufs, int* const* flag_bufs,
                         float* const* scale_bufs, fluxb_ag_gemm_t* out) {
  FLUXB_REQUIRE(comm != nullptr && out != nullptr, "ag_gemm_create: NULL argument");
  FLUXB_REQUIRE(gather_bufs != nullptr && flag_bufs != nullptr, "ag_gemm_create: NULL buffer table");
  FLUXB_REQUIRE(full_m >= comm->world, "ag_gemm_create: full_m=%d < world=%d", full_m, comm->world);
  int rc = check_gemm_shapes("ag_gemm_create", full_m, n_dim, k_dim, in_dtype, out_dtype);
  if (rc != FLUXB_OK) return rc;
  int ot;
  rc = out_type_of(out_dtype, &ot);
  if (rc != FLUXB_OK) return rc;
  fluxb_ag_gemm* op = new fluxb_ag_gemm();
  op->calls = 0;
  op->comm = comm;
  op->full_m = full_m;
  op->n_dim = n_dim;
  op->k_dim = k_dim;
  op->in_dtype = in_dtype;
  op->out_dtype = out_dtype;
  op->flag_stride = ag_flag_stride(full_m, comm->world);
  op->has_scales = scale_bufs != nullptr;
  for (int r = 0; r < comm->world; ++r) {
    if (gather_bufs[r] == nullptr || flag_bufs[r] == nullptr ||
        (scale_bufs != nullptr && scale_bufs[r] == nullptr)) {
      delete op;
      FLUXB_FAIL(FLUXB_ERR_INVALID, "ag_gemm_create: buffer of rank %d is NULL", r);
    }
    op->gather[r] = static_cast<uint8_t*>(gather_bufs[r]);
    op->flags[r] = flag_bufs[r];
    op->scales[r] = scale_bufs != nullptr ? scale_bufs[r] : nullptr;
  }
  if (comm->world > 1) {
    rc = ag_dma_create(&op->dma, op->flag_stride);
    if (rc != FLUXB_OK) {
      ag_dma_destroy(&op->dma);
      delete op;
      return rc;
    }
  }
  *out = op;
  return FLUXB_OK;
}

int fluxb_ag_gemm_destroy(fluxb_ag_gemm_t op) {
  if (op != nullptr) ag_dma_destroy(&op->dma);
  delete op;
  return FLUXB_OK;
}

int fluxb_ag_gemm_reset(fluxb_ag_gemm_t op, fluxb_stream_t stream) {
  FLUXB_REQUIRE(op != nullptr, "ag_gemm_reset: op is NULL");
  FLUXB_CUDA(cudaMemsetAsync(op->flags[op->comm->rank], 0, fluxb_ag_gemm_flag_bytes(op->full_m, op->comm->world),
                             static_cast<cudaStream_t>(stream)));
  op->calls = 0;
  return FLUXB_OK;
}

int fluxb_ag_gemm_forward(fluxb_ag_gemm_t op, const void* a_shard, int m_local, const void* b,
                          int n, int k, void* c, const void* bias, int bias_mode,
                          const float* scale_a_shard, const float* scale_b, float alpha, int flags,
                          void* gathered_out, const fluxb_tuning* tuning, fluxb_stream_t stream_) {
  FLUXB_REQUIRE(op != nullptr && a_shard != nullptr && b != nullptr && c != nullptr,
                "ag_gemm_forward: NULL argument");
  fluxb_comm* comm = op->comm;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int world = comm->world;
  const long long m = static_cast<long long>(m_local) * world;
  FLUXB_REQUIRE(m_local >= 1 && m <= op->full_m, "ag_gemm_forward: m_local=%d * world=%d exceeds full_m=%d",
                m_local, world, op->full_m);
  FLUXB_REQUIRE(k == op->k_dim, "ag_gemm_forward: k=%d differs from k_dim=%d", k, op->k_dim);
  FLUXB_REQUIRE(n >= 1 && n <= op->n_dim, "ag_gemm_forward: n=%d exceeds n_dim=%d", n, op->n_dim);
  int rc = check_gemm_shapes("ag_gemm_forward", static_cast<int>(m), n, k, op->in_dtype, op->out_dtype);
  if (rc != FLUXB_OK) return rc;
  FLUXB_REQUIRE(bias_mode == FLUXB_BIAS_NONE || bias != nullptr, "ag_gemm_forward: bias is NULL");
  FLUXB_REQUIRE(scale_a_shard == nullptr || op->has_scales,
                "ag_gemm_forward: per-row input scales need scale buffers at create time");
  const int eb = dtype_bytes(op->in_dtype);
  const long long row_bytes = static_cast<long long>(k) * eb;

  if (world == 1) {
    rc = fluxb_gemm(comm, a_shard, b, c, m_local, n, k, op->in_dtype, op->out_dtype, bias, bias_mode,
                    scale_a_shard, scale_b, alpha, flags, tuning, stream_);
    if (rc != FLUXB_OK) return rc;
    if (gathered_out != nullptr)
      FLUXB_CUDA(cudaMemcpyAsync(gathered_out, a_shard, m_local * row_bytes, cudaMemcpyDeviceToDevice, stream));
    return FLUXB_OK;
  }

  const int parity = static_cast<int>(op->calls & 1ull);
  const size_t half_gather = (static_cast<size_t>(op->full_m) + kBM) * op->k_dim * eb;
  const size_t half_flags = static_cast<size_t>(world) * op->flag_stride;
  // The other parity's counters were consumed by the previous call and are next written by
  // peers only after they have seen this call's pushes: clear them now.
  FLUXB_CUDA(cudaMemsetAsync(op->flags[comm->rank] + (parity ^ 1) * half_flags, 0,
                             half_flags * sizeof(int), stream));

  GemmParams p;
  zero_params(p);
  rc = out_type_of(op->out_dtype, &p.out_type);
  if (rc != FLUXB_OK) return rc;
  p.M = static_cast<int>(m);
  p.N = n;
  p.K = k;
  p.nseg = world;
  p.seg_rows = m_local;
  p.seg_first = comm->rank;
  p.epi_mode = kEpiStore;
  p.bias_mode = bias_mode;
  p.out = c;
  p.ldo = n;
  p.bias = bias;
  p.ldbias = n;
  p.scale_b = scale_b;
  p.alpha = alpha;
  p.ag_flags = op->flags[comm->rank] + parity * half_flags;
  p.ag_flag_stride = op->flag_stride;
  p.ag_groups = kAgMaxGroups;
  p.ag_spf = ag_slices_per_flag(row_bytes);
  p.ag_unit_rows = resolve_ag_unit_rows(tuning);
  p.ag_src = static_cast<const uint8_t*>(a_shard);
  p.ag_row_bytes = row_bytes;
  p.ag_src_scale = scale_a_shard;
  for (int r = 0; r < world; ++r) {
    p.ag_dst[r] = op->gather[r] + parity * half_gather;
    p.ag_dst_flags[r] = op->flags[r] + parity * half_flags;
    p.ag_dst_scale[r] = op->has_scales ? op->scales[r] + parity * op->full_m : nullptr;
  }
  if (scale_a_shard != nullptr) p.scale_a = op->scales[comm->rank] + parity * op->full_m;
  const bool dma = resolve_ag_mode(tuning) == kAgModeCopyEngine;
  if (dma) {
    // the copy engines carry the shard to the peers; the kernel's comm warps have nothing to push
    uint8_t* gather_p[kMaxWorld];
    int* flags_p[kMaxWorld];
    float* scale_p[kMaxWorld];
    for (int r = 0; r < world; ++r) {
      gather_p[r] = p.ag_dst[r];
      flags_p[r] = p.ag_dst_flags[r];
      scale_p[r] = p.ag_dst_scale[r];
    }
    if (scale_a_shard != nullptr)  // this rank's own rows of the gathered scale vector
      FLUXB_CUDA(cudaMemcpyAsync(scale_p[comm->rank] + static_cast<size_t>(comm->rank) * m_local, scale_a_shard,
                                 static_cast<size_t>(m_local) * sizeof(float), cudaMemcpyDeviceToDevice, stream));
    rc = ag_dma_push(comm, &op->dma, a_shard, m_local, row_bytes, gather_p, flags_p, scale_a_shard, scale_p, false, stream);
    if (rc != FLUXB_OK) return rc;
    p.ag_src = nullptr;
    p.ag_src_scale = nullptr;
  }
  p.b_mn_major = (flags & FLUXB_WEIGHT_KN) ? 1 : 0;
  if (tuning == nullptr || tuning->group_m <= 0) {
    // own shard first, then bands that double (1, 2, 4 shards ...) so that tiles follow the arrival order
    const int tile_m = resolve_cta_group(p, tuning) == 2 ? 2 * kBM : kBM;
    const int tps = (m_local + tile_m - 1) / tile_m;
    p.group_m = tps < 8 ? tps : 8;
    make_bands(p, world, tps, /*first_single=*/true, /*last_single=*/false);
  }
  const int bn = resolve_block_n(comm, p, tuning, 0);
  uint8_t* local_gather = op->gather[comm->rank] + parity * half_gather;
  rc = encode_tmap_2d(&p.tmap_a, local_gather, op->in_dtype, m, k, row_bytes, kBM);
  if (rc != FLUXB_OK) return rc;
  rc = encode_tmap_2d(&p.tmap_a_own, a_shard, op->in_dtype, m_local, k, row_bytes, kBM);
  if (rc != FLUXB_OK) return rc;
  encode_out_map(p, c, m, n, p.out_type);
  // kernel push: per-row scales travel through the scale buffer under the same flags as the data, so the
  // own shard takes the flagged path too in that case (the copy-engine form has put the own scales in place)
  p.a_own_valid = (scale_a_shard == nullptr || dma) ? 1 : 0;
  rc = encode_b(p, b, op->in_dtype, n, k, resolve_cta_group(p, tuning) == 2 ? bn / 2 : bn, flags);
  if (rc != FLUXB_OK) return rc;
  fluxb_tuning t = tuning != nullptr ? *tuning : fluxb_tuning{0, 0, 0, 0, 0};
  t.block_n = bn;
  rc = launch_fused_gemm(comm, p, op->in_dtype, &t, stream);
  if (rc != FLUXB_OK) return rc;
  op->calls += 1;
  // the caller's tensor and this call's counters stay in use until the copies are done
  if (dma) FLUXB_CUDA(cudaStreamWaitEvent(stream, op->dma.ev_done, 0));
  if (gathered_out != nullptr) {
    // peers' shards come from the gather buffer, this rank's own shard from the caller's tensor
    const size_t all_bytes = static_cast<size_t>(m) * row_bytes, own_bytes = static_cast<size_t>(m_local) * row_bytes;
    uint8_t* own_dst = static_cast<uint8_t*>(gathered_out) + static_cast<size_t>(comm->rank) * own_bytes;
    return enqueue_or_defer(comm, stream, [=](cudaStream_t st) -> int {
      FLUXB_CUDA(cudaMemcpyAsync(gathered_out, local_gather, all_bytes, cudaMemcpyDeviceToDevice, st));
      FLUXB_CUDA(cudaMemcpyAsync(own_dst, a_shard, own_bytes, cudaMemcpyDeviceToDevice, st));
      return FLUXB_OK;
    });
  }
  return FLUXB_OK;
}

// ------------------------------------------------------------------ GEMM-RS
static long long rs_cnt_cap(int max_m, int n_dim, int world) {
  const int mpr = (max_m + world - 1) / world;
  return static_cast<long long>((mpr + kBM - 1) / kBM) * ((n_dim + 63) / 64);
}
size_t fluxb_gemm_rs_stage_bytes(int max_m, int n_dim, int world) {
  (void)world;
  return 2ull * static_cast<size_t>(max_m) * n_dim * sizeof(float);
}
size_t fluxb_gemm_rs_cnt_bytes(int max_m, int n_dim, int world) {
  // two parities x (arrival counters of the early peers + ready flags + arrival counters of the late peers)
  return 2ull * 3ull * rs_cnt_cap(max_m, n_dim, world) * sizeof(int);
}

int fluxb_gemm_rs_create(fluxb_comm_t comm, int max_m, int n_dim, int in_dtype, int out_dtype,
                         float* const* stage_bufs, int* const* cnt_bufs, fluxb_gemm_rs_t* out) {
  FLUXB_REQUIRE(comm != nullptr && out != nullptr, "gemm_rs_create: NULL argument");
  FLUXB_REQUIRE(stage_bufs != nullptr && cnt_bufs != nullptr, "gemm_rs_create: NULL buffer table");
  FLUXB_REQUIRE(max_m >= comm->world && n_dim >= 8 && n_dim % 8 == 0,
                "gemm_rs_create: max_m=%d n_dim=%d invalid (n_dim must be a multiple of 8)", max_m, n_dim);
  FLUXB_REQUIRE(is_16bit(in_dtype) || is_8bit(in_dtype), "gemm_rs_create: input dtype %d unsupported", in_dtype);
  int ot;
  int rc = out_type_of(out_dtype, &ot);
  if (rc != FLUXB_OK) return rc;
  fluxb_gemm_rs* op = new fluxb_gemm_rs();
  memset(op, 0, sizeof(*op));
  op->comm = comm;
  op->max_m = max_m;
  op->n_dim = n_dim;
  op->in_dtype = in_dtype;
  op->out_dtype = out_dtype;
  op->cnt_cap = rs_cnt_cap(max_m, n_dim, comm->world);
  for (int r = 0; r < comm->world; ++r) {
    if (stage_bufs[r] == nullptr || cnt_bufs[r] == nullptr) {
      delete op;
      FLUXB_FAIL(FLUXB_ERR_INVALID, "gemm_rs_create: buffer of rank %d is NULL", r);
    }
    op->stage[r] = stage_bufs[r];
    op->cnt[r] = cnt_bufs[r];
  }
  *out = op;
  return FLUXB_OK;
}

int fluxb_gemm_rs_destroy(fluxb_gemm_rs_t op) {
  delete op;
  return FLUXB_OK;
}

int fluxb_gemm_rs_reset(fluxb_gemm_rs_t op, fluxb_stream_t stream) {
  FLUXB_REQUIRE(op != nullptr, "gemm_rs_reset: op is NULL");
  FLUXB_CUDA(cudaMemsetAsync(op->cnt[op->comm->rank], 0, fluxb_gemm_rs_cnt_bytes(op->max_m, op->n_dim, op->comm->world),
                             static_cast<cudaStream_t>(stream)));
  op->calls = 0;
  return FLUXB_OK;
}

int fluxb_gemm_rs_forward(fluxb_gemm_rs_t op, const void* a, const void* b, int m, int n,
                          int k_local, void* out, const void* bias, int bias_mode,
                          const float* scale_a, const float* scale_b, float alpha, int flags,
                          const fluxb_tuning* tuning, fluxb_stream_t stream_) {
  FLUXB_REQUIRE(op != nullptr && a != nullptr && b != nullptr && out != nullptr,
                "gemm_rs_forward: NULL argument");
  fluxb_comm* comm = op->comm;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int world = comm->world;
  FLUXB_REQUIRE(m >= world && m <= op->max_m, "gemm_rs_forward: m=%d out of [%d, max_m=%d]", m, world, op->max_m);
  FLUXB_REQUIRE(m % world == 0, "gemm_rs_forward: m=%d is not a multiple of world=%d", m, world);
  FLUXB_REQUIRE(n == op->n_dim, "gemm_rs_forward: n=%d differs from n_dim=%d", n, op->n_dim);
  int rc = check_gemm_shapes("gemm_rs_forward", m, n, k_local, op->in_dtype, op->out_dtype);
  if (rc != FLUXB_OK) return rc;
  FLUXB_REQUIRE(bias_mode == FLUXB_BIAS_NONE || bias != nullptr, "gemm_rs_forward: bias is NULL");
  if (world == 1)
    return fluxb_gemm(comm, a, b, out, m, n, k_local, op->in_dtype, op->out_dtype, bias, bias_mode,
                      scale_a, scale_b, alpha, flags, tuning, stream_);
  FLUXB_REQUIRE(bias_mode == FLUXB_BIAS_NONE || op->out_dtype == FLUXB_BF16,
                "gemm_rs_forward: bias needs a bf16 output");
  // w8a8: the bias is applied by rank 0 only (src/gemm_rs/ths_op/gemm_reduce_scatter.cc:596-599)
  if (is_int8(op->in_dtype) && comm->rank != 0) bias_mode = FLUXB_BIAS_NONE;

  const int eb = dtype_bytes(op->in_dtype);
  const int mpr = m / world;
  const int parity = static_cast<int>(op->calls & 1ull);
  // The other parity's counters and flags were consumed by the previous call and are next written by
  // peers only after they have seen this call's pushes: clear them now.
  FLUXB_CUDA(cudaMemsetAsync(op->cnt[comm->rank] + (parity ^ 1) * 3 * op->cnt_cap, 0,
                             3 * op->cnt_cap * sizeof(int), stream));
  GemmParams p;
  zero_params(p);
  int ot;
  rc = out_type_of(op->out_dtype, &ot);
  if (rc != FLUXB_OK) return rc;
  p.M = m;
  p.N = n;
  p.K = k_local;
  p.nseg = world;
  p.seg_rows = mpr;
  p.seg_first = (comm->rank + 1) % world;  // rows owned by peers first, own rows last
  p.epi_mode = kEpiRsPush;
  p.out_type = kOutF32;
  p.bias_mode = bias_mode;
  p.bias = bias;
  p.ldbias = n;
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  p.alpha = alpha;
  p.b_mn_major = (flags & FLUXB_WEIGHT_KN) ? 1 : 0;
  // Partials cross NVLink in the output's 16-bit format (half the bytes of fp32; the owner still sums in
  // fp32 and rounds once more at the end). Slots keep their fp32-sized stride; 16-bit data fills the
  // first half of a peer's slot, the owner's own slot holds the fp32 sum of the peers' partials.
  p.rs_wire16 = (ot == kOutBf16 || ot == kOutF16) && !(flags & FLUXB_RS_FP32_WIRE) ? 1 : 0;
  p.rs_ring = (p.rs_wire16 && (flags & FLUXB_RS_RING_ORDER)) ? 1 : 0;
  const size_t half_stage = static_cast<size_t>(op->max_m) * op->n_dim;
  for (int r = 0; r < world; ++r) {
    p.rs_stage[r] = op->stage[r] + parity * half_stage + static_cast<size_t>(comm->rank) * mpr * n;
    p.rs_cnt[r] = op->cnt[r] + parity * 3 * op->cnt_cap;
    rc = p.rs_wire16 ? encode_tmap_b16_store(&p.tmap_rs[r], p.rs_stage[r], mpr, n)
                     : encode_tmap_f32_store(&p.tmap_rs[r], p.rs_stage[r], mpr, n);
    if (rc != FLUXB_OK) return rc;
  }
  if (tuning == nullptr || tuning->group_m <= 0) {
    // rows owned by peers first, in bands of up to 8 M tiles; this rank's own rows as the last band
    const int tile_m = resolve_cta_group(p, tuning) == 2 ? 2 * kBM : kBM;
    const int tps = (mpr + tile_m - 1) / tile_m;
    p.group_m = tps < 8 ? tps : 8;
    make_bands(p, world, tps, /*first_single=*/false, /*last_single=*/true);
  }
  const int bn = resolve_block_n(comm, p, tuning, 0);
  const long long row_bytes = static_cast<long long>(k_local) * eb;
  rc = encode_tmap_2d(&p.tmap_a, a, op->in_dtype, m, k_local, row_bytes, kBM);
  if (rc != FLUXB_OK) return rc;
  rc = encode_b(p, b, op->in_dtype, n, k_local, resolve_cta_group(p, tuning) == 2 ? bn / 2 : bn, flags);
  if (rc != FLUXB_OK) return rc;
  fluxb_tuning t = tuning != nullptr ? *tuning : fluxb_tuning{0, 0, 0, 0, 0};
  t.block_n = bn;
  // the owner-side reduction runs in the same kernel (comm warps)
  p.rs_local_stage = op->stage[comm->rank] + parity * half_stage;
  p.rs_local_cnt = op->cnt[comm->rank] + parity * 3 * op->cnt_cap;
  p.rs_local_ready = p.rs_local_cnt + op->cnt_cap;
  p.rs_late_off = static_cast<int>(2 * op->cnt_cap);
  // Late peers: those that compute this rank's rows in their last band of peer rows (by symmetry, the ranks
  // rank+1 .. rank+n_late, where n_late is the number of owners in that band). Not with the ring-order
  // reduction (its order and roundings are fixed) nor with fp32 partials.
  p.rs_n_late = 0;
  if (p.rs_wire16 && !p.rs_ring) {
    const int tile_m = resolve_cta_group(p, tuning) == 2 ? 2 * kBM : kBM;
    p.rs_n_late = rs_late_peers(p, world, (mpr + tile_m - 1) / tile_m);
  }
  p.rs_out = out;
  p.rs_out_type = ot;
  rc = launch_fused_gemm(comm, p, op->in_dtype, &t, stream);
  if (rc != FLUXB_OK) return rc;
  op->calls += 1;
  return FLUXB_OK;
}

}  // extern "C"
