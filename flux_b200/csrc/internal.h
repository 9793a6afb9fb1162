// Host-side internals shared by the .cu files of the library: error
// reporting, the communicator object, tensor-map encoding, launch helpers.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include <functional>
#include <string>
#include <vector>

#include "../../include/fluxb.h"
#include "gemm_kernel.cuh"

namespace fluxb {

void set_error(const char* fmt, ...);

#define FLUXB_FAIL(code, ...)          \
  do {                                 \
    ::fluxb::set_error(__VA_ARGS__);   \
    return (code);                     \
  } while (0)

#define FLUXB_REQUIRE(cond, ...)                        \
  do {                                                  \
    if (!(cond)) FLUXB_FAIL(FLUXB_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define FLUXB_CUDA(expr)                                                              \
  do {                                                                                \
    cudaError_t e_ = (expr);                                                          \
    if (e_ != cudaSuccess)                                                            \
      FLUXB_FAIL(FLUXB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                 __FILE__, __LINE__);                                                 \
  } while (0)

inline int dtype_bytes(int dt) {
  switch (dt) {
    case FLUXB_BF16:
    case FLUXB_F16:
      return 2;
    case FLUXB_F32:
      return 4;
    case FLUXB_E4M3:
    case FLUXB_E5M2:
    case FLUXB_S8:
      return 1;
    default:
      return 0;
  }
}
inline bool is_fp8(int dt) { return dt == FLUXB_E4M3 || dt == FLUXB_E5M2; }
inline bool is_int8(int dt) { return dt == FLUXB_S8; }
inline bool is_8bit(int dt) { return is_fp8(dt) || is_int8(dt); }
inline bool is_16bit(int dt) { return dt == FLUXB_BF16 || dt == FLUXB_F16; }

}  // namespace fluxb

namespace fluxb {
// One piece of work a forward call would have put on the stream, kept back while several ranks share one
// GPU (fluxb_comm_set_ranks_on_gpu): either a launch of the fused kernel (its parameters and template
// choice) or any other stream work (a closure).
struct DeferredItem {
  bool fused = false;
  GemmParams p;
  uint32_t idesc = 0;
  int bn = 0, kind = 0, cta_group = 1, grid = 0;
  std::function<int(cudaStream_t)> plain;
};
}  // namespace fluxb

struct fluxb_comm {
  int rank = 0;
  int world = 1;
  int device = 0;
  int sm_count = 0;
  int* status_host = nullptr;  // pinned + mapped; kernels write, host reads
  int* status_dev = nullptr;   // device alias of status_host
  unsigned long long timeout_ns = 10ull * 1000 * 1000 * 1000;
  int barrier_epoch = 0;
  unsigned long long* trace = nullptr;  // optional per-CTA timeline buffer (caller-owned device memory)
  float* splitk_scratch = nullptr;  // sm_count x 128 x 256 fp32: parked partial accumulators of split tail tiles
  int* splitk_cnt = nullptr;        // per (tail tile, half, epilogue warp) arrivals, zero between launches
  // several ranks on one GPU (test harness): forwards queue their stream work here, fluxb_run_ranks issues it
  int ranks_on_gpu = 1;
  std::vector<fluxb::DeferredItem> deferred;
  fluxb::GemmParams* ranks_params_dev = nullptr;   // [kMaxRankItems][kMaxWorld] parameter blocks of merged launches
  fluxb::GemmParams* ranks_params_host = nullptr;  // pinned staging of the same
};

namespace fluxb {

// 2-D tensor map over a row-major [rows, k] matrix whose rows are `ld_bytes`
// apart; box = 128 bytes of K x `box_rows` rows, 128-byte swizzle.
int encode_tmap_2d(CUtensorMap* out, const void* base, int elt_dtype, long long rows, long long k,
                   long long ld_bytes, int box_rows);

// 16-bit [k, n] row-major matrix (n contiguous) read as 64-column x `box_k`-row boxes, 128-byte swizzle
int encode_tmap_kn(CUtensorMap* out, const void* base, int elt_dtype, long long k, long long n, long long ld_bytes,
                   int box_k);

// fp32 [rows, n] row-major matrix, 32 x 32 element boxes, 128-byte swizzle (reduce-scatter pushes)
int encode_tmap_f32_store(CUtensorMap* out, const void* base, long long rows, long long n);
int encode_tmap_b16_store(CUtensorMap* out, const void* base, long long rows, long long n);

// Output tile width for a problem: the caller's choice, else a wave-quantisation heuristic.
// `m_tiles_hint` > 0 overrides the M-tile count derived from the segments (grouped problems).
int resolve_block_n(const fluxb_comm* comm, const GemmParams& p, const fluxb_tuning* tuning,
                    long long m_tiles_hint);

// Tiled-store map over a plain 16-bit output (see GemmParams::tmap_out); never fails, it only leaves the map invalid.
void encode_out_map(GemmParams& p, void* out, long long rows, long long n, int out_type);

// 2 KB slices of a row that share one arrival counter (1 unless the row has more than kAgMaxGroups slices)
int ag_slices_per_flag(long long row_bytes);

// All-gather carried by the copy engines instead of the kernel's comm warps: a side stream copies this rank's
// shard into every peer's gather buffer, piece by piece (256 rows), in the order the peers consume it
// (rank-1 first), and after each piece copies the piece's expected counter values into the peer's arrival
// counters, so the consuming kernel cannot tell the two transports apart. This is the reference's default
// transport (cudaMemcpyAsync per peer + flag writes, src/coll/ths_op/all_gather_op.cc:529-574).
struct AgDma {
  cudaStream_t side = nullptr;
  cudaEvent_t ev_start = nullptr, ev_done = nullptr;
  int* expected_dev = nullptr;       // [flag_stride] counter values of a complete shard for `expected_row_bytes`
  long long expected_row_bytes = -1;
  int flag_stride = 0;
};
int ag_dma_create(AgDma* d, int flag_stride);
void ag_dma_destroy(AgDma* d);
// Queue the copies (after everything already on `main`) and record d->ev_done behind them; the caller launches
// its kernel on `main` and then makes `main` wait for d->ev_done. `gather` / `flags` / `dst_scale` are the
// per-rank bases of the buffer parity in use.
// `include_self`: also copy the shard into this rank's own gather buffer (consumers that read every shard from
// the buffer), before the peers'.
int ag_dma_push(const fluxb_comm* comm, AgDma* d, const void* src, int m_local, long long row_bytes,
                uint8_t* const* gather, int* const* flags, const float* src_scale, float* const* dst_scale,
                bool include_self, cudaStream_t main);

enum : int { kAgModeDefault = 0, kAgModeKernelPush = 1, kAgModeCopyEngine = 2 };
int resolve_ag_mode(const fluxb_tuning* tuning);
int resolve_ag_unit_rows(const fluxb_tuning* tuning);  // rows of a push unit for the chosen mode

// 1 = one CTA per 128-row tile, 2 = CTA pair per 256-row tile (the caller's choice or a heuristic).
int resolve_cta_group(const GemmParams& p, const fluxb_tuning* tuning);

// Fill the problem-independent fields and launch the fused kernel (or queue the launch while several
// ranks share the GPU).
int launch_fused_gemm(fluxb_comm* comm, GemmParams& p, int in_dtype,
                      const fluxb_tuning* tuning, cudaStream_t stream);

// Run `fn(stream)` now, or queue it behind the queued launches while several ranks share the GPU.
int enqueue_or_defer(fluxb_comm* comm, cudaStream_t stream, std::function<int(cudaStream_t)> fn);

constexpr int kMaxRankItems = 16;  // queued fused launches per fluxb_run_ranks call

// pipeline depth of each tile width: one CTA per tile / CTA pair
constexpr int stages_for(int bn, bool cta2) {
  return bn == 256 ? (cta2 ? 6 : 4) : bn == 192 ? (cta2 ? 7 : 5) : bn == 128 ? (cta2 ? 8 : 6) : 8;
}

// One launch that runs `nranks` problems side by side (loopback.cu).
int launch_ranks_kernel(int bn, int kind, int cta_group, const GemmParams* ps_dev, int nranks, int ctas_per_rank,
                        uint32_t idesc, cudaStream_t stream);

}  // namespace fluxb
