// Integer routing work of the MoE ops. Everything here is exact integer
// arithmetic and deterministic (no atomics decide an order).
//
// scatter index (stable): rows are sorted by expert, ties keep (token, k)
// order - the definition of the reference's calc_scatter_index_stable
// (python/flux/testing/moe_utils.py:141-144). The reference's device kernel
// (src/cuda/moe_utils.cu:23-75) orders rows inside an expert with shared
// memory atomics; this one does not.
// gather index: inverse permutation (src/moe_ag_scatter/sort_util.cu:39-92).
#include "internal.h"

namespace fluxb {

constexpr int kIdxThreads = 1024;
constexpr int kMaxExperts = 1024;

// Single block: per-thread contiguous slices keep (token,k) order, a block
// scan per expert turns per-slice counts into stable positions.
__global__ void __launch_bounds__(kIdxThreads)
scatter_index_kernel(const int* __restrict__ chosen, int total, int nexperts, int* splits,
                     int* scatter_index) {
  extern __shared__ int sh[];  // [nexperts] running base + [kIdxThreads] scan scratch
  int* base = sh;
  int* scan = sh + nexperts;
  const int tid = threadIdx.x;
  const int per = (total + kIdxThreads - 1) / kIdxThreads;
  const int lo = imin(tid * per, total);
  const int hi = imin(lo + per, total);
  for (int e = tid; e < nexperts; e += kIdxThreads) base[e] = 0;
  __syncthreads();
  // pass 1: histogram
  for (int i = lo; i < hi; ++i) {
    const int e = chosen[i];
    if (e >= 0 && e < nexperts) atomicAdd(&base[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < nexperts; ++e) {
      const int c = base[e];
      splits[e] = c;
      base[e] = run;
      run += c;
    }
  }
  __syncthreads();
  // pass 2: one expert at a time, exclusive scan of per-slice counts
  for (int e = 0; e < nexperts; ++e) {
    int cnt = 0;
    for (int i = lo; i < hi; ++i) cnt += (chosen[i] == e) ? 1 : 0;
    scan[tid] = cnt;
    __syncthreads();
    for (int off = 1; off < kIdxThreads; off <<= 1) {
      int v = (tid >= off) ? scan[tid - off] : 0;
      __syncthreads();
      scan[tid] += v;
      __syncthreads();
    }
    int pos = base[e] + scan[tid] - cnt;
    for (int i = lo; i < hi; ++i)
      if (chosen[i] == e) scatter_index[i] = pos++;
    __syncthreads();
  }
}

__global__ void gather_index_kernel(const int* __restrict__ scatter_index, int total, int topk,
                                    int* gather_index, int* topk_index) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int row = scatter_index[i];
  if (row < 0 || row >= total) return;
  gather_index[row] = i / topk;
  if (topk_index != nullptr) topk_index[row] = i % topk;
}

}  // namespace fluxb

using namespace fluxb;

extern "C" {

int fluxb_moe_scatter_index(const int* chosen_experts, int ntokens, int topk, int nexperts,
                            int* splits_out, int* scatter_index_out, fluxb_stream_t stream) {
  FLUXB_REQUIRE(chosen_experts != nullptr && splits_out != nullptr && scatter_index_out != nullptr,
                "moe_scatter_index: NULL argument");
  FLUXB_REQUIRE(ntokens >= 0 && topk >= 1, "moe_scatter_index: ntokens=%d topk=%d invalid", ntokens, topk);
  FLUXB_REQUIRE(nexperts >= 1 && nexperts <= kMaxExperts, "moe_scatter_index: nexperts=%d out of [1,%d]",
                nexperts, kMaxExperts);
  const long long total = static_cast<long long>(ntokens) * topk;
  FLUXB_REQUIRE(total < (1ll << 30), "moe_scatter_index: too many routed rows");
  const size_t sh = (nexperts + kIdxThreads) * sizeof(int);
  scatter_index_kernel<<<1, kIdxThreads, sh, static_cast<cudaStream_t>(stream)>>>(
      chosen_experts, static_cast<int>(total), nexperts, splits_out, scatter_index_out);
  FLUXB_CUDA(cudaGetLastError());
  return FLUXB_OK;
}

int fluxb_moe_gather_index(const int* scatter_index, int ntokens, int topk, int* gather_index_out,
                           int* topk_index_out, fluxb_stream_t stream) {
  FLUXB_REQUIRE(scatter_index != nullptr && gather_index_out != nullptr, "moe_gather_index: NULL argument");
  FLUXB_REQUIRE(ntokens >= 0 && topk >= 1, "moe_gather_index: ntokens=%d topk=%d invalid", ntokens, topk);
  const long long total = static_cast<long long>(ntokens) * topk;
  FLUXB_REQUIRE(total < (1ll << 30), "moe_gather_index: too many routed rows");
  if (total == 0) return FLUXB_OK;
  const int blocks = static_cast<int>((total + 255) / 256);
  gather_index_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      scatter_index, static_cast<int>(total), topk, gather_index_out, topk_index_out);
  FLUXB_CUDA(cudaGetLastError());
  return FLUXB_OK;
}

}  // extern "C"
