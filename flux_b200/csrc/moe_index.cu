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

constexpr int kExpertChunk = 32;  // experts handled per sweep: one row of per-thread counts per warp

// Single block. Every thread owns a contiguous slice of the (token, k) pairs, so positions inside an expert
// follow (token, k) order. Experts are handled 32 at a time: the threads count their slice's pairs per expert
// into a [32][1024] table in shared memory (one column per thread), each of the 32 warps turns one expert's
// row into exclusive prefixes over the threads, and a second walk over the slice hands out the positions.
// Three barriers per 32 experts, whatever the number of experts.
__global__ void __launch_bounds__(kIdxThreads)
scatter_index_kernel(const int* __restrict__ chosen, int total, int nexperts, int* splits,
                     int* scatter_index) {
  extern __shared__ int sh[];  // [nexperts] first row of every expert + [kExpertChunk][kIdxThreads] counts
  int* base = sh;
  int* cnt = sh + nexperts;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int per = (total + kIdxThreads - 1) / kIdxThreads;
  const int lo = imin(tid * per, total);
  const int hi = imin(lo + per, total);
  for (int e = tid; e < nexperts; e += kIdxThreads) base[e] = 0;
  __syncthreads();
  // histogram -> splits and the first row of every expert
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
  for (int e0 = 0; e0 < nexperts; e0 += kExpertChunk) {
    for (int j = 0; j < kExpertChunk; ++j) cnt[j * kIdxThreads + tid] = 0;
    for (int i = lo; i < hi; ++i) {
      const int j = chosen[i] - e0;
      if (j >= 0 && j < kExpertChunk && j + e0 < nexperts) cnt[j * kIdxThreads + tid] += 1;
    }
    __syncthreads();  // counts complete (and `base` written, first time round)
    {
      // warp w scans the row of expert e0 + w: lane l owns threads 32l .. 32l+31
      int* row = cnt + warp * kIdxThreads + lane * 32;
      int sum = 0;
      for (int q = 0; q < 32; ++q) sum += row[q];
      int incl = sum;
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
      }
      int run = incl - sum;
      for (int q = 0; q < 32; ++q) {
        const int c = row[q];
        row[q] = run;
        run += c;
      }
    }
    __syncthreads();  // prefixes complete
    for (int i = lo; i < hi; ++i) {
      const int j = chosen[i] - e0;
      if (j >= 0 && j < kExpertChunk && j + e0 < nexperts) scatter_index[i] = base[j + e0] + cnt[j * kIdxThreads + tid]++;
    }
    __syncthreads();  // the table is reused by the next 32 experts
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
  const size_t sh = (static_cast<size_t>(nexperts) + static_cast<size_t>(kExpertChunk) * kIdxThreads) * sizeof(int);
  static bool configured[64] = {};
  int dev = 0;
  FLUXB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {  // 132 KB of dynamic shared memory: above the default limit
    FLUXB_CUDA(cudaFuncSetAttribute(scatter_index_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>((kMaxExperts + kExpertChunk * kIdxThreads) * sizeof(int))));
    configured[dev] = true;
  }
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
