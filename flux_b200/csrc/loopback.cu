// Several ranks on ONE GPU, for machines with fewer GPUs than ranks (test harnesses, bring-up).
//
// The fused kernels of different ranks wait on one another's arrival flags. Launched one after the other, or
// on different streams of one GPU, nothing guarantees that they run at the same time, so they would wait
// for each other until their budgets expire. Here every rank's forward call only queues its stream work
// (fluxb_comm_set_ranks_on_gpu), and fluxb_run_ranks issues the queued fused launches of all ranks as ONE
// cooperative launch in which each rank owns a slice of the grid (fused_gemm_ranks_kernel): all CTAs are
// resident together, each slice behaves exactly like that rank's own launch, and the pushes, counters and
// owner-side sums run through the same code as on separate GPUs (peer pointers are simply local pointers).
// The reference's own C++ unit test drives all ranks from one process in the same spirit
// (src/gemm_rs/test/test_gemm_rs.cc:43-130).
#include <string.h>

#include "internal.h"

namespace fluxb {

template <int BN, int STAGES, int KIND, bool CTA2>
static int launch_ranks_inst(const GemmParams* ps_dev, int nranks, int ctas_per_rank, uint32_t idesc,
                             cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES, CTA2>;
  auto kern = fused_gemm_ranks_kernel<BN, STAGES, KIND, CTA2>;
  FLUXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.gridDim = dim3(nranks * ctas_per_rank, 1, 1);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTA2 ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // cooperative: the launch fails (instead of waiting forever) unless every CTA can be resident at once
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (CTA2) {
    int n = 0;
    FLUXB_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    FLUXB_REQUIRE(2 * n >= nranks * ctas_per_rank,
                  "run_ranks: %d CTAs do not fit on the device at once (%d CTA pairs can be resident)",
                  nranks * ctas_per_rank, n);
  }
  FLUXB_CUDA(cudaLaunchKernelEx(&cfg, kern, ps_dev, ctas_per_rank, idesc));
  return FLUXB_OK;
}

int launch_ranks_kernel(int bn, int kind, int cta_group, const GemmParams* ps_dev, int nranks, int ctas_per_rank,
                        uint32_t idesc, cudaStream_t stream) {
#define FLUXB_RANKS(BN_)                                                                                          \
  (cta_group == 2                                                                                                  \
       ? (kind == 0 ? launch_ranks_inst<BN_, stages_for(BN_, true), 0, true>(ps_dev, nranks, ctas_per_rank, idesc, stream)   \
                    : launch_ranks_inst<BN_, stages_for(BN_, true), 1, true>(ps_dev, nranks, ctas_per_rank, idesc, stream))  \
       : (kind == 0 ? launch_ranks_inst<BN_, stages_for(BN_, false), 0, false>(ps_dev, nranks, ctas_per_rank, idesc, stream) \
                    : launch_ranks_inst<BN_, stages_for(BN_, false), 1, false>(ps_dev, nranks, ctas_per_rank, idesc, stream)))
  switch (bn) {
    case 256: return FLUXB_RANKS(256);
    case 192: return FLUXB_RANKS(192);
    case 128: return FLUXB_RANKS(128);
    case 64: return FLUXB_RANKS(64);
    default: FLUXB_FAIL(FLUXB_ERR_INVALID, "run_ranks: block_n=%d not in {64,128,192,256}", bn);
  }
#undef FLUXB_RANKS
}

}  // namespace fluxb

using namespace fluxb;

extern "C" {

int fluxb_comm_set_ranks_on_gpu(fluxb_comm_t comm, int nranks) {
  FLUXB_REQUIRE(comm != nullptr, "set_ranks_on_gpu: comm is NULL");
  FLUXB_REQUIRE(nranks >= 1 && nranks <= kMaxWorld, "set_ranks_on_gpu: nranks=%d out of [1,%d]", nranks, kMaxWorld);
  FLUXB_REQUIRE(comm->deferred.empty(), "set_ranks_on_gpu: %zu queued items are still waiting for fluxb_run_ranks",
                comm->deferred.size());
  if (nranks > 1 && comm->ranks_params_dev == nullptr) {
    const size_t bytes = sizeof(GemmParams) * kMaxRankItems * kMaxWorld;
    FLUXB_CUDA(cudaMalloc(reinterpret_cast<void**>(&comm->ranks_params_dev), bytes));
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&comm->ranks_params_host), bytes, cudaHostAllocDefault);
    if (e != cudaSuccess) {
      cudaFree(comm->ranks_params_dev);
      comm->ranks_params_dev = nullptr;
      FLUXB_FAIL(FLUXB_ERR_CUDA, "cudaHostAlloc(rank parameter staging) failed: %s", cudaGetErrorString(e));
    }
  }
  comm->ranks_on_gpu = nranks;
  return FLUXB_OK;
}

int fluxb_run_ranks(fluxb_comm_t const* comms, int nranks, fluxb_stream_t stream_) {
  FLUXB_REQUIRE(comms != nullptr && nranks >= 2 && nranks <= kMaxWorld, "run_ranks: bad argument (nranks=%d)", nranks);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  for (int r = 0; r < nranks; ++r)
    FLUXB_REQUIRE(comms[r] != nullptr && comms[r]->ranks_on_gpu == nranks,
                  "run_ranks: communicator %d is NULL or was not set up for %d ranks on one GPU", r, nranks);
  fluxb_comm* c0 = comms[0];
  const size_t nitems = c0->deferred.size();
  int rc = FLUXB_OK;
  int fused_seen = 0;
  for (int r = 1; r < nranks && rc == FLUXB_OK; ++r)
    if (comms[r]->deferred.size() != nitems) {
      set_error("run_ranks: rank 0 queued %zu items, rank %d queued %zu (every rank must make the same calls)", nitems,
                r, comms[r]->deferred.size());
      rc = FLUXB_ERR_INVALID;
    }
  for (size_t i = 0; i < nitems && rc == FLUXB_OK; ++i) {
    const DeferredItem& a = c0->deferred[i];
    if (!a.fused) {
      for (int r = 0; r < nranks && rc == FLUXB_OK; ++r) {
        const DeferredItem& it = comms[r]->deferred[i];
        if (it.fused) {
          set_error("run_ranks: item %zu is a fused launch on rank %d but not on rank 0", i, r);
          rc = FLUXB_ERR_INVALID;
        } else {
          rc = it.plain(stream);
        }
      }
      continue;
    }
    if (fused_seen >= kMaxRankItems) {
      set_error("run_ranks: more than %d fused launches queued", kMaxRankItems);
      rc = FLUXB_ERR_INVALID;
      break;
    }
    GemmParams* host = c0->ranks_params_host + static_cast<size_t>(fused_seen) * kMaxWorld;
    GemmParams* dev = c0->ranks_params_dev + static_cast<size_t>(fused_seen) * kMaxWorld;
    int per = a.grid;
    for (int r = 0; r < nranks && rc == FLUXB_OK; ++r) {
      const DeferredItem& it = comms[r]->deferred[i];
      if (!it.fused || it.bn != a.bn || it.kind != a.kind || it.cta_group != a.cta_group || it.idesc != a.idesc) {
        set_error("run_ranks: item %zu differs between rank 0 and rank %d (tile shape or dtype)", i, r);
        rc = FLUXB_ERR_INVALID;
        break;
      }
      if (it.grid < per) per = it.grid;
      host[r] = it.p;
    }
    if (rc != FLUXB_OK) break;
    if (a.cta_group == 2) per &= ~1;
    if (per < a.cta_group) {
      set_error("run_ranks: no CTAs left per rank");
      rc = FLUXB_ERR_INVALID;
      break;
    }
    cudaError_t e = cudaMemcpyAsync(dev, host, sizeof(GemmParams) * nranks, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) {
      set_error("run_ranks: parameter upload failed: %s", cudaGetErrorString(e));
      rc = FLUXB_ERR_CUDA;
      break;
    }
    rc = launch_ranks_kernel(a.bn, a.kind, a.cta_group, dev, nranks, per, a.idesc, stream);
    fused_seen += 1;
  }
  // the pinned staging is reused by the next call: wait until this call's uploads have been read
  if (fused_seen > 0 && cudaStreamSynchronize(stream) != cudaSuccess && rc == FLUXB_OK) {
    set_error("run_ranks: the stream reported an error after the launches");
    rc = FLUXB_ERR_CUDA;
  }
  for (int r = 0; r < nranks; ++r) comms[r]->deferred.clear();
  return rc;
}

}  // extern "C"
