// Runtime of the library: error text, communicator, symmetric memory through
// CUDA IPC handles, the bounded all-rank barrier, tensor-map encoding.
// Stands in for src/ths_op/flux_shm.cc and src/cuda/cudaipc_barrier_all.cu of
// the reference (no NVSHMEM, no NCCL).
#include <string.h>

#include "internal.h"

namespace fluxb {

static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved at run time so that the library loads on
// machines without a driver (build hosts, symbol checks).
static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn != nullptr) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || ptr == nullptr) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elt_dtype, long long rows, long long k,
                   long long ld_bytes, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const int eb = dtype_bytes(elt_dtype);
  FLUXB_REQUIRE(eb == 1 || eb == 2, "tensor map: unsupported element type %d", elt_dtype);
  FLUXB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0,
                "tensor map: base address must be 16-byte aligned");
  FLUXB_REQUIRE((ld_bytes & 15) == 0, "tensor map: row pitch (%lld bytes) must be a multiple of 16",
                ld_bytes);
  FLUXB_REQUIRE(rows > 0 && k > 0, "tensor map: empty matrix");
  CUtensorMapDataType dt = eb == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : (elt_dtype == FLUXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / eb), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld k=%lld ld=%lld box_rows=%d)",
               static_cast<int>(r), rows, k, ld_bytes, box_rows);
  return FLUXB_OK;
}

int encode_tmap_kn(CUtensorMap* out, const void* base, int elt_dtype, long long k, long long n, long long ld_bytes,
                   int box_k) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  FLUXB_REQUIRE(dtype_bytes(elt_dtype) == 2, "[K,N] weights need a 16-bit element type");
  FLUXB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0 && (ld_bytes & 15) == 0 && k > 0 && n > 0,
                "[K,N] tensor map: base and row pitch must be 16-byte aligned");
  CUtensorMapDataType dt = elt_dtype == FLUXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(k)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_bytes)};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_k)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled ([K,N] map) failed with CUresult %d", static_cast<int>(r));
  return FLUXB_OK;
}

int encode_tmap_f32_store(CUtensorMap* out, const void* base, long long rows, long long n) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  FLUXB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0 && (n * 4) % 16 == 0 && rows > 0 && n > 0,
                "store tensor map: base and row pitch must be 16-byte aligned (rows=%lld n=%lld)", rows, n);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(n) * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled (store map) failed with CUresult %d", static_cast<int>(r));
  return FLUXB_OK;
}

// Store map over a [rows, n] matrix of 16-bit elements: 32-row x 64-column boxes (128-byte rows, 128-byte swizzle).
int encode_tmap_b16_store(CUtensorMap* out, const void* base, long long rows, long long n) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  FLUXB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0 && (n * 2) % 16 == 0 && rows > 0 && n > 0,
                "store tensor map: base and row pitch must be 16-byte aligned (rows=%lld n=%lld)", rows, n);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(n) * 2};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled (16-bit store map) failed with CUresult %d", static_cast<int>(r));
  return FLUXB_OK;
}

// One block, one thread per peer. Epoch-valued handshake: rank r stores the
// epoch into slot r of every peer's array, then waits until every slot of its
// own array has reached the epoch. Values only grow, so nothing is reset.
__global__ void barrier_all_kernel(int* const* sync_bufs_unused, int* b0, int* b1, int* b2, int* b3,
                                   int* b4, int* b5, int* b6, int* b7, int rank, int world,
                                   int epoch, int* status, unsigned long long budget_ns) {
  int* bufs[kMaxWorld] = {b0, b1, b2, b3, b4, b5, b6, b7};
  const int peer = threadIdx.x;
  if (peer >= world) return;
  __threadfence_system();
  st_release_sys(bufs[peer] + rank, epoch);
  const int* mine = bufs[rank] + peer;
  const uint64_t t0 = globaltimer_ns();
  uint32_t n = 0;
  while (ld_acquire_sys(mine) < epoch) {
    __nanosleep(100);
    if ((++n & 15u) == 0u && globaltimer_ns() - t0 > budget_ns) {
      *reinterpret_cast<volatile int*>(status) = kStatusTimeoutBarrier;
      __threadfence_system();
      return;
    }
  }
}

}  // namespace fluxb

using namespace fluxb;

extern "C" {

const char* fluxb_last_error(void) { return g_err; }
int fluxb_version(void) { return 100; }

int fluxb_device_supported(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

int fluxb_comm_create(int rank, int world, fluxb_comm_t* out) {
  FLUXB_REQUIRE(out != nullptr, "comm_create: out is NULL");
  FLUXB_REQUIRE(world >= 1 && world <= FLUXB_MAX_WORLD, "comm_create: world=%d out of [1,%d]", world,
                FLUXB_MAX_WORLD);
  FLUXB_REQUIRE(rank >= 0 && rank < world, "comm_create: rank=%d out of [0,%d)", rank, world);
  FLUXB_REQUIRE((world & (world - 1)) == 0, "comm_create: world=%d must be a power of two", world);
  int dev = 0;
  FLUXB_CUDA(cudaGetDevice(&dev));
  int major = 0, sms = 0;
  FLUXB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  FLUXB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (major != 10)
    FLUXB_FAIL(FLUXB_ERR_UNSUPPORTED,
               "comm_create: device %d has compute capability %d.x; this library only holds "
               "sm_100a code and has no fallback",
               dev, major);
  fluxb_comm* c = new fluxb_comm();
  c->rank = rank;
  c->world = world;
  c->device = dev;
  c->sm_count = sms;
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&c->status_host), 64, cudaHostAllocMapped);
  if (e != cudaSuccess) {
    delete c;
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cudaHostAlloc(status) failed: %s", cudaGetErrorString(e));
  }
  memset(c->status_host, 0, 64);
  e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_dev), c->status_host, 0);
  if (e != cudaSuccess) {
    cudaFreeHost(c->status_host);
    delete c;
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cudaHostGetDevicePointer failed: %s", cudaGetErrorString(e));
  }
  // scratch of the split-K tail: one 128 x 256 fp32 tile per SM bounds every launch's need
  const size_t sk_bytes = static_cast<size_t>(sms) * kBM * 256 * sizeof(float);
  const size_t cnt_bytes = static_cast<size_t>(sms) * 16 * sizeof(int);  // "parked" and "seen" counters
  if (cudaMalloc(reinterpret_cast<void**>(&c->splitk_scratch), sk_bytes) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&c->splitk_cnt), cnt_bytes) != cudaSuccess ||
      cudaMemset(c->splitk_cnt, 0, cnt_bytes) != cudaSuccess) {
    cudaGetLastError();
    if (c->splitk_scratch != nullptr) cudaFree(c->splitk_scratch);
    if (c->splitk_cnt != nullptr) cudaFree(c->splitk_cnt);
    cudaFreeHost(c->status_host);
    delete c;
    FLUXB_FAIL(FLUXB_ERR_CUDA, "could not allocate the split-K scratch (%zu bytes)", sk_bytes);
  }
  *out = c;
  return FLUXB_OK;
}

int fluxb_comm_destroy(fluxb_comm_t comm) {
  if (comm == nullptr) return FLUXB_OK;
  if (comm->splitk_scratch != nullptr) cudaFree(comm->splitk_scratch);
  if (comm->splitk_cnt != nullptr) cudaFree(comm->splitk_cnt);
  if (comm->ranks_params_dev != nullptr) cudaFree(comm->ranks_params_dev);
  if (comm->ranks_params_host != nullptr) cudaFreeHost(comm->ranks_params_host);
  if (comm->status_host != nullptr) cudaFreeHost(comm->status_host);
  delete comm;
  return FLUXB_OK;
}

int fluxb_comm_set_timeout_ms(fluxb_comm_t comm, int timeout_ms) {
  FLUXB_REQUIRE(comm != nullptr, "set_timeout: comm is NULL");
  FLUXB_REQUIRE(timeout_ms > 0 && timeout_ms <= 600000, "set_timeout: %d ms out of (0, 600000]",
                timeout_ms);
  comm->timeout_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  return FLUXB_OK;
}

int fluxb_comm_set_trace(fluxb_comm_t comm, void* device_buffer) {
  FLUXB_REQUIRE(comm != nullptr, "set_trace: comm is NULL");
  comm->trace = static_cast<unsigned long long*>(device_buffer);
  return FLUXB_OK;
}

int fluxb_status_peek(fluxb_comm_t comm, int* status) {
  FLUXB_REQUIRE(comm != nullptr && status != nullptr, "status_peek: NULL argument");
  *status = *reinterpret_cast<volatile int*>(comm->status_host);
  return FLUXB_OK;
}

int fluxb_status_clear(fluxb_comm_t comm) {
  FLUXB_REQUIRE(comm != nullptr, "status_clear: comm is NULL");
  *reinterpret_cast<volatile int*>(comm->status_host) = 0;
  // a launch that gave up may have left the split-K tail's self-clearing counters part-way
  if (comm->splitk_cnt != nullptr) {
    int cur = -1;
    FLUXB_CUDA(cudaGetDevice(&cur));
    if (cur != comm->device) FLUXB_CUDA(cudaSetDevice(comm->device));
    const cudaError_t e = cudaMemset(comm->splitk_cnt, 0, static_cast<size_t>(comm->sm_count) * 16 * sizeof(int));
    if (cur != comm->device) cudaSetDevice(cur);
    FLUXB_CUDA(e);
  }
  return FLUXB_OK;
}

int fluxb_symm_alloc(size_t bytes, void** local_ptr, void* ipc_handle_out) {
  FLUXB_REQUIRE(local_ptr != nullptr, "symm_alloc: local_ptr is NULL");
  FLUXB_REQUIRE(bytes > 0, "symm_alloc: zero bytes");
  void* p = nullptr;
  FLUXB_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cudaMemset failed: %s", cudaGetErrorString(e));
  }
  if (ipc_handle_out != nullptr) {
    static_assert(sizeof(cudaIpcMemHandle_t) == FLUXB_IPC_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
      cudaFree(p);
      FLUXB_FAIL(FLUXB_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    }
    memcpy(ipc_handle_out, &h, sizeof(h));
  }
  *local_ptr = p;
  return FLUXB_OK;
}

int fluxb_symm_free(void* local_ptr) {
  if (local_ptr != nullptr) FLUXB_CUDA(cudaFree(local_ptr));
  return FLUXB_OK;
}

int fluxb_symm_open(const void* ipc_handle, void** peer_ptr) {
  FLUXB_REQUIRE(ipc_handle != nullptr && peer_ptr != nullptr, "symm_open: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  FLUXB_CUDA(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FLUXB_OK;
}

int fluxb_symm_close(void* peer_ptr) {
  if (peer_ptr != nullptr) FLUXB_CUDA(cudaIpcCloseMemHandle(peer_ptr));
  return FLUXB_OK;
}

int fluxb_enable_peer_access(int device, int peer_device) {
  if (device == peer_device) return FLUXB_OK;
  int prev = 0;
  FLUXB_CUDA(cudaGetDevice(&prev));
  int can = 0;
  FLUXB_CUDA(cudaDeviceCanAccessPeer(&can, device, peer_device));
  FLUXB_REQUIRE(can == 1, "device %d cannot access device %d", device, peer_device);
  FLUXB_CUDA(cudaSetDevice(device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    e = cudaSuccess;
  }
  cudaSetDevice(prev);
  if (e != cudaSuccess)
    FLUXB_FAIL(FLUXB_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d -> %d) failed: %s", device, peer_device,
               cudaGetErrorString(e));
  return FLUXB_OK;
}

int fluxb_barrier_all(fluxb_comm_t comm, int* const* sync_bufs, fluxb_stream_t stream) {
  FLUXB_REQUIRE(comm != nullptr && sync_bufs != nullptr, "barrier_all: NULL argument");
  int* b[kMaxWorld] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int r = 0; r < comm->world; ++r) {
    FLUXB_REQUIRE(sync_bufs[r] != nullptr, "barrier_all: sync_bufs[%d] is NULL", r);
    b[r] = sync_bufs[r];
  }
  comm->barrier_epoch += 1;
  barrier_all_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      nullptr, b[0], b[1], b[2], b[3], b[4], b[5], b[6], b[7], comm->rank, comm->world,
      comm->barrier_epoch, comm->status_dev, comm->timeout_ns);
  FLUXB_CUDA(cudaGetLastError());
  return FLUXB_OK;
}

}  // extern "C"
