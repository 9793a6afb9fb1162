// Thin inline-PTX wrappers for the Blackwell (sm_100a) primitives the fused
// kernels use: mbarrier, TMA (cp.async.bulk.tensor, never with cluster
// multicast), tcgen05 (TMEM alloc, UMMA, commit, ld) and the system-scope
// flag operations that order peer-GPU traffic.
//
// Every wait in this file is bounded: it polls, checks a CTA-wide abort word
// and a wall-clock budget, and returns false instead of spinning forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fluxb {

// ----------------------------------------------------------------------------
// status codes written by kernels into the status word (0 = ok)
// ----------------------------------------------------------------------------
enum : int {
  kStatusOk = 0,
  kStatusTimeoutSmemFull = 1,   // MMA warp: operand stage never became full
  kStatusTimeoutSmemEmpty = 2,  // TMA warp: operand stage never drained
  kStatusTimeoutTmemFull = 3,   // epilogue: accumulator never completed
  kStatusTimeoutTmemEmpty = 4,  // MMA warp: accumulator never drained
  kStatusTimeoutFlag = 5,       // a peer's arrival flag never reached its value
  kStatusTimeoutBarrier = 6,    // all-rank barrier kernel gave up
  kStatusTimeoutReduce = 7,     // reduce-scatter tail: partial tiles missing
  kStatusBadTable = 8,          // grouped GEMM: tile table is inconsistent
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// The suspend-time hint lets the hardware park the thread (up to that many nanoseconds) until the
// phase completes, instead of returning at once: a waiting role then costs no issue slots or power,
// and still wakes up as soon as the barrier flips.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(20000u)
      : "memory");
  return ok != 0;
}

// The abort word of a CTA: non-zero means some role has given up, and every other role must leave
// its loop too. In a CTA pair the word of the partner CTA is raised as well (a store through
// distributed shared memory; `peer` is the cluster address of the partner's word, 0 = no partner),
// so that the partner does not have to run into a timeout of its own.
struct AbortWord {
  volatile int* local;
  uint32_t peer;
};
__device__ __forceinline__ void abort_raise(const AbortWord& ab, int code) {
  if (ab.local == nullptr) return;
  atomicCAS(const_cast<int*>(ab.local), 0, code);
  if (ab.peer != 0u)
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(ab.peer), "r"(code) : "memory");
}
__device__ __forceinline__ bool abort_seen(const AbortWord& ab) {
  return ab.local != nullptr && *ab.local != 0;
}

// Bounded mbarrier wait.
// `backoff_ns` > 0 sleeps between polls: for waits that normally last many microseconds (an
// accumulator that is still being computed), so that idle warps do not burn issue slots and power.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortWord& ab,
                                          int code, uint64_t budget_ns, uint32_t backoff_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t n = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (backoff_ns != 0) __nanosleep(backoff_ns);
    if ((++n & 31u) == 0u) {
      if (abort_seen(ab)) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        abort_raise(ab, code);
        return false;
      }
    }
  }
  return true;
}

// ----------------------------------------------------------------------------
// proxy / scope fences
// ----------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// ----------------------------------------------------------------------------
// system-scope flags (live in symmetric memory, written by peers)
// ----------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void red_add_release_gpu(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// 16-byte load that is not served from a stale L1 line (data another SM stored earlier in this launch)
__device__ __forceinline__ uint4 ld_relaxed_gpu_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Bounded wait until *flag == want (acquire, system scope).
__device__ __forceinline__ bool flag_wait_eq(const int* flag, int want, const AbortWord& ab,
                                             int code, uint64_t budget_ns) {
  if (ld_acquire_sys(flag) == want) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t n = 0;
  while (ld_acquire_sys(flag) != want) {
    __nanosleep(64);
    if ((++n & 15u) == 0u) {
      if (abort_seen(ab)) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        abort_raise(ab, code);
        return false;
      }
    }
  }
  return true;
}

// ----------------------------------------------------------------------------
// TMA (tiled tensor copies global -> shared). No multicast anywhere.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// x = innermost (element) coordinate, y = row coordinate.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tmap, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// Four independent rows (y0..y3) of one 2-D tensor, `box_x` elements each,
// land as four consecutive smem rows.
__device__ __forceinline__ void tma_gather4_2d(uint32_t smem_dst, const void* tmap, uint32_t bar,
                                               int x, int y0, int y1, int y2, int y3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y0), "r"(y1),
        "r"(y2), "r"(y3)
      : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: tensor memory + UMMA
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// arrives (count 1) on `bar` once every tcgen05.mma issued so far by this thread has retired
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, 16-bit inputs (f16/bf16), fp32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// same for 8-bit float inputs (e4m3/e5m2)
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// same for signed 8-bit integer inputs, int32 accumulate
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread `lane` receives row
// (taddr.lane + lane), columns taddr.col .. +31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------
// CTA pairs (cluster of 2): the even CTA ("leader") issues cta_group::2 UMMAs
// that read both CTAs' shared memory and write both CTAs' tensor memory.
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory object in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// arrives on `bar` (same offset) in every CTA of `cta_mask` once the UMMAs issued so far retire
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}
__device__ __forceinline__ void umma_f16_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f8_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// TMA loads of a CTA pair: data lands in this CTA's shared memory, the byte count is credited
// to `bar_cluster_addr`, a barrier of the leader CTA (cluster address). No multicast.
__device__ __forceinline__ void tma_load_2d_2cta(uint32_t smem_dst, const void* tmap,
                                                 uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_gather4_2d_2cta(uint32_t smem_dst, const void* tmap,
                                                    uint32_t bar_cluster_addr, int x, int y0, int y1,
                                                    int y2, int y3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y0),
        "r"(y1), "r"(y2), "r"(y3)
      : "memory");
}

// ----------------------------------------------------------------------------
// bulk copies shared -> global (used to push row segments to peer memory in
// full 128-byte pieces instead of per-lane 16-byte stores)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src),
               "r"(bytes)
               : "memory");
}
// 2-D tiled store shared -> global (tensor map decides box and swizzle; out-of-range parts are clipped)
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the shared-memory sources of all committed groups have been read
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... of all but the most recent committed group
__device__ __forceinline__ void bulk_wait_read_keep1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// all committed groups are complete (their global writes are performed)
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// all committed groups except the most recent N are complete
template <int N>
__device__ __forceinline__ void bulk_wait_all_but() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------
// descriptors
// ----------------------------------------------------------------------------
// Shared-memory operand descriptor for a K-major tile whose rows are exactly
// one 128-byte swizzle span (64 bf16 or 128 fp8): rows are 128 B apart,
// groups of 8 rows are 1024 B apart (stride byte offset), the tile base is
// 1024-byte aligned, and TMA wrote it with CU_TENSOR_MAP_SWIZZLE_128B.
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) descriptor version (1)
//   bits [61,64) swizzle mode (2 = 128 B)
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Shared-memory operand descriptor for an MN-major tile (the operand is stored [K][MN] with MN
// contiguous): TMA wrote it as boxes of 64 elements of MN (128 B) x `k` rows with 128-byte swizzle, one
// box after the other. Inside a box the K rows are 128 B apart and groups of 8 rows 1024 B (stride byte
// offset); the next 64 elements of MN start one box later (leading byte offset = box_bytes).
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t box_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((box_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor (dense, both operands K-major unless b_mn_major).
//   [4,6) D format (1 = f32, 2 = s32)   [7,10) A format   [10,13) B format
//   [15] A major (0 = K)       [16] B major (0 = K)
//   [17,23) N >> 3             [24,29) M >> 4
// A/B format: kind::f16 -> 0 = f16, 1 = bf16; kind::f8f6f4 -> 0 = e4m3, 1 = e5m2; kind::i8 -> 0 = u8, 1 = s8
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t m, uint32_t n,
                                                  uint32_t b_mn_major = 0, uint32_t d_format = 1) {
  return (d_format << 4) | (ab_format << 7) | (ab_format << 10) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

}  // namespace fluxb
