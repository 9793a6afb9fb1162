/*
 * fluxb.h - C ABI of the B200-native fused tensor-parallel GEMM library.
 *
 * Plain C: opaque handles, raw device pointers and sizes, no torch types.
 * Every function returns FLUXB_OK (0) or a negative error code and stores a
 * message retrievable with fluxb_last_error() (thread local). Nothing here
 * falls back to a CPU or library path: if the GPU code cannot run, the call
 * fails.
 *
 * One process drives one GPU (the usual case, peers mapped through CUDA IPC
 * handles exchanged by the caller), or one process drives several GPUs with
 * peer access enabled (test harnesses): the entry points only see pointer
 * tables, one pointer per rank, valid in the calling process.
 *
 * Each entry point names the reference interface it stands in for, by the
 * file's path inside bytedance/flux.
 */
#ifndef FLUXB_H_
#define FLUXB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLUXB_OK 0
#define FLUXB_ERR_INVALID (-1)     /* bad argument / shape / dtype              */
#define FLUXB_ERR_CUDA (-2)        /* a CUDA runtime or driver call failed      */
#define FLUXB_ERR_TIMEOUT (-3)     /* a bounded device wait expired             */
#define FLUXB_ERR_UNSUPPORTED (-4) /* valid in the reference, not built here    */

#define FLUXB_MAX_WORLD 8 /* ranks of one NVSwitch domain (include/flux/flux.h:53 kMaxLocalWorldSize) */
#define FLUXB_IPC_HANDLE_BYTES 64

/* element types (include/flux/flux.h DataTypeEnum) */
#define FLUXB_BF16 0
#define FLUXB_F16 1
#define FLUXB_F32 2
#define FLUXB_E4M3 3
#define FLUXB_E5M2 4
#define FLUXB_S8 5 /* w8a8: int8 operands, int32 accumulation, output = (scale_a[m] * scale_b[n]) * acc in the 16-bit
                      output type (AGS8KernelArguments, include/flux/args/ag_gemm.h:38-54) */

/* bias layouts (src/ag_gemm/ths_op/gemm_with_barrier.cc:201-205) */
#define FLUXB_BIAS_NONE 0
#define FLUXB_BIAS_MN 1 /* [M,N], added elementwise        */
#define FLUXB_BIAS_1N 2 /* [1,N], broadcast over rows      */

/* `flags` of the GEMM entry points */
#define FLUXB_WEIGHT_KN 1 /* the weight is [K,N] with N contiguous ("RRR", transpose_weight=True in the
                             reference, src/ag_gemm/ths_op/gemm_with_barrier.cc:55,196-197); 16-bit inputs only */
#define FLUXB_RS_FP32_WIRE 2 /* fluxb_gemm_rs_forward: send the partial sums to their owner as fp32 instead of
                                the 16-bit output format (the reference reduces in the output format,
                                src/gemm_rs/ths_op/gemm_reduce_scatter.cc:335-899); twice the NVLink bytes */

#define FLUXB_RS_RING_ORDER 4 /* fluxb_gemm_rs_forward: reduce in the order and precision of the reference's
                                `ring_reduction` (src/gemm_rs/ring_reduce.cu:54-80): partials of rank+1, rank+2, ...,
                                own partial last, the running sum rounded to the 16-bit element type after every
                                addition. Default: the same order, summed in fp32 and rounded once. */

typedef struct fluxb_comm* fluxb_comm_t;
typedef struct fluxb_ag_gemm* fluxb_ag_gemm_t;
typedef struct fluxb_gemm_rs* fluxb_gemm_rs_t;
typedef struct fluxb_moe_ag_scatter* fluxb_moe_ag_scatter_t;
typedef struct fluxb_moe_gather_rs* fluxb_moe_gather_rs_t;
typedef void* fluxb_stream_t; /* a cudaStream_t */

/* Optional launch tuning; zero in a field means "choose for me". */
typedef struct fluxb_tuning {
  int block_n;  /* output tile width: 64, 128, 192 or 256             */
  int group_m;  /* rasterisation band height, in 128-row tiles         */
  int num_ctas; /* persistent grid size (<= SM count)                  */
  int cta_group; /* 1 = one CTA per 128-row tile, 2 = CTA pair per 256-row tile */
  int ag_mode;  /* transport of the all-gather: 1 = pushed by the fused kernel's communication warps (units of 32
                   rows x 2 KB per system-scope release; 3 = units of 64 rows, 4 = units of 128 rows), 2 = copy
                   engines on a side stream (AllGatherOption.use_cuda_core_ag = true / false in the reference,
                   src/coll/ths_op/all_gather_types.h:35-43); the consuming kernel is the same; 0 = the environment variable
                   FLUXB_AG_MODE (1 or 2) if set, else 1 */
} fluxb_tuning;

const char* fluxb_last_error(void);
int fluxb_version(void);
/* 1 when the library holds sm_100a code and a device that can run it is current. */
int fluxb_device_supported(void);

/* ------------------------------------------------------------------ runtime
 * Replaces src/ths_op/flux_shm.cc (init_flux_shm :379-408,
 * cudaipc_create_tensor_list :275-366, GroupBarrier :656-733) and
 * src/cuda/cudaipc_barrier_all.cu:45-113. Handle exchange between processes
 * is the caller's job (any byte transport; the torch binding uses the
 * process group, as Group::all_gather_cpu does, flux_shm.cc:161-168). */
int fluxb_comm_create(int rank, int world, fluxb_comm_t* out);
int fluxb_comm_destroy(fluxb_comm_t comm);
int fluxb_comm_set_timeout_ms(fluxb_comm_t comm, int timeout_ms);
/* Optional timeline of the fused kernel (the reference has only host-side profiling,
 * python/flux/util.py:111-172): device_buffer = 8 x uint64 per CTA (64 B x SM count), filled by every
 * later launch with %globaltimer stamps: kernel start, first operands landed, last UMMA issued, epilogue
 * done, comm warps done, ns waited on arrival flags, ns waited on peers-summed flags, work items.
 * NULL switches it off (default). */
int fluxb_comm_set_trace(fluxb_comm_t comm, void* device_buffer);
/* Device-written status word: 0 = ok, else the code of the wait that expired. */
int fluxb_status_peek(fluxb_comm_t comm, int* status);
int fluxb_status_clear(fluxb_comm_t comm);

int fluxb_symm_alloc(size_t bytes, void** local_ptr, void* ipc_handle_out /* 64 bytes */);
int fluxb_symm_free(void* local_ptr);
int fluxb_symm_open(const void* ipc_handle /* 64 bytes */, void** peer_ptr);
int fluxb_symm_close(void* peer_ptr);
/* single-process multi-GPU harnesses: let `device` access `peer_device` */
int fluxb_enable_peer_access(int device, int peer_device);

/* All-rank barrier on a stream. sync_bufs[r] points at rank r's sync array
 * (>= 2*FLUXB_MAX_WORLD ints, zero-initialised once). Bounded: expiry sets
 * the status word and the kernel returns. */
int fluxb_barrier_all(fluxb_comm_t comm, int* const* sync_bufs, fluxb_stream_t stream);

/* Several ranks on ONE GPU (machines with fewer GPUs than ranks; the reference's C++ unit test drives all
 * ranks from one process in the same spirit, src/gemm_rs/test/test_gemm_rs.cc:43-130). Kernels of different
 * ranks wait on one another's flags, so they cannot be separate launches on one GPU. After
 * fluxb_comm_set_ranks_on_gpu(comm, n) on each of the n communicators (rank r of world n, all on the current
 * device, pointer tables filled with local allocations), the forward calls only queue their stream work;
 * fluxb_run_ranks(comms, n, stream) then issues every rank's queued fused launch as ONE cooperative launch in
 * which each rank owns 1/n of the grid, and the other queued work rank by rank. Every rank must have made
 * the same calls in the same order. The call synchronises the stream. n = 1 switches back to normal. */
int fluxb_comm_set_ranks_on_gpu(fluxb_comm_t comm, int nranks);
int fluxb_run_ranks(fluxb_comm_t const* comms, int nranks, fluxb_stream_t stream);

/* -------------------------------------------------------------- plain GEMM
 * C[M,N] = alpha * (A[M,K] . B[N,K]^T) * scale_a[m] * scale_b[n] + bias.
 * The TP=1 degenerate of both fused ops; also what AGKernel.gemm_only runs
 * (src/ag_gemm/ths_op/all_gather_gemm_op.cc:166-194). A and B are row-major
 * with K contiguous. scale_a / scale_b may be NULL. */
int fluxb_gemm(fluxb_comm_t comm, const void* a, const void* b, void* c, int m, int n, int k,
               int in_dtype, int out_dtype, const void* bias, int bias_mode, const float* scale_a,
               const float* scale_b, float alpha, int flags, const fluxb_tuning* tuning, fluxb_stream_t stream);

/* ----------------------------------------------------------------- AG-GEMM
 * Replaces AllGatherGemmOp (src/ag_gemm/ths_op/all_gather_gemm_op.cc:97-123
 * ctor, :132-163 forward) together with AllGatherOp
 * (src/coll/ths_op/all_gather_op.cc:193-276, :352-404).
 *
 * Symmetric buffers (one per rank, same size on every rank, zero-filled
 * before the first forward and followed by an all-rank barrier):
 *   gather_bufs[r]: fluxb_ag_gemm_gather_bytes(...) bytes
 *   flag_bufs[r]  : fluxb_ag_gemm_flag_bytes(...) bytes
 *   scale_bufs[r] : fluxb_ag_gemm_scale_bytes(...) bytes, or NULL table if the
 *                   op never receives per-row input scales                   */
size_t fluxb_ag_gemm_gather_bytes(int full_m, int k_dim, int in_dtype);
size_t fluxb_ag_gemm_flag_bytes(int full_m, int world);
size_t fluxb_ag_gemm_scale_bytes(int full_m);
int fluxb_ag_gemm_create(fluxb_comm_t comm, int full_m, int n_dim, int k_dim, int in_dtype,
                         int out_dtype, void* const* gather_bufs, int* const* flag_bufs,
                         float* const* scale_bufs, fluxb_ag_gemm_t* out);
int fluxb_ag_gemm_destroy(fluxb_ag_gemm_t op);
/* Re-arm after a call that ended with a non-zero status word (a bounded wait expired, so arrival counters
 * hold partial counts): clears this rank's counters of both buffer parities and restarts the parity
 * sequence. Collective: every rank calls it, with an all-rank barrier (fluxb_barrier_all or the caller's)
 * before the next forward. The reference has no recovery path: its waits are unbounded
 * (include/flux/cuda/system_barrier.hpp:66-103). The other ops have the same call. */
int fluxb_ag_gemm_reset(fluxb_ag_gemm_t op, fluxb_stream_t stream);
/* c[M, n] = all_gather(a_shard)[M, k] . b[n, k]^T, M = m_local * world.
 * scale_a_shard: [m_local] fp32 or NULL; scale_b: [n] fp32 or NULL.
 * gathered_out: optional [M,k] device buffer that receives the gathered input
 * (all_gather_gemm_op.cc:292-301). Collective: every rank calls with the same
 * m_local, n, k. Asynchronous on `stream`. */
int fluxb_ag_gemm_forward(fluxb_ag_gemm_t op, const void* a_shard, int m_local, const void* b,
                          int n, int k, void* c, const void* bias, int bias_mode,
                          const float* scale_a_shard, const float* scale_b, float alpha, int flags,
                          void* gathered_out, const fluxb_tuning* tuning, fluxb_stream_t stream);

/* ----------------------------------------------------------------- GEMM-RS
 * Replaces GemmRS (src/gemm_rs/ths_op/gemm_reduce_scatter.cc:335-408 ctor,
 * :552-660 forward_gemm_impl, :690-788 forward_reduce_scatter_impl).
 *   stage_bufs[r]: fluxb_gemm_rs_stage_bytes(...)   (partial tiles, slots of fp32 size)
 *   cnt_bufs[r]  : fluxb_gemm_rs_cnt_bytes(...)     (per-tile arrival counters) */
size_t fluxb_gemm_rs_stage_bytes(int max_m, int n_dim, int world);
size_t fluxb_gemm_rs_cnt_bytes(int max_m, int n_dim, int world);
int fluxb_gemm_rs_create(fluxb_comm_t comm, int max_m, int n_dim, int in_dtype, int out_dtype,
                         float* const* stage_bufs, int* const* cnt_bufs, fluxb_gemm_rs_t* out);
int fluxb_gemm_rs_destroy(fluxb_gemm_rs_t op);
/* GemmRS::zero_buffers (src/gemm_rs/ths_op/gemm_reduce_scatter.cc:654-657); see fluxb_ag_gemm_reset. */
int fluxb_gemm_rs_reset(fluxb_gemm_rs_t op, fluxb_stream_t stream);
/* out[m/world, n] = reduce_scatter_rows( a[m, k_local] . b[n, k_local]^T (+ bias) ).
 * With a 16-bit output the partials travel to the owner of their rows in that
 * format, as in the reference, are summed there in fp32 and rounded once more;
 * FLUXB_RS_FP32_WIRE in `flags` (or an fp32 output) sends them as fp32. */
int fluxb_gemm_rs_forward(fluxb_gemm_rs_t op, const void* a, const void* b, int m, int n,
                          int k_local, void* out, const void* bias, int bias_mode,
                          const float* scale_a, const float* scale_b, float alpha, int flags,
                          const fluxb_tuning* tuning, fluxb_stream_t stream);

/* ---------------------------------------------------------- MoE index work
 * Integer routing helpers, bit-exact against the reference's stable forms.
 * fluxb_moe_scatter_index: stable scatter index + splits from the chosen
 * experts (python/flux/testing/moe_utils.py:141-144 calc_scatter_index_stable;
 * device counterpart src/cuda/moe_utils.cu:23-75 calc_scatter_index, whose
 * order inside an expert is not deterministic).
 * fluxb_moe_gather_index: inverse permutation (src/moe_ag_scatter/sort_util.cu:39-92). */
int fluxb_moe_scatter_index(const int* chosen_experts, int ntokens, int topk, int nexperts,
                            int* splits_out, int* scatter_index_out, fluxb_stream_t stream);
int fluxb_moe_gather_index(const int* scatter_index, int ntokens, int topk, int* gather_index_out,
                           int* topk_index_out, fluxb_stream_t stream);

/* ------------------------------------------------------ MoE AG + scatter
 * Replaces GemmGroupedV3AGScatterOp
 * (src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc:112-126, :227-447).
 * out[scatter_index[t,k], :] = token_t . W[expert]^T * out_scale[expert].
 * gather_bufs / flag_bufs sized with the fluxb_ag_gemm_* helpers
 * (full_m = max_ntokens, k_dim = hidden). */
size_t fluxb_moe_ag_scatter_workspace_bytes(int max_ntokens, int topk, int nexperts, int hidden, int in_dtype);
int fluxb_moe_ag_scatter_create(fluxb_comm_t comm, int max_ntokens, int hidden, int ffn_local,
                                int nexperts, int topk, int in_dtype, int out_dtype,
                                void* const* gather_bufs, int* const* flag_bufs, void* workspace,
                                fluxb_moe_ag_scatter_t* out);
int fluxb_moe_ag_scatter_destroy(fluxb_moe_ag_scatter_t op);
/* GemmGroupedV3AGScatterOp::clear_buffers (src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc:112-126);
 * see fluxb_ag_gemm_reset. */
int fluxb_moe_ag_scatter_reset(fluxb_moe_ag_scatter_t op, fluxb_stream_t stream);
/* Expert parallelism (DistEnvTPWithEP with an ep_group, src/ths_op/ths_op.cc:334-346): the `world` ranks form
 * ep_size groups of world / ep_size ranks; group ep_rank holds experts [ep_rank, ep_rank + 1) * nexperts / ep_size
 * with the ffn dimension sharded over the ranks of the group (`ffn_local` = ffn / (world / ep_size)). Tokens are
 * still gathered from all `world` ranks. After this call `weights` is [nexperts / ep_size, ffn_local, hidden] and
 * `out` receives only the rows of this rank's experts, numbered from the first of them
 * (python/flux/testing/moe_ag_scatter_utils.py:228-262). */
int fluxb_moe_ag_scatter_set_ep(fluxb_moe_ag_scatter_t op, int ep_rank, int ep_size);
int fluxb_moe_ag_scatter_forward(fluxb_moe_ag_scatter_t op, const void* tokens_shard,
                                 int ntokens_local, const void* weights, const int* splits_dev,
                                 const int* scatter_index_dev, const float* out_scale, void* out,
                                 void* gathered_out, const fluxb_tuning* tuning,
                                 fluxb_stream_t stream);

/* ------------------------------------- scatter + grouped GEMM, no allocation
 * No counterpart in the reference. The single-GPU form of the MoE layer-0 product
 *     out[scatter_index[t,k], :] = tokens[t, :] . W[expert(t,k)]^T * out_scale[expert]
 * for callers that must not allocate device memory at call time: serving processes that hand all
 * free device memory to their own pool at start-up (a later cudaMalloc fails or fragments the pool),
 * and latency-critical loops that cannot afford the device-wide synchronisation an allocation may
 * imply. The routing tables the grouped kernel needs (inverse permutation, per-expert tile list) live
 * in a fixed device array inside the library instead of a caller-provided workspace, so the entry
 * point itself calls no cudaMalloc / cudaFree and no allocating library routine.
 * Limits: ntokens * topk <= FLUXB_STATIC_MAX_ROWS and nexperts <= FLUXB_STATIC_MAX_EXPERTS; larger
 * problems are rejected with FLUXB_ERR_INVALID. Every GPU that loads the library holds the array
 * (about 300 KB) until the process exits.
 * The first call on a device looks up the array's device address and configures the kernel; make
 * that first call outside any stream capture. All calls on a device share the one array, which keeps
 * the previous call's contents (everything a call reads is rewritten by that call first): calls that
 * overlap on the GPU (different streams) race and must be serialised by the caller.
 * `comm` is a world-1 communicator whose device is current; tokens [ntokens, hidden], weights
 * [nexperts, ffn, hidden], splits_dev int32 [nexperts], scatter_index_dev int32 [ntokens, topk],
 * out_scale fp32 [nexperts] or NULL, out [ntokens*topk, ffn]. */
#define FLUXB_STATIC_MAX_ROWS 65536
#define FLUXB_STATIC_MAX_EXPERTS 256
int fluxb_moe_scatter_gemm_static(fluxb_comm_t comm, const void* tokens, int ntokens, int hidden,
                                  const void* weights, int nexperts, int ffn, int topk,
                                  const int* splits_dev, const int* scatter_index_dev,
                                  const float* out_scale, void* out, int in_dtype, int out_dtype,
                                  const fluxb_tuning* tuning, fluxb_stream_t stream);

/* ------------------------------------------------------ MoE gather + RS
 * Replaces GemmGroupedV3GatherRS
 * (src/moe_gather_rs/ths_op/gemm_grouped_v3_gather_rs.cc:549-584, :595-820).
 * out[t_local, :] = sum over ranks, sum over k of
 *     (x[scatter_index[t,k], :] . W[expert]^T) * in_scale * w_scale[expert] * vec_scale[row]. */
size_t fluxb_moe_gather_rs_workspace_bytes(int max_m, int n_dim, int topk, int nexperts);
size_t fluxb_moe_gather_rs_stage_bytes(int max_m, int n_dim, int topk, int world);
size_t fluxb_moe_gather_rs_cnt_bytes(int max_m, int n_dim, int topk, int world);
int fluxb_moe_gather_rs_create(fluxb_comm_t comm, int nexperts, int max_m, int n_dim, int topk,
                               int in_dtype, int out_dtype, float* const* stage_bufs,
                               int* const* cnt_bufs, void* workspace, fluxb_moe_gather_rs_t* out);
int fluxb_moe_gather_rs_destroy(fluxb_moe_gather_rs_t op);
/* GemmGroupedV3GatherRS::ep_zero_buffer (src/moe_gather_rs/ths_op/gemm_grouped_v3_gather_rs.cc:549-584); see
 * fluxb_ag_gemm_reset. */
int fluxb_moe_gather_rs_reset(fluxb_moe_gather_rs_t op, fluxb_stream_t stream);
int fluxb_moe_gather_rs_forward(fluxb_moe_gather_rs_t op, const void* x, int m, int k_local,
                                const void* weights, const int* splits_host,
                                const int* routing_idx_dev, const float* in_scale,
                                const float* w_scale, const float* vec_scale, void* out,
                                const fluxb_tuning* tuning, fluxb_stream_t stream);
/* Expert parallelism (see fluxb_moe_ag_scatter_set_ep): `x` [m, k_local] and `vec_scale` [m] hold only the rows
 * of this rank's experts (m = sum of their splits), `weights` is [nexperts / ep_size, n, k_local], `splits_host`
 * and `routing_idx_dev` stay global ([nexperts] and [ntokens * topk]); every rank pushes its share of every
 * token's top-k sum to the token's owner (python/flux/testing/moe_gather_rs_utils.py:26-125). */
int fluxb_moe_gather_rs_set_ep(fluxb_moe_gather_rs_t op, int ep_rank, int ep_size);
int fluxb_moe_gather_rs_forward_ep(fluxb_moe_gather_rs_t op, const void* x, int m, int ntokens, int k_local,
                                   const void* weights, const int* splits_host,
                                   const int* routing_idx_dev, const float* in_scale,
                                   const float* w_scale, const float* vec_scale, void* out,
                                   const fluxb_tuning* tuning, fluxb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FLUXB_H_ */
