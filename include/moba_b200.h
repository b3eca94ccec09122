/*
 * moba_b200 -- C ABI of the B200 (sm_100a) MoBA causal-prefill forward.
 *
 * Drop-in boundary for the operator the reference exposes as
 *   parallel_moba(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
 *   (backends/_mthreads/ops/moba/parallel.py:377-457, inference body :253-374).
 *
 * Conventions
 *   - plain pointers and sizes only; every device pointer must belong to the
 *     CUDA device that is current on the calling thread;
 *   - every entry point is stream ordered on `stream` (a cudaStream_t passed as
 *     void*), performs no device-to-host read and no allocation, so a caller
 *     may capture it in a CUDA graph, exactly like the reference path
 *     (parallel.py:262-275).  The one exception is moba_forward_host, which
 *     creates two copy streams per device on first use and short-lived events
 *     on every call: it is not meant to be captured;
 *   - return value: 0 success, < 0 invalid argument (MOBA_E_*), > 0 a
 *     cudaError_t raised by a launch or a copy.  Nothing throws or aborts;
 *   - tensors are bf16 or fp16 (moba_problem.dtype), head_dim 64, 96, 128 or 256
 *     (the head dims of the reference's benchmark suite, moba_compare.py:63, :70),
 *     innermost dimension contiguous; token and head strides are given in
 *     elements (the reference kernels also take strides, attention.py:431-439).
 *     Both dense stages exist for all four head dims (the tcgen05 one with its own
 *     kernel at 256).  Anything else returns MOBA_E_UNSUPPORTED: there is no
 *     fallback path.
 */
#ifndef MOBA_B200_H_
#define MOBA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MOBA_OK = 0,
  MOBA_E_SHAPE = -1,        /* parallel.py:410-443 ValueError cases              */
  MOBA_E_UNSUPPORTED = -2,  /* dtype / head_dim / stride outside the build       */
  MOBA_E_WORKSPACE = -3,    /* workspace pointer null or too small               */
  MOBA_E_NULL = -4,         /* a required pointer is null                        */
  MOBA_E_TOPK = -5,         /* moba_topk outside 1..64 (parallel.py:434-437)     */
  MOBA_E_ALIGN = -6,        /* base pointer or stride not 16-byte aligned        */
  MOBA_E_DEVICE = -7,       /* not an sm_100 device, or driver entry point missing */
  MOBA_E_STATIC_LIMIT = -8, /* problem too large for the built-in scratch of moba_route_static */
  MOBA_E_NCCL = -9          /* an NCCL call failed or no NCCL library could be loaded */
};

/* Which implementation of the dense stage moba_attend/moba_forward run. */
enum {
  MOBA_ATTEND_TCGEN05 = 0,  /* tcgen05.mma + TMEM accumulators + TMA K/V tiles                   */
  MOBA_ATTEND_MMA_SYNC = 1  /* legacy mma.sync tensor path, kept as cross-check  */
};

/* Element type of q, k, v and out (parallel.py:448-457 accepts both; the
 * reference's suite runs bf16 and fp16, moba_compare.py:56, :69-71). */
enum {
  MOBA_DTYPE_BF16 = 0,
  MOBA_DTYPE_FP16 = 1
};

/* Problem description.  Mirrors the arguments of parallel_moba
 * (parallel.py:377-385) plus the strides its kernels receive. */
typedef struct moba_problem {
  int64_t total_tokens;     /* T = q.shape[0] = cu_seqlens[batch]                */
  int32_t batch;            /* B = len(cu_seqlens) - 1                           */
  int32_t num_q_heads;      /* Hq                                                */
  int32_t num_kv_heads;     /* Hkv, Hq % Hkv == 0                                */
  int32_t head_dim;         /* D: 64, 96, 128 or 256                             */
  int32_t max_seqlen;       /* >= the longest sequence                           */
  int32_t chunk_size;       /* moba_chunk_size                                   */
  int32_t topk;             /* moba_topk, counts the query's own chunk           */
  int32_t attend_impl;      /* MOBA_ATTEND_*                                     */
  int64_t q_stride_token, q_stride_head;   /* elements                           */
  int64_t k_stride_token, k_stride_head;
  int64_t v_stride_token, v_stride_head;
  int64_t o_stride_token, o_stride_head;
  /* Query window, for context-parallel, incremental-prefill and decode callers
   * (the reference has none: it is rendered with enable_cp=False,
   * native_moba.py:69).  With q_tokens > 0 only the packed tokens
   * [q_token_begin, q_token_begin + q_tokens) are queries: q, out, lse_out and
   * selected_out then hold q_tokens tokens (token 0 of q is packed token
   * q_token_begin) while k, v and cu_seqlens still describe all total_tokens.
   * The window may start and end at any token (a decode step is a window of one
   * token at the end of the prefix); its rows equal those of the run over all
   * tokens bit for bit.  moba_cp_forward alone wants chunk-aligned windows.
   * q_tokens == 0: every token is a query. */
  int64_t q_token_begin, q_tokens;
  int32_t dtype;            /* MOBA_DTYPE_*; 0 (bf16) in a zero-initialised struct */
  int32_t reserved;         /* must be 0                                         */
} moba_problem_t;

/* Derived sizes: mc = ceil(max_seqlen / chunk), slots = B*mc,
 * hist = min(topk-1, mc-1)  (parallel.py:303, routing.py:604-605). */
typedef struct moba_dims {
  int32_t chunks_per_seq;   /* mc                                                */
  int32_t slots;            /* B * mc                                            */
  int32_t hist;             /* historical chunks selected per query, may be <= 0 */
  int32_t partials;         /* max(hist,0) + 1 partial results per (token, head) */
  int64_t rows;             /* query tokens * Hq                                 */
  int64_t lists;            /* slots * Hkv routed query lists                    */
} moba_dims_t;

int moba_b200_abi_version(void);
const char* moba_b200_strerror(int code);

/* Validation of parallel.py:410-443 without touching the device. */
int moba_problem_check(const moba_problem_t* p);
int moba_problem_dims(const moba_problem_t* p, moba_dims_t* dims);

/* Bytes of caller-owned scratch that moba_forward needs for `p`.  Replaces the
 * per-call torch allocations of parallel.py:283-374 (table of buffers:
 * routing.py:1653-1658, attention.py:418-419, :727-728). */
int moba_workspace_size(const moba_problem_t* p, size_t* bytes);

/* Smallest workspace moba_forward accepts for `p`: enough for one kv head and its
 * query heads.  With anything between the two sizes moba_forward processes the kv
 * heads in groups that fit, one after the other on the stream, with identical
 * results; the reference bounds its scratch with a 512 MiB budget and a loop over
 * rank passes instead (parallel.py:56, :322-373). */
int moba_workspace_size_min(const moba_problem_t* p, size_t* bytes);

/* The whole operator: replaces _moba_attn_varlen_inference (parallel.py:253-374).
 *   q [T,Hq,D], k,v [T,Hkv,D], out [T,Hq,D] bf16 on device; cu_seqlens int32[B+1] on device.
 *   lse_out       optional fp32 [Hq,T]   (natural log, layout of attention.py:419)
 *   selected_out  optional int32 [hist,Hq,T] (layout of routing.py:1221-1226);
 *                 when null the selection lives in the workspace only. */
int moba_forward(const moba_problem_t* p, const void* q, const void* k, const void* v,
                 const int32_t* cu_seqlens, void* out, float* lse_out, int32_t* selected_out,
                 void* workspace, size_t workspace_bytes, void* stream);

/* moba_forward with CUDA events (cudaEvent_t, may be null) recorded on `stream`
 * between the stages, for per-kernel timing without a profiler:
 *   [0] before the first launch   [1] after the chunk means   [2] after scores/top-k
 *   [3] after the compaction      [4] after the dense stage   [5] after the merge
 * The reference has no such hook: its harness times the whole call with
 * perf_counter (benchmarks/moba_compare.py:111-128). */
int moba_forward_events(const moba_problem_t* p, const void* q, const void* k, const void* v,
                        const int32_t* cu_seqlens, void* out, float* lse_out, int32_t* selected_out,
                        void* workspace, size_t workspace_bytes, void* stream, void* const* events);

/* moba_forward with a caller-held cache of chunk means, for incremental prefill and decode: a
 * sequence (or batch) is processed in several calls, each with a later query window
 * (q_token_begin / q_tokens; any number of tokens, down to the single token of a decode step)
 * over a longer K/V prefix, and the means of chunks that were complete at an earlier call are
 * not computed again.  The reference recomputes all chunk means
 * on every call (parallel.py:306-311); it has no incremental mode.
 *   means_cache   [slots, Hkv, D] in the tensors' dtype, slots = batch * ceil(max_seqlen / chunk)
 *                 (use the same max_seqlen, the capacity, for every call so that slots keep their
 *                 place); 16-byte aligned
 *   cached_slots  slots [0, cached_slots) of the cache hold final means and are read only; the
 *                 means of the slots from there on are computed from k and stored into the cache.
 *                 A chunk's mean is final once its sequence has grown past the chunk: with batch 1
 *                 and a prefix of T >= 1 tokens the next call may pass cached_slots =
 *                 (T - 1) / chunk, the chunks before the prefix's last one (that one was the
 *                 sequence's last chunk, which is never a candidate and is not computed).
 * Results are bit-identical to moba_forward on the same window.  The workspace must have the
 * full moba_workspace_size (one pass over all kv heads). */
int moba_forward_cached(const moba_problem_t* p, const void* q, const void* k, const void* v,
                        const int32_t* cu_seqlens, void* out, float* lse_out, int32_t* selected_out,
                        void* means_cache, int32_t cached_slots, void* workspace, size_t workspace_bytes,
                        void* stream);

/* Same call with HOST buffers (pinned memory; cu_seqlens_host is also read by the
 * CPU): copies q, k, v to staging buffers inside `workspace`, runs the operator
 * and copies `out` back.  The caller synchronises `stream`, which completes after
 * the last copy out.  Without the optional outputs the call is pipelined: every
 * sequence is cut into chunk-aligned query windows (causality makes window w need
 * K/V only up to its own end), and window w+1 is copied in and window w-1 copied
 * out on two internal streams (created once per device) while window w computes;
 * results are identical to moba_forward.  With lse_out / selected_out the whole
 * batch runs as one call on `stream`.  Calls on distinct (stream, workspace) pairs may
 * be in flight together (they share the two internal copy streams, which keep the copies
 * in order of the calls): alternating between two pairs hides the first copy in and the
 * last copy out of every call behind its neighbours' kernels.  Use
 * moba_workspace_size_host for sizing. */
int moba_workspace_size_host(const moba_problem_t* p, size_t* bytes);
int moba_forward_host(const moba_problem_t* p, const void* q_host, const void* k_host,
                      const void* v_host, const int32_t* cu_seqlens_host, void* out_host,
                      float* lse_out_host, int32_t* selected_out_host,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ---- staged entry points (unit tests, context-parallel driver) ------------ */

/* Chunk slot tables: replaces _build_dense_chunk_metadata_triton
 * (routing.py:595-632).  cu_chunk int32[slots+1], chunk_end int32[slots],
 * valid_hist int8[slots]. */
int moba_chunk_metadata(const moba_problem_t* p, const int32_t* cu_seqlens, int32_t* cu_chunk,
                        int32_t* chunk_end, int8_t* valid_hist, void* stream);

/* Mean-pooled keys: replaces _compute_dense_chunk_means_triton
 * (routing.py:740-775).  means bf16 [slots,Hkv,D], zeros for slots that are
 * not historical. */
int moba_chunk_means(const moba_problem_t* p, const void* k, const int32_t* cu_seqlens,
                     void* means, void* stream);

/* Scores + causal chunk mask + top-k: replaces
 * _compute_selected_chunks_batched_streaming_triton (routing.py:1185-1262).
 * selected int32 [hist,Hq,T]; list_counts int32[lists] (optional) receives the
 * number of (token, head) rows routed to every (slot, kv head) list and must be
 * zero on entry. */
int moba_gate_topk(const moba_problem_t* p, const void* q, const void* means,
                   const int32_t* cu_seqlens, int32_t* selected, int32_t* list_counts,
                   void* stream);

/* moba_gate_topk with its decision path observable and steerable, for tests and profiling
 * (the reference kernel has one path only, routing.py:1056-1182).  The kernel estimates all
 * scores of a row on the tensor core and evaluates in the reference-compatible fp32 order
 * only the candidates the estimate cannot rank with certainty; `selected` is the same
 * whatever path a row takes.
 *   stats  optional int32[4], added to (zero it first):
 *          [0] rows whose near-ties were scored again, [1] largest |estimate - exact| / bound
 *          seen while doing so, in units of 2^-16, [2] rows where that ratio exceeded 1 (never
 *          expected), [3] rows ranked over all their candidates
 *   flags  0 normal; 1 rank every row over all candidates in the exact order (no estimate
 *          used); 2 score the kept candidates of every row again. */
int moba_gate_topk_stats(const moba_problem_t* p, const void* q, const void* means,
                         const int32_t* cu_seqlens, int32_t* selected, int32_t* list_counts,
                         int32_t* stats, int32_t flags, void* stream);

/* Grouping of the routed rows: replaces _build_sparse_routes_device_triton
 * (routing.py:1642-1718), grouped by (slot, kv head) instead of (slot, q head)
 * so the query heads of a GQA group share one K/V stream.
 *   list_offsets  int32[lists+1]  exclusive prefix of list_counts
 *   tile_prefix   int32[lists+1]  exclusive prefix of ceil(count / tile_rows)
 *   row_list      int32[hist*T*Hq] entry ids  (t*Hq + h) * partials + rank + 1
 *   partial_lse   fp32 [T*Hq, partials, 2] = {natural-log LSE, 1 / scale of the partial row};
 *                 entries of ranks that selected nothing are set to {-inf, 0} here
 *   cursors       int32[lists] scratch */
int moba_compact_routes(const moba_problem_t* p, const int32_t* cu_seqlens,
                        const int32_t* selected, const int32_t* list_counts,
                        int32_t* list_offsets, int32_t* tile_prefix, int32_t* cursors,
                        int32_t* row_list, float* partial_lse, int32_t tile_rows, void* stream);

/* Dense stage: own-chunk causal attention (replaces _varlen_attn_fwd_kernel,
 * attention.py:53-160) and the routed historical-chunk attention (replaces
 * native_moba.routed / _routed_gqa_attn_fwd_kernel, native_moba.py:120-135,
 * attention.py:610-707) in one persistent launch.  Writes the normalised
 * partial outputs [T*Hq, partials, D] as fp16 (the reference keeps them in the
 * input dtype, attention.py:727), each row scaled by a power of two that puts
 * its largest magnitude into [2^13, 2^14) - 11 significant bits on every
 * element whatever the range of V - and {natural-log LSE, 1 / scale} per row
 * into partial_lse [T*Hq, partials, 2].  partial_out 16-byte, partial_lse
 * 8-byte aligned.
 *   work_counter int32[2] must be zero on entry: [0] is the item counter, [1]
 *   receives a non-zero status if a bounded device-side wait gave up. */
int moba_attend(const moba_problem_t* p, const void* q, const void* k, const void* v,
                const int32_t* cu_seqlens, const int32_t* list_counts,
                const int32_t* list_offsets, const int32_t* tile_prefix,
                const int32_t* row_list, void* partial_out, float* partial_lse,
                int32_t* work_counter, void* stream);

/* LSE-weighted combine: replaces _fused_merge_softmax_triton
 * (attention.py:892-945), all partials of a row in one pass, fp32 arithmetic,
 * one rounding to the output dtype.  `status` (optional) is work_counter + 1 of moba_attend:
 * when it is non-zero the output is filled with NaN instead of partial data. */
int moba_merge(const moba_problem_t* p, const void* partial_out, const float* partial_lse,
               const int32_t* status, void* out, float* lse_out, void* stream);

/* Self-test of the device-side wait limit (no counterpart in the reference, whose kernels
 * never wait on one another).  Every wait inside the dense-stage and gradient kernels is
 * bounded; one that gives up sets the status word next to the work counter, the kernel drains
 * and moba_merge then writes NaN instead of partial data.  This call launches one warp that
 * waits `limit_us` microseconds (1 .. 100000) on a barrier nothing will ever arrive on and then
 * sets `*status` (device int32, zero on entry) the way the kernels do.  Nothing faults, traps
 * or spins without limit. */
int moba_selftest_bounded_wait(int32_t* status, uint32_t limit_us, void* stream);

/* Routing without a workspace.  No counterpart in the reference, whose stages
 * all allocate through torch; it exists for callers that cannot give the library
 * device memory at call time (a server whose memory pool is fixed after start-up,
 * a plugin called where allocation is not allowed, a client that owns nothing but
 * its inputs and outputs).  Computes selected int32 [hist,Hq,T] from q and k like
 * moba_chunk_means + moba_gate_topk, keeping the chunk means in a 4 MiB array that
 * is part of the library image (held by every GPU that loads the library).
 *   - limit: slots * num_kv_heads * head_dim <= 2 Mi elements, otherwise
 *     MOBA_E_STATIC_LIMIT;
 *   - the first call on a device looks up the device address of that array; make
 *     that first call outside any stream capture;
 *   - all calls on a device share the array: calls whose kernels may overlap on the
 *     GPU (unordered streams) race on it.  It needs no clearing between calls;
 *   - performs no allocation and no host synchronisation. */
int moba_route_static(const moba_problem_t* p, const void* q, const void* k, const int32_t* cu_seqlens,
                      int32_t* selected, void* stream);

/* Training path: gradients of the operator (MixedAttention.backward, parallel.py:149-250;
 * dq and dk/dv kernels attention.py:163-369).  Inputs are those of the forward plus what it
 * returned: out [T,Hq,D], lse fp32 [Hq,T] and selected int32 [hist,Hq,T] (may be NULL when
 * hist <= 0), and dout [T,Hq,D].  Writes dq [T,Hq,D], dk and dv [T,Hkv,D] in the input
 * dtype; dout, dq, dk, dv are contiguous, q, k, v, out use the strides of the problem.  Like
 * the reference, both branches are differentiated with the merged LSE and output, and the
 * chunk selection is a constant.  No atomic accumulation: dq is bit-identical run to run,
 * dk and dv up to the order in which the rows of a routed list are added.  With
 * attend_impl = MOBA_ATTEND_TCGEN05 the dq and dk/dv kernels run on tcgen05 (accumulators in
 * tensor memory) up to head_dim 128; with MOBA_ATTEND_MMA_SYNC, and at head_dim 256, on mma.sync.
 * Whole problems only (q_tokens == 0), T*Hq*(hist+1) < 2^31; otherwise
 * MOBA_E_UNSUPPORTED.  The workspace holds, besides the route lists, one fp32 [D] slot per
 * (row, partial) for dQ and the Q / dO rows of the routed lists packed in list order. */
int moba_backward_workspace_size(const moba_problem_t* p, size_t* bytes);
int moba_backward(const moba_problem_t* p, const void* q, const void* k, const void* v, const int32_t* cu_seqlens,
                  const void* out, const float* lse, const int32_t* selected, const void* dout, void* dq, void* dk,
                  void* dv, void* workspace, size_t workspace_bytes, void* stream);

/* ---- context parallelism: one long sequence split over the GPUs of a communicator ----------
 *
 * The reference has no multi-device path (its native kernel is rendered with enable_cp=False,
 * native_moba.py:69); this is the partition BASELINE.json's million-token configuration asks
 * for.  Rank i owns the tokens [bounds[i], bounds[i+1]) of ONE sequence (bounds[0] = 0,
 * bounds[world] = total_tokens, inner bounds on chunk boundaries): its queries, its output rows
 * and its K/V rows.  `p` describes the whole sequence (batch 1, cu_seqlens = {0, total_tokens} on
 * the device) with the query window q_token_begin / q_tokens equal to this rank's range.
 *   k_full, v_full  contiguous [total_tokens, Hkv, D] buffers in this GPU's memory; on entry the
 *                   rank's own rows are in place at their token positions, on return (stream
 *                   order) the rows of all earlier ranks are too.  Later ranks' rows are not
 *                   needed (causal) and not transferred: rank i receives bounds[i] rows, not all.
 *   nccl_comm       an ncclComm_t of `world` ranks (the host framework's, or the caller's own),
 *                   used on `comm_stream` only.  NCCL is bound at run time from the library
 *                   already in the process.
 *   Schedule: the means of the rank's own chunks are computed from its own K rows, all ranks'
 *   means are exchanged (a few hundred KB), gating and compaction run on `stream` while K and V
 *   rows travel on `comm_stream`; the dense stage waits for them.  Every kernel reads local
 *   memory only.  Results are bit-identical to a single-device moba_forward on the same window.
 *   events          optional, as for moba_forward_events.
 * The call creates two short-lived events and is not meant to be captured in a CUDA graph.
 * All ranks must call with the same bounds; a rank that does not leaves the others waiting in
 * NCCL, which is what moba_cp_poll / moba_cp_abort are for: poll returns the communicator's
 * asynchronous error state (ncclCommGetAsyncError: 0 ok, 7 still in progress), abort tears the
 * communicator down (ncclCommAbort) so that a host that gave up waiting gets its stream back. */
int moba_cp_workspace_size(const moba_problem_t* p, size_t* bytes);
int moba_cp_forward(const moba_problem_t* p, void* nccl_comm, int32_t rank, int32_t world, const int64_t* bounds,
                    const void* q_local, void* k_full, void* v_full, const int32_t* cu_seqlens, void* out_local,
                    float* lse_out, int32_t* selected_out, void* workspace, size_t workspace_bytes, void* stream,
                    void* comm_stream, void* const* events);
int moba_cp_poll(void* nccl_comm, int32_t* async_error);
int moba_cp_abort(void* nccl_comm);

/* Rows per routed work item that the dense stage wants (the tile_rows argument of
 * moba_compact_routes).  moba_problem_tile_rows answers for a problem and is what callers
 * of the staged entry points should use: the tcgen05 stage takes 256 rows per item, 128 at
 * head_dim 256 and for chunks of at most 256 keys (its kernel for short items), the
 * mma.sync stage 128.  moba_attend_tile_rows / _for answer for long chunks at head_dim
 * <= 128 / any head_dim. */
int moba_attend_tile_rows(int attend_impl);
int moba_attend_tile_rows_for(int attend_impl, int head_dim);
int moba_problem_tile_rows(const moba_problem_t* p);

#ifdef __cplusplus
}
#endif
#endif /* MOBA_B200_H_ */
