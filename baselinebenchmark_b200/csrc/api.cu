// C ABI of the MoBA forward and backward (declared in include/moba_b200.h): argument
// validation, workspace carving and the launch sequences.  Host-side only.
//
// Mirrors backends/_mthreads/ops/moba/parallel.py:253-457 of the reference:
// the checks of parallel_moba (:410-443) and the dataflow of
// _moba_attn_varlen_inference (:283-374), with all ranks handled in one pass
// and every scratch buffer taken from a caller-owned workspace.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "nccl_dl.cuh"

using namespace moba;

namespace {

// rows per work item of the dense stage: the tcgen05 kernel takes two 128-row tiles per item up to
// head_dim 128 and one at head_dim 256, the mma.sync kernel one
int tile_rows_of(int impl, int head_dim, int chunk = 1 << 30) {
  if (impl == MOBA_ATTEND_MMA_SYNC) return kMmaTileRows;
  return head_dim > 128 || tc5_small_items(head_dim, chunk) ? kTileRowsWide : kTc5TileRows;
}
constexpr size_t kAlign = 256;
inline size_t align_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

Params make_params(const moba_problem_t* p);

int check_problem(const moba_problem_t* p) {
  if (p == nullptr) return MOBA_E_NULL;
  if (p->total_tokens <= 0 || p->batch <= 0 || p->num_q_heads <= 0 || p->num_kv_heads <= 0 || p->head_dim <= 0)
    return MOBA_E_SHAPE;                                   // parallel.py:440-441
  if (p->num_q_heads % p->num_kv_heads != 0) return MOBA_E_SHAPE;          // :442-443
  if (p->max_seqlen <= 0 || p->chunk_size <= 0) return MOBA_E_SHAPE;       // :428-431
  if (p->topk < 1 || p->topk > kMaxTopk) return MOBA_E_TOPK;               // :432-437
  if (p->head_dim > 256) return MOBA_E_SHAPE;                              // :445-446
  if (p->head_dim != 64 && p->head_dim != 96 && p->head_dim != 128 && p->head_dim != 256) return MOBA_E_UNSUPPORTED;
  if (p->num_q_heads / p->num_kv_heads > 128) return MOBA_E_UNSUPPORTED;
  if (p->attend_impl != MOBA_ATTEND_TCGEN05 && p->attend_impl != MOBA_ATTEND_MMA_SYNC) return MOBA_E_UNSUPPORTED;
  if ((p->dtype != MOBA_DTYPE_BF16 && p->dtype != MOBA_DTYPE_FP16) || p->reserved != 0) return MOBA_E_UNSUPPORTED;
  const int64_t strides[8] = {p->q_stride_token, p->q_stride_head, p->k_stride_token, p->k_stride_head,
                              p->v_stride_token, p->v_stride_head, p->o_stride_token, p->o_stride_head};
  for (int i = 0; i < 8; ++i) {
    if (strides[i] <= 0) return MOBA_E_SHAPE;
    if (strides[i] % 8 != 0) return MOBA_E_ALIGN;          // 16-byte vector and TMA accesses
  }
  if (p->q_tokens < 0 || p->q_token_begin < 0) return MOBA_E_SHAPE;
  if (p->q_tokens > 0 && p->q_token_begin + p->q_tokens > p->total_tokens) return MOBA_E_SHAPE;
  if (p->q_tokens == 0 && p->q_token_begin != 0) return MOBA_E_SHAPE;
  if (p->total_tokens >= ((int64_t)1 << 31)) return MOBA_E_UNSUPPORTED;
  const int64_t mc = (p->max_seqlen + (int64_t)p->chunk_size - 1) / p->chunk_size;
  if (mc * p->batch > (int64_t)1 << 24) return MOBA_E_UNSUPPORTED;
  if (mc > 16384) return MOBA_E_UNSUPPORTED;               // per-CTA list tables live in shared memory
  const int64_t hist = (p->topk - 1 < mc - 1) ? p->topk - 1 : mc - 1;
  const int64_t np = (hist > 0 ? hist : 0) + 1;
  // entry ids (row * partials + rank) are int32, like the reference's int32 offsets (routing.py:1094-1100)
  // a pass covers at least one kv head with its query heads (forward_impl splits larger problems)
  const int64_t tq = p->q_tokens > 0 ? p->q_tokens : p->total_tokens;
  if (tq * (p->num_q_heads / p->num_kv_heads) * np >= ((int64_t)1 << 31)) return MOBA_E_UNSUPPORTED;
  // launch limits: the gating and scatter grids put the sequence in grid.z and the kv head in
  // grid.y; the gating kernel's lists must fit the shared memory of an SM; work items of the
  // dense stage are counted in int32 (routed tiles <= hist * rows / tile + lists, own-chunk
  // tiles = slots * Hq * tiles per chunk, per pass of one kv-head group at least)
  if (p->batch > 65535 || p->num_kv_heads > 65535) return MOBA_E_UNSUPPORTED;
  const int64_t g = p->num_q_heads / p->num_kv_heads;
  const int64_t tile = tile_rows_of(p->attend_impl, p->head_dim, p->chunk_size);
  const int64_t own_items = mc * p->batch * g * ((p->chunk_size + tile - 1) / tile);
  const int64_t routed_items = (hist > 0 ? hist : 0) * tq * g / tile + mc * p->batch;
  if (own_items + routed_items >= ((int64_t)1 << 31)) return MOBA_E_UNSUPPORTED;
  if (!gate_topk_fits(make_params(p))) return MOBA_E_UNSUPPORTED;
  return MOBA_OK;
}

Params make_params(const moba_problem_t* p) {
  Params r;
  r.T = p->total_tokens;
  r.Tq = p->q_tokens > 0 ? p->q_tokens : p->total_tokens;
  r.win_lo = p->q_tokens > 0 ? (int)p->q_token_begin : 0;
  r.B = p->batch;
  r.Hq = p->num_q_heads;
  r.Hkv = p->num_kv_heads;
  r.G = r.Hq / r.Hkv;
  r.D = p->head_dim;
  r.fp16 = p->dtype == MOBA_DTYPE_FP16;
  r.max_seqlen = p->max_seqlen;
  r.C = p->chunk_size;
  r.topk = p->topk;
  r.mc = (int)((p->max_seqlen + (int64_t)p->chunk_size - 1) / p->chunk_size);
  r.slots = r.B * r.mc;
  r.hist = (r.topk - 1 < r.mc - 1) ? r.topk - 1 : r.mc - 1;       // parallel.py:303
  if (r.hist < 0) r.hist = 0;
  r.NP = r.hist + 1;
  r.rows = r.Tq * r.Hq;
  r.sel_rs = (int64_t)r.Hq * r.Tq;
  r.lists = (int64_t)r.slots * r.Hkv;
  r.sq_t = p->q_stride_token; r.sq_h = p->q_stride_head;
  r.sk_t = p->k_stride_token; r.sk_h = p->k_stride_head;
  r.sv_t = p->v_stride_token; r.sv_h = p->v_stride_head;
  r.so_t = p->o_stride_token; r.so_h = p->o_stride_head;
  return r;
}

// Carves the workspace; with base == nullptr only sizes are computed.
struct Workspace {
  __nv_bfloat16* means;
  int32_t* selected;
  int32_t* list_counts;      // [lists] + work counter + status, zeroed per call in one memset
  int32_t* work_counter;
  int32_t* status;
  int32_t* list_offsets;
  int32_t* tile_prefix;
  int32_t* cursors;
  int32_t* row_list;
  void* partial_out;         // forward: fp16 [rows * NP][D]; backward: fp32 dq contributions of the same shape
  float2* partial_lse;       // {lse, 1 / scale} per entry
  size_t zero_bytes;
  size_t total;
};

Workspace carve(const Params& r, void* base, bool backward = false) {
  Workspace w;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* ptr = base ? static_cast<char*>(base) + off : nullptr;
    off += align_up(bytes);
    return ptr;
  };
  const size_t lists = (size_t)r.lists;
  w.zero_bytes = (lists + 512) * sizeof(int32_t);        // + work counter, status, debug counters
  w.list_counts = static_cast<int32_t*>(take(w.zero_bytes));
  w.work_counter = w.list_counts ? w.list_counts + lists : nullptr;
  w.status = w.list_counts ? w.list_counts + lists + 1 : nullptr;
  w.list_offsets = static_cast<int32_t*>(take((lists + 1) * sizeof(int32_t)));
  w.tile_prefix = static_cast<int32_t*>(take((lists + 1) * sizeof(int32_t)));
  w.cursors = static_cast<int32_t*>(take(lists * sizeof(int32_t)));
  w.means = static_cast<__nv_bfloat16*>(take((size_t)r.slots * r.Hkv * r.D * 2));
  w.selected = static_cast<int32_t*>(take((size_t)r.hist * r.rows * sizeof(int32_t)));
  w.row_list = static_cast<int32_t*>(take((size_t)r.hist * r.rows * sizeof(int32_t)));
  w.partial_lse = static_cast<float2*>(take((size_t)r.rows * r.NP * sizeof(float2)));
  w.partial_out = take((size_t)r.rows * r.NP * r.D * (backward ? sizeof(float) : sizeof(__half)));
  w.total = off;
  return w;
}



int attend_dispatch(const moba_problem_t* p, const Params& r, const void* q, const void* k, const void* v,
                    const int32_t* cu, const int32_t* list_counts, const int32_t* list_offsets,
                    const int32_t* tile_prefix, const int32_t* row_list, __half* partial_out,
                    float2* partial_lse, int32_t* work_counter, int32_t* status, cudaStream_t st) {
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(k);
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(v);
  if (p->attend_impl == MOBA_ATTEND_MMA_SYNC)
    return (int)launch_attend_mma(r, qb, kb, vb, cu, list_counts, list_offsets, tile_prefix, row_list,
                                  partial_out, partial_lse, work_counter, st);
  return (int)launch_attend_tc5(r, qb, kb, vb, cu, list_counts, list_offsets, tile_prefix, row_list,
                                partial_out, partial_lse, work_counter, status, st);
}

// ---- host-buffer variant: side streams and window bookkeeping ----------------
constexpr int kHostWindowsPerSeq = 8;     // query windows a sequence is cut into
constexpr int kHostMaxUnits = 256;        // [0, prefix] pairs kept alive in the workspace

struct HostStreams {
  cudaStream_t h2d, d2h;
};
// Two copy streams per device, created on first use (once, whatever thread asks first) and
// kept for the process.
HostStreams* host_streams() {
  constexpr int kMaxDev = 64;
  static HostStreams streams[kMaxDev];
  static std::once_flag once[kMaxDev];
  static bool ready[kMaxDev] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::call_once(once[dev], [dev]() {
    if (cudaStreamCreateWithFlags(&streams[dev].h2d, cudaStreamNonBlocking) != cudaSuccess) return;
    if (cudaStreamCreateWithFlags(&streams[dev].d2h, cudaStreamNonBlocking) != cudaSuccess) return;
    ready[dev] = true;
  });
  return ready[dev] ? &streams[dev] : nullptr;
}

// A cudaEvent_t that is destroyed on every exit path.
struct ScopedEvent {
  cudaEvent_t ev = nullptr;
  cudaError_t create() { return cudaEventCreateWithFlags(&ev, cudaEventDisableTiming); }
  ~ScopedEvent() { if (ev) cudaEventDestroy(ev); }
};
// `to` waits for everything queued on `from` so far.
cudaError_t chain(cudaStream_t from, cudaStream_t to) {
  ScopedEvent e;
  cudaError_t rc = e.create();
  if (rc != cudaSuccess) return rc;
  if ((rc = cudaEventRecord(e.ev, from)) != cudaSuccess) return rc;
  return cudaStreamWaitEvent(to, e.ev, 0);
}

__global__ void set_pair_kernel(int32_t* dst, int32_t a, int32_t b) {
  dst[0] = a;
  dst[1] = b;
}

}  // namespace

// Workspace of the problem restricted to `kv_heads` kv heads (and their query heads).
static size_t pass_bytes(const moba_problem_t* p, int kv_heads) {
  moba_problem_t sub = *p;
  sub.num_kv_heads = kv_heads;
  sub.num_q_heads = kv_heads * (p->num_q_heads / p->num_kv_heads);
  return carve(make_params(&sub), nullptr).total;
}


extern "C" {

int moba_b200_abi_version(void) { return 3; }

const char* moba_b200_strerror(int code) {
  switch (code) {
    case MOBA_OK: return "ok";
    case MOBA_E_SHAPE: return "q, k, v, cu_seqlens or the integer arguments have an invalid shape or value";
    case MOBA_E_UNSUPPORTED: return "configuration outside this build (bf16 or fp16; head_dim 64, 96, 128 or 256, backward up to 128 only)";
    case MOBA_E_WORKSPACE: return "workspace is null or too small";
    case MOBA_E_NULL: return "a required pointer is null";
    case MOBA_E_TOPK: return "moba_topk must be in 1..64";
    case MOBA_E_ALIGN: return "pointers and strides must be multiples of 16 bytes";
    case MOBA_E_DEVICE: return "needs an sm_100 device and a driver that exports cuTensorMapEncodeTiled";
    case MOBA_E_NCCL: return "an NCCL call failed, or no NCCL library with the needed entry points could be loaded";
    case MOBA_E_STATIC_LIMIT: return "problem exceeds the built-in scratch of moba_route_static (slots * kv heads * head_dim <= 2 Mi elements)";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

int moba_problem_check(const moba_problem_t* p) { return check_problem(p); }

int moba_problem_dims(const moba_problem_t* p, moba_dims_t* d) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (d == nullptr) return MOBA_E_NULL;
  const Params r = make_params(p);
  d->chunks_per_seq = r.mc;
  d->slots = r.slots;
  d->hist = (p->topk - 1 < r.mc - 1) ? p->topk - 1 : r.mc - 1;
  d->partials = r.NP;
  d->rows = r.rows;
  d->lists = r.lists;
  return MOBA_OK;
}

int moba_attend_tile_rows(int impl) { return tile_rows_of(impl, 128); }
int moba_attend_tile_rows_for(int impl, int head_dim) { return tile_rows_of(impl, head_dim); }
int moba_problem_tile_rows(const moba_problem_t* p) {
  const int rc = check_problem(p);
  return rc != MOBA_OK ? rc : tile_rows_of(p->attend_impl, p->head_dim, p->chunk_size);
}

int moba_workspace_size(const moba_problem_t* p, size_t* bytes) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (bytes == nullptr) return MOBA_E_NULL;
  const Params r = make_params(p);
  int per = r.Hkv;                                          // the largest pass whose entry ids fit int32
  while (per > 1 && r.Tq * (int64_t)(per * r.G) * r.NP >= ((int64_t)1 << 31)) --per;
  *bytes = pass_bytes(p, per);
  return MOBA_OK;
}

int moba_workspace_size_min(const moba_problem_t* p, size_t* bytes) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (bytes == nullptr) return MOBA_E_NULL;
  moba_problem_t sub = *p;
  sub.num_kv_heads = 1;
  sub.num_q_heads = p->num_q_heads / p->num_kv_heads;
  *bytes = carve(make_params(&sub), nullptr).total;
  return MOBA_OK;
}

int moba_chunk_metadata(const moba_problem_t* p, const int32_t* cu, int32_t* cu_chunk, int32_t* chunk_end,
                        int8_t* valid, void* stream) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!cu || !cu_chunk || !chunk_end || !valid) return MOBA_E_NULL;
  return (int)launch_chunk_metadata(make_params(p), cu, cu_chunk, chunk_end, valid, (cudaStream_t)stream);
}

int moba_chunk_means(const moba_problem_t* p, const void* k, const int32_t* cu, void* means, void* stream) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!k || !cu || !means) return MOBA_E_NULL;
  if (((uintptr_t)k | (uintptr_t)means) & 15) return MOBA_E_ALIGN;   // 16-byte loads of k, 16-byte loads of means later
  return (int)launch_chunk_means(make_params(p), static_cast<const __nv_bfloat16*>(k), cu,
                                 static_cast<__nv_bfloat16*>(means), (cudaStream_t)stream);
}

int moba_gate_topk_stats(const moba_problem_t* p, const void* q, const void* means, const int32_t* cu,
                         int32_t* selected, int32_t* list_counts, int32_t* stats, int32_t flags, void* stream) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!q || !means || !cu || !selected) return MOBA_E_NULL;
  if (((uintptr_t)q | (uintptr_t)means) & 15) return MOBA_E_ALIGN;
  const Params r = make_params(p);
  if (r.hist <= 0) return MOBA_OK;
  return (int)launch_gate_topk_stats(r, static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(means),
                                     cu, selected, list_counts, stats, flags, (cudaStream_t)stream);
}

int moba_gate_topk(const moba_problem_t* p, const void* q, const void* means, const int32_t* cu,
                   int32_t* selected, int32_t* list_counts, void* stream) {
  return moba_gate_topk_stats(p, q, means, cu, selected, list_counts, nullptr, 0, stream);
}

int moba_compact_routes(const moba_problem_t* p, const int32_t* cu, const int32_t* selected,
                        const int32_t* list_counts, int32_t* list_offsets, int32_t* tile_prefix,
                        int32_t* cursors, int32_t* row_list, float* partial_lse, int32_t tile_rows,
                        void* stream) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!cu || !selected || !list_counts || !list_offsets || !tile_prefix || !cursors || !row_list || !partial_lse)
    return MOBA_E_NULL;
  if (tile_rows <= 0) return MOBA_E_SHAPE;
  const Params r = make_params(p);
  if (r.hist <= 0) return MOBA_OK;
  return (int)launch_compact(r, cu, selected, list_counts, list_offsets, tile_prefix, cursors, row_list,
                             reinterpret_cast<float2*>(partial_lse), tile_rows, (cudaStream_t)stream);
}

int moba_attend(const moba_problem_t* p, const void* q, const void* k, const void* v, const int32_t* cu,
                const int32_t* list_counts, const int32_t* list_offsets, const int32_t* tile_prefix,
                const int32_t* row_list, void* partial_out, float* partial_lse, int32_t* work_counter,
                void* stream) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !v || !cu || !partial_out || !partial_lse || !work_counter) return MOBA_E_NULL;
  const Params r = make_params(p);
  if (r.hist > 0 && (!list_counts || !list_offsets || !tile_prefix || !row_list)) return MOBA_E_NULL;
  if (((uintptr_t)partial_out & 15) || ((uintptr_t)partial_lse & 7)) return MOBA_E_ALIGN;
  return attend_dispatch(p, r, q, k, v, cu, list_counts, list_offsets, tile_prefix, row_list,
                         static_cast<__half*>(partial_out), reinterpret_cast<float2*>(partial_lse), work_counter,
                         work_counter + 1, (cudaStream_t)stream);
}

int moba_merge(const moba_problem_t* p, const void* partial_out, const float* partial_lse,
               const int32_t* status, void* out, float* lse_out, void* stream) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!partial_out || !partial_lse || !out) return MOBA_E_NULL;
  if ((((uintptr_t)partial_out | (uintptr_t)out) & 15) || ((uintptr_t)partial_lse & 7)) return MOBA_E_ALIGN;
  return (int)launch_merge(make_params(p), static_cast<const __half*>(partial_out),
                           reinterpret_cast<const float2*>(partial_lse), status, static_cast<__nv_bfloat16*>(out),
                           lse_out, (cudaStream_t)stream);
}

// One pass over all query heads of `p` (the whole problem, or a group of kv heads
// carved out of it by forward_impl).  `sel_rs`: rank stride of `selected_out`.
// Variations of a pass:
//   means_ready  the chunk means already are in the workspace (context-parallel callers gather them)
//   kv_ready     an event the dense stage waits for (K and V rows still arriving), or null
//   means_ext    a caller-held means array [slots, Hkv, D] used instead of the workspace's, of which
//                the slots below means_from are valid already and the rest is computed here
struct PassOptions {
  bool means_ready = false;
  cudaEvent_t kv_ready = nullptr;
  __nv_bfloat16* means_ext = nullptr;
  int means_from = 0;
};
static int forward_pass(const moba_problem_t* p, int64_t sel_rs, const void* q, const void* k, const void* v,
                        const int32_t* cu, void* out, float* lse_out, int32_t* selected_out, void* workspace,
                        cudaStream_t st, void* const* events, bool first, bool last, const PassOptions& opt = {}) {
  Params r = make_params(p);
  if (selected_out) r.sel_rs = sel_rs;
  const Workspace w = carve(r, workspace);
  cudaError_t e;
  auto mark = [&](int i) -> cudaError_t {
    return (events && events[i]) ? cudaEventRecord((cudaEvent_t)events[i], st) : cudaSuccess;
  };
  if (first && (e = mark(0)) != cudaSuccess) return (int)e;
  if ((e = cudaMemsetAsync(w.list_counts, 0, w.zero_bytes, st)) != cudaSuccess) return (int)e;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(k);
  if (r.hist > 0) {
    int32_t* sel = selected_out ? selected_out : w.selected;
    __nv_bfloat16* means = opt.means_ext ? opt.means_ext : w.means;
    if (!opt.means_ready &&
        (e = launch_chunk_means_range(r, opt.means_ext ? opt.means_from : 0, r.slots, kb, cu, means, st)) != cudaSuccess)
      return (int)e;
    if (last && (e = mark(1)) != cudaSuccess) return (int)e;
    if ((e = launch_gate_topk(r, qb, means, cu, sel, w.list_counts, st)) != cudaSuccess) return (int)e;
    if (last && (e = mark(2)) != cudaSuccess) return (int)e;
    if ((e = launch_compact(r, cu, sel, w.list_counts, w.list_offsets, w.tile_prefix, w.cursors, w.row_list,
                            w.partial_lse, tile_rows_of(p->attend_impl, p->head_dim, p->chunk_size), st)) != cudaSuccess)
      return (int)e;
  } else if (last) {
    if ((e = mark(1)) != cudaSuccess || (e = mark(2)) != cudaSuccess) return (int)e;
  }
  if (opt.kv_ready != nullptr && (e = cudaStreamWaitEvent(st, opt.kv_ready, 0)) != cudaSuccess) return (int)e;
  if (last && (e = mark(3)) != cudaSuccess) return (int)e;
  const int arc = attend_dispatch(p, r, q, k, v, cu, w.list_counts, w.list_offsets, w.tile_prefix, w.row_list,
                                  static_cast<__half*>(w.partial_out), w.partial_lse, w.work_counter, w.status, st);
  if (arc != 0) return arc;
  if (last && (e = mark(4)) != cudaSuccess) return (int)e;
  e = launch_merge(r, static_cast<const __half*>(w.partial_out), w.partial_lse, w.status,
                   static_cast<__nv_bfloat16*>(out), lse_out, st);
  if (e != cudaSuccess) return (int)e;
  return last ? (int)mark(5) : MOBA_OK;
}

// The operator.  With a workspace smaller than moba_workspace_size the kv heads are
// processed in groups that fit (routing and attention never cross a kv-head group,
// routing.py:1089, attention.py:649-650); the reference bounds its memory with rank
// passes instead (parallel.py:322-373).  Events, when given, bracket the stages of the
// last group ([0] is recorded before the first).
static int forward_impl(const moba_problem_t* p, const void* q, const void* k, const void* v, const int32_t* cu,
                        void* out, float* lse_out, int32_t* selected_out, void* workspace, size_t workspace_bytes,
                        void* stream, void* const* events) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !v || !cu || !out) return MOBA_E_NULL;
  const uintptr_t ptrs[5] = {(uintptr_t)q, (uintptr_t)k, (uintptr_t)v, (uintptr_t)out, (uintptr_t)workspace};
  for (int i = 0; i < 5; ++i)
    if (ptrs[i] % 16 != 0) return MOBA_E_ALIGN;
  if (workspace == nullptr) return MOBA_E_WORKSPACE;
  const Params r = make_params(p);
  cudaStream_t st = (cudaStream_t)stream;
  int per = r.Hkv;                                          // kv heads per pass: the most that fit
  while (per > 1 && (pass_bytes(p, per) > workspace_bytes ||
                     r.Tq * (int64_t)(per * r.G) * r.NP >= ((int64_t)1 << 31)))
    --per;
  if (pass_bytes(p, per) > workspace_bytes) return MOBA_E_WORKSPACE;
  for (int g0 = 0; g0 < r.Hkv; g0 += per) {
    const int ng = g0 + per <= r.Hkv ? per : r.Hkv - g0;
    moba_problem_t sub = *p;
    sub.num_kv_heads = ng;
    sub.num_q_heads = ng * r.G;
    const int64_t h0 = (int64_t)g0 * r.G;
    const int prc = forward_pass(
        &sub, r.sel_rs, static_cast<const __nv_bfloat16*>(q) + h0 * r.sq_h,
        static_cast<const __nv_bfloat16*>(k) + (int64_t)g0 * r.sk_h,
        static_cast<const __nv_bfloat16*>(v) + (int64_t)g0 * r.sv_h, cu,
        static_cast<__nv_bfloat16*>(out) + h0 * r.so_h, lse_out ? lse_out + h0 * r.Tq : nullptr,
        selected_out ? selected_out + h0 * r.Tq : nullptr, workspace, st, events, g0 == 0, g0 + ng >= r.Hkv);
    if (prc != MOBA_OK) return prc;
  }
  return MOBA_OK;
}

int moba_forward(const moba_problem_t* p, const void* q, const void* k, const void* v, const int32_t* cu,
                 void* out, float* lse_out, int32_t* selected_out, void* workspace, size_t workspace_bytes,
                 void* stream) {
  return forward_impl(p, q, k, v, cu, out, lse_out, selected_out, workspace, workspace_bytes, stream, nullptr);
}

int moba_forward_events(const moba_problem_t* p, const void* q, const void* k, const void* v, const int32_t* cu,
                        void* out, float* lse_out, int32_t* selected_out, void* workspace,
                        size_t workspace_bytes, void* stream, void* const* events) {
  return forward_impl(p, q, k, v, cu, out, lse_out, selected_out, workspace, workspace_bytes, stream, events);
}

int moba_selftest_bounded_wait(int32_t* status, uint32_t limit_us, void* stream) {
  if (status == nullptr) return MOBA_E_NULL;
  if (limit_us == 0 || limit_us > 100000) return MOBA_E_SHAPE;            // at most 0.1 s
  return (int)launch_bounded_wait_probe(status, (unsigned long long)limit_us * 1000ull, (cudaStream_t)stream);
}

int moba_forward_cached(const moba_problem_t* p, const void* q, const void* k, const void* v, const int32_t* cu,
                        void* out, float* lse_out, int32_t* selected_out, void* means_cache, int32_t cached_slots,
                        void* workspace, size_t workspace_bytes, void* stream) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !v || !cu || !out || !means_cache) return MOBA_E_NULL;
  const uintptr_t ptrs[6] = {(uintptr_t)q, (uintptr_t)k, (uintptr_t)v, (uintptr_t)out, (uintptr_t)workspace,
                             (uintptr_t)means_cache};
  for (int i = 0; i < 6; ++i)
    if (ptrs[i] % 16 != 0) return MOBA_E_ALIGN;
  const Params r = make_params(p);
  if (cached_slots < 0 || cached_slots > r.slots) return MOBA_E_SHAPE;
  if (r.rows * (int64_t)r.NP >= ((int64_t)1 << 31)) return MOBA_E_UNSUPPORTED;   // the cache covers all kv heads: one pass
  if (workspace == nullptr || workspace_bytes < pass_bytes(p, r.Hkv)) return MOBA_E_WORKSPACE;
  PassOptions opt;
  opt.means_ext = static_cast<__nv_bfloat16*>(means_cache);
  opt.means_from = cached_slots;
  return forward_pass(p, r.sel_rs, q, k, v, cu, out, lse_out, selected_out, workspace, (cudaStream_t)stream, nullptr, true,
                      true, opt);
}

// ---------------------------------------------------------------------------
// training path: backward of the operator
// ---------------------------------------------------------------------------
static int check_backward(const moba_problem_t* p) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (p->q_tokens != 0) return MOBA_E_UNSUPPORTED;           // whole problems only
  const Params r = make_params(p);
  if (r.rows * r.NP >= ((int64_t)1 << 31)) return MOBA_E_UNSUPPORTED;
  return MOBA_OK;
}

int moba_backward_workspace_size(const moba_problem_t* p, size_t* bytes) {
  const int rc = check_backward(p);
  if (rc != MOBA_OK) return rc;
  if (bytes == nullptr) return MOBA_E_NULL;
  const Params r = make_params(p);
  // + delta and lse per row + the packed Q / dO rows of the routed lists (tcgen05 dk/dv kernel)
  *bytes = carve(r, nullptr, true).total + 2 * align_up((size_t)r.rows * sizeof(float)) +
           align_up((size_t)bwd_packed_elems(r) * 2);
  return MOBA_OK;
}

int moba_backward(const moba_problem_t* p, const void* q, const void* k, const void* v, const int32_t* cu,
                  const void* out, const float* lse, const int32_t* selected, const void* dout, void* dq, void* dk,
                  void* dv, void* workspace, size_t workspace_bytes, void* stream) {
  size_t need = 0;
  const int rc = moba_backward_workspace_size(p, &need);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !v || !cu || !out || !lse || !dout || !dq || !dk || !dv) return MOBA_E_NULL;
  if (workspace == nullptr || workspace_bytes < need) return MOBA_E_WORKSPACE;
  if (((uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv | (uintptr_t)out | (uintptr_t)q |
       (uintptr_t)k | (uintptr_t)v | (uintptr_t)workspace) & 15)
    return MOBA_E_ALIGN;
  const Params r = make_params(p);
  if (r.hist > 0 && selected == nullptr) return MOBA_E_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = carve(r, workspace, true);
  float* partial_dq = static_cast<float*>(w.partial_out);
  float* delta = reinterpret_cast<float*>(static_cast<char*>(workspace) + w.total);
  float* lse2 = reinterpret_cast<float*>(reinterpret_cast<char*>(delta) + align_up((size_t)r.rows * sizeof(float)));
  __nv_bfloat16* packed =
      reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(lse2) + align_up((size_t)r.rows * sizeof(float)));
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(k);
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(v);
  const __nv_bfloat16* gb = static_cast<const __nv_bfloat16*>(dout);
  // dout, dq: contiguous [T, Hq, D]; dk, dv: contiguous [T, Hkv, D]
  const int64_t qt = (int64_t)r.Hq * r.D, kt = (int64_t)r.Hkv * r.D, hd = r.D;
  // the gradient kernels run on the tcgen05 path where the forward's dense stage does, on
  // mma.sync otherwise
  const bool dq_tc5 = p->attend_impl == MOBA_ATTEND_TCGEN05 && r.D <= 128;
  cudaError_t e;
  if ((e = cudaMemsetAsync(w.list_counts, 0, w.zero_bytes, st)) != cudaSuccess) return (int)e;
  if (r.hist > 0) {
    if ((e = launch_count_lists(r, selected, w.list_counts, st)) != cudaSuccess) return (int)e;
    if ((e = launch_compact(r, cu, selected, w.list_counts, w.list_offsets, w.tile_prefix, w.cursors, w.row_list,
                            w.partial_lse, dq_tc5 ? kTc5TileRows : kMmaTileRows, st)) != cudaSuccess)
      return (int)e;
  }
  if ((e = launch_bwd_delta(r, static_cast<const __nv_bfloat16*>(out), gb, qt, hd, lse, delta, lse2, st)) != cudaSuccess)
    return (int)e;
  if (dq_tc5)
    e = launch_bwd_dq_tc5(r, qb, kb, vb, gb, cu, w.list_counts, w.list_offsets, w.tile_prefix, w.row_list, lse2, delta,
                          partial_dq, w.work_counter, w.status, st);
  else
    e = launch_bwd_dq(r, qb, kb, vb, gb, qt, hd, cu, w.list_counts, w.list_offsets, w.tile_prefix, w.row_list, lse2,
                      delta, partial_dq, w.work_counter, st);
  if (e != cudaSuccess) return (int)e;
  if ((e = launch_bwd_sum_dq(r, partial_dq, selected, w.status, static_cast<__nv_bfloat16*>(dq), qt, hd, st)) !=
      cudaSuccess)
    return (int)e;
  if (dq_tc5)
    e = launch_bwd_dkdv_tc5(r, qb, kb, vb, gb, cu, w.list_counts, w.list_offsets, w.row_list, lse2, delta,
                            static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), packed,
                            w.work_counter + 8, w.status, st);
  else
    e = launch_bwd_dkdv(r, qb, kb, vb, gb, qt, hd, cu, w.list_counts, w.list_offsets, w.row_list, lse2, delta,
                        static_cast<__nv_bfloat16*>(dk), kt, hd, static_cast<__nv_bfloat16*>(dv), kt, hd,
                        w.work_counter + 8, st);
  if (e != cudaSuccess) return (int)e;
  return MOBA_OK;
}

int moba_workspace_size_host(const moba_problem_t* p, size_t* bytes) {
  size_t core = 0;
  const int rc = moba_workspace_size(p, &core);
  if (rc != MOBA_OK) return rc;
  if (bytes == nullptr) return MOBA_E_NULL;
  const Params r = make_params(p);
  size_t extra = align_up((size_t)r.T * r.Hq * r.D * 2) * 2 +      // q, out
                 align_up((size_t)r.T * r.Hkv * r.D * 2) * 2 +     // k, v
                 align_up((size_t)(r.B + 1) * 4) +                      // cu_seqlens
                 align_up((size_t)kHostMaxUnits * 2 * 4) +              // [0, prefix] pairs of the windows
                 align_up((size_t)r.rows * 4);                          // lse
  *bytes = core + extra;
  return MOBA_OK;
}

int moba_forward_host(const moba_problem_t* p, const void* q_host, const void* k_host, const void* v_host,
                      const int32_t* cu_host, void* out_host, float* lse_out_host, int32_t* selected_out_host,
                      void* workspace, size_t workspace_bytes, void* stream) {
  size_t need = 0, core = 0;
  int rc = moba_workspace_size_host(p, &need);
  if (rc != MOBA_OK) return rc;
  moba_workspace_size(p, &core);
  if (!q_host || !k_host || !v_host || !cu_host || !out_host) return MOBA_E_NULL;
  if (workspace == nullptr || workspace_bytes < need) return MOBA_E_WORKSPACE;
  const Params r = make_params(p);
  if (r.Tq != r.T) return MOBA_E_UNSUPPORTED;             // the host variant runs whole problems
  // host tensors are taken as contiguous [T, H, D]
  if (r.sq_h != r.D || r.sq_t != (int64_t)r.Hq * r.D || r.sk_h != r.D ||
      r.sk_t != (int64_t)r.Hkv * r.D || r.sv_h != r.D || r.sv_t != (int64_t)r.Hkv * r.D ||
      r.so_h != r.D || r.so_t != (int64_t)r.Hq * r.D)
    return MOBA_E_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  char* base = static_cast<char*>(workspace) + core;
  const size_t qrow = (size_t)r.Hq * r.D * 2, krow = (size_t)r.Hkv * r.D * 2;
  const size_t qbytes = (size_t)r.T * qrow, kbytes = (size_t)r.T * krow;
  char* dq = base;               base += align_up(qbytes);
  char* dout = base;             base += align_up(qbytes);
  char* dk = base;               base += align_up(kbytes);
  char* dv = base;               base += align_up(kbytes);
  int32_t* dcu = (int32_t*)base; base += align_up((size_t)(r.B + 1) * 4);
  int32_t* dpairs = (int32_t*)base; base += align_up((size_t)kHostMaxUnits * 2 * 4);
  float* dlse = (float*)base;
  cudaError_t e;

  if (lse_out_host || selected_out_host) {
    // one call on the whole batch: the extra outputs keep their whole-batch layouts.  The
    // selection is copied out of the workspace, which holds all heads only when the problem
    // runs as one pass.
    if (selected_out_host && r.hist > 0 && pass_bytes(p, r.Hkv) > core) return MOBA_E_UNSUPPORTED;
    if ((e = cudaMemcpyAsync(dq, q_host, qbytes, cudaMemcpyHostToDevice, st)) != cudaSuccess) return (int)e;
    if ((e = cudaMemcpyAsync(dk, k_host, kbytes, cudaMemcpyHostToDevice, st)) != cudaSuccess) return (int)e;
    if ((e = cudaMemcpyAsync(dv, v_host, kbytes, cudaMemcpyHostToDevice, st)) != cudaSuccess) return (int)e;
    if ((e = cudaMemcpyAsync(dcu, cu_host, (size_t)(r.B + 1) * 4, cudaMemcpyHostToDevice, st)) != cudaSuccess)
      return (int)e;
    const Workspace w = carve(r, workspace);
    rc = moba_forward(p, dq, dk, dv, dcu, dout, lse_out_host ? dlse : nullptr, nullptr, workspace, core, stream);
    if (rc != MOBA_OK) return rc;
    if ((e = cudaMemcpyAsync(out_host, dout, qbytes, cudaMemcpyDeviceToHost, st)) != cudaSuccess) return (int)e;
    if (lse_out_host &&
        (e = cudaMemcpyAsync(lse_out_host, dlse, (size_t)r.rows * 4, cudaMemcpyDeviceToHost, st)) != cudaSuccess)
      return (int)e;
    if (selected_out_host && r.hist > 0 &&
        (e = cudaMemcpyAsync(selected_out_host, w.selected, (size_t)r.hist * r.rows * 4, cudaMemcpyDeviceToHost,
                             st)) != cudaSuccess)
      return (int)e;
    return MOBA_OK;
  }

  // Pipelined path.  A query only sees keys at or before its own position, so a
  // sequence can be processed in chunk-aligned query windows, window w needing K/V
  // of the sequence only up to the end of w: copy window w+1 in and window w-1 out
  // on two side streams while window w computes.  All copies are contiguous.
  HostStreams* hs = host_streams();
  if (hs == nullptr) return (int)cudaErrorUnknown;
  // side streams start after everything already queued on the caller's stream
  if ((e = chain(st, hs->h2d)) != cudaSuccess) return (int)e;
  if ((e = chain(st, hs->d2h)) != cudaSuccess) return (int)e;
  int unit = 0;
  int status = MOBA_OK;
  for (int b = 0; b < r.B && status == MOBA_OK; ++b) {
    const int64_t s0 = cu_host[b], s1 = cu_host[b + 1];
    const int64_t nchunks = (s1 - s0 + r.C - 1) / r.C;
    int64_t per = (nchunks + kHostWindowsPerSeq - 1) / kHostWindowsPerSeq;      // chunks per window
    if ((int64_t)r.B * kHostWindowsPerSeq > kHostMaxUnits) per = nchunks;        // many sequences: one window each
    if (per < 1) per = 1;
    for (int64_t c0 = 0; c0 < nchunks && status == MOBA_OK; c0 += per, ++unit) {
      const int64_t lo = s0 + c0 * r.C;
      const int64_t hi = (c0 + per) * r.C < s1 - s0 ? s0 + (c0 + per) * r.C : s1;
      if ((e = cudaMemcpyAsync(dq + lo * qrow, (const char*)q_host + lo * qrow, (hi - lo) * qrow,
                               cudaMemcpyHostToDevice, hs->h2d)) != cudaSuccess ||
          (e = cudaMemcpyAsync(dk + lo * krow, (const char*)k_host + lo * krow, (hi - lo) * krow,
                               cudaMemcpyHostToDevice, hs->h2d)) != cudaSuccess ||
          (e = cudaMemcpyAsync(dv + lo * krow, (const char*)v_host + lo * krow, (hi - lo) * krow,
                               cudaMemcpyHostToDevice, hs->h2d)) != cudaSuccess ||
          (e = chain(hs->h2d, st)) != cudaSuccess) {
        status = (int)e;
        break;
      }
      // the window as a problem of its own: the prefix [s0, hi) is the sequence
      moba_problem_t sub = *p;
      sub.total_tokens = hi - s0;
      sub.batch = 1;
      sub.q_token_begin = lo - s0;
      sub.q_tokens = hi - lo;
      int32_t* pair = dpairs + 2 * (unit % kHostMaxUnits);
      set_pair_kernel<<<1, 1, 0, st>>>(pair, 0, (int32_t)(hi - s0));
      if ((e = cudaGetLastError()) != cudaSuccess) { status = (int)e; break; }
      status = moba_forward(&sub, dq + lo * qrow, dk + s0 * krow, dv + s0 * krow, pair, dout + lo * qrow, nullptr,
                            nullptr, workspace, core, stream);
      if (status != MOBA_OK) break;
      if ((e = chain(st, hs->d2h)) != cudaSuccess ||
          (e = cudaMemcpyAsync((char*)out_host + lo * qrow, dout + lo * qrow, (hi - lo) * qrow,
                               cudaMemcpyDeviceToHost, hs->d2h)) != cudaSuccess) {
        status = (int)e;
        break;
      }
    }
  }
  // the caller's stream completes when the last copy in and the last copy out have, also
  // after an error: nothing of this call is then still running on the side streams
  const cudaError_t j1 = chain(hs->h2d, st), j2 = chain(hs->d2h, st);
  if (status != MOBA_OK) return status;
  if (j1 != cudaSuccess) return (int)j1;
  return (int)j2;
}

// ---------------------------------------------------------------------------
// context parallelism: one sequence split contiguously over the ranks of an NCCL communicator
// ---------------------------------------------------------------------------
int moba_cp_workspace_size(const moba_problem_t* p, size_t* bytes) {
  const int rc = check_problem(p);
  if (rc != MOBA_OK) return rc;
  if (bytes == nullptr) return MOBA_E_NULL;
  if (p->batch != 1 || p->q_tokens <= 0) return MOBA_E_SHAPE;
  *bytes = pass_bytes(p, p->num_kv_heads);                  // one pass: the gathered means cover all kv heads
  return MOBA_OK;
}

int moba_cp_forward(const moba_problem_t* p, void* nccl_comm, int32_t rank, int32_t world, const int64_t* bounds,
                    const void* q_local, void* k_full, void* v_full, const int32_t* cu, void* out_local,
                    float* lse_out, int32_t* selected_out, void* workspace, size_t workspace_bytes, void* stream,
                    void* comm_stream, void* const* events) {
  size_t need = 0;
  const int rc = moba_cp_workspace_size(p, &need);
  if (rc != MOBA_OK) return rc;
  if (!nccl_comm || !bounds || !q_local || !k_full || !v_full || !cu || !out_local) return MOBA_E_NULL;
  if (workspace == nullptr || workspace_bytes < need) return MOBA_E_WORKSPACE;
  if (world < 1 || rank < 0 || rank >= world) return MOBA_E_SHAPE;
  const Params r = make_params(p);
  if (r.rows * (int64_t)r.NP >= ((int64_t)1 << 31)) return MOBA_E_UNSUPPORTED;   // one pass over all heads
  // windows: increasing, chunk aligned, covering the sequence; this rank's is the query window of `p`
  if (bounds[0] != 0 || bounds[world] != p->total_tokens) return MOBA_E_SHAPE;
  for (int i = 0; i < world; ++i)
    if (bounds[i + 1] < bounds[i] || (bounds[i + 1] % r.C != 0 && bounds[i + 1] != p->total_tokens)) return MOBA_E_SHAPE;
  if (bounds[rank] != p->q_token_begin || bounds[rank + 1] - bounds[rank] != p->q_tokens) return MOBA_E_SHAPE;
  // K and V are taken as contiguous [T, Hkv, D] buffers that every rank lays out alike
  if (r.sk_h != r.D || r.sk_t != (int64_t)r.Hkv * r.D || r.sv_h != r.D || r.sv_t != (int64_t)r.Hkv * r.D)
    return MOBA_E_UNSUPPORTED;
  const uintptr_t ptrs[5] = {(uintptr_t)q_local, (uintptr_t)k_full, (uintptr_t)v_full, (uintptr_t)out_local,
                             (uintptr_t)workspace};
  for (int i = 0; i < 5; ++i)
    if (ptrs[i] % 16 != 0) return MOBA_E_ALIGN;
  const NcclApi* nc = nccl_api();
  if (nc == nullptr) return MOBA_E_NCCL;
  ncclComm_t comm = static_cast<ncclComm_t>(nccl_comm);
  cudaStream_t st = (cudaStream_t)stream, cs = (cudaStream_t)comm_stream;
  const Workspace w = carve(r, workspace);
  cudaError_t e;

  // 1. means of this rank's own chunks, from its own K rows (already in place inside k_full)
  const int slot_lo = (int)(bounds[rank] / r.C), slot_hi = (int)((bounds[rank + 1] + r.C - 1) / r.C);
  if (events && events[0] && (e = cudaEventRecord((cudaEvent_t)events[0], st)) != cudaSuccess) return (int)e;
  if (r.hist > 0 &&
      (e = launch_chunk_means_range(r, slot_lo, slot_hi, static_cast<const __nv_bfloat16*>(k_full), cu, w.means, st)) !=
          cudaSuccess)
    return (int)e;
  // 2. on the communication stream: every rank's means to every rank (a few hundred KB), then the K
  //    and V rows of the earlier ranks to the later ones (rank r receives tokens [0, bounds[r]) only).
  //    The gating of step 3 runs while the rows travel.
  if ((e = chain(st, cs)) != cudaSuccess) return (int)e;
  const size_t mean_row = (size_t)r.Hkv * r.D * 2, kv_row = (size_t)r.Hkv * r.D * 2;
  ncclResult_t nrc = ncclSuccess;
  auto ok = [&](ncclResult_t x) { if (x != ncclSuccess && nrc == ncclSuccess) nrc = x; };
  if (r.hist > 0 && world > 1) {
    ok(nc->GroupStart());
    for (int s = 0; s < world; ++s) {
      const int64_t lo = bounds[s] / r.C, hi = (bounds[s + 1] + r.C - 1) / r.C;
      char* buf = reinterpret_cast<char*>(w.means) + lo * mean_row;
      if (hi > lo) ok(nc->Broadcast(buf, buf, (size_t)(hi - lo) * mean_row, ncclChar, s, comm, cs));
    }
    ok(nc->GroupEnd());
  }
  ScopedEvent means_ready, kv_ready;
  if ((e = means_ready.create()) != cudaSuccess || (e = kv_ready.create()) != cudaSuccess) return (int)e;
  if ((e = cudaEventRecord(means_ready.ev, cs)) != cudaSuccess) return (int)e;
  if (world > 1) {
    ok(nc->GroupStart());
    for (int pass = 0; pass < 2; ++pass) {
      char* base = static_cast<char*>(pass == 0 ? k_full : v_full);
      for (int s = 0; s < rank; ++s)                          // rows of the earlier ranks
        if (bounds[s + 1] > bounds[s])
          ok(nc->Recv(base + bounds[s] * kv_row, (size_t)(bounds[s + 1] - bounds[s]) * kv_row, ncclChar, s, comm, cs));
      for (int d = rank + 1; d < world; ++d)                  // this rank's rows to the later ranks
        if (bounds[rank + 1] > bounds[rank] && bounds[d + 1] > bounds[d])
          ok(nc->Send(base + bounds[rank] * kv_row, (size_t)(bounds[rank + 1] - bounds[rank]) * kv_row, ncclChar, d, comm, cs));
    }
    ok(nc->GroupEnd());
  }
  if ((e = cudaEventRecord(kv_ready.ev, cs)) != cudaSuccess) return (int)e;
  if (nrc != ncclSuccess) return MOBA_E_NCCL;
  // 3. gating and compaction once the means are complete, dense stage and merge once K and V are
  if ((e = cudaStreamWaitEvent(st, means_ready.ev, 0)) != cudaSuccess) return (int)e;
  PassOptions opt;
  opt.means_ready = true;
  opt.kv_ready = kv_ready.ev;
  return forward_pass(p, r.sel_rs, q_local, k_full, v_full, cu, out_local, lse_out, selected_out, workspace, st, events,
                      false, true, opt);
}

int moba_cp_poll(void* nccl_comm, int32_t* async_error) {
  if (!nccl_comm || !async_error) return MOBA_E_NULL;
  const NcclApi* nc = nccl_api();
  if (nc == nullptr) return MOBA_E_NCCL;
  ncclResult_t state = ncclSuccess;
  if (nc->CommGetAsyncError(static_cast<ncclComm_t>(nccl_comm), &state) != ncclSuccess) return MOBA_E_NCCL;
  *async_error = (int32_t)state;
  return MOBA_OK;
}

int moba_cp_abort(void* nccl_comm) {
  if (!nccl_comm) return MOBA_E_NULL;
  const NcclApi* nc = nccl_api();
  if (nc == nullptr) return MOBA_E_NCCL;
  return nc->CommAbort(static_cast<ncclComm_t>(nccl_comm)) == ncclSuccess ? MOBA_OK : MOBA_E_NCCL;
}

}  // extern "C"
