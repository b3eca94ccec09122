// Shared declarations of the MoBA forward kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "moba_b200.h"

namespace moba {

constexpr int kHeadDim = 128;            // largest head dim of the tcgen05 dense stage (64 and 128; others: mma.sync stage)
constexpr int kMeanLanes = 32;           // row accumulators of a chunk mean
constexpr int kMaxTopk = 64;             // parallel.py:436

// Launch-time view of a problem, passed to kernels by value.
struct Params {
  int64_t T;                             // tokens of k / v (and of cu_seqlens)
  int64_t Tq;                            // query tokens: the window [win_lo, win_lo + Tq) of the packed tokens
  int win_lo;                            // q, out, selected and the partials are indexed by token - win_lo
  int B, Hq, Hkv, G, D;
  int max_seqlen, C, topk;
  int mc, slots, hist, NP;               // NP = partial results per row
  int64_t rows, lists;
  int fp16;                              // element type of q, k, v, out: 0 bf16, 1 fp16
  int64_t sel_rs;                        // elements between two ranks of `selected` (heads of the full tensor * Tq)
  int64_t sq_t, sq_h, sk_t, sk_h, sv_t, sv_h, so_t, so_h;
};

__host__ inline int cdiv_i(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// Token tiles of `tile` tokens per sequence that the gating and scatter grids enumerate: those
// of max_seqlen when every token is a query; with a query window only as many as Tq tokens can
// overlap (one more than they fill), counted from window_tile0 of the sequence, so that a
// decode step on a long prefix does not walk over the tiles of the whole prefix.
__host__ __device__ inline int window_tiles(const Params& p, int tile) {
  const int64_t all = ((int64_t)p.max_seqlen + tile - 1) / tile;
  if (p.Tq == p.T) return (int)all;
  const int64_t w = (p.Tq + tile - 1) / tile + 1;
  return (int)(w < all ? w : all);
}
// First tile of the sequence starting at packed token s0 that can hold a token of the window.
__device__ __forceinline__ int window_tile0(const Params& p, int s0, int tile) {
  return (p.Tq == p.T || p.win_lo <= s0) ? 0 : (p.win_lo - s0) / tile;
}

__device__ __forceinline__ float bf16_lo(uint32_t x) { return __uint_as_float(x << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t x) { return __uint_as_float(x & 0xffff0000u); }

// 16-bit element helpers; kHalf selects fp16, otherwise bf16.  Tensors are passed as
// __nv_bfloat16* whatever their element type: only these helpers interpret the bits.
template <bool kHalf>
__device__ __forceinline__ float2 unpack2(uint32_t x) {
  if (kHalf) return __half22float2(*reinterpret_cast<const __half2*>(&x));
  return make_float2(bf16_lo(x), bf16_hi(x));
}
template <bool kHalf>
__device__ __forceinline__ uint32_t pack2_16(float lo, float hi) {       // round to nearest even
  if (kHalf) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <bool kHalf>
__device__ __forceinline__ void unpack8(const uint4 x, float (&f)[8]) {
  const float2 a = unpack2<kHalf>(x.x), b = unpack2<kHalf>(x.y), c = unpack2<kHalf>(x.z), d = unpack2<kHalf>(x.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// Partial results of the dense stage (one per row and attended chunk; the reference keeps them
// in the input dtype, attention.py:727).  The normalised O row is stored as fp16 scaled by a
// power of two chosen per row, so that its largest magnitude lands in [2^13, 2^14): 11
// significant bits on every element whatever the range of V, no overflow.  partial_lse holds
// two floats per entry: the natural-log LSE (-inf: the entry contributes nothing) and 1 / scale.
struct PartialScale { float scale, inv; };
__device__ __forceinline__ PartialScale partial_scale(float amax) {
  // floor(log2 amax) from the exponent field: -127 for zero and subnormals, 128 for inf / NaN
  int s = 13 - ((int)((__float_as_uint(amax) >> 23) & 0xFF) - 127);
  s = s < -100 ? -100 : (s > 100 ? 100 : s);
  PartialScale r;
  r.scale = __uint_as_float((uint32_t)(127 + s) << 23);
  r.inv = __uint_as_float((uint32_t)(127 - s) << 23);
  return r;
}
__device__ __forceinline__ uint32_t pack2_half(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Chunk slot geometry (routing.py:565-579).
struct Slot {
  int start, end;        // token range [start, end)
  bool historical;       // may be selected by later queries
};
__device__ __forceinline__ Slot slot_of(const int32_t* __restrict__ cu, int b, int j, int C) {
  const int s0 = cu[b], s1 = cu[b + 1];
  Slot s;
  const long long st = (long long)s0 + (long long)j * C;
  s.start = st < s1 ? (int)st : s1;
  const long long en = (long long)s.start + C;
  s.end = en < s1 ? (int)en : s1;
  s.historical = s.end < s1;
  return s;
}

// Work item of the dense stage.
struct Item {
  int valid;             // 0: nothing to do
  int causal;            // 1: own chunk, rows are consecutive tokens of one head
  int nrows;             // rows in this item (<= tile rows)
  int row_start;         // routed: first index into row_list; own: first row inside the query window
  int tok0;              // own: first query token
  int head;              // own: query head
  int kv_head;
  int kv_tok0;           // first key token
  int kv_len;            // keys to visit
};

// Slots that can hold tokens of the query window: [lo, lo + n).  All slots when every token
// is a query; otherwise from the slot of the window's first token to that of its last one
// (packed tokens rise with the slot index), so that a short window - a decode step is one
// token - does not enumerate the own-chunk tiles of the whole batch.
struct SlotRange { int lo, n; };
__device__ __forceinline__ SlotRange own_slot_range(const Params& p, const int32_t* __restrict__ cu) {
  SlotRange sr;
  sr.lo = 0;
  sr.n = (int)p.slots;
  if (p.Tq == p.T) return sr;
  int at[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int tok = e == 0 ? p.win_lo : p.win_lo + (int)p.Tq - 1;
    int l = 0, r = p.B;                       // last sequence with cu[b] <= tok
    while (r - l > 1) {
      const int mid = (l + r) >> 1;
      if (__ldg(cu + mid) <= tok) l = mid; else r = mid;
    }
    at[e] = l * p.mc + (tok - __ldg(cu + l)) / p.C;
  }
  sr.lo = at[0];
  sr.n = at[1] - at[0] + 1;
  return sr;
}

// Decode work item `i`.  Routed items come first (list-major, tiles of
// `tile_rows` rows), own-chunk items follow with the longest tiles first, over the
// slots [own.lo, own.lo + own.n) (own.n < 0: all slots).
// `list_hint` >= 0: the list of a routed item, found by the caller (the last l with
// tile_prefix[l] <= i); otherwise it is searched for in tile_prefix.
__device__ __forceinline__ Item decode_item(const Params& p, int i, int n_routed, int tile_rows,
                                            const int32_t* __restrict__ cu,
                                            const int32_t* __restrict__ list_counts,
                                            const int32_t* __restrict__ list_offsets,
                                            const int32_t* __restrict__ tile_prefix, int list_hint = -1,
                                            SlotRange own = SlotRange{0, -1}) {
  Item it;
  it.valid = 0;
  if (i < n_routed) {
    int l = list_hint;
    if (l < 0) {
      int lo = 0, hi = (int)p.lists;         // last l with tile_prefix[l] <= i
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_prefix[mid] <= i) lo = mid; else hi = mid;
      }
      l = lo;
    }
    const int tile = i - tile_prefix[l];
    const int slot = l / p.Hkv;
    const int b = slot / p.mc, j = slot - b * p.mc;
    it.valid = 1;
    it.causal = 0;
    it.row_start = list_offsets[l] + tile * tile_rows;
    const int left = list_counts[l] - tile * tile_rows;
    it.nrows = left < tile_rows ? left : tile_rows;
    it.kv_head = l - slot * p.Hkv;
    it.kv_tok0 = cu[b] + j * p.C;
    it.kv_len = p.C;
    it.tok0 = 0;
    it.head = 0;
    return it;
  }
  const int tiles_per_chunk = (p.C + tile_rows - 1) / tile_rows;
  const int per_tile = (own.n < 0 ? (int)p.slots : own.n) * p.Hq;
  int idx = i - n_routed;
  const int ti = tiles_per_chunk - 1 - idx / per_tile;
  idx -= (idx / per_tile) * per_tile;
  const int slot = own.lo + idx / p.Hq;
  const int h = idx - (slot - own.lo) * p.Hq;
  const int b = slot / p.mc, j = slot - b * p.mc;
  const Slot s = slot_of(cu, b, j, p.C);
  const int tok0 = s.start + ti * tile_rows;
  if (ti < 0) return it;
  // the tile keeps its place in the chunk; of its rows, those inside the query window
  // [first, nrows) are computed (a window may start and end anywhere)
  const int win_hi = p.win_lo + (int)p.Tq;
  const int tok_end = s.end < win_hi ? s.end : win_hi;
  const int first = p.win_lo > tok0 ? p.win_lo - tok0 : 0;
  const int nrows = tok_end - tok0 < tile_rows ? tok_end - tok0 : tile_rows;
  if (first >= nrows) return it;
  it.valid = 1;
  it.causal = 1;
  it.tok0 = tok0;
  it.nrows = nrows;
  it.head = h;
  it.kv_head = h / p.G;
  it.kv_tok0 = s.start;
  it.kv_len = tok0 + nrows - s.start;
  it.row_start = first;
  return it;
}

__host__ __device__ inline int own_item_count(int slots, int Hq, int C, int tile_rows) {
  return slots * Hq * ((C + tile_rows - 1) / tile_rows);
}

// ---- launchers implemented in the kernel files -----------------------------
cudaError_t launch_chunk_metadata(const Params& p, const int32_t* cu, int32_t* cu_chunk,
                                  int32_t* chunk_end, int8_t* valid, cudaStream_t st);
cudaError_t launch_chunk_means(const Params& p, const __nv_bfloat16* k, const int32_t* cu,
                               __nv_bfloat16* means, cudaStream_t st);
cudaError_t launch_chunk_means_range(const Params& p, int slot_begin, int slot_end, const __nv_bfloat16* k,
                                     const int32_t* cu, __nv_bfloat16* means, cudaStream_t st);
cudaError_t launch_gate_topk(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* means,
                             const int32_t* cu, int32_t* selected, int32_t* list_counts,
                             cudaStream_t st);
// The same with optional statistics (int32[4], added to: [0] rows whose near-ties were ranked
// again in the contract order, [1] largest |estimate - contract score| / eps seen there in
// units of 2^-16, [2] rows where that ratio exceeded 1, [3] rows ranked over all candidates)
// and flags (1: rank every row over all candidates, 2: rank the kept candidates of every row again).
cudaError_t launch_gate_topk_stats(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* means,
                                   const int32_t* cu, int32_t* selected, int32_t* list_counts, int32_t* stats,
                                   int flags, cudaStream_t st);
// false when the shared memory the gating kernel needs for `p` exceeds what an SM offers
bool gate_topk_fits(const Params& p);
cudaError_t launch_compact(const Params& p, const int32_t* cu, const int32_t* selected,
                           const int32_t* list_counts, int32_t* list_offsets, int32_t* tile_prefix,
                           int32_t* cursors, int32_t* row_list, float2* partial_lse, int tile_rows,
                           cudaStream_t st);
cudaError_t launch_merge(const Params& p, const __half* partial_out, const float2* partial_lse,
                         const int32_t* status, __nv_bfloat16* out, float* lse_out, cudaStream_t st);

constexpr int kMmaTileRows = 128;        // rows per work item, mma.sync kernel
constexpr int kTc5TileRows = 256;        // rows per work item, tcgen05 kernel (two 128-row MMA tiles)
constexpr int kTileRowsWide = 128;       // rows per work item, tcgen05 kernel at head_dim 256 (one tile)
// Chunks of at most this many keys run the tcgen05 kernel for short items (128-row items, two CTAs per SM).
#ifndef MOBA_SMALL_CHUNK
#define MOBA_SMALL_CHUNK 256
#endif
constexpr int kSmallChunk = MOBA_SMALL_CHUNK;
__host__ __device__ inline bool tc5_small_items(int head_dim, int chunk) { return head_dim <= 128 && chunk <= kSmallChunk; }

cudaError_t launch_attend_mma(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                              const __nv_bfloat16* v, const int32_t* cu, const int32_t* list_counts,
                              const int32_t* list_offsets, const int32_t* tile_prefix,
                              const int32_t* row_list, __half* partial_out, float2* partial_lse,
                              int32_t* work_counter, cudaStream_t st);
cudaError_t launch_attend_tc5(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                              const __nv_bfloat16* v, const int32_t* cu, const int32_t* list_counts,
                              const int32_t* list_offsets, const int32_t* tile_prefix,
                              const int32_t* row_list, __half* partial_out, float2* partial_lse,
                              int32_t* work_counter, int32_t* status, cudaStream_t st);

cudaError_t launch_bounded_wait_probe(int32_t* status, unsigned long long limit_ns, cudaStream_t st);

// ---- backward (training path), attend_bwd.cu ---------------------------------
cudaError_t launch_count_lists(const Params& p, const int32_t* selected, int32_t* list_counts, cudaStream_t st);
cudaError_t launch_bwd_delta(const Params& p, const __nv_bfloat16* out, const __nv_bfloat16* dout, int64_t do_t,
                             int64_t do_h, const float* lse, float* delta, float* lse2, cudaStream_t st);
cudaError_t launch_bwd_dq(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                          const __nv_bfloat16* dout, int64_t do_t, int64_t do_h, const int32_t* cu,
                          const int32_t* list_counts, const int32_t* list_offsets, const int32_t* tile_prefix,
                          const int32_t* row_list, const float* lse2, const float* delta, float* partial_dq,
                          int32_t* work_counter, cudaStream_t st);
cudaError_t launch_bwd_dq_tc5(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                              const __nv_bfloat16* v, const __nv_bfloat16* dout, const int32_t* cu,
                              const int32_t* list_counts, const int32_t* list_offsets, const int32_t* tile_prefix,
                              const int32_t* row_list, const float* lse2, const float* delta, float* partial_dq,
                              int32_t* work_counter, int32_t* status, cudaStream_t st);
cudaError_t launch_bwd_dkdv_tc5(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                                const __nv_bfloat16* v, const __nv_bfloat16* dout, const int32_t* cu,
                                const int32_t* list_counts, const int32_t* list_offsets, const int32_t* row_list,
                                const float* lse2, const float* delta, __nv_bfloat16* dk, __nv_bfloat16* dv,
                                __nv_bfloat16* packed, int32_t* work_counter, int32_t* status, cudaStream_t st);
// 16-bit elements of the `packed` scratch of launch_bwd_dkdv_tc5 (Q and dO rows of the routed lists)
inline int64_t bwd_packed_elems(const Params& p) { return 2 * ((int64_t)p.hist * p.rows + 64) * p.D; }
cudaError_t launch_bwd_sum_dq(const Params& p, const float* partial_dq, const int32_t* selected, const int32_t* status,
                              __nv_bfloat16* dq, int64_t dq_t, int64_t dq_h, cudaStream_t st);
cudaError_t launch_bwd_dkdv(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                            const __nv_bfloat16* dout, int64_t do_t, int64_t do_h, const int32_t* cu,
                            const int32_t* list_counts, const int32_t* list_offsets, const int32_t* row_list,
                            const float* lse2, const float* delta, __nv_bfloat16* dk, int64_t dk_t, int64_t dk_h,
                            __nv_bfloat16* dv, int64_t dv_t, int64_t dv_h, int32_t* work_counter, cudaStream_t st);

}  // namespace moba
