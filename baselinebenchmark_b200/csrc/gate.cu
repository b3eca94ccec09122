// Gating stage of MoBA: chunk slot tables, mean-pooled keys, q.mean scores with
// the causal chunk mask and a per-(token, head) top-k.
//
// Replaces, for the inference path of the reference,
//   _dense_chunk_metadata_kernel            backends/_mthreads/ops/moba/routing.py:553-592
//   _dense_chunk_mean_kernel                routing.py:690-737
//   _chunk_topk_batched_streaming_kernel    routing.py:1056-1182
//
// K and Q are read once.  The selection is defined by one fixed fp32 summation
// order, so that a CPU restatement reproduces it bit for bit; the scores of all
// candidates are first estimated on the tensor core and only the candidates the
// estimate cannot rank with certainty are evaluated in that order (see the
// scores section below):
//   mean : row r of a chunk is added to accumulator r % 32 in increasing r, the
//          32 accumulators are added in increasing index, the total is divided
//          by C and rounded to bf16 (round to nearest even);
//   score: products of two 16-bit values are exact in fp32; each block of 8
//          dims is added left to right, then a halving tree combines the D/8
//          block sums (for D = 128: block l + block l+8, then l + l+4, l + l+2,
//          l + l+1); a block count that is no power of two (D = 96) is padded
//          with blocks of +0.0 to the next one.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "topk_network.cuh"

namespace moba {

// ---------------------------------------------------------------------------
// slot tables
// ---------------------------------------------------------------------------
__global__ void chunk_metadata_kernel(Params p, const int32_t* __restrict__ cu,
                                      int32_t* __restrict__ cu_chunk,
                                      int32_t* __restrict__ chunk_end,
                                      int8_t* __restrict__ valid) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s == 0) cu_chunk[p.slots] = cu[p.B];
  if (s >= p.slots) return;
  const int b = s / p.mc, j = s - b * p.mc;
  const Slot sl = slot_of(cu, b, j, p.C);
  cu_chunk[s] = sl.start;
  chunk_end[s] = sl.historical ? sl.end : 0;
  valid[s] = sl.historical ? 1 : 0;
}

cudaError_t launch_chunk_metadata(const Params& p, const int32_t* cu, int32_t* cu_chunk,
                                  int32_t* chunk_end, int8_t* valid, cudaStream_t st) {
  const int threads = 256;
  chunk_metadata_kernel<<<cdiv_i(p.slots, threads), threads, 0, st>>>(p, cu, cu_chunk, chunk_end, valid);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// chunk means: one CTA per (slot, kv head), 32 row lanes x D/8 dim lanes
// (16-byte loads).
// ---------------------------------------------------------------------------
template <bool kHalf, int D>
__global__ void __launch_bounds__(kMeanLanes * (D / 8))
chunk_mean_kernel(Params p, int slot_begin, const __nv_bfloat16* __restrict__ k, const int32_t* __restrict__ cu,
                  __nv_bfloat16* __restrict__ means) {
  const int slot = slot_begin + blockIdx.x, hk = blockIdx.y;
  const int b = slot / p.mc, j = slot - b * p.mc;
  const Slot sl = slot_of(cu, b, j, p.C);
  constexpr int kDimLanes = D / 8;
  const int dl = threadIdx.x % kDimLanes;  // dims 8*dl .. 8*dl+7
  const int rl = threadIdx.x / kDimLanes;  // row lane 0..31
  __nv_bfloat16* dst = means + ((int64_t)slot * p.Hkv + hk) * D;

  __shared__ float part[kMeanLanes][D + 4];
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  if (sl.historical) {                     // historical chunks are always full: C rows
    const __nv_bfloat16* base = k + (int64_t)sl.start * p.sk_t + (int64_t)hk * p.sk_h + dl * 8;
    int r = rl;
    // four rows in flight per thread, accumulated in increasing r
    for (; r + 3 * kMeanLanes < p.C; r += 4 * kMeanLanes) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        x[u] = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)(r + u * kMeanLanes) * p.sk_t));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        unpack8<kHalf>(x[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    for (; r < p.C; r += kMeanLanes) {
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)r * p.sk_t));
      float f[8];
      unpack8<kHalf>(x, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[rl][dl * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float tot = part[0][threadIdx.x];
#pragma unroll
    for (int a = 1; a < kMeanLanes; ++a) tot += part[a][threadIdx.x];
    const float mean = sl.historical ? __fdiv_rn(tot, (float)p.C) : 0.f;
    if (kHalf) reinterpret_cast<__half*>(dst)[threadIdx.x] = __float2half_rn(mean);
    else dst[threadIdx.x] = __float2bfloat16_rn(mean);
  }
}

// Means of the slots [slot_begin, slot_end) only (context-parallel ranks compute those of their own chunks).
cudaError_t launch_chunk_means_range(const Params& p, int slot_begin, int slot_end, const __nv_bfloat16* k,
                                     const int32_t* cu, __nv_bfloat16* means, cudaStream_t st) {
  if (slot_end <= slot_begin) return cudaSuccess;
  dim3 grid(slot_end - slot_begin, p.Hkv);
#define MOBA_MEANS(HALF, DIM) \
  chunk_mean_kernel<HALF, DIM><<<grid, kMeanLanes * (DIM / 8), 0, st>>>(p, slot_begin, k, cu, means)
  switch (p.D) {
    case 64:  if (p.fp16) MOBA_MEANS(true, 64);  else MOBA_MEANS(false, 64);  break;
    case 96:  if (p.fp16) MOBA_MEANS(true, 96);  else MOBA_MEANS(false, 96);  break;
    case 128: if (p.fp16) MOBA_MEANS(true, 128); else MOBA_MEANS(false, 128); break;
    case 256: if (p.fp16) MOBA_MEANS(true, 256); else MOBA_MEANS(false, 256); break;
    default: return cudaErrorInvalidValue;
  }
#undef MOBA_MEANS
  return cudaGetLastError();
}

cudaError_t launch_chunk_means(const Params& p, const __nv_bfloat16* k, const int32_t* cu,
                               __nv_bfloat16* means, cudaStream_t st) {
  return launch_chunk_means_range(p, 0, p.slots, k, cu, means, st);
}

// ---------------------------------------------------------------------------
// scores + mask + top-k
//
// Two steps per (token, head) row, with the same result as scoring every
// candidate in the contract order above:
//
//   1. estimate on the tensor core.  A row tile is 128 rows: the tokens of a
//      tile x the query heads of one kv head.  Persistent CTAs (128 threads)
//      walk the row tiles; TMA brings the Q rows of a tile and a tile of up to
//      256 candidate means into shared memory in the 128-byte swizzled K-major
//      layout, tcgen05.mma multiplies them (fp32 accumulators in tensor
//      memory, one lane per row), and thread r reads the estimates a_c of its
//      row 32 at a time and keeps the L = hist + 1 (+ 3 when a row can have
//      more than 32 candidates) largest, sorted, in shared memory.  For
//      L <= 32 the 32 estimates become order-preserving integer keys whose
//      five lowest bits hold the position (a change of less than 2^-18 of
//      the score, counted in eps), a compare-exchange network over the 32
//      registers brings the largest 8, 16 or 32 keys to the front, and they
//      are merged with the list; longer lists are kept as a min-heap.
//   2. recheck.  With e_c the score in the contract order, |a_c - e_c| <= eps
//      for every candidate of the row (bound below).  If neighbours in the
//      sorted list differ by more than 2 eps down to the entry after the
//      hist-th, the order of the a_c is the order of the e_c and the list is
//      the answer.  Otherwise the candidates with a_c >= a_(hist) - 2 eps (the
//      only ones that can be among the hist best e_c) are scored again by the
//      warp on CUDA cores in the contract order, one candidate per lane, and
//      ranked by the packed key of the reference
//      (order-preserving score bits << 32 | 0xFFFFFFFF - slot,
//      routing.py:778-784, :1151-1153: ties go to the lower slot).  A row
//      whose near-ties overflow the list, whose scores are not finite, or
//      whose tensor-core result did not arrive is ranked over all its
//      candidates the same way.
//
// Error bound.  Products of two 16-bit inputs are exact in fp32, so both
// results differ from the real dot product by summation error only.  Contract
// order: 7 + log2(D/8) roundings on a path, each <= 2^-24 of a partial sum
// that is <= S = sum_i |q_i m_i|.  Tensor core: per 16-dim step the 16
// products and the accumulator are aligned to the largest exponent and
// truncated; assuming no more than one unit of the 24-bit significand of that
// exponent is lost per term and one more when the sum is normalised, a step
// loses <= 18 * 2^-23 * S.  Together eps = ((18 * D/16 + 16) * 2^-23 + 2^-18) * S
// with S <= |q|_2 |m|_2 (Cauchy-Schwarz, the largest norm over the staged means),
// plus 2^-100 for products flushed to zero.  The recheck step measures
// |a_c - e_c| / eps on every candidate it scores again (optional statistics
// output), so the assumption is observable: on random inputs the largest
// ratio seen is below 0.01.
// ---------------------------------------------------------------------------
namespace {

using namespace ptx;

constexpr int kGateThreads = 128;         // one thread per row = one TMEM lane
constexpr int kGateRows = 128;            // (token, head) rows per tile
constexpr int kListExtra = 3;             // list places beyond hist + 1 that absorb near-ties at the cut
constexpr int kCntSmemMax = 4096;         // chunks per sequence up to which the list histogram is kept in shared memory
constexpr int kQBlockBytes = 128 * 128;   // one [128 rows][64 dims] swizzled block of 16-bit values
constexpr int kScratchStride = 36;        // floats per row of the score scratch (144 bytes: conflict-free 16-byte stores)

__device__ __forceinline__ uint32_t float_key(float x) {      // routing.py:778-784
  const uint32_t b = __float_as_uint(x);
  return b ^ ((b & 0x80000000u) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {      // inverse of float_key
  return __uint_as_float(k ^ ((k & 0x80000000u) ? 0x80000000u : 0xFFFFFFFFu));
}
__device__ __forceinline__ float dot8(const float (&q)[8], const float (&m)[8]) {
  float s = __fmul_rn(q[0], m[0]);
#pragma unroll
  for (int i = 1; i < 8; ++i) s = __fmaf_rn(q[i], m[i], s);
  return s;
}

// shared-memory matrix descriptor of a K-major, 128-byte swizzled tile (8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t gate_desc(uint32_t addr) {
  constexpr uint64_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (hi << 32) | (uint64_t)(((addr & 0x3FFFFu) >> 4) | (1u << 16));
}

// byte offset of the 16-byte piece `ch` of row `r` inside a tile of [rows][64]-element blocks
__device__ __forceinline__ uint32_t swz_piece(int r, int ch, int block_bytes) {
  return (uint32_t)((ch >> 3) * block_bytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4));
}

struct GateCtrl {
  uint64_t q_full[2];
  uint64_t b_full;
  uint64_t mma_done;
  uint32_t tmem_slot;
  int32_t mean_ssq_max;                    // largest squared norm over the means seen so far of this (sequence, kv head)
  unsigned long long exact[kGateThreads / 32][64];   // per warp: keys of the row being ranked exactly
};

// Squared norm of row `r` of a swizzled tile.
template <bool kHalf, int D>
__device__ __forceinline__ float row_ssq(const unsigned char* tile, int r, int block_bytes) {
  float ssq = 0.f;
#pragma unroll 4
  for (int ch = 0; ch < D / 8; ++ch) {
    float f[8];
    unpack8<kHalf>(*reinterpret_cast<const uint4*>(tile + swz_piece(r, ch, block_bytes)), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) ssq = __fmaf_rn(f[e], f[e], ssq);
  }
  return ssq;
}
// Squared norm of the D values at `row` (global memory).
template <bool kHalf, int D>
__device__ __forceinline__ float global_ssq(const __nv_bfloat16* row) {
  float ssq = 0.f;
#pragma unroll 4
  for (int ch = 0; ch < D / 8; ++ch) {
    float f[8];
    unpack8<kHalf>(__ldg(reinterpret_cast<const uint4*>(row + ch * 8)), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) ssq = __fmaf_rn(f[e], f[e], ssq);
  }
  return ssq;
}

// Score of row `r` (Q tile in shared memory) against the mean at `mrow` (global), in the contract order.
// (not inlined: it is called from the two rarely taken recheck paths, and one copy keeps the
// kernel's hot loop small in the instruction cache)
template <bool kHalf, int D>
__device__ __noinline__ float contract_score(const unsigned char* sQ, int r, const __nv_bfloat16* mrow) {
  constexpr int kNB = D / 8;
  constexpr int kNBPad = kNB <= 8 ? 8 : (kNB <= 16 ? 16 : 32);
  uint4 mraw[kNB];
#pragma unroll
  for (int l = 0; l < kNB; ++l) mraw[l] = __ldg(reinterpret_cast<const uint4*>(mrow + l * 8));
  float b[kNBPad];
#pragma unroll
  for (int l = 0; l < kNBPad; ++l) {
    if (l < kNB) {
      float qf[8], mf[8];
      unpack8<kHalf>(*reinterpret_cast<const uint4*>(sQ + swz_piece(r, l, kQBlockBytes)), qf);
      unpack8<kHalf>(mraw[l], mf);
      b[l] = dot8(qf, mf);
    } else {
      b[l] = 0.f;
    }
  }
#pragma unroll
  for (int h = kNBPad / 2; h >= 1; h >>= 1)
#pragma unroll
    for (int l = 0; l < h; ++l) b[l] = __fadd_rn(b[l], b[l + h]);
  return b[0];
}

// Min-heap of {chunk, key} on the key: `heap[0]` is the smallest key kept.  Replaces the
// root by (key, chunk) and restores the heap.
__device__ __forceinline__ void heap_replace_root(uint2* heap, int n, uint32_t key, uint32_t chunk) {
  int k = 0;
  for (;;) {
    const int l = 2 * k + 1;
    if (l >= n) break;
    uint2 child = heap[l];
    int s = l;
    if (l + 1 < n) {
      const uint2 right = heap[l + 1];
      if (right.y < child.y) { child = right; s = l + 1; }
    }
    if (!(child.y < key)) break;
    heap[k] = child;
    k = s;
  }
  heap[k] = make_uint2(chunk, key);
}

enum { GATE_FORCE_EXACT = 1, GATE_FORCE_RECHECK = 2 };
// marks in the chunk word of a list entry (chunk indices are below 2^24; an empty place is 0xFFFFFFFF)
constexpr uint32_t kTied = 1u << 30, kRunStart = 1u << 29, kChunkMask = 0x00FFFFFFu;

// Resident CTAs per SM the register budget is set for: four with the narrow network (its
// working set is small and the kernel is bound by the latency of dependent instructions, which
// more warps hide), three otherwise (a fourth would spill the 32 keys of the wide network).
template <int kW> constexpr int kGateMinCtas = kW == 8 ? 4 : 3;

struct GateTile {
  int valid, b, hk, s0, tok_lo, ntok, max_cand;
};

__device__ __forceinline__ GateTile gate_tile(const Params& p, const int32_t* __restrict__ cu, int i, int tiles_x,
                                              int tokens_per_cta) {
  GateTile t;
  const int rest = i / tiles_x;
  t.hk = rest % p.Hkv;
  t.b = rest / p.Hkv;
  t.s0 = cu[t.b];
  const int s1 = cu[t.b + 1];
  const int x = i - rest * tiles_x + window_tile0(p, t.s0, tokens_per_cta);
  // tokens of the tile, clipped to the sequence and to the query window
  t.tok_lo = max(t.s0 + x * tokens_per_cta, p.win_lo);
  const int tok_hi = min(min(t.s0 + (x + 1) * tokens_per_cta, s1), p.win_lo + (int)p.Tq);
  t.valid = t.tok_lo < tok_hi;
  t.ntok = tok_hi - t.tok_lo;
  // candidates of the last token of the tile bound the chunks to stage
  t.max_cand = t.valid ? (tok_hi - 1 - t.s0) / p.C : 0;
  return t;
}

// kW: width of the compare-exchange network (8, 16 or 32 >= list_len), 0: lists longer than 32 (min-heap)
template <bool kHalf, int D, int kW>
__global__ void __launch_bounds__(kGateThreads, kGateMinCtas<kW>)
gate_topk_kernel(const Params p, const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_m,
                 int tokens_per_cta, int nt, int list_len, int nbuf, int cnt_in_smem,
                 const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ means,
                 const int32_t* __restrict__ cu, int32_t* __restrict__ selected,
                 int32_t* __restrict__ list_counts, int32_t* __restrict__ stats, int flags) {
  extern __shared__ unsigned char gate_smem_raw[];
  constexpr int kNBlk = (D + 63) / 64;                 // 64-dim blocks of a row
  const int hist = p.hist;
  const int lstride = list_len | 1;                    // odd: the rows' lists start in different banks

  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)gate_smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ0 = smem;                                             // nbuf x kNBlk blocks [128][64]
  unsigned char* sB = sQ0 + (size_t)nbuf * kNBlk * kQBlockBytes;        // kNBlk blocks [nt][64]
  uint2* lists = reinterpret_cast<uint2*>(sB + (size_t)kNBlk * nt * 128);   // [128][lstride] {chunk, score bits}
  float* scratch = reinterpret_cast<float*>(lists + (size_t)kGateRows * lstride);   // [128][36], absent when unused
  const bool has_scratch = kW == 0 || p.mc - 1 > 32;   // one 32-candidate step per row needs no merge
  GateCtrl& c = *reinterpret_cast<GateCtrl*>(scratch + (has_scratch ? kGateRows * kScratchStride : 0));
  int32_t* cnt_s = reinterpret_cast<int32_t*>(&c + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_x = window_tiles(p, tokens_per_cta);
  const int n_tiles = tiles_x * p.Hkv * p.B;
  const int rows_box = tokens_per_cta * p.G;           // rows one Q box brings

  if (tid == 0) {
    mbar_init(smem_u32(&c.q_full[0]), 1);
    mbar_init(smem_u32(&c.q_full[1]), 1);
    mbar_init(smem_u32(&c.b_full), 1);
    mbar_init(smem_u32(&c.mma_done), 1);
    c.mean_ssq_max = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_m);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&c.tmem_slot), (uint32_t)nt);
    tmem_relinquish();
  }
  if (cnt_in_smem)
    for (int i = tid; i < p.mc; i += kGateThreads) cnt_s[i] = 0;       // every tile leaves them at zero again
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c.tmem_slot;
  const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);          // this thread's lane, column 0

  // producer state (thread 0): Q tiles requested so far, tile index to look for the next one from
  int q_requested = 0, q_next_from = blockIdx.x;
  uint32_t b_phase = 0, mma_phase = 0;
  int n = 0;                                           // tiles with candidates processed so far
  // mean norms: the (sequence, kv head) the running maximum belongs to and the candidates it covers
  int norm_b = -1, norm_hk = -1, norm_covered = 0;

  auto request_q = [&](const GateTile& t, int buf) {
    const uint32_t bar = smem_u32(&c.q_full[buf]);
    mbar_expect_tx(bar, (uint32_t)(kNBlk * rows_box * 128));
#pragma unroll
    for (int blk = 0; blk < kNBlk; ++blk)
      tma_load_3d(smem_u32(sQ0 + ((size_t)buf * kNBlk + blk) * kQBlockBytes), &tmap_q, bar, blk * 64, t.hk * p.G,
                  t.tok_lo - p.win_lo);
  };
  auto request_b = [&](const GateTile& t, int c0) {
    const uint32_t bar = smem_u32(&c.b_full);
    mbar_expect_tx(bar, (uint32_t)(kNBlk * nt * 128));
#pragma unroll
    for (int blk = 0; blk < kNBlk; ++blk)
      tma_load_3d(smem_u32(sB + (size_t)blk * nt * 128), &tmap_m, bar, blk * 64, t.hk, t.b * p.mc + c0);
  };

  for (int ti = blockIdx.x; ti < n_tiles; ti += gridDim.x) {
    const GateTile t = gate_tile(p, cu, ti, tiles_x, tokens_per_cta);
    if (!t.valid) continue;
    const int nrows = t.ntok * p.G;
    const int slot0 = t.b * p.mc;
    // selected[r][head][tok]: `ntok` consecutive ints per (rank, head)
    auto store_selected = [&](int i, int slot) {
      const int r = i / nrows, rem = i - r * nrows;
      const int hl = rem / t.ntok, tl = rem - hl * t.ntok;
      selected[(int64_t)r * p.sel_rs + (int64_t)(t.hk * p.G + hl) * p.Tq + (t.tok_lo - p.win_lo) + tl] = slot;
    };
    if (t.max_cand <= 0) {                             // first chunk of a sequence: nothing to select
      for (int i = tid; i < hist * nrows; i += kGateThreads) store_selected(i, -1);
      continue;
    }
    const int buf = nbuf == 2 ? (n & 1) : 0;
    const uint32_t q_phase = nbuf == 2 ? ((n >> 1) & 1) : (n & 1);
    unsigned char* sQ = sQ0 + (size_t)buf * kNBlk * kQBlockBytes;
    if (tid == 0) {
      if (q_requested == n) {                          // not prefetched (first tile, or a single buffer)
        request_q(t, buf);
        q_requested = n + 1;
        q_next_from = ti + gridDim.x;
      }
      request_b(t, 0);
      if (nbuf == 2 && q_requested == n + 1) {         // the next tile with candidates, into the other buffer
        for (; q_next_from < n_tiles; q_next_from += gridDim.x) {
          const GateTile nx = gate_tile(p, cu, q_next_from, tiles_x, tokens_per_cta);
          if (nx.valid && nx.max_cand > 0) {
            request_q(nx, buf ^ 1);
            q_requested = n + 2;
            q_next_from += gridDim.x;
            break;
          }
        }
      }
    }

    // Largest squared norm over the means this tile's rows can meet: kept per (sequence, kv head)
    // and extended when a tile reaches further than the ones before it (a CTA walks the tiles
    // of a sequence in order, so every mean is read once per CTA).
    if (t.b != norm_b || t.hk != norm_hk || t.max_cand > norm_covered) {
      const bool fresh = t.b != norm_b || t.hk != norm_hk;
      if (fresh) {                                   // every thread is past its last read of the old maximum
        if (tid == 0) c.mean_ssq_max = 0;
        __syncthreads();
      }
      int ssq_max = 0;
      for (int cc = (fresh ? 0 : norm_covered) + tid; cc < t.max_cand; cc += kGateThreads)
        // floats >= 0 order like their bit patterns; +inf and NaN have the largest patterns
        ssq_max = max(ssq_max, __float_as_int(global_ssq<kHalf, D>(means + ((int64_t)(slot0 + cc) * p.Hkv + t.hk) * D)) &
                                   0x7FFFFFFF);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq_max = max(ssq_max, __shfl_xor_sync(0xffffffffu, ssq_max, o));
      if (lane == 0 && ssq_max > 0) atomicMax(&c.mean_ssq_max, ssq_max);
      __syncthreads();
      norm_b = t.b;
      norm_hk = t.hk;
      norm_covered = t.max_cand;
    }

    // this thread's row
    const int row = tid;
    const int ncand = row < nrows ? (t.tok_lo + row / p.G - t.s0) / p.C : 0;     // chunks before the row's own chunk
    uint2* mylist = lists + (size_t)row * lstride;
    for (int i = 0; i < list_len; ++i) mylist[i] = make_uint2(0xFFFFFFFFu, 0u);   // chunk -1, key 0: empty place
    uint32_t tau = 0;                                  // smallest key kept (heap root / last place); 0 while places are free
    uint32_t* myscratch = reinterpret_cast<uint32_t*>(scratch + row * kScratchStride);

    // A wait that gives up is remembered by the thread: its row is then ranked exactly, from Q rows
    // read with plain loads (see the recheck).
    bool failed = !mbar_wait(smem_u32(&c.q_full[buf]), q_phase);
    const float q_ssq = failed ? 0.f : row_ssq<kHalf, D>(sQ, row, kQBlockBytes);

    for (int c0 = 0; c0 < t.max_cand; c0 += nt) {
      const int ct = min(nt, t.max_cand - c0);
      if (!mbar_wait(smem_u32(&c.b_full), b_phase)) failed = true;
      b_phase ^= 1;
      if (tid == 0) {
        tc_fence_after();
        const uint32_t idesc = idesc_16_f32(kHalf, 128, nt, 0, 0);
        const uint32_t aQ = smem_u32(sQ), aB = smem_u32(sB);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          mma_ss(tmem, gate_desc(aQ + (ks >> 2) * kQBlockBytes + (ks & 3) * 32),
                 gate_desc(aB + (ks >> 2) * nt * 128 + (ks & 3) * 32), idesc, ks > 0);
        tc_commit(smem_u32(&c.mma_done));
      }
      if (!mbar_wait(smem_u32(&c.mma_done), mma_phase)) failed = true;
      mma_phase ^= 1;
      tc_fence_after();
      // ---- estimates of this row: keep the largest in the heap -------------------------------
      const int cend = min(ct, ncand - c0);                   // this row's candidates in the tile
      int wend = cend;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) wend = max(wend, __shfl_xor_sync(0xffffffffu, wend, o));
      for (int col = 0; col < wend; col += 32) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld32(trow + col, v);
        tmem_wait_ld();
        // estimates -> order-preserving keys; places past the row's candidates get key 0
        const int rem = cend - col;
        uint32_t vmax = 0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          uint32_t key = float_key(__uint_as_float(v[i]));
          if (kW > 0) key = (key & ~31u) | (uint32_t)(31 - i);         // position in the low bits: earlier wins ties
          v[i] = i < rem ? key : 0u;
          vmax = max(vmax, v[i]);
        }
        if (!__any_sync(0xffffffffu, vmax > tau)) continue;             // nothing here enters any list of the warp
        const uint32_t chunk0 = (uint32_t)(c0 + col);
        if (kW > 0) {
          topk::top_of_32<(kW > 0 ? kW : 32)>(v);
          if (c0 == 0 && col == 0) {
            // first candidates of the row: the list is the head of the sorted keys
#pragma unroll
            for (int i = 0; i < kW; ++i)
              if (i < list_len) mylist[i] = make_uint2(v[i] ? chunk0 + 31u - (v[i] & 31u) : 0xFFFFFFFFu, v[i]);
          } else {
            // s_t enters the list iff it beats the entry t places from the end (both are sorted)
            int j = 0;
#pragma unroll
            for (int t2 = 0; t2 < kW; ++t2)
              if (t2 < list_len) j += v[t2] > mylist[list_len - 1 - t2].y;
            if (j > 0) {
#pragma unroll
              for (int i = 0; i < kW; i += 4)
                *reinterpret_cast<uint4*>(myscratch + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
              // in-place merge from the bottom: the smaller of the two tails goes to `pos`; equal keys
              // keep the list's entry (an earlier chunk) above
              int i = list_len - j - 1, jj = j - 1;
              for (int pos = list_len - 1; jj >= 0; --pos) {
                const uint32_t sk = myscratch[jj];
                if (i >= 0 && mylist[i].y < sk) {
                  mylist[pos] = mylist[i];
                  --i;
                } else {
                  mylist[pos] = make_uint2(chunk0 + 31u - (sk & 31u), sk);
                  --jj;
                }
              }
            }
          }
          tau = mylist[list_len - 1].y;
        } else {
          uint32_t hits = 0;
#pragma unroll
          for (int i = 0; i < 32; ++i) hits |= v[i] > tau ? (1u << i) : 0u;
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<uint4*>(myscratch + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          // every lane walks its own hits; tau rises as it goes
          while (hits) {
            const int i = __ffs(hits) - 1;
            hits &= hits - 1;
            const uint32_t key = myscratch[i];
            if (key > tau) {
              heap_replace_root(mylist, list_len, key, chunk0 + (uint32_t)i);
              tau = mylist[0].y;
            }
          }
        }
      }
      tc_fence_before();
      if (c0 + nt < t.max_cand) {
        __syncthreads();                                      // the means and their estimates are consumed
        if (tid == 0) request_b(t, c0 + nt);
      }
    }

    // ---- a heap is sorted now: largest key first (equal scores in any order: they are rechecked) ----
    if (kW == 0)
      for (int m = list_len - 1; m > 0; --m) {
        const uint2 last = mylist[m];
        mylist[m] = mylist[0];
        heap_replace_root(mylist, m, last.y, last.x);
      }

    // ---- recheck ------------------------------------------------------------------------------
    // eps of this row (see the head of this section); inf or NaN sends the row to the exact ranking
    constexpr float kKappa = (18.f * (D / 16) + 16.f) / 8388608.f + (kW > 0 ? 1.f / 262144.f : 0.f);
    const float eps = kKappa * 1.001f * sqrtf(q_ssq) * sqrtf(__int_as_float(c.mean_ssq_max)) + 7.9e-31f;
    const int n_keep = min(hist, ncand);
    // 0: list is exact; 3: order the runs of near-ties (marked in the list); 1: rank all survivors;
    // 2: rank all candidates
    int mode = 0, n_surv = 0;
    if (ncand > 0) {
      int n_real = 0;
      for (int i = 0; i < list_len; ++i) n_real += (int32_t)mylist[i].x >= 0;
      if ((flags & GATE_FORCE_EXACT) || failed || n_real < min(ncand, list_len)) {
        mode = 2;
      } else {
        const float eps2 = 2.f * eps;
        const bool all = (flags & GATE_FORCE_RECHECK) != 0;
        // settled by the estimates alone? (the common case: nothing else is computed for the row)
        bool amb = all;
        {
          float prev = key_float(mylist[0].y);
          for (int i = 0; i < n_keep && i + 1 < n_real; ++i) {
            const float next = key_float(mylist[i + 1].y);
            if (!(prev - next > eps2)) amb = true;
            prev = next;
          }
        }
        // survivors: the only candidates that can be among the n_keep best exact scores
        if (amb) {
          const float theta = key_float(mylist[n_keep - 1].y) - eps2;
          while (n_surv < n_real && key_float(mylist[n_surv].y) >= theta) ++n_surv;
        }
        if (!amb) {
          mode = 0;
        } else if ((n_surv == list_len && ncand > list_len) || !(eps2 < INFINITY) || n_surv < n_keep) {
          mode = 2;            // the near-ties may go on below the list, or eps is not finite
        } else {
          // Runs of neighbours closer than 2 eps: entries of different runs are certainly in the
          // order of their estimates, entries of one run are ordered by their exact scores.  The
          // members of a run are marked in the chunk word (kTied, kRunStart on its first member).
          int tied = 0;
          bool in_run = false;
          float prev = key_float(mylist[0].y);
          for (int i = 0; i + 1 < n_surv; ++i) {
            const float next = key_float(mylist[i + 1].y);
            if (all || !(prev - next > eps2)) {
              if (!in_run) { mylist[i].x |= kTied | kRunStart; ++tied; }
              mylist[i + 1].x |= kTied;
              ++tied;
              in_run = true;
            } else {
              in_run = false;
            }
            prev = next;
          }
          if (all && tied == 0) {                             // a single survivor, scored again on request
            mylist[0].x |= kTied | kRunStart;
            tied = 1;
          }
          if (tied > 32) {     // more near-ties than one round of the warp ranks: rank all survivors instead
            for (int i = 0; i < n_surv; ++i) mylist[i].x &= kChunkMask;
            mode = 1;
          } else if (tied > 0) {
            mode = 3;
          }
        }
      }
    }
    __syncwarp();                                             // the marks are visible to the warp
    unsigned need = __ballot_sync(0xffffffffu, mode != 0);
    unsigned long long* lx = c.exact[warp];
    while (need) {
      const int src = __ffs(need) - 1;
      need &= need - 1;
      const int r = warp * 32 + src;
      const int r_mode = __shfl_sync(0xffffffffu, mode, src);
      const int r_total = r_mode == 2 ? __shfl_sync(0xffffffffu, ncand, src) : __shfl_sync(0xffffffffu, n_surv, src);
      const int r_keep = __shfl_sync(0xffffffffu, n_keep, src);
      const float r_eps = __shfl_sync(0xffffffffu, eps, src);
      uint2* rlist = lists + (size_t)r * lstride;
      if (r_mode == 3) {
        // runs of near-ties: one marked entry per lane (at most 32), exact keys, rank inside the run
        int cnt = 0, runs = 0, my_e = -1, my_run = 0;
        for (int e0 = 0; e0 < r_total; e0 += 32) {
          const int e = e0 + lane;
          const uint32_t x = e < r_total ? rlist[e].x : 0u;
          const unsigned bt = __ballot_sync(0xffffffffu, (x & kTied) != 0 && x != 0xFFFFFFFFu);
          const unsigned bs = __ballot_sync(0xffffffffu, (x & kRunStart) != 0 && x != 0xFFFFFFFFu);
          if ((bt >> lane) & 1) {
            const int slot = cnt + __popc(bt & ((1u << lane) - 1));
            const int run = runs + __popc(bs & ((2u << lane) - 1));
            lx[slot] = (unsigned long long)e | ((unsigned long long)run << 8);
          }
          cnt += __popc(bt);
          runs += __popc(bs);
        }
        __syncwarp();
        unsigned long long key = 0ull;
        uint32_t cc = 0;
        if (lane < cnt) {
          my_e = (int)(lx[lane] & 0xFF);
          my_run = (int)(lx[lane] >> 8);
          const uint2 ent = rlist[my_e];
          cc = ent.x & kChunkMask;
          const float e = contract_score<kHalf, D>(sQ, r, means + ((int64_t)(slot0 + (int)cc) * p.Hkv + t.hk) * D);
          key = ((unsigned long long)float_key(e) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)(slot0 + (int)cc));
          if (stats != nullptr) {
            const float diff = fabsf(key_float(ent.y) - e);
            if (!(diff <= r_eps)) atomicAdd(&stats[2], 1);
            atomicMax(&stats[1], (int)fminf(diff / r_eps * 65536.f, 1.0e9f));
          }
        }
        int rank = 0, first = my_e;
        for (int t2 = 0; t2 < cnt; ++t2) {
          const unsigned long long kt = __shfl_sync(0xffffffffu, key, t2);
          const int rt = __shfl_sync(0xffffffffu, my_run, t2), et = __shfl_sync(0xffffffffu, my_e, t2);
          if (lane < cnt && rt == my_run) {
            rank += kt > key;
            first = min(first, et);
          }
        }
        __syncwarp();
        if (lane < cnt) rlist[first + rank].x = cc;          // a run occupies consecutive places; marks are cleared
        __syncwarp();
        if (stats != nullptr && lane == 0) atomicAdd(&stats[0], 1);
        continue;
      }
      lx[lane] = 0ull;
      lx[lane + 32] = 0ull;
      if (__shfl_sync(0xffffffffu, (int)failed, src)) {
        // the row's thread gave up waiting for the Q tile: fetch the row with plain loads into its place
        if (lane < D / 8) {
          const int tl = r / p.G, hl = r - tl * p.G;
          const uint4 val = __ldg(reinterpret_cast<const uint4*>(
              q + (int64_t)(t.tok_lo + tl - p.win_lo) * p.sq_t + (int64_t)(t.hk * p.G + hl) * p.sq_h + lane * 8));
          *reinterpret_cast<uint4*>(sQ + swz_piece(r, lane, kQBlockBytes)) = val;
        }
      }
      __syncwarp();
      int viol = 0, ratio = 0;
      for (int base = 0; base < r_total; base += 32) {
        const int idx = base + lane;
        unsigned long long key = 0ull;
        if (idx < r_total) {
          const int cc = r_mode == 2 ? idx : (int)rlist[idx].x;
          const float e = contract_score<kHalf, D>(sQ, r, means + ((int64_t)(slot0 + cc) * p.Hkv + t.hk) * D);
          key = ((unsigned long long)float_key(e) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)(slot0 + cc));
          if (r_mode == 1 && stats != nullptr) {
            const float diff = fabsf(key_float(rlist[idx].y) - e);
            if (!(diff <= r_eps)) viol = 1;
            ratio = (int)fminf(diff / r_eps * 65536.f, 1.0e9f);
          }
        }
        // the keys of this batch, in lane order, into the ordered list lx[0, r_keep)
        unsigned hits = __ballot_sync(0xffffffffu, key > lx[r_keep - 1]);
        while (hits) {
          const int l = __ffs(hits) - 1;
          hits &= hits - 1;
          const unsigned long long kk = __shfl_sync(0xffffffffu, key, l);
          const unsigned long long k0 = lane < r_keep ? lx[lane] : 0ull;
          const unsigned long long k1 = lane + 32 < r_keep ? lx[lane + 32] : 0ull;
          const int pos = __popc(__ballot_sync(0xffffffffu, k0 > kk)) + __popc(__ballot_sync(0xffffffffu, k1 > kk));
          if (pos < r_keep) {                                  // uniform; false when the list filled up meanwhile
            if (lane >= pos && lane + 1 < r_keep) lx[lane + 1] = k0;
            if (lane + 32 >= pos && lane + 33 < r_keep) lx[lane + 33] = k1;
            if (lane == 0) lx[pos] = kk;
          }
          __syncwarp();
        }
      }
      // the exact ranking replaces the chunk ids of the row's list
      for (int i = lane; i < hist; i += 32) {
        const unsigned long long key = i < r_keep ? lx[i] : 0ull;
        rlist[i].x = key ? (0xFFFFFFFFu - (uint32_t)(key & 0xFFFFFFFFull)) - (uint32_t)slot0 : 0xFFFFFFFFu;
      }
      __syncwarp();
      if (stats != nullptr) {
        viol = __any_sync(0xffffffffu, viol);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ratio = max(ratio, __shfl_xor_sync(0xffffffffu, ratio, o));
        if (lane == 0) {
          atomicAdd(&stats[r_mode == 2 ? 3 : 0], 1);
          if (r_mode == 1) atomicMax(&stats[1], ratio);
          if (viol) atomicAdd(&stats[2], 1);
        }
      }
    }
    // selected[rank][head][token]: every thread stores the chunks of its own row (its list was
    // written by its own warp); neighbouring lanes are neighbouring heads, then tokens
    if (row < nrows) {
      const int tl = row / p.G, hl = row - tl * p.G;
      int32_t* dst = selected + (int64_t)(t.hk * p.G + hl) * p.Tq + (t.tok_lo - p.win_lo) + tl;
      for (int r = 0; r < hist; ++r) {
        const uint32_t x = mylist[r].x;
        const int cc = x == 0xFFFFFFFFu ? -1 : (int)(x & kChunkMask);
        dst[(int64_t)r * p.sel_rs] = cc >= 0 ? slot0 + cc : -1;
        if (cc >= 0 && list_counts != nullptr) {
          if (cnt_in_smem) atomicAdd(&cnt_s[cc], 1);
          else atomicAdd(&list_counts[(int64_t)(slot0 + cc) * p.Hkv + t.hk], 1);
        }
      }
    }
    __syncthreads();                                          // lists, scratch and the Q buffer are free again
    if (cnt_in_smem && list_counts != nullptr)
      for (int cc = tid; cc < t.max_cand; cc += kGateThreads) {        // flush and clear this thread's counters
        const int m = cnt_s[cc];
        if (m > 0) {
          atomicAdd(&list_counts[(int64_t)(slot0 + cc) * p.Hkv + t.hk], m);
          cnt_s[cc] = 0;
        }
      }
    ++n;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, (uint32_t)nt);
}

struct GateLaunch {
  int nt, list_len, nbuf, cnt_in_smem, ctas_per_sm;
  size_t smem;
};

// Candidate tile, Q buffers, list length and shared memory of a launch: the combination that puts
// the most CTAs on an SM (more warps hide the latency of the heap updates), then two Q buffers,
// then the wider candidate tile.  smem == 0: nothing fits.
GateLaunch gate_launch_config(const Params& p) {
  GateLaunch best{};
  const int nblk = (p.D + 63) / 64;
  // hist + 1 places settle the cut; more only help rows with more than 32 candidates (a row with
  // fewer is ranked over all of them in one round of the exact path anyway)
  const int list_len = p.hist + 1 + (p.mc - 1 > 32 ? kListExtra : 0);
  const int cnt_in_smem = p.mc <= kCntSmemMax;
  int want = 32;
  while (want < p.mc - 1 && want < 256) want *= 2;            // a row has at most mc - 1 candidates
  for (int nbuf = 2; nbuf >= 1; --nbuf)
    for (int nt = want; nt >= 32; nt /= 2) {
      const bool has_scratch = list_len > 32 || p.mc - 1 > 32;
      const size_t smem = 1024 + (size_t)nbuf * nblk * kQBlockBytes + (size_t)nblk * nt * 128 +
                          (size_t)kGateRows * (list_len | 1) * sizeof(uint2) +
                          (has_scratch ? (size_t)kGateRows * kScratchStride * sizeof(float) : 0) + sizeof(GateCtrl) +
                          (cnt_in_smem ? (size_t)p.mc * sizeof(int32_t) : 0);
      if (smem > 227 * 1024) continue;
      int ctas = (int)((228 * 1024) / (smem + 1024));         // 1 KB per CTA is reserved by the system
      if (ctas > 512 / nt) ctas = 512 / nt;                   // tensor memory columns
      if (ctas > 4) ctas = 4;
      if (ctas < 1) continue;
      if (ctas > best.ctas_per_sm) best = GateLaunch{nt, list_len, nbuf, cnt_in_smem, ctas, smem};
    }
  return best;
}

}  // namespace

bool make_tile_map(CUtensorMap* m, bool fp16, int D, const __nv_bfloat16* base, int64_t T, int H, int64_t st,
                   int64_t sh, int box_heads, int box_rows);

bool gate_topk_fits(const Params& p) { return p.hist <= 0 || gate_launch_config(p).smem != 0; }

cudaError_t launch_gate_topk_stats(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* means,
                                   const int32_t* cu, int32_t* selected, int32_t* list_counts, int32_t* stats,
                                   int flags, cudaStream_t st) {
  int tokens_per_cta = kGateRows / p.G;
  if (tokens_per_cta < 1) return cudaErrorInvalidConfiguration;
  const GateLaunch g = gate_launch_config(p);
  if (g.smem == 0) return cudaErrorInvalidConfiguration;
  CUtensorMap mq, mm;
  if (!make_tile_map(&mq, p.fp16 != 0, p.D, q, p.Tq, p.Hq, p.sq_t, p.sq_h, p.G, tokens_per_cta) ||
      !make_tile_map(&mm, p.fp16 != 0, p.D, means, p.slots, p.Hkv, (int64_t)p.Hkv * p.D, p.D, 1, g.nt))
    return cudaErrorNotSupported;
  typedef void (*Kernel)(Params, CUtensorMap, CUtensorMap, int, int, int, int, int, const __nv_bfloat16*,
                         const __nv_bfloat16*, const int32_t*, int32_t*, int32_t*, int32_t*, int);
  Kernel kernel = nullptr;
  const int w = g.list_len <= 8 ? 8 : (g.list_len <= 16 ? 16 : (g.list_len <= 32 ? 32 : 0));
#define MOBA_GATE_W(HALF, DIM)                                                                       \
  kernel = w == 8 ? (Kernel)gate_topk_kernel<HALF, DIM, 8> : w == 16 ? (Kernel)gate_topk_kernel<HALF, DIM, 16> \
         : w == 32 ? (Kernel)gate_topk_kernel<HALF, DIM, 32> : (Kernel)gate_topk_kernel<HALF, DIM, 0>
  switch (p.D) {
    case 64:  if (p.fp16) MOBA_GATE_W(true, 64);  else MOBA_GATE_W(false, 64);  break;
    case 96:  if (p.fp16) MOBA_GATE_W(true, 96);  else MOBA_GATE_W(false, 96);  break;
    case 128: if (p.fp16) MOBA_GATE_W(true, 128); else MOBA_GATE_W(false, 128); break;
    case 256: if (p.fp16) MOBA_GATE_W(true, 256); else MOBA_GATE_W(false, 256); break;
    default: return cudaErrorInvalidValue;
  }
#undef MOBA_GATE_W
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t n_tiles = (int64_t)window_tiles(p, tokens_per_cta) * p.Hkv * p.B;
  if (n_tiles >= ((int64_t)1 << 31)) return cudaErrorInvalidConfiguration;
  // persistent CTAs: as many as are resident at once, by shared memory (1 KB per CTA is reserved),
  // registers (allocated in units of 8 per thread) and tensor memory (512 columns per SM)
  cudaFuncAttributes attr;
  if ((e = cudaFuncGetAttributes(&attr, kernel)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100)) != cudaSuccess) return e;
  int smem_per_sm = 0, regs_per_sm = 0;
  cudaDeviceGetAttribute(&smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  cudaDeviceGetAttribute(&regs_per_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev);
  int resident = (int)(smem_per_sm / (g.smem + 1024));
  const int regs_per_cta = ((attr.numRegs + 7) / 8 * 8) * kGateThreads;
  if (regs_per_cta > 0 && resident > regs_per_sm / regs_per_cta) resident = regs_per_sm / regs_per_cta;
  if (resident > 512 / g.nt) resident = 512 / g.nt;
  if (resident < 1) resident = 1;
  int64_t grid = (int64_t)sms * resident;
  if (grid > n_tiles) grid = n_tiles;
  kernel<<<(int)grid, kGateThreads, g.smem, st>>>(p, mq, mm, tokens_per_cta, g.nt, g.list_len, g.nbuf, g.cnt_in_smem, q,
                                                  means, cu, selected, list_counts, stats, flags);
  return cudaGetLastError();
}

cudaError_t launch_gate_topk(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* means,
                             const int32_t* cu, int32_t* selected, int32_t* list_counts,
                             cudaStream_t st) {
  return launch_gate_topk_stats(p, q, means, cu, selected, list_counts, nullptr, 0, st);
}

}  // namespace moba
