// Gating stage of MoBA: chunk slot tables, mean-pooled keys, q.mean scores with
// the causal chunk mask and a per-(token, head) top-k.
//
// Replaces, for the inference path of the reference,
//   _dense_chunk_metadata_kernel            backends/_mthreads/ops/moba/routing.py:553-592
//   _dense_chunk_mean_kernel                routing.py:690-737
//   _chunk_topk_batched_streaming_kernel    routing.py:1056-1182
//
// The stage is bound by HBM traffic (K and Q are read once); the arithmetic
// runs on CUDA cores in one fixed fp32 summation order so that the selection
// is reproducible bit for bit by a CPU restatement:
//   mean : row r of a chunk is added to accumulator r % 32 in increasing r, the
//          32 accumulators are added in increasing index, the total is divided
//          by C and rounded to bf16 (round to nearest even);
//   score: products of two 16-bit values are exact in fp32; each block of 8
//          dims is added left to right, then a halving tree combines the D/8
//          block sums (for D = 128: block l + block l+8, then l + l+4, l + l+2,
//          l + l+1); a block count that is no power of two (D = 96) is padded
//          with blocks of +0.0 to the next one.
#include "common.cuh"

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
chunk_mean_kernel(Params p, const __nv_bfloat16* __restrict__ k, const int32_t* __restrict__ cu,
                  __nv_bfloat16* __restrict__ means) {
  const int slot = blockIdx.x, hk = blockIdx.y;
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

cudaError_t launch_chunk_means(const Params& p, const __nv_bfloat16* k, const int32_t* cu,
                               __nv_bfloat16* means, cudaStream_t st) {
  dim3 grid(p.slots, p.Hkv);
#define MOBA_MEANS(HALF, DIM) chunk_mean_kernel<HALF, DIM><<<grid, kMeanLanes * (DIM / 8), 0, st>>>(p, k, cu, means)
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

// ---------------------------------------------------------------------------
// scores + mask + top-k
//   grid (token tiles of one sequence, kv head, sequence); 256 threads = 64 row
//   groups of 4 lanes.  The CTA stages the means of its kv head for a tile of
//   candidate chunks in shared memory as fp32; every row group then scores its
//   rows against them and keeps the `hist` largest packed keys
//   (order-preserving score bits << 32 | 0xFFFFFFFF - slot, routing.py:1151-1153)
//   in an ordered list: the keys of a candidate tile are held in registers,
//   extracted largest first and merged with the list.  Keys are unique, so ties
//   in the score fall to the lower slot.
//   Lane t of a group owns the 8-dim blocks t, t+4, t+8, ..., so all levels of
//   the halving tree but the last two stay inside the lane and only those two
//   cross lanes: same summation order as one lane per block, a fraction of the
//   shuffles.
// ---------------------------------------------------------------------------
constexpr int kGateThreads = 256;
constexpr int kGateGroups = kGateThreads / 4;
constexpr int kGateRows = 128;            // (token, head) rows per CTA
constexpr int kCandTile = 32;             // candidate chunks staged per pass

__device__ __forceinline__ uint32_t float_key(float x) {      // routing.py:778-784
  const uint32_t b = __float_as_uint(x);
  return b ^ ((b & 0x80000000u) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float dot8(const float (&q)[8], const float4 a, const float4 b) {
  float s = q[0] * a.x;
  s = __fmaf_rn(q[1], a.y, s);
  s = __fmaf_rn(q[2], a.z, s);
  s = __fmaf_rn(q[3], a.w, s);
  s = __fmaf_rn(q[4], b.x, s);
  s = __fmaf_rn(q[5], b.y, s);
  s = __fmaf_rn(q[6], b.z, s);
  s = __fmaf_rn(q[7], b.w, s);
  return s;
}

#ifndef MOBA_GATE_CTAS
#define MOBA_GATE_CTAS 3             // resident CTAs per SM the register budget is set for (D <= 128)
#endif
template <bool kHalf, int D>
__global__ void __launch_bounds__(kGateThreads, D > 128 ? 2 : MOBA_GATE_CTAS)
gate_topk_kernel(Params p, int tokens_per_cta, const __nv_bfloat16* __restrict__ q,
                 const __nv_bfloat16* __restrict__ means, const int32_t* __restrict__ cu,
                 int32_t* __restrict__ selected, int32_t* __restrict__ list_counts) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int hist = p.hist;
  constexpr int kBlocks = D / 8;                       // 8-dim blocks per row
  constexpr int kOwn = (kBlocks + 3) / 4;              // blocks owned by a lane: t, t+4, ...
  constexpr int kOwnPad = kOwn <= 2 ? 2 : (kOwn <= 4 ? 4 : 8);   // padded to a power of two with +0.0
  // layout: means tile fp32 | scratch[groups][2 * hist] | best[rows][hist] | counts[mc]
  float4* means_s = reinterpret_cast<float4*>(smem_raw);                            // kCandTile * D/4 float4
  unsigned long long* wins_s = reinterpret_cast<unsigned long long*>(means_s + kCandTile * (D / 4));
  unsigned long long* best_s = wins_s + kGateGroups * 2 * hist;
  int32_t* cnt_s = reinterpret_cast<int32_t*>(best_s + (size_t)kGateRows * hist);

  const int b = blockIdx.z, hk = blockIdx.y;
  const int s0 = cu[b], s1 = cu[b + 1];
  // tokens of this CTA, clipped to the sequence and to the query window
  const int tok_lo = max(s0 + blockIdx.x * tokens_per_cta, p.win_lo);
  const int tok_hi = min(min(s0 + (blockIdx.x + 1) * tokens_per_cta, s1), p.win_lo + (int)p.Tq);
  if (tok_lo >= tok_hi) return;
  const int ntok = tok_hi - tok_lo;
  const int nrows = ntok * p.G;
  const int grp = threadIdx.x >> 2, t = threadIdx.x & 3;
  const unsigned gmask = 0xFu << (threadIdx.x & 28);          // the 4 lanes of this group

  for (int i = threadIdx.x; i < p.mc; i += kGateThreads) cnt_s[i] = 0;
  for (int i = threadIdx.x; i < kGateRows * hist; i += kGateThreads) best_s[i] = 0ull;
  // candidates of the last token of the tile bound the chunks to stage
  const int max_cand = (tok_lo + ntok - 1 - s0) / p.C;
  const int slot0 = b * p.mc;

  for (int c0 = 0; c0 < max_cand; c0 += kCandTile) {
    const int ct = min(kCandTile, max_cand - c0);
    __syncthreads();                                          // previous tile fully consumed
    for (int i = threadIdx.x; i < ct * kBlocks; i += kGateThreads) {
      const int c = i / kBlocks, part = i - c * kBlocks;
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(
          means + ((int64_t)(slot0 + c0 + c) * p.Hkv + hk) * D + part * 8));
      float f[8];
      unpack8<kHalf>(x, f);
      means_s[c * (D / 4) + part * 2] = make_float4(f[0], f[1], f[2], f[3]);
      means_s[c * (D / 4) + part * 2 + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncthreads();
    for (int row = grp; row < nrows; row += kGateGroups) {    // row = token-major, head-minor
      const int tl = row / p.G, hl = row - tl * p.G;
      const int tok = tok_lo + tl;
      const int cend = min(ct, (tok - s0) / p.C - c0);        // this row's candidates in the tile
      if (cend <= 0) continue;                                // uniform over the 4 lanes
      float qf[kOwn][8];
      {
        const __nv_bfloat16* qrow = q + (int64_t)(tok - p.win_lo) * p.sq_t + (int64_t)(hk * p.G + hl) * p.sq_h;
#pragma unroll
        for (int k = 0; k < kOwn; ++k)
          unpack8<kHalf>(__ldg(reinterpret_cast<const uint4*>(qrow + (t + 4 * k) * 8)), qf[k]);
      }
      // packed key of candidate c of this tile; the same value in the 4 lanes
      auto score_key = [&](int c) -> unsigned long long {
        const float4* m = means_s + c * (D / 4);
        float acc[kOwnPad];
#pragma unroll
        for (int k = 0; k < kOwnPad; ++k)
          acc[k] = k < kOwn ? dot8(qf[k < kOwn ? k : 0], m[(t + 4 * k) * 2], m[(t + 4 * k) * 2 + 1]) : 0.f;
        // halving tree over the block sums: every level but the last two pairs blocks of
        // the same lane (block l with block l + half), the last two cross lanes
#pragma unroll
        for (int h = kOwnPad / 2; h >= 1; h >>= 1)
#pragma unroll
          for (int k = 0; k < h; ++k) acc[k] = __fadd_rn(acc[k], acc[k + h]);
        float s = acc[0];
        s = __fadd_rn(s, __shfl_xor_sync(gmask, s, 2));
        s = __fadd_rn(s, __shfl_xor_sync(gmask, s, 1));
        return ((unsigned long long)float_key(s) << 32) |
               (unsigned long long)(0xFFFFFFFFu - (uint32_t)(slot0 + c0 + c));
      };
      // The row's list best[0..hist) is kept ordered, largest key first, 0 = empty place.
      // Lane t keeps the keys of candidates c = 4e + t of this tile in registers (only those
      // that beat the smallest key of a full list) and the group extracts them largest first:
      // no shared-memory round trip per candidate.  First tile: straight into the list.
      // Later tiles: into a scratch list that is then merged with the old one.
      unsigned long long* best = best_s + (size_t)row * hist;
      unsigned long long* fresh = wins_s + (size_t)grp * 2 * hist;       // [hist] new keys, [hist] merge output
      const unsigned long long tau = c0 > 0 ? best[hist - 1] : 0ull;
      unsigned long long mine[kCandTile / 4];
#pragma unroll
      for (int e = 0; e < kCandTile / 4; ++e) {
        mine[e] = 0ull;
        if (4 * e < cend) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int c = 4 * e + cc;
            const unsigned long long key = score_key(c < cend ? c : 0);
            if (cc == t && c < cend && key > tau) mine[e] = key;
          }
        }
      }
      unsigned long long* dst = c0 > 0 ? fresh : best;
      int n_new = 0;
      for (; n_new < hist; ++n_new) {
        unsigned long long top = 0ull;
        int top_e = 0;
#pragma unroll
        for (int e = 0; e < kCandTile / 4; ++e)
          if (mine[e] > top) { top = mine[e]; top_e = e; }
        unsigned long long all = top;
#pragma unroll
        for (int o = 2; o > 0; o >>= 1) {
          const unsigned long long other = __shfl_xor_sync(gmask, all, o);
          all = other > all ? other : all;
        }
        if (all == 0ull) break;                               // nothing left
        if (top == all) {                                     // keys are unique: exactly one owner
#pragma unroll
          for (int e = 0; e < kCandTile / 4; ++e)
            if (e == top_e) mine[e] = 0ull;
          dst[n_new] = all;
        }
      }
      if (c0 > 0 && n_new > 0) {
        // merge the two ordered lists (every lane follows the same steps, lane 0 writes)
        __syncwarp(gmask);
        unsigned long long a = best[0], b = fresh[0];
        int ia = 0, ib = 0;
        for (int o = 0; o < hist; ++o) {
          const bool take = b > a;
          if (t == 0) fresh[hist + o] = take ? b : a;
          if (take) { ++ib; b = ib < n_new ? fresh[ib] : 0ull; }
          else      { ++ia; a = ia < hist ? best[ia] : 0ull; }
        }
        __syncwarp(gmask);
        for (int i = t; i < hist; i += 4) best[i] = fresh[hist + i];
        __syncwarp(gmask);
      }
    }
  }
  __syncthreads();
  // selected[r][head][tok]: `ntok` consecutive ints per (rank, head)
  for (int i = threadIdx.x; i < hist * nrows; i += kGateThreads) {
    const int r = i / nrows, rem = i - r * nrows;
    const int hl = rem / ntok, tl = rem - hl * ntok;
    const unsigned long long w = best_s[(size_t)(tl * p.G + hl) * hist + r];
    const int slot = w ? (int)(0xFFFFFFFFu - (uint32_t)(w & 0xFFFFFFFFull)) : -1;
    selected[(int64_t)r * p.sel_rs + (int64_t)(hk * p.G + hl) * p.Tq + (tok_lo - p.win_lo) + tl] = slot;
    if (slot >= 0) atomicAdd(&cnt_s[slot - slot0], 1);
  }
  __syncthreads();
  if (list_counts != nullptr)
    for (int c = threadIdx.x; c < p.mc; c += kGateThreads)
      if (cnt_s[c] > 0) atomicAdd(&list_counts[(int64_t)(slot0 + c) * p.Hkv + hk], cnt_s[c]);
}

static size_t gate_smem_bytes(const Params& p) {
  return (size_t)kCandTile * (p.D / 4) * sizeof(float4) + (size_t)kGateGroups * 2 * p.hist * 8 +
         (size_t)kGateRows * p.hist * 8 + (size_t)p.mc * 4;
}

cudaError_t launch_gate_topk(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* means,
                             const int32_t* cu, int32_t* selected, int32_t* list_counts,
                             cudaStream_t st) {
  int tokens_per_cta = kGateRows / p.G;
  if (tokens_per_cta < 1) tokens_per_cta = 1;
  const size_t smem = gate_smem_bytes(p);
  if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
  void (*kernel)(Params, int, const __nv_bfloat16*, const __nv_bfloat16*, const int32_t*, int32_t*, int32_t*);
  switch (p.D) {
    case 64:  kernel = p.fp16 ? gate_topk_kernel<true, 64>  : gate_topk_kernel<false, 64>;  break;
    case 96:  kernel = p.fp16 ? gate_topk_kernel<true, 96>  : gate_topk_kernel<false, 96>;  break;
    case 128: kernel = p.fp16 ? gate_topk_kernel<true, 128> : gate_topk_kernel<false, 128>; break;
    case 256: kernel = p.fp16 ? gate_topk_kernel<true, 256> : gate_topk_kernel<false, 256>; break;
    default: return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(cdiv_i(p.max_seqlen, tokens_per_cta), p.Hkv, p.B);
  kernel<<<grid, kGateThreads, smem, st>>>(p, tokens_per_cta, q, means, cu, selected, list_counts);
  return cudaGetLastError();
}

}  // namespace moba
