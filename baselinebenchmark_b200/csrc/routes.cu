// Compaction of the per-(token, head) selections into per-(chunk slot, kv head)
// query lists, and the LSE-weighted merge of the partial results.
//
// Replaces, for the inference path of the reference,
//   _count_sparse_routes_kernel / _exclusive_prefix_sum_triton /
//   _scatter_sparse_routes_device_kernel / _build_route_block_descriptors_kernel
//                              backends/_mthreads/ops/moba/routing.py:1311-1429, 1561-1718
//   _fused_merge_softmax_kernel                      attention.py:787-889
//
// Differences by design: lists are keyed by (slot, kv head) so the query heads
// of a GQA group share one K/V stream; all ranks are compacted at once (the
// reference loops over rank passes, parallel.py:335); tile descriptors are not
// materialised, the dense stage finds its tile by binary search in a prefix of
// tile counts; the merge sees every partial of a row at once and rounds once.
#include "common.cuh"

namespace moba {

// ---------------------------------------------------------------------------
// exclusive prefix sums over the lists (single CTA, any number of lists)
// ---------------------------------------------------------------------------
constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads)
scan_lists_kernel(int64_t lists, int tile_rows, const int32_t* __restrict__ counts,
                  int32_t* __restrict__ offsets, int32_t* __restrict__ tile_prefix,
                  int32_t* __restrict__ cursors) {
  __shared__ int warp_rows[32], warp_tiles[32];
  __shared__ int carry_rows, carry_tiles;
  if (threadIdx.x == 0) { carry_rows = 0; carry_tiles = 0; }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t base = 0; base < lists; base += kScanThreads) {
    const int64_t l = base + threadIdx.x;
    const int n = l < lists ? counts[l] : 0;
    const int t = (n + tile_rows - 1) / tile_rows;
    int xr = n, xt = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int yr = __shfl_up_sync(0xffffffffu, xr, o);
      const int yt = __shfl_up_sync(0xffffffffu, xt, o);
      if (lane >= o) { xr += yr; xt += yt; }
    }
    if (lane == 31) { warp_rows[warp] = xr; warp_tiles[warp] = xt; }
    __syncthreads();
    if (warp == 0) {
      int wr = warp_rows[lane], wt = warp_tiles[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int yr = __shfl_up_sync(0xffffffffu, wr, o);
        const int yt = __shfl_up_sync(0xffffffffu, wt, o);
        if (lane >= o) { wr += yr; wt += yt; }
      }
      warp_rows[lane] = wr; warp_tiles[lane] = wt;            // inclusive over warps
    }
    __syncthreads();
    const int pre_r = carry_rows + (warp ? warp_rows[warp - 1] : 0) + xr - n;
    const int pre_t = carry_tiles + (warp ? warp_tiles[warp - 1] : 0) + xt - t;
    if (l < lists) { offsets[l] = pre_r; tile_prefix[l] = pre_t; cursors[l] = 0; }
    __syncthreads();
    if (threadIdx.x == 0) { carry_rows += warp_rows[31]; carry_tiles += warp_tiles[31]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { offsets[lists] = carry_rows; tile_prefix[lists] = carry_tiles; }
}

// ---------------------------------------------------------------------------
// scatter: grid (token tiles of one sequence, kv head, sequence), like the
// gating kernel, so a CTA touches the lists of one (sequence, kv head) only and
// can reserve list space with one global atomic per list.
// ---------------------------------------------------------------------------
constexpr int kScatterThreads = 256;
constexpr int kScatterTokens = 64;

__global__ void __launch_bounds__(kScatterThreads)
scatter_routes_kernel(Params p, const int32_t* __restrict__ cu, const int32_t* __restrict__ selected,
                      const int32_t* __restrict__ offsets, int32_t* __restrict__ cursors,
                      int32_t* __restrict__ row_list, float* __restrict__ partial_lse) {
  extern __shared__ int32_t sm[];
  int32_t* cnt_s = sm;               // [mc] rows of this CTA per list, then running index
  int32_t* base_s = sm + p.mc;       // [mc] first position reserved for this CTA
  const int b = blockIdx.z, hk = blockIdx.y;
  const int s0 = cu[b], s1 = cu[b + 1];
  const int tok_lo = max(s0 + blockIdx.x * kScatterTokens, p.win_lo);
  const int tok_hi = min(min(s0 + (blockIdx.x + 1) * kScatterTokens, s1), p.win_lo + (int)p.Tq);
  if (tok_lo >= tok_hi) return;
  const int ntok = tok_hi - tok_lo;
  const int loc = tok_lo - p.win_lo;             // window-relative token of the first row
  const int slot0 = b * p.mc;
  const int n = p.hist * p.G * ntok;             // entries (rank, head, token), token fastest
  for (int i = threadIdx.x; i < p.mc; i += kScatterThreads) cnt_s[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += kScatterThreads) {
    const int tl = i % ntok, rh = i / ntok;
    const int hl = rh % p.G, r = rh / p.G;
    const int slot = selected[(int64_t)r * p.sel_rs + (int64_t)(hk * p.G + hl) * p.Tq + loc + tl];
    if (slot >= 0) atomicAdd(&cnt_s[slot - slot0], 1);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < p.mc; c += kScatterThreads) {
    const int m = cnt_s[c];
    base_s[c] = m > 0 ? atomicAdd(&cursors[(int64_t)(slot0 + c) * p.Hkv + hk], m) : 0;
    cnt_s[c] = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += kScatterThreads) {
    const int tl = i % ntok, rh = i / ntok;
    const int hl = rh % p.G, r = rh / p.G;
    const int head = hk * p.G + hl;
    const int slot = selected[(int64_t)r * p.sel_rs + (int64_t)head * p.Tq + loc + tl];
    const int64_t entry = ((int64_t)(loc + tl) * p.Hq + head) * p.NP + r + 1;
    if (slot >= 0) {
      const int c = slot - slot0;
      const int pos = offsets[(int64_t)slot * p.Hkv + hk] + base_s[c] + atomicAdd(&cnt_s[c], 1);
      row_list[pos] = (int32_t)entry;
    } else {
      partial_lse[entry] = -INFINITY;            // this rank contributes nothing to the merge
    }
  }
}

cudaError_t launch_compact(const Params& p, const int32_t* cu, const int32_t* selected,
                           const int32_t* list_counts, int32_t* list_offsets, int32_t* tile_prefix,
                           int32_t* cursors, int32_t* row_list, float* partial_lse, int tile_rows,
                           cudaStream_t st) {
  scan_lists_kernel<<<1, kScanThreads, 0, st>>>(p.lists, tile_rows, list_counts, list_offsets, tile_prefix, cursors);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const size_t smem = (size_t)p.mc * 2 * sizeof(int32_t);
  if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
  e = cudaFuncSetAttribute(scatter_routes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(cdiv_i(p.max_seqlen, kScatterTokens), p.Hkv, p.B);
  scatter_routes_kernel<<<grid, kScatterThreads, smem, st>>>(p, cu, selected, list_offsets, cursors, row_list, partial_lse);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// merge: one warp per (token, head) row.
//   lse_tot = log sum_j exp(lse_j);  out = sum_j O_j * exp(lse_j - lse_tot)
// ---------------------------------------------------------------------------
constexpr int kMergeThreads = 256;

// A row has D/4 float4 pieces: one per lane for D <= 128 (lanes beyond D/4 idle), two for D = 256.
template <bool kHalf, int D>
__global__ void __launch_bounds__(kMergeThreads)
merge_kernel(Params p, const float* __restrict__ partial_out, const float* __restrict__ partial_lse,
             const int32_t* __restrict__ status, __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out) {
  const int lane = threadIdx.x & 31;
  // a dense stage that gave up on a wait leaves a non-zero status: poison the result
  const bool failed = status != nullptr && *status != 0;
  const int64_t warps = (int64_t)gridDim.x * (kMergeThreads / 32);
  for (int64_t row = (int64_t)blockIdx.x * (kMergeThreads / 32) + (threadIdx.x >> 5); row < p.rows; row += warps) {
    const float* lse = partial_lse + row * p.NP;
    float mx = -INFINITY;
    for (int j = lane; j < p.NP; j += 32) mx = fmaxf(mx, lse[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float tot = 0.f;
    for (int j = lane; j < p.NP; j += 32) tot += expf(lse[j] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float inv = failed ? __int_as_float(0x7fc00000) : 1.f / tot;
    constexpr int nvec = D / 4, kVecs = (nvec + 31) / 32;
    float4 acc[kVecs];
#pragma unroll
    for (int u = 0; u < kVecs; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* src = reinterpret_cast<const float4*>(partial_out + row * p.NP * D) + lane;
    for (int j = 0; j < p.NP; ++j) {
      const float lj = lse[j];                                // same address for all lanes
      if (lj == -INFINITY) continue;
      const float w = expf(lj - mx) * inv;
#pragma unroll
      for (int u = 0; u < kVecs; ++u) {
        if (nvec % 32 == 0 || lane + 32 * u < nvec) {
          const float4 o = __ldg(src + j * nvec + 32 * u);
          acc[u].x += w * o.x; acc[u].y += w * o.y; acc[u].z += w * o.z; acc[u].w += w * o.w;
        }
      }
    }
    const int64_t t = row / p.Hq;
    const int h = (int)(row - t * p.Hq);
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
      if (nvec % 32 == 0 || lane + 32 * u < nvec) {
        uint2 pk;
        pk.x = pack2_16<kHalf>(acc[u].x, acc[u].y);
        pk.y = pack2_16<kHalf>(acc[u].z, acc[u].w);
        *reinterpret_cast<uint2*>(out + t * p.so_t + (int64_t)h * p.so_h + (lane + 32 * u) * 4) = pk;
      }
    }
    if (lse_out != nullptr && lane == 0) lse_out[(int64_t)h * p.Tq + t] = logf(tot) + mx;
  }
}

cudaError_t launch_merge(const Params& p, const float* partial_out, const float* partial_lse,
                         const int32_t* status, __nv_bfloat16* out, float* lse_out, cudaStream_t st) {
  int64_t blocks = (p.rows + (kMergeThreads / 32) - 1) / (kMergeThreads / 32);
  if (blocks > 148 * 64) blocks = 148 * 64;
#define MOBA_MERGE(HALF, DIM) \
  merge_kernel<HALF, DIM><<<(int)blocks, kMergeThreads, 0, st>>>(p, partial_out, partial_lse, status, out, lse_out)
  switch (p.D) {
    case 64:  if (p.fp16) MOBA_MERGE(true, 64);  else MOBA_MERGE(false, 64);  break;
    case 96:  if (p.fp16) MOBA_MERGE(true, 96);  else MOBA_MERGE(false, 96);  break;
    case 128: if (p.fp16) MOBA_MERGE(true, 128); else MOBA_MERGE(false, 128); break;
    case 256: if (p.fp16) MOBA_MERGE(true, 256); else MOBA_MERGE(false, 256); break;
    default: return cudaErrorInvalidValue;
  }
#undef MOBA_MERGE
  return cudaGetLastError();
}

}  // namespace moba
