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
                      int32_t* __restrict__ row_list, float2* __restrict__ partial_lse) {
  extern __shared__ int32_t sm[];
  int32_t* cnt_s = sm;               // [mc] rows of this CTA per list, then running index
  int32_t* base_s = sm + p.mc;       // [mc] first position reserved for this CTA
  const int b = blockIdx.z, hk = blockIdx.y;
  const int s0 = cu[b], s1 = cu[b + 1];
  const int x = blockIdx.x + window_tile0(p, s0, kScatterTokens);
  const int tok_lo = max(s0 + x * kScatterTokens, p.win_lo);
  const int tok_hi = min(min(s0 + (x + 1) * kScatterTokens, s1), p.win_lo + (int)p.Tq);
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
      partial_lse[entry] = make_float2(-INFINITY, 0.f);   // this rank contributes nothing to the merge
    }
  }
}

cudaError_t launch_compact(const Params& p, const int32_t* cu, const int32_t* selected,
                           const int32_t* list_counts, int32_t* list_offsets, int32_t* tile_prefix,
                           int32_t* cursors, int32_t* row_list, float2* partial_lse, int tile_rows,
                           cudaStream_t st) {
  scan_lists_kernel<<<1, kScanThreads, 0, st>>>(p.lists, tile_rows, list_counts, list_offsets, tile_prefix, cursors);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const size_t smem = (size_t)p.mc * 2 * sizeof(int32_t);
  if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
  e = cudaFuncSetAttribute(scatter_routes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(window_tiles(p, kScatterTokens), p.Hkv, p.B);
  scatter_routes_kernel<<<grid, kScatterThreads, smem, st>>>(p, cu, selected, list_offsets, cursors, row_list, partial_lse);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// merge: one warp per (token, head) row.
//   lse_tot = log sum_j exp(lse_j);  out = sum_j O_j * exp(lse_j - lse_tot)
// (exponentials through ex2.approx: relative error 2^-22, far below the rounding of the output)
// ---------------------------------------------------------------------------
constexpr int kMergeThreads = 256;

// A partial row is D/8 pieces of eight fp16 values (16 bytes), one per lane: 32 / (D/8) rows fit
// one load instruction of the warp (2 at head dim 128 and 96, 4 at 64, 1 at 256), so the lanes form
// that many groups, group g takes the partials g, g + groups, ... of the row, four of them in
// flight at a time, and the groups' sums are added at the end.
template <bool kHalf, int D>
// five CTAs per SM (at most 51 registers): more warps to wait for partial rows; six would spill
__global__ void __launch_bounds__(kMergeThreads, 5)
merge_kernel(Params p, const __half* __restrict__ partial_out, const float2* __restrict__ partial_lse,
             const int32_t* __restrict__ status, __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out) {
  constexpr int kLanes = D / 8;                  // lanes per partial row
  constexpr int kGroups = 32 / kLanes;
  constexpr int kAhead = 4;                      // partial rows a group has in flight
  const int lane = threadIdx.x & 31;
  const int grp = lane / kLanes, piece = lane - grp * kLanes;
  const bool active = grp < kGroups;             // head dim 96: lanes 24-31 idle
  // a dense stage that gave up on a wait leaves a non-zero status: poison the result
  const bool failed = status != nullptr && *status != 0;
  const int64_t warps = (int64_t)gridDim.x * (kMergeThreads / 32);
  // Up to 32 partials per row (top-k up to 32): lane j holds {lse, 1 / scale} of partial j, and the
  // pair of the warp's next row is requested before this row is worked on, so that a row starts
  // with its partial rows as the only loads it has to wait for.
  const bool in_regs = p.NP <= 32;
  const int64_t row0 = (int64_t)blockIdx.x * (kMergeThreads / 32) + (threadIdx.x >> 5);
  float2 mine = make_float2(-INFINITY, 0.f);
  if (in_regs && row0 < p.rows && lane < p.NP) mine = __ldg(partial_lse + row0 * p.NP + lane);
  for (int64_t row = row0; row < p.rows; row += warps) {
    const float2* lse = partial_lse + row * p.NP;
    const float2 cur = mine;
    if (in_regs && row + warps < p.rows && lane < p.NP) mine = __ldg(partial_lse + (row + warps) * p.NP + lane);
    float mx = -INFINITY;
    if (in_regs) mx = cur.x;
    else for (int j = lane; j < p.NP; j += 32) mx = fmaxf(mx, lse[j].x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float tot = 0.f;
    if (in_regs) tot = __expf(cur.x - mx);                    // 0 for lanes past the partials (lse -inf)
    else for (int j = lane; j < p.NP; j += 32) tot += __expf(lse[j].x - mx);
    const float wlane = tot * cur.y;                          // in_regs: weight of partial `lane` up to 1 / sum
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float inv = failed ? __int_as_float(0x7fc00000) : 1.f / tot;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    const uint4* src = reinterpret_cast<const uint4*>(partial_out + row * p.NP * D) + piece;
    for (int j0 = 0; j0 < p.NP; j0 += kGroups * kAhead) {
      float w[kAhead];
      uint4 o[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int j = j0 + u * kGroups + grp;
        w[u] = 0.f;
        o[u] = make_uint4(0u, 0u, 0u, 0u);
        // the row's power-of-two scale is undone with the weight
        const float wj = __shfl_sync(0xffffffffu, wlane, j & 31) * inv;
        if (in_regs) {
          if (active && j < p.NP && wj != 0.f) {
            w[u] = wj;
            o[u] = __ldg(src + j * kLanes);
          }
        } else if (active && j < p.NP) {
          const float2 lj = lse[j];
          if (lj.x != -INFINITY) {
            w[u] = __expf(lj.x - mx) * inv * lj.y;
            o[u] = __ldg(src + j * kLanes);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const uint32_t words[4] = {o[u].x, o[u].y, o[u].z, o[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&words[i]));
          acc[2 * i] += w[u] * a.x;
          acc[2 * i + 1] += w[u] * a.y;
        }
      }
    }
    // sum of the groups into group 0
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (kGroups == 4) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], 2 * kLanes);
      if (kGroups >= 2) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], kLanes);
    }
    const int64_t t = row / p.Hq;
    const int h = (int)(row - t * p.Hq);
    if (grp == 0) {
      uint4 pk;
      pk.x = pack2_16<kHalf>(acc[0], acc[1]);
      pk.y = pack2_16<kHalf>(acc[2], acc[3]);
      pk.z = pack2_16<kHalf>(acc[4], acc[5]);
      pk.w = pack2_16<kHalf>(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + t * p.so_t + (int64_t)h * p.so_h + piece * 8) = pk;
    }
    if (lse_out != nullptr && lane == 0) lse_out[(int64_t)h * p.Tq + t] = logf(tot) + mx;
  }
}

cudaError_t launch_merge(const Params& p, const __half* partial_out, const float2* partial_lse,
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
