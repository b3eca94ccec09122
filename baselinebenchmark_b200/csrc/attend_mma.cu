// Dense stage of MoBA on the legacy tensor path (mma.sync m16n8k16, bf16 in,
// fp32 accumulate).  Same work items, inputs and outputs as the tcgen05 kernel;
// kept as an independently written cross-check of it.
//
// Replaces, for the inference path of the reference,
//   _varlen_attn_fwd_kernel        backends/_mthreads/ops/moba/attention.py:53-160  (own chunk, causal)
//   _routed_gqa_attn_fwd_kernel    attention.py:610-707                           (selected chunks)
// Numerics follow attention.py:116-155: scores * (D^-0.5 * log2 e) in fp32,
// running row maximum, P rounded to bf16 before P.V, fp32 accumulators,
// natural-log LSE.
//
// A CTA of 8 warps owns a tile of 128 query rows (16 per warp) and walks the
// keys of its item in tiles of 64; K/V tiles are double buffered with cp.async
// into XOR-swizzled shared memory.  CTAs are persistent and draw items from a
// global counter (routed items first, then own-chunk tiles, longest first).
#include "common.cuh"

namespace moba {

namespace {

constexpr int kRows = kMmaTileRows;   // 128
constexpr int kBN = 64;
constexpr int kThreads = 256;
// Bytes of one tile row in shared memory: the head dim rounded up to 64, 128 or 256 elements.
__host__ __device__ constexpr int row_bytes(int d) { return d <= 64 ? 128 : (d <= 128 ? 256 : 512); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
// byte offset of 16-byte chunk `ch` of row `r` in a [rows][D] tile of 16-bit elements
template <int D>
__device__ __forceinline__ uint32_t swz(int r, int ch) {
  return (uint32_t)(r * row_bytes(D) + (((ch & ~7) | ((ch ^ r) & 7)) << 4));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
template <bool kHalf>
__device__ __forceinline__ void mma_16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (kHalf)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int D>
struct Smem {
  unsigned char q[kRows * row_bytes(D)];
  unsigned char k[2][kBN * row_bytes(D)];
  unsigned char v[2][kBN * row_bytes(D)];
  int64_t qoff[kRows];
  int32_t entry[kRows];
  int32_t item;
};

template <int D>
__device__ __forceinline__ void load_kv_tile(const Params& p, const Item& it, int tile, Smem<D>& s, int buf,
                                             const __nv_bfloat16* __restrict__ k,
                                             const __nv_bfloat16* __restrict__ v) {
  const uint32_t kb = smem_u32(s.k[buf]), vb = smem_u32(s.v[buf]);
  constexpr int kChunks = D / 8;
  for (int i = threadIdx.x; i < kBN * kChunks; i += kThreads) {
    const int r = i / kChunks, ch = i - r * kChunks;
    const int key = tile * kBN + r;
    const bool ok = key < it.kv_len;
    const int64_t tok = (int64_t)it.kv_tok0 + (ok ? key : 0);
    cp_async16(kb + swz<D>(r, ch), k + tok * p.sk_t + (int64_t)it.kv_head * p.sk_h + ch * 8, ok);
    cp_async16(vb + swz<D>(r, ch), v + tok * p.sv_t + (int64_t)it.kv_head * p.sv_h + ch * 8, ok);
  }
}

template <bool kHalf, int D>
__global__ void __launch_bounds__(kThreads, D > 128 ? 1 : 2)
attend_mma_kernel(Params p, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                  const __nv_bfloat16* __restrict__ v, const int32_t* __restrict__ cu,
                  const int32_t* __restrict__ list_counts, const int32_t* __restrict__ list_offsets,
                  const int32_t* __restrict__ tile_prefix, const int32_t* __restrict__ row_list,
                  __half* __restrict__ partial_out, float2* __restrict__ partial_lse,
                  int32_t* __restrict__ work_counter) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  Smem<D>& s = *reinterpret_cast<Smem<D>*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_routed = p.hist > 0 ? tile_prefix[p.lists] : 0;
  const SlotRange own = own_slot_range(p, cu);
  const int n_items = n_routed + own_item_count(own.n, p.Hq, p.C, kRows);
  const float sl2 = rsqrtf((float)D) * 1.4426950408889634f;
  constexpr int kChunks = D / 8;

  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) s.item = atomicAdd(work_counter, 1);
    __syncthreads();
    const int idx = s.item;
    if (idx >= n_items) break;
    const Item it = decode_item(p, idx, n_routed, kRows, cu, list_counts, list_offsets, tile_prefix, -1, own);
    if (!it.valid) continue;

    for (int r = threadIdx.x; r < kRows; r += kThreads) {
      int32_t e = -1;
      int64_t off = 0;
      if (r < it.nrows && !(it.causal && r < it.row_start)) {   // own chunk: rows before the query window stay absent
        if (it.causal) {
          const int64_t tl = it.tok0 - p.win_lo + r;          // window-relative token
          e = (int32_t)((tl * p.Hq + it.head) * p.NP);
          off = tl * p.sq_t + (int64_t)it.head * p.sq_h;
        } else {
          e = row_list[it.row_start + r];
          const int64_t row = e / p.NP;
          const int64_t t = row / p.Hq;
          off = t * p.sq_t + (row - t * p.Hq) * p.sq_h;
        }
      }
      s.entry[r] = e;
      s.qoff[r] = off;
    }
    __syncthreads();
    {
      const uint32_t qb = smem_u32(s.q);
      for (int i = threadIdx.x; i < kRows * kChunks; i += kThreads) {
        const int r = i / kChunks, ch = i - r * kChunks;
        cp_async16(qb + swz<D>(r, ch), q + s.qoff[r] + ch * 8, s.entry[r] >= 0);
      }
    }
    const int ntiles = (it.kv_len + kBN - 1) / kBN;
    load_kv_tile<D>(p, it, 0, s, 0, k, v);
    cp_async_commit();

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int row0 = warp * 16 + (lane >> 2);          // this thread's rows: row0 and row0 + 8
    const int qpos0 = it.tok0 + row0, qpos1 = qpos0 + 8;

    for (int j = 0; j < ntiles; ++j) {
      if (j + 1 < ntiles) load_kv_tile<D>(p, it, j + 1, s, (j + 1) & 1, k, v);
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      const uint32_t qb = smem_u32(s.q);
      const int qr = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const uint32_t kb = smem_u32(s.k[j & 1]), vb = smem_u32(s.v[j & 1]);
      float sc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t qa[4];
        ldsm_x4(qb + swz<D>(qr, 2 * ks + (lane >> 4)), qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
          ldsm_x4(kb + swz<D>(r, 2 * ks + ((lane >> 3) & 1)), b0, b1, b2, b3);
          mma_16<kHalf>(sc[2 * np], qa, b0, b1);
          mma_16<kHalf>(sc[2 * np + 1], qa, b2, b3);
        }
      }
      // scale, mask, row maxima
      const int key_base = j * kBN + 2 * (lane & 3);
      const bool need_mask = (j + 1) * kBN > it.kv_len || (it.causal && it.kv_tok0 + (j + 1) * kBN - 1 > it.tok0);
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = sc[nt][e] * sl2;
          if (need_mask) {
            const int key = key_base + nt * 8 + (e & 1);
            const int qpos = (e & 2) ? qpos1 : qpos0;
            const bool ok = key < it.kv_len && (!it.causal || it.kv_tok0 + key <= qpos);
            x = ok ? x : -INFINITY;
          }
          sc[nt][e] = x;
        }
        mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // the first key of an item is visible to every row, so mn* is finite from tile 0 on
      const float a0 = exp2f(m0 - mn0), a1 = exp2f(m1 - mn1);
      m0 = mn0; m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
      uint32_t pa[4][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float p0 = exp2f(sc[nt][0] - mn0), p1 = exp2f(sc[nt][1] - mn0);
        const float p2 = exp2f(sc[nt][2] - mn1), p3 = exp2f(sc[nt][3] - mn1);
        ps0 += p0 + p1;
        ps1 += p2 + p3;
        pa[nt >> 1][(nt & 1) * 2 + 0] = pack2_16<kHalf>(p0, p1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack2_16<kHalf>(p2, p3);
      }
      l0 = l0 * a0 + ps0;
      l1 = l1 * a1 + ps1;
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt) { o[dt][0] *= a0; o[dt][1] *= a0; o[dt][2] *= a1; o[dt][3] *= a1; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
          uint32_t b0, b1, b2, b3;
          const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldsm_x4_t(vb + swz<D>(r, 2 * dp + (lane >> 4)), b0, b1, b2, b3);
          mma_16<kHalf>(o[2 * dp], pa[kk], b0, b1);
          mma_16<kHalf>(o[2 * dp + 1], pa[kk], b2, b3);
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();
    // epilogue: normalise, write the partial rows (fp16, scaled by a power of two per row)
    // and {natural-log LSE, 1 / scale}; a row lives in the four lanes of a quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int e0 = s.entry[row0], e1 = s.entry[row0 + 8];
    const float i0 = 1.f / l0, i1 = 1.f / l1;
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      a0 = fmaxf(a0, fmaxf(fabsf(o[dt][0]), fabsf(o[dt][1])));
      a1 = fmaxf(a1, fmaxf(fabsf(o[dt][2]), fabsf(o[dt][3])));
    }
    a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, 1));
    a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, 2));
    a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, 1));
    a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, 2));
    const PartialScale ps0 = partial_scale(a0 * i0), ps1 = partial_scale(a1 * i1);
    const float f0 = i0 * ps0.scale, f1 = i1 * ps1.scale;
    if (e0 >= 0) {
      __half* dst = partial_out + (int64_t)e0 * D + 2 * (lane & 3);
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<uint32_t*>(dst + dt * 8) = pack2_half(o[dt][0] * f0, o[dt][1] * f0);
      if ((lane & 3) == 0) partial_lse[e0] = make_float2((m0 + log2f(l0)) * 0.6931471805599453f, ps0.inv);
    }
    if (e1 >= 0) {
      __half* dst = partial_out + (int64_t)e1 * D + 2 * (lane & 3);
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<uint32_t*>(dst + dt * 8) = pack2_half(o[dt][2] * f1, o[dt][3] * f1);
      if ((lane & 3) == 0) partial_lse[e1] = make_float2((m1 + log2f(l1)) * 0.6931471805599453f, ps1.inv);
    }
  }
}

}  // namespace

cudaError_t launch_attend_mma(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                              const __nv_bfloat16* v, const int32_t* cu, const int32_t* list_counts,
                              const int32_t* list_offsets, const int32_t* tile_prefix,
                              const int32_t* row_list, __half* partial_out, float2* partial_lse,
                              int32_t* work_counter, cudaStream_t st) {
  void (*kernel)(Params, const __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*, const int32_t*,
                 const int32_t*, const int32_t*, const int32_t*, const int32_t*, __half*, float2*, int32_t*);
  size_t smem;
  switch (p.D) {
    case 64:  kernel = p.fp16 ? attend_mma_kernel<true, 64>  : attend_mma_kernel<false, 64>;  smem = sizeof(Smem<64>);  break;
    case 96:  kernel = p.fp16 ? attend_mma_kernel<true, 96>  : attend_mma_kernel<false, 96>;  smem = sizeof(Smem<96>);  break;
    case 128: kernel = p.fp16 ? attend_mma_kernel<true, 128> : attend_mma_kernel<false, 128>; smem = sizeof(Smem<128>); break;
    case 256: kernel = p.fp16 ? attend_mma_kernel<true, 256> : attend_mma_kernel<false, 256>; smem = sizeof(Smem<256>); break;
    default: return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  kernel<<<sms * (p.D > 128 ? 1 : 2), kThreads, smem, st>>>(p, q, k, v, cu, list_counts, list_offsets, tile_prefix,
                                                    row_list, partial_out, partial_lse, work_counter);
  return cudaGetLastError();
}

}  // namespace moba
