// Backward of the MoBA dense stage (training path) on mma.sync m16n8k16.
//
// Replaces, for the training path of the reference,
//   MixedAttention.backward            backends/_mthreads/ops/moba/parallel.py:149-250
//   _triton_varlen_backward            backends/_mthreads/ops/moba/attention.py:163-369 (dq and dk/dv kernels)
//   gather / scatter of routed rows    backends/_mthreads/ops/moba/routing.py:394-463, :1776-1896
// Like the reference, both branches (own chunk, selected chunks) are differentiated with
// the merged LSE and the merged output (parallel.py:171-236): with
//   p_ij = exp(s_ij * scale - lse_i),  delta_i = sum_d dO_id * O_id,
//   dV_j = sum_i p_ij dO_i,  dS_ij = p_ij (dO_i . V_j - delta_i),
//   dQ_i = scale * sum_j dS_ij K_j,  dK_j = scale * sum_i dS_ij Q_i
// over exactly the (query, key) pairs the forward attends; the chunk selection is constant.
//
// Two kernels, neither accumulates with atomics.  dQ is bit-identical run to run; dK and dV
// add the rows of a routed list in list order, which the compaction's atomics leave
// unspecified, so they vary in the last bits:
//   bwd_dq_kernel    row-stationary over the forward's work items (128 rows x one chunk);
//                    each item writes its fp32 dQ contribution into the row's partial slot
//                    (own chunk = 0, rank r = r+1) and sum_dq_kernel adds the slots;
//   bwd_dkdv_kernel  key-stationary: a CTA owns 64 keys of one (chunk, kv head), visits every
//                    row tile that attends them (the routed list of the chunk, then the
//                    chunk's own rows of each query head of the group) and writes dK, dV once.
// P and dS are rounded to the input dtype before they enter an MMA, accumulation is fp32.
#include "common.cuh"

namespace moba {

namespace {

constexpr int kRows = 128;      // rows per tile
constexpr int kBN = 64;         // keys per tile
constexpr int kThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

__host__ __device__ constexpr int row_bytes(int d) { return d <= 64 ? 128 : (d <= 128 ? 256 : 512); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// byte offset of 16-byte chunk `ch` of row `r` in a tile whose rows hold D 16-bit elements
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

// acc[nt] (16 rows x 64 keys of this warp) = X[rows of the warp] . Y[64 keys]^T over D dims;
// X, Y: swizzled tiles in shared memory with rows of D elements.
template <bool kHalf, int D>
__device__ __forceinline__ void rows_times_keys(float (&acc)[8][4], uint32_t xb, uint32_t yb, int warp, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  const int xr = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t xa[4];
    ldsm_x4(xb + swz<D>(xr, 2 * ks + (lane >> 4)), xa[0], xa[1], xa[2], xa[3]);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b0, b1, b2, b3;
      const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
      ldsm_x4(yb + swz<D>(r, 2 * ks + ((lane >> 3) & 1)), b0, b1, b2, b3);
      mma_16<kHalf>(acc[2 * np], xa, b0, b1);
      mma_16<kHalf>(acc[2 * np + 1], xa, b2, b3);
    }
  }
}

// ---------------------------------------------------------------------------
// delta[row] = sum_d dO * O,  lse2[row] = lse * log2(e);  row = t * Hq + h
// ---------------------------------------------------------------------------
template <bool kHalf>
__global__ void __launch_bounds__(256)
delta_kernel(Params p, const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
             int64_t do_t, int64_t do_h, const float* __restrict__ lse, float* __restrict__ delta,
             float* __restrict__ lse2) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < p.rows; row += warps) {
    const int64_t t = row / p.Hq;
    const int h = (int)(row - t * p.Hq);
    const __nv_bfloat16* o = out + t * p.so_t + (int64_t)h * p.so_h;
    const __nv_bfloat16* g = dout + t * do_t + (int64_t)h * do_h;
    float s = 0.f;
    for (int c = lane; c < p.D / 8; c += 32) {
      float a[8], b[8];
      unpack8<kHalf>(__ldg(reinterpret_cast<const uint4*>(o + c * 8)), a);
      unpack8<kHalf>(__ldg(reinterpret_cast<const uint4*>(g + c * 8)), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) s = fmaf(a[i], b[i], s);
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
    if (lane == 0) {
      delta[row] = s;
      lse2[row] = lse[(int64_t)h * p.Tq + t] * kLog2e;
    }
  }
}

// list_counts[slot * Hkv + h / G] = rows that selected the slot.  With up to kSmemLists lists a
// block counts in shared memory and adds its totals once; the warp-aggregated global
// atomics of the general path serialise on a few hundred hot counters.
constexpr int kSmemLists = 8192;

__global__ void count_lists_kernel(Params p, const int32_t* __restrict__ selected, int32_t* __restrict__ list_counts) {
  __shared__ int32_t hist[kSmemLists];
  const bool local = p.lists <= kSmemLists;
  if (local) {
    for (int i = threadIdx.x; i < (int)p.lists; i += blockDim.x) hist[i] = 0;
    __syncthreads();
  }
  const int64_t n = (int64_t)p.hist * p.Hq * p.Tq;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / (p.Hq * p.Tq);
    const int64_t rem = i - r * (p.Hq * p.Tq);
    const int h = (int)(rem / p.Tq);
    const int slot = selected[r * p.sel_rs + rem];
    // lanes of a warp that hit the same list add once (neighbouring tokens mostly do)
    const int list = slot >= 0 ? slot * p.Hkv + h / p.G : -1;
    const unsigned active = __activemask();
    const unsigned same = __match_any_sync(active, list);
    if (list >= 0 && (int)(threadIdx.x & 31) == __ffs(same) - 1) {
      if (local) atomicAdd(&hist[list], __popc(same));
      else atomicAdd(&list_counts[list], __popc(same));
    }
  }
  if (local) {
    __syncthreads();
    for (int i = threadIdx.x; i < (int)p.lists; i += blockDim.x)
      if (hist[i] != 0) atomicAdd(&list_counts[i], hist[i]);
  }
}

// ---------------------------------------------------------------------------
// dQ: row-stationary
// ---------------------------------------------------------------------------
template <int D>
struct DqSmem {
  static constexpr int kBuf = D > 128 ? 1 : 2;  // K / V tiles in flight (head dim 256: one, 192 KB of tiles)
  unsigned char q[kRows * row_bytes(D)];
  unsigned char g[kRows * row_bytes(D)];        // dO rows
  unsigned char k[kBuf][kBN * row_bytes(D)];
  unsigned char v[kBuf][kBN * row_bytes(D)];
  int64_t qoff[kRows];
  int64_t goff[kRows];
  float lse2[kRows];
  float delta[kRows];
  int32_t entry[kRows];
  int32_t item;
};

template <int D, typename S>
__device__ __forceinline__ void load_kv_tile(const Params& p, int kv_tok0, int kv_len, int kv_head, int tile, S& s,
                                             int buf, const __nv_bfloat16* __restrict__ k,
                                             const __nv_bfloat16* __restrict__ v) {
  const uint32_t kb = smem_u32(s.k[buf]), vb = smem_u32(s.v[buf]);
  constexpr int kChunks = D / 8;
  for (int i = threadIdx.x; i < kBN * kChunks; i += kThreads) {
    const int r = i / kChunks, ch = i - r * kChunks;
    const int key = tile * kBN + r;
    const bool ok = key < kv_len;
    const int64_t tok = (int64_t)kv_tok0 + (ok ? key : 0);
    cp_async16(kb + swz<D>(r, ch), k + tok * p.sk_t + (int64_t)kv_head * p.sk_h + ch * 8, ok);
    cp_async16(vb + swz<D>(r, ch), v + tok * p.sv_t + (int64_t)kv_head * p.sv_h + ch * 8, ok);
  }
}

template <bool kHalf, int D>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_kernel(Params p, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
              const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ dout, int64_t do_t, int64_t do_h,
              const int32_t* __restrict__ cu, const int32_t* __restrict__ list_counts,
              const int32_t* __restrict__ list_offsets, const int32_t* __restrict__ tile_prefix,
              const int32_t* __restrict__ row_list, const float* __restrict__ lse2, const float* __restrict__ delta,
              float* __restrict__ partial_dq, int32_t* __restrict__ work_counter) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  DqSmem<D>& s = *reinterpret_cast<DqSmem<D>*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_routed = p.hist > 0 ? tile_prefix[p.lists] : 0;
  const int n_items = n_routed + own_item_count(p.slots, p.Hq, p.C, kRows);
  const float scale = rsqrtf((float)D);
  const float sl2 = scale * kLog2e;
  constexpr int kChunks = D / 8;

  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) s.item = atomicAdd(work_counter, 1);
    __syncthreads();
    const int idx = s.item;
    if (idx >= n_items) break;
    const Item it = decode_item(p, idx, n_routed, kRows, cu, list_counts, list_offsets, tile_prefix);
    if (!it.valid) continue;

    for (int r = threadIdx.x; r < kRows; r += kThreads) {
      int32_t e = -1;
      int64_t off = 0, goff = 0;
      float l2 = INFINITY, dl = 0.f;              // rows that do not exist: p = exp2(-inf) = 0
      if (r < it.nrows) {
        int64_t row;
        if (it.causal) {
          row = (int64_t)(it.tok0 - p.win_lo + r) * p.Hq + it.head;
          e = (int32_t)(row * p.NP);
        } else {
          e = row_list[it.row_start + r];
          row = e / p.NP;
        }
        const int64_t t = row / p.Hq;
        const int64_t h = row - t * p.Hq;
        off = t * p.sq_t + h * p.sq_h;
        goff = t * do_t + h * do_h;
        l2 = lse2[row];
        dl = delta[row];
      }
      s.entry[r] = e;
      s.qoff[r] = off;
      s.goff[r] = goff;
      s.lse2[r] = l2;
      s.delta[r] = dl;
    }
    __syncthreads();
    {
      const uint32_t qb = smem_u32(s.q), gb = smem_u32(s.g);
      for (int i = threadIdx.x; i < kRows * kChunks; i += kThreads) {
        const int r = i / kChunks, ch = i - r * kChunks;
        cp_async16(qb + swz<D>(r, ch), q + s.qoff[r] + ch * 8, s.entry[r] >= 0);
        cp_async16(gb + swz<D>(r, ch), dout + s.goff[r] + ch * 8, s.entry[r] >= 0);
      }
    }
    const int ntiles = (it.kv_len + kBN - 1) / kBN;
    load_kv_tile<D>(p, it.kv_tok0, it.kv_len, it.kv_head, 0, s, 0, k, v);
    cp_async_commit();

    float dq[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f; }
    const int row0 = warp * 16 + (lane >> 2);          // this thread's rows: row0 and row0 + 8
    const int qpos0 = it.tok0 + row0, qpos1 = qpos0 + 8;

    constexpr int kBuf = DqSmem<D>::kBuf;
    for (int j = 0; j < ntiles; ++j) {
      // two buffers: tile j + 1 travels while tile j is used; one: it is requested behind tile j
      if (kBuf == 2) {
        if (j + 1 < ntiles) load_kv_tile<D>(p, it.kv_tok0, it.kv_len, it.kv_head, j + 1, s, (j + 1) & 1, k, v);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const uint32_t kb = smem_u32(s.k[j & (kBuf - 1)]), vb = smem_u32(s.v[j & (kBuf - 1)]);
      float sc[8][4], dp[8][4];
      rows_times_keys<kHalf, D>(sc, smem_u32(s.q), kb, warp, lane);
      rows_times_keys<kHalf, D>(dp, smem_u32(s.g), vb, warp, lane);
      const float l0 = s.lse2[row0], l1 = s.lse2[row0 + 8];
      const float d0 = s.delta[row0], d1 = s.delta[row0 + 8];
      const int key_base = j * kBN + 2 * (lane & 3);
      uint32_t da[4][4];                               // dS as A fragments (16 rows x 64 keys)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float ds[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key_base + nt * 8 + (e & 1);
          const int qpos = (e & 2) ? qpos1 : qpos0;
          const bool ok = key < it.kv_len && (!it.causal || it.kv_tok0 + key <= qpos);
          const float pij = ok ? exp2f(sc[nt][e] * sl2 - ((e & 2) ? l1 : l0)) : 0.f;
          ds[e] = pij * (dp[nt][e] - ((e & 2) ? d1 : d0));
        }
        da[nt >> 1][(nt & 1) * 2 + 0] = pack2_16<kHalf>(ds[0], ds[1]);
        da[nt >> 1][(nt & 1) * 2 + 1] = pack2_16<kHalf>(ds[2], ds[3]);
      }
      // dQ += dS . K   (K tile rows are the contraction index)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int dpi = 0; dpi < D / 16; ++dpi) {
          uint32_t b0, b1, b2, b3;
          const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldsm_x4_t(kb + swz<D>(r, 2 * dpi + (lane >> 4)), b0, b1, b2, b3);
          mma_16<kHalf>(dq[2 * dpi], da[kk], b0, b1);
          mma_16<kHalf>(dq[2 * dpi + 1], da[kk], b2, b3);
        }
      }
      __syncthreads();
      if (kBuf == 1 && j + 1 < ntiles) {
        load_kv_tile<D>(p, it.kv_tok0, it.kv_len, it.kv_head, j + 1, s, 0, k, v);
        cp_async_commit();
      }
    }
    cp_async_wait<0>();
    const int e0 = s.entry[row0], e1 = s.entry[row0 + 8];
    if (e0 >= 0) {
      float* dst = partial_dq + (int64_t)e0 * D + 2 * (lane & 3);
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<float2*>(dst + dt * 8) = make_float2(dq[dt][0] * scale, dq[dt][1] * scale);
    }
    if (e1 >= 0) {
      float* dst = partial_dq + (int64_t)e1 * D + 2 * (lane & 3);
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<float2*>(dst + dt * 8) = make_float2(dq[dt][2] * scale, dq[dt][3] * scale);
    }
  }
}

// dq[row] = sum of the row's partial slots (slot 0 always, slot r+1 if rank r has a chunk)
template <bool kHalf>
__global__ void __launch_bounds__(256)
sum_dq_kernel(Params p, const float* __restrict__ partial_dq, const int32_t* __restrict__ selected,
              const int32_t* __restrict__ status, __nv_bfloat16* __restrict__ dq, int64_t dq_t, int64_t dq_h) {
  const int lane = threadIdx.x & 31;
  // a dq kernel that gave up on a wait leaves a non-zero status: poison the result
  const bool failed = status != nullptr && *status != 0;
  const int nvec = p.D / 4;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < p.rows; row += warps) {
    const int64_t t = row / p.Hq;
    const int h = (int)(row - t * p.Hq);
    for (int c = lane; c < nvec; c += 32) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < p.NP; ++j) {
        if (j > 0 && selected[(int64_t)(j - 1) * p.sel_rs + (int64_t)h * p.Tq + t] < 0) continue;
        const float4 x = __ldg(reinterpret_cast<const float4*>(partial_dq + (row * p.NP + j) * p.D) + c);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      }
      if (failed) acc.x = acc.y = acc.z = acc.w = __int_as_float(0x7fc00000);
      uint2 pk;
      pk.x = pack2_16<kHalf>(acc.x, acc.y);
      pk.y = pack2_16<kHalf>(acc.z, acc.w);
      *reinterpret_cast<uint2*>(dq + t * dq_t + (int64_t)h * dq_h + c * 4) = pk;
    }
  }
}

// ---------------------------------------------------------------------------
// dK, dV: key-stationary
// ---------------------------------------------------------------------------
template <int D>
struct DkvSmem {
  unsigned char k[kBN * row_bytes(D)];
  unsigned char v[kBN * row_bytes(D)];
  unsigned char q[2][kRows * row_bytes(D)];     // row tiles, double buffered
  unsigned char g[2][kRows * row_bytes(D)];
  unsigned char ps[kRows * 128];                // P  [128 rows][64 keys], 16-bit, swizzled
  unsigned char ds[kRows * 128];                // dS
  int64_t qoff[3][kRows];                       // row descriptions run two tiles ahead
  int64_t goff[3][kRows];
  float lse2[3][kRows];
  float delta[3][kRows];
  int32_t tok[3][kRows];                        // query token of the row, -1: no row
  int32_t unit;
};

template <bool kHalf, int D>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dkdv_kernel(Params p, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ dout, int64_t do_t, int64_t do_h,
                const int32_t* __restrict__ cu, const int32_t* __restrict__ list_counts,
                const int32_t* __restrict__ list_offsets, const int32_t* __restrict__ row_list,
                const float* __restrict__ lse2, const float* __restrict__ delta,
                __nv_bfloat16* __restrict__ dk, int64_t dk_t, int64_t dk_h,
                __nv_bfloat16* __restrict__ dv, int64_t dv_t, int64_t dv_h, int32_t* __restrict__ work_counter) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  DkvSmem<D>& s = *reinterpret_cast<DkvSmem<D>*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = rsqrtf((float)D);
  const float sl2 = scale * kLog2e;
  constexpr int kChunks = D / 8;
  const int key_tiles = (p.C + kBN - 1) / kBN;
  const int64_t n_units = p.lists * key_tiles;
  // second phase: this warp owns keys mt*16 .. +15 and dims dh*D/2 .. +D/2 of dK and dV
  const int mt = warp & 3, dh = warp >> 2;

  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) s.unit = atomicAdd(work_counter, 1);
    __syncthreads();
    const int64_t u = s.unit;
    if (u >= n_units) break;
    // key tiles of late keys first: they have the fewest own-chunk rows, lists are equal
    const int l = (int)(u / key_tiles), kt = (int)(u - (int64_t)l * key_tiles);
    const int slot = l / p.Hkv, kvh = l - slot * p.Hkv;
    const int b = slot / p.mc, jc = slot - b * p.mc;
    const Slot sl = slot_of(cu, b, jc, p.C);
    const int key0 = sl.start + kt * kBN;                    // first key token of the tile
    if (key0 >= sl.end) continue;
    const int nkeys = min(kBN, sl.end - key0);
    {
      const uint32_t kb = smem_u32(s.k), vb = smem_u32(s.v);
      for (int i = threadIdx.x; i < kBN * kChunks; i += kThreads) {
        const int r = i / kChunks, ch = i - r * kChunks;
        const bool ok = r < nkeys;
        const int64_t tok = key0 + (ok ? r : 0);
        cp_async16(kb + swz<D>(r, ch), k + tok * p.sk_t + (int64_t)kvh * p.sk_h + ch * 8, ok);
        cp_async16(vb + swz<D>(r, ch), v + tok * p.sv_t + (int64_t)kvh * p.sv_h + ch * 8, ok);
      }
      cp_async_commit();
    }
    float acc_k[D / 16][4], acc_v[D / 16][4];
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      acc_k[i][0] = acc_k[i][1] = acc_k[i][2] = acc_k[i][3] = 0.f;
      acc_v[i][0] = acc_v[i][1] = acc_v[i][2] = acc_v[i][3] = 0.f;
    }
    // row tiles: the routed list of (slot, kv head), then the chunk's own rows head by head
    const int n_routed = p.hist > 0 ? list_counts[l] : 0;
    const int routed_tiles = (n_routed + kRows - 1) / kRows;
    const int own_rows = sl.end - key0;                      // tokens key0 .. end see at least one key of the tile
    const int own_tiles = (own_rows + kRows - 1) / kRows;
    const int total_tiles = routed_tiles + own_tiles * p.G;
    // describes the rows of row tile `rt` into slot rt % 3
    auto describe = [&](int rt) {
      const int m = rt % 3;
      const bool routed = rt < routed_tiles;
      int hl = 0, ot = 0;
      if (!routed) { hl = (rt - routed_tiles) / own_tiles; ot = (rt - routed_tiles) - hl * own_tiles; }
      for (int r = threadIdx.x; r < kRows; r += kThreads) {
        int64_t row = -1;
        int tokq = -1;
        if (routed) {
          const int i = rt * kRows + r;
          if (i < n_routed) {
            row = row_list[list_offsets[l] + i] / p.NP;
            tokq = 0x7fffffff;                                // routed rows see every key of the chunk
          }
        } else {
          const int tok = key0 + ot * kRows + r;
          if (tok < sl.end) { row = (int64_t)(tok - p.win_lo) * p.Hq + (kvh * p.G + hl); tokq = tok; }
        }
        int64_t off = 0, goff = 0;
        float l2 = INFINITY, dl = 0.f;
        if (row >= 0) {
          const int64_t t = row / p.Hq;
          const int64_t h = row - t * p.Hq;
          off = t * p.sq_t + h * p.sq_h;
          goff = t * do_t + h * do_h;
          l2 = lse2[row];
          dl = delta[row];
        }
        s.qoff[m][r] = off; s.goff[m][r] = goff; s.lse2[m][r] = l2; s.delta[m][r] = dl; s.tok[m][r] = tokq;
      }
    };
    // requests the Q and dO rows of row tile `rt` into buffer rt & 1
    auto request = [&](int rt) {
      const int m = rt % 3, bf = rt & 1;
      const uint32_t qb = smem_u32(s.q[bf]), gb = smem_u32(s.g[bf]);
      for (int i = threadIdx.x; i < kRows * kChunks; i += kThreads) {
        const int r = i / kChunks, ch = i - r * kChunks;
        cp_async16(qb + swz<D>(r, ch), q + s.qoff[m][r] + ch * 8, s.tok[m][r] >= 0);
        cp_async16(gb + swz<D>(r, ch), dout + s.goff[m][r] + ch * 8, s.tok[m][r] >= 0);
      }
      cp_async_commit();
    };
    describe(0);
    __syncthreads();
    request(0);
    if (total_tiles > 1) describe(1);
    __syncthreads();
    for (int rt = 0; rt < total_tiles; ++rt) {
      const int m = rt % 3, bf = rt & 1;
      if (rt + 1 < total_tiles) { request(rt + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
      __syncthreads();
      // phase 1: this warp's 16 rows x 64 keys of P and dS
      {
        float sc[8][4], dp[8][4];
        rows_times_keys<kHalf, D>(sc, smem_u32(s.q[bf]), smem_u32(s.k), warp, lane);
        rows_times_keys<kHalf, D>(dp, smem_u32(s.g[bf]), smem_u32(s.v), warp, lane);
        const int row0 = warp * 16 + (lane >> 2);
        const float l0 = s.lse2[m][row0], l1 = s.lse2[m][row0 + 8];
        const float d0 = s.delta[m][row0], d1 = s.delta[m][row0 + 8];
        const int t0 = s.tok[m][row0], t1 = s.tok[m][row0 + 8];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          float pv[4], ds[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = nt * 8 + 2 * (lane & 3) + (e & 1);
            const int tq = (e & 2) ? t1 : t0;
            const bool ok = key < nkeys && key0 + key <= tq;
            pv[e] = ok ? exp2f(sc[nt][e] * sl2 - ((e & 2) ? l1 : l0)) : 0.f;
            ds[e] = pv[e] * (dp[nt][e] - ((e & 2) ? d1 : d0));
          }
          // element (row, key) at byte row*128 + swizzled 16-byte chunk (key / 8) + (key % 8) * 2
          const uint32_t c0 = (uint32_t)(((nt ^ row0) & 7) << 4) + 4 * (lane & 3);
          const uint32_t c1 = (uint32_t)(((nt ^ (row0 + 8)) & 7) << 4) + 4 * (lane & 3);
          *reinterpret_cast<uint32_t*>(s.ps + row0 * 128 + c0) = pack2_16<kHalf>(pv[0], pv[1]);
          *reinterpret_cast<uint32_t*>(s.ps + (row0 + 8) * 128 + c1) = pack2_16<kHalf>(pv[2], pv[3]);
          *reinterpret_cast<uint32_t*>(s.ds + row0 * 128 + c0) = pack2_16<kHalf>(ds[0], ds[1]);
          *reinterpret_cast<uint32_t*>(s.ds + (row0 + 8) * 128 + c1) = pack2_16<kHalf>(ds[2], ds[3]);
        }
      }
      if (rt + 2 < total_tiles) describe(rt + 2);            // its loads overlap the other warps' MMAs
      __syncthreads();
      // phase 2: dV += P^T . dO,  dK += dS^T . Q  over the 128 rows of the tile
      {
        const uint32_t pb = smem_u32(s.ps), sb = smem_u32(s.ds), qb = smem_u32(s.q[bf]), gb = smem_u32(s.g[bf]);
#pragma unroll
        for (int ks = 0; ks < kRows / 16; ++ks) {
          // A = transposed 16 keys x 16 rows: stored [row][key], loaded with .trans
          const int ar = ks * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
          const int ach = 2 * mt + ((lane >> 3) & 1);
          const uint32_t aoff = (uint32_t)(ar * 128 + (((ach ^ ar) & 7) << 4));
          uint32_t pa[4], sa[4];
          ldsm_x4_t(pb + aoff, pa[0], pa[1], pa[2], pa[3]);
          ldsm_x4_t(sb + aoff, sa[0], sa[1], sa[2], sa[3]);
          const int br = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
          for (int dpi = 0; dpi < D / 32; ++dpi) {
            const int ch = dh * (D / 16) + 2 * dpi + (lane >> 4);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(gb + swz<D>(br, ch), b0, b1, b2, b3);
            mma_16<kHalf>(acc_v[2 * dpi], pa, b0, b1);
            mma_16<kHalf>(acc_v[2 * dpi + 1], pa, b2, b3);
            ldsm_x4_t(qb + swz<D>(br, ch), b0, b1, b2, b3);
            mma_16<kHalf>(acc_k[2 * dpi], sa, b0, b1);
            mma_16<kHalf>(acc_k[2 * dpi + 1], sa, b2, b3);
          }
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();
    // write dK (scaled) and dV rows of this tile: thread holds keys mt*16 + lane/4 (+8), dims dh*D/2 + nt*8 + 2*(lane%4)
    const int kr0 = mt * 16 + (lane >> 2), kr1 = kr0 + 8;
#pragma unroll
    for (int nt = 0; nt < D / 16; ++nt) {
      const int dim = dh * (D / 2) + nt * 8 + 2 * (lane & 3);
      if (kr0 < nkeys) {
        const int64_t tok = key0 + kr0;
        *reinterpret_cast<uint32_t*>(dk + tok * dk_t + (int64_t)kvh * dk_h + dim) =
            pack2_16<kHalf>(acc_k[nt][0] * scale, acc_k[nt][1] * scale);
        *reinterpret_cast<uint32_t*>(dv + tok * dv_t + (int64_t)kvh * dv_h + dim) = pack2_16<kHalf>(acc_v[nt][0], acc_v[nt][1]);
      }
      if (kr1 < nkeys) {
        const int64_t tok = key0 + kr1;
        *reinterpret_cast<uint32_t*>(dk + tok * dk_t + (int64_t)kvh * dk_h + dim) =
            pack2_16<kHalf>(acc_k[nt][2] * scale, acc_k[nt][3] * scale);
        *reinterpret_cast<uint32_t*>(dv + tok * dv_t + (int64_t)kvh * dv_h + dim) = pack2_16<kHalf>(acc_v[nt][2], acc_v[nt][3]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// dK, dV at head dim 256: the tiles of the kernel above would need 320 KB of shared memory.
// One buffer of row tiles (no prefetch of the next one), and P / dS take the place of the K tile,
// which - with the V tile - is fetched again for every row tile.
// ---------------------------------------------------------------------------
struct DkvWideSmem {
  unsigned char k[kBN * 512];                   // K tile; in the second phase P (16 KB) and dS (16 KB)
  unsigned char v[kBN * 512];
  unsigned char q[kRows * 512];
  unsigned char g[kRows * 512];
  int64_t qoff[kRows];
  int64_t goff[kRows];
  float lse2[kRows];
  float delta[kRows];
  int32_t tok[kRows];
  int32_t unit;
};

template <bool kHalf>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dkdv_wide_kernel(Params p, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                     const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ dout, int64_t do_t,
                     int64_t do_h, const int32_t* __restrict__ cu, const int32_t* __restrict__ list_counts,
                     const int32_t* __restrict__ list_offsets, const int32_t* __restrict__ row_list,
                     const float* __restrict__ lse2, const float* __restrict__ delta,
                     __nv_bfloat16* __restrict__ dk, int64_t dk_t, int64_t dk_h,
                     __nv_bfloat16* __restrict__ dv, int64_t dv_t, int64_t dv_h, int32_t* __restrict__ work_counter) {
  constexpr int D = 256;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  DkvWideSmem& s = *reinterpret_cast<DkvWideSmem*>(smem_raw);
  unsigned char* ps = s.k;                       // P  [128 rows][64 keys], 16-bit, swizzled
  unsigned char* ds = s.k + kRows * 128;         // dS
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = rsqrtf((float)D);
  const float sl2 = scale * kLog2e;
  constexpr int kChunks = D / 8;
  const int key_tiles = (p.C + kBN - 1) / kBN;
  const int64_t n_units = p.lists * key_tiles;
  const int mt = warp & 3, dh = warp >> 2;       // second phase: keys mt*16 .. +15, dims dh*128 .. +127

  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) s.unit = atomicAdd(work_counter, 1);
    __syncthreads();
    const int64_t u = s.unit;
    if (u >= n_units) break;
    const int l = (int)(u / key_tiles), kt = (int)(u - (int64_t)l * key_tiles);
    const int slot = l / p.Hkv, kvh = l - slot * p.Hkv;
    const int b = slot / p.mc, jc = slot - b * p.mc;
    const Slot sl = slot_of(cu, b, jc, p.C);
    const int key0 = sl.start + kt * kBN;
    if (key0 >= sl.end) continue;
    const int nkeys = min(kBN, sl.end - key0);
    float acc_k[D / 16][4], acc_v[D / 16][4];
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      acc_k[i][0] = acc_k[i][1] = acc_k[i][2] = acc_k[i][3] = 0.f;
      acc_v[i][0] = acc_v[i][1] = acc_v[i][2] = acc_v[i][3] = 0.f;
    }
    const int n_routed = p.hist > 0 ? list_counts[l] : 0;
    const int routed_tiles = (n_routed + kRows - 1) / kRows;
    const int own_rows = sl.end - key0;
    const int own_tiles = (own_rows + kRows - 1) / kRows;
    const int total_tiles = routed_tiles + own_tiles * p.G;
    for (int rt = 0; rt < total_tiles; ++rt) {
      // rows of the tile
      {
        const bool routed = rt < routed_tiles;
        int hl = 0, ot = 0;
        if (!routed) { hl = (rt - routed_tiles) / own_tiles; ot = (rt - routed_tiles) - hl * own_tiles; }
        for (int r = threadIdx.x; r < kRows; r += kThreads) {
          int64_t row = -1;
          int tokq = -1;
          if (routed) {
            const int i = rt * kRows + r;
            if (i < n_routed) { row = row_list[list_offsets[l] + i] / p.NP; tokq = 0x7fffffff; }
          } else {
            const int tok = key0 + ot * kRows + r;
            if (tok < sl.end) { row = (int64_t)(tok - p.win_lo) * p.Hq + (kvh * p.G + hl); tokq = tok; }
          }
          int64_t off = 0, goff = 0;
          float l2 = INFINITY, dl = 0.f;
          if (row >= 0) {
            const int64_t t = row / p.Hq;
            const int64_t h = row - t * p.Hq;
            off = t * p.sq_t + h * p.sq_h;
            goff = t * do_t + h * do_h;
            l2 = lse2[row];
            dl = delta[row];
          }
          s.qoff[r] = off; s.goff[r] = goff; s.lse2[r] = l2; s.delta[r] = dl; s.tok[r] = tokq;
        }
      }
      __syncthreads();                                       // rows described; the second phase of the tile before is over
      {
        const uint32_t kb = smem_u32(s.k), vb = smem_u32(s.v), qb = smem_u32(s.q), gb = smem_u32(s.g);
        for (int i = threadIdx.x; i < kBN * kChunks; i += kThreads) {
          const int r = i / kChunks, ch = i - r * kChunks;
          const bool ok = r < nkeys;
          const int64_t tok = key0 + (ok ? r : 0);
          cp_async16(kb + swz<D>(r, ch), k + tok * p.sk_t + (int64_t)kvh * p.sk_h + ch * 8, ok);
          cp_async16(vb + swz<D>(r, ch), v + tok * p.sv_t + (int64_t)kvh * p.sv_h + ch * 8, ok);
        }
        for (int i = threadIdx.x; i < kRows * kChunks; i += kThreads) {
          const int r = i / kChunks, ch = i - r * kChunks;
          cp_async16(qb + swz<D>(r, ch), q + s.qoff[r] + ch * 8, s.tok[r] >= 0);
          cp_async16(gb + swz<D>(r, ch), dout + s.goff[r] + ch * 8, s.tok[r] >= 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
      }
      __syncthreads();
      // phase 1: this warp's 16 rows x 64 keys of P and dS, kept in registers until every warp has read K and V
      uint32_t wp[8][2], wd[8][2];
      const int row0 = warp * 16 + (lane >> 2);
      {
        float sc[8][4], dp[8][4];
        rows_times_keys<kHalf, D>(sc, smem_u32(s.q), smem_u32(s.k), warp, lane);
        rows_times_keys<kHalf, D>(dp, smem_u32(s.g), smem_u32(s.v), warp, lane);
        const float l0 = s.lse2[row0], l1 = s.lse2[row0 + 8];
        const float d0 = s.delta[row0], d1 = s.delta[row0 + 8];
        const int t0 = s.tok[row0], t1 = s.tok[row0 + 8];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          float pv[4], dsv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = nt * 8 + 2 * (lane & 3) + (e & 1);
            const int tq = (e & 2) ? t1 : t0;
            const bool ok = key < nkeys && key0 + key <= tq;
            pv[e] = ok ? exp2f(sc[nt][e] * sl2 - ((e & 2) ? l1 : l0)) : 0.f;
            dsv[e] = pv[e] * (dp[nt][e] - ((e & 2) ? d1 : d0));
          }
          wp[nt][0] = pack2_16<kHalf>(pv[0], pv[1]);
          wp[nt][1] = pack2_16<kHalf>(pv[2], pv[3]);
          wd[nt][0] = pack2_16<kHalf>(dsv[0], dsv[1]);
          wd[nt][1] = pack2_16<kHalf>(dsv[2], dsv[3]);
        }
      }
      __syncthreads();                                       // K is no longer needed: P and dS take its place
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const uint32_t c0 = (uint32_t)(((nt ^ row0) & 7) << 4) + 4 * (lane & 3);
        const uint32_t c1 = (uint32_t)(((nt ^ (row0 + 8)) & 7) << 4) + 4 * (lane & 3);
        *reinterpret_cast<uint32_t*>(ps + row0 * 128 + c0) = wp[nt][0];
        *reinterpret_cast<uint32_t*>(ps + (row0 + 8) * 128 + c1) = wp[nt][1];
        *reinterpret_cast<uint32_t*>(ds + row0 * 128 + c0) = wd[nt][0];
        *reinterpret_cast<uint32_t*>(ds + (row0 + 8) * 128 + c1) = wd[nt][1];
      }
      __syncthreads();
      // phase 2: dV += P^T . dO,  dK += dS^T . Q  over the 128 rows of the tile
      {
        const uint32_t pb = smem_u32(ps), sb = smem_u32(ds), qb = smem_u32(s.q), gb = smem_u32(s.g);
#pragma unroll
        for (int ks = 0; ks < kRows / 16; ++ks) {
          const int ar = ks * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
          const int ach = 2 * mt + ((lane >> 3) & 1);
          const uint32_t aoff = (uint32_t)(ar * 128 + (((ach ^ ar) & 7) << 4));
          uint32_t pa[4], sa[4];
          ldsm_x4_t(pb + aoff, pa[0], pa[1], pa[2], pa[3]);
          ldsm_x4_t(sb + aoff, sa[0], sa[1], sa[2], sa[3]);
          const int br = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
          for (int dpi = 0; dpi < D / 32; ++dpi) {
            const int ch = dh * (D / 16) + 2 * dpi + (lane >> 4);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(gb + swz<D>(br, ch), b0, b1, b2, b3);
            mma_16<kHalf>(acc_v[2 * dpi], pa, b0, b1);
            mma_16<kHalf>(acc_v[2 * dpi + 1], pa, b2, b3);
            ldsm_x4_t(qb + swz<D>(br, ch), b0, b1, b2, b3);
            mma_16<kHalf>(acc_k[2 * dpi], sa, b0, b1);
            mma_16<kHalf>(acc_k[2 * dpi + 1], sa, b2, b3);
          }
        }
      }
      // the barrier at the top of the next tile (after its rows are described) ends this phase
    }
    const int kr0 = mt * 16 + (lane >> 2), kr1 = kr0 + 8;
#pragma unroll
    for (int nt = 0; nt < D / 16; ++nt) {
      const int dim = dh * (D / 2) + nt * 8 + 2 * (lane & 3);
      if (kr0 < nkeys) {
        const int64_t tok = key0 + kr0;
        *reinterpret_cast<uint32_t*>(dk + tok * dk_t + (int64_t)kvh * dk_h + dim) =
            pack2_16<kHalf>(acc_k[nt][0] * scale, acc_k[nt][1] * scale);
        *reinterpret_cast<uint32_t*>(dv + tok * dv_t + (int64_t)kvh * dv_h + dim) = pack2_16<kHalf>(acc_v[nt][0], acc_v[nt][1]);
      }
      if (kr1 < nkeys) {
        const int64_t tok = key0 + kr1;
        *reinterpret_cast<uint32_t*>(dk + tok * dk_t + (int64_t)kvh * dk_h + dim) =
            pack2_16<kHalf>(acc_k[nt][2] * scale, acc_k[nt][3] * scale);
        *reinterpret_cast<uint32_t*>(dv + tok * dv_t + (int64_t)kvh * dv_h + dim) = pack2_16<kHalf>(acc_v[nt][2], acc_v[nt][3]);
      }
    }
  }
}

template <typename K>
cudaError_t set_smem(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace

cudaError_t launch_count_lists(const Params& p, const int32_t* selected, int32_t* list_counts, cudaStream_t st) {
  if (p.hist <= 0) return cudaSuccess;
  count_lists_kernel<<<sm_count() * (p.lists <= kSmemLists ? 2 : 8), 512, 0, st>>>(p, selected, list_counts);
  return cudaGetLastError();
}

cudaError_t launch_bwd_delta(const Params& p, const __nv_bfloat16* out, const __nv_bfloat16* dout, int64_t do_t,
                             int64_t do_h, const float* lse, float* delta, float* lse2, cudaStream_t st) {
  int64_t blocks = (p.rows + 7) / 8;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (p.fp16) delta_kernel<true><<<(int)blocks, 256, 0, st>>>(p, out, dout, do_t, do_h, lse, delta, lse2);
  else delta_kernel<false><<<(int)blocks, 256, 0, st>>>(p, out, dout, do_t, do_h, lse, delta, lse2);
  return cudaGetLastError();
}

template <bool kHalf, int D>
static cudaError_t launch_dq_t(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                               const __nv_bfloat16* dout, int64_t do_t, int64_t do_h, const int32_t* cu,
                               const int32_t* list_counts, const int32_t* list_offsets, const int32_t* tile_prefix,
                               const int32_t* row_list, const float* lse2, const float* delta, float* partial_dq,
                               int32_t* work_counter, cudaStream_t st) {
  cudaError_t e = set_smem(bwd_dq_kernel<kHalf, D>, sizeof(DqSmem<D>));
  if (e != cudaSuccess) return e;
  bwd_dq_kernel<kHalf, D><<<sm_count(), kThreads, sizeof(DqSmem<D>), st>>>(
      p, q, k, v, dout, do_t, do_h, cu, list_counts, list_offsets, tile_prefix, row_list, lse2, delta, partial_dq,
      work_counter);
  return cudaGetLastError();
}

cudaError_t launch_bwd_dq(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                          const __nv_bfloat16* dout, int64_t do_t, int64_t do_h, const int32_t* cu,
                          const int32_t* list_counts, const int32_t* list_offsets, const int32_t* tile_prefix,
                          const int32_t* row_list, const float* lse2, const float* delta, float* partial_dq,
                          int32_t* work_counter, cudaStream_t st) {
#define MOBA_DQ(HALF, DIM) launch_dq_t<HALF, DIM>(p, q, k, v, dout, do_t, do_h, cu, list_counts, list_offsets, \
                                                  tile_prefix, row_list, lse2, delta, partial_dq, work_counter, st)
  switch (p.D) {
    case 64:  return p.fp16 ? MOBA_DQ(true, 64) : MOBA_DQ(false, 64);
    case 96:  return p.fp16 ? MOBA_DQ(true, 96) : MOBA_DQ(false, 96);
    case 128: return p.fp16 ? MOBA_DQ(true, 128) : MOBA_DQ(false, 128);
    case 256: return p.fp16 ? MOBA_DQ(true, 256) : MOBA_DQ(false, 256);
    default: return cudaErrorInvalidValue;
  }
#undef MOBA_DQ
}

cudaError_t launch_bwd_sum_dq(const Params& p, const float* partial_dq, const int32_t* selected, const int32_t* status,
                              __nv_bfloat16* dq, int64_t dq_t, int64_t dq_h, cudaStream_t st) {
  int64_t blocks = (p.rows + 7) / 8;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (p.fp16) sum_dq_kernel<true><<<(int)blocks, 256, 0, st>>>(p, partial_dq, selected, status, dq, dq_t, dq_h);
  else sum_dq_kernel<false><<<(int)blocks, 256, 0, st>>>(p, partial_dq, selected, status, dq, dq_t, dq_h);
  return cudaGetLastError();
}

template <bool kHalf, int D>
static cudaError_t launch_dkdv_t(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, int64_t do_t, int64_t do_h,
                                 const int32_t* cu, const int32_t* list_counts, const int32_t* list_offsets,
                                 const int32_t* row_list, const float* lse2, const float* delta, __nv_bfloat16* dk,
                                 int64_t dk_t, int64_t dk_h, __nv_bfloat16* dv, int64_t dv_t, int64_t dv_h,
                                 int32_t* work_counter, cudaStream_t st) {
  cudaError_t e = set_smem(bwd_dkdv_kernel<kHalf, D>, sizeof(DkvSmem<D>));
  if (e != cudaSuccess) return e;
  bwd_dkdv_kernel<kHalf, D><<<sm_count(), kThreads, sizeof(DkvSmem<D>), st>>>(
      p, q, k, v, dout, do_t, do_h, cu, list_counts, list_offsets, row_list, lse2, delta, dk, dk_t, dk_h, dv, dv_t,
      dv_h, work_counter);
  return cudaGetLastError();
}

cudaError_t launch_bwd_dkdv(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                            const __nv_bfloat16* dout, int64_t do_t, int64_t do_h, const int32_t* cu,
                            const int32_t* list_counts, const int32_t* list_offsets, const int32_t* row_list,
                            const float* lse2, const float* delta, __nv_bfloat16* dk, int64_t dk_t, int64_t dk_h,
                            __nv_bfloat16* dv, int64_t dv_t, int64_t dv_h, int32_t* work_counter, cudaStream_t st) {
#define MOBA_DKDV(HALF, DIM) launch_dkdv_t<HALF, DIM>(p, q, k, v, dout, do_t, do_h, cu, list_counts, list_offsets, \
                                                      row_list, lse2, delta, dk, dk_t, dk_h, dv, dv_t, dv_h,       \
                                                      work_counter, st)
  switch (p.D) {
    case 64:  return p.fp16 ? MOBA_DKDV(true, 64) : MOBA_DKDV(false, 64);
    case 96:  return p.fp16 ? MOBA_DKDV(true, 96) : MOBA_DKDV(false, 96);
    case 128: return p.fp16 ? MOBA_DKDV(true, 128) : MOBA_DKDV(false, 128);
    case 256: {
      auto kernel = p.fp16 ? bwd_dkdv_wide_kernel<true> : bwd_dkdv_wide_kernel<false>;
      const cudaError_t e = set_smem(kernel, sizeof(DkvWideSmem));
      if (e != cudaSuccess) return e;
      kernel<<<sm_count(), kThreads, sizeof(DkvWideSmem), st>>>(p, q, k, v, dout, do_t, do_h, cu, list_counts,
                                                              list_offsets, row_list, lse2, delta, dk, dk_t, dk_h, dv,
                                                              dv_t, dv_h, work_counter);
      return cudaGetLastError();
    }
    default: return cudaErrorInvalidValue;
  }
#undef MOBA_DKDV
}

}  // namespace moba
