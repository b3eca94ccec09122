// Dense stage of MoBA on the Blackwell tensor path: block-sparse flash-attention
// forward with tcgen05.mma, accumulators in tensor memory (TMEM) and K/V tiles
// staged by TMA.
//
// Replaces, for the inference path of the reference,
//   _varlen_attn_fwd_kernel        backends/_mthreads/ops/moba/attention.py:53-160  (own chunk, causal)
//   native_moba.routed / MATE FMHA backends/_mthreads/ops/moba/native_moba.py:120-135
//   _routed_gqa_attn_fwd_kernel    attention.py:610-707                           (selected chunks)
// Numerics follow attention.py:116-155 (fp32 scores * D^-0.5 * log2 e, P rounded
// to bf16 before P.V, fp32 accumulation, natural-log LSE); the running maximum is
// only refreshed when it grows by more than 8 (factor 256), which changes the
// rounding pattern but not the value of the softmax.
//
// Work item = up to 256 query rows (two 128-row MMA tiles, "A" and "B") against
// the keys of one chunk.  Routed items gather their rows through row_list (the
// rows of all query heads of a GQA group share the K/V stream of their kv
// head); own-chunk items are 256 consecutive tokens of one head with a causal
// mask.  CTAs are persistent (one per SM) and draw items from a global counter.
//
// Warp roles (384 threads):
//   warp 0      TMA producer: K and V tiles of 128 keys, two stages each
//   warp 1      MMA issuer (one lane): S = Q.K^T into TMEM, O += P.V with P read
//               from TMEM; owns the TMEM allocation
//   warps 4-7   softmax of tile A: one thread per row (TMEM lane)
//   warps 8-11  softmax of tile B
//   all warps   gather of the Q rows into 128B-swizzled shared memory
// TMEM columns: S_A 0-127, S_B 128-255, O_A 256-383, O_B 384-511; the bf16 P
// tile overwrites the first 64 columns of its S tile.
// The tensor core alternates  QK_A(j+1) | PV_B(j) | QK_B(j+1) | PV_A(j+1) ...
// so that the softmax of one tile runs while the MMAs of the other execute.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace moba {

namespace {

using namespace ptx;

constexpr int kThreads = 384;
constexpr int kTileM = 128;              // rows per MMA tile
constexpr int kBN = 128;                 // keys per K/V tile
constexpr int kHalfBytes = 128 * 64 * 2; // one [128][64] bf16 swizzled block
constexpr int kTileBytes = 2 * kHalfBytes;
constexpr uint32_t kTmemCols = 512;

constexpr uint32_t kIdescQK = idesc_bf16_f32(128, kBN, 0, 0);
constexpr uint32_t kIdescPV = idesc_bf16_f32(128, kHeadDim, 0, 1);

enum { ST_OK = 0, ST_PRODUCER = 1, ST_MMA = 2, ST_SOFTMAX = 3 };

struct Ctrl {
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint32_t tmem_slot;
  int32_t item;
  volatile int32_t abort;
  int32_t pad;
  int64_t qoff[2 * kTileM];
  int32_t entry[2 * kTileM];
};

constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + 6 * kTileBytes + sizeof(Ctrl);

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
attend_tc5_kernel(const Params p, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const __nv_bfloat16* __restrict__ q,
                  const int32_t* __restrict__ cu, const int32_t* __restrict__ list_counts,
                  const int32_t* __restrict__ list_offsets, const int32_t* __restrict__ tile_prefix,
                  const int32_t* __restrict__ row_list, float* __restrict__ partial_out,
                  float* __restrict__ partial_lse, int32_t* __restrict__ work_counter,
                  int32_t* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sQ = smem_u32(smem);                       // tile A, tile B
  const uint32_t sK = sQ + 2 * kTileBytes;                  // 2 stages
  const uint32_t sV = sK + 2 * kTileBytes;                  // 2 stages
  Ctrl& c = *reinterpret_cast<Ctrl*>(smem + 6 * kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&c.k_full[i]), 1);
      mbar_init(smem_u32(&c.k_empty[i]), 1);
      mbar_init(smem_u32(&c.v_full[i]), 1);
      mbar_init(smem_u32(&c.v_empty[i]), 1);
      mbar_init(smem_u32(&c.s_full[i]), 1);
      mbar_init(smem_u32(&c.p_full[i]), kTileM);
      mbar_init(smem_u32(&c.o_full[i]), 1);
    }
    c.abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&c.tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c.tmem_slot;

  const int n_routed = p.hist > 0 ? tile_prefix[p.lists] : 0;
  const int n_items = n_routed + own_item_count(p.slots, p.Hq, p.C, 2 * kTileM);
  const float sl2 = rsqrtf((float)kHeadDim) * 1.4426950408889634f;

  // running pipeline counters; every role advances its own copy identically
  uint32_t kc = 0, vc = 0;                 // K / V tiles produced or consumed so far
  uint32_t sph = 0, oph = 0;               // softmax: s_full / o_full phases of its tile
  uint32_t pph0 = 0, pph1 = 0;             // MMA: p_full phases of tile A / B

  for (;;) {
    __syncthreads();                       // every role has finished the previous item
    if (threadIdx.x == 0) c.item = c.abort ? 0x7fffffff : atomicAdd(work_counter, 1);
    __syncthreads();
    const int idx = c.item;
    if (idx >= n_items) break;
    const Item it = decode_item(p, idx, n_routed, 2 * kTileM, cu, list_counts, list_offsets, tile_prefix);
    if (!it.valid) continue;

    for (int r = threadIdx.x; r < 2 * kTileM; r += kThreads) {
      int32_t e = -1;
      int64_t off = 0;
      if (r < it.nrows) {
        if (it.causal) {
          e = (int32_t)(((int64_t)(it.tok0 + r) * p.Hq + it.head) * p.NP);
          off = (int64_t)(it.tok0 + r) * p.sq_t + (int64_t)it.head * p.sq_h;
        } else {
          e = row_list[it.row_start + r];
          const int64_t row = e / p.NP;
          const int64_t t = row / p.Hq;
          off = t * p.sq_t + (row - t * p.Hq) * p.sq_h;
        }
      }
      c.entry[r] = e;
      c.qoff[r] = off;
    }
    __syncthreads();
    // gather Q rows into two [2][128][64] blocks with the 128-byte swizzle TMA would produce
    for (int i0 = threadIdx.x; i0 < 2 * kTileM * 16; i0 += 4 * kThreads) {
      uint4 val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kThreads;
        val[u] = make_uint4(0, 0, 0, 0);
        if (i < 2 * kTileM * 16) {
          const int r = i >> 4, ch = i & 15;
          if (c.entry[r] >= 0) val[u] = __ldg(reinterpret_cast<const uint4*>(q + c.qoff[r] + ch * 8));
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kThreads;
        if (i < 2 * kTileM * 16) {
          const int r = i >> 4, ch = i & 15;
          const uint32_t dst = (uint32_t)((r >> 7) * kTileBytes + (ch >> 3) * kHalfBytes + (r & 127) * 128 +
                                          (((ch & 7) ^ (r & 7)) << 4));
          *reinterpret_cast<uint4*>(smem + dst) = val[u];
        }
      }
    }
    fence_proxy_async_smem();
    __syncthreads();

    const int ntiles = (it.kv_len + kBN - 1) / kBN;

    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      if (lane == 0) {
        for (int j = 0; j < ntiles; ++j) {
          const int tok = it.kv_tok0 + j * kBN;
          {
            const uint32_t s = kc & 1;
            if (!mbar_wait(smem_u32(&c.k_empty[s]), ((kc >> 1) & 1) ^ 1)) { atomicExch(status, ST_PRODUCER); c.abort = 1; break; }
            const uint32_t bar = smem_u32(&c.k_full[s]);
            mbar_expect_tx(bar, kTileBytes);
            tma_load_3d(sK + s * kTileBytes, &tmap_k, bar, 0, it.kv_head, tok);
            tma_load_3d(sK + s * kTileBytes + kHalfBytes, &tmap_k, bar, 64, it.kv_head, tok);
            ++kc;
          }
          {
            const uint32_t s = vc & 1;
            if (!mbar_wait(smem_u32(&c.v_empty[s]), ((vc >> 1) & 1) ^ 1)) { atomicExch(status, ST_PRODUCER); c.abort = 1; break; }
            const uint32_t bar = smem_u32(&c.v_full[s]);
            mbar_expect_tx(bar, kTileBytes);
            tma_load_3d(sV + s * kTileBytes, &tmap_v, bar, 0, it.kv_head, tok);
            tma_load_3d(sV + s * kTileBytes + kHalfBytes, &tmap_v, bar, 64, it.kv_head, tok);
            ++vc;
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        bool ok = true;
        auto issue_qk = [&](int x, uint32_t stage) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t koff = (uint32_t)((ks >> 2) * kHalfBytes + (ks & 3) * 32);
            mma_ss(tmem + x * kBN, smem_desc_sw128(sQ + x * kTileBytes + koff, 16, 1024),
                   smem_desc_sw128(sK + stage * kTileBytes + koff, 16, 1024), kIdescQK, ks > 0);
          }
        };
        auto issue_pv = [&](int x, uint32_t stage, bool first) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            mma_ts(tmem + 256 + x * kHeadDim, tmem + x * kBN + ks * 8,
                   smem_desc_sw128(sV + stage * kTileBytes + ks * 2048, kHalfBytes, 1024), kIdescPV,
                   (!first) || ks > 0);
        };
        tc_fence_after();
        ok = mbar_wait(smem_u32(&c.k_full[kc & 1]), (kc >> 1) & 1);
        if (ok) {
          tc_fence_after();
          issue_qk(0, kc & 1);
          tc_commit(smem_u32(&c.s_full[0]));
          issue_qk(1, kc & 1);
          tc_commit(smem_u32(&c.s_full[1]));
          tc_commit(smem_u32(&c.k_empty[kc & 1]));
          ++kc;
        }
        for (int j = 0; ok && j < ntiles; ++j) {
          const bool more = j + 1 < ntiles;
          ok = mbar_wait(smem_u32(&c.v_full[vc & 1]), (vc >> 1) & 1);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&c.p_full[0]), pph0);
          if (!ok) break;
          pph0 ^= 1;
          tc_fence_after();
          issue_pv(0, vc & 1, j == 0);
          if (more) {
            ok = mbar_wait(smem_u32(&c.k_full[kc & 1]), (kc >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            issue_qk(0, kc & 1);
            tc_commit(smem_u32(&c.s_full[0]));
          } else {
            tc_commit(smem_u32(&c.o_full[0]));
          }
          ok = mbar_wait(smem_u32(&c.p_full[1]), pph1);
          if (!ok) break;
          pph1 ^= 1;
          tc_fence_after();
          issue_pv(1, vc & 1, j == 0);
          tc_commit(smem_u32(&c.v_empty[vc & 1]));
          ++vc;
          if (more) {
            issue_qk(1, kc & 1);
            tc_commit(smem_u32(&c.s_full[1]));
            tc_commit(smem_u32(&c.k_empty[kc & 1]));
            ++kc;
          } else {
            tc_commit(smem_u32(&c.o_full[1]));
          }
        }
        if (!ok) { atomicExch(status, ST_MMA); c.abort = 1; }
      }
      __syncwarp();
    } else if (warp >= 4) {
      // ------------------------------------------------------------ softmax + epilogue
      const int x = (warp - 4) >> 2;                       // 0: tile A, 1: tile B
      const int row = (warp & 3) * 32 + lane;              // row inside the tile = TMEM lane
      const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
      const uint32_t tS = tmem + lane_base + x * kBN;
      const uint32_t tO = tmem + lane_base + 256 + x * kHeadDim;
      const int qpos = it.tok0 + x * kTileM + row;
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      uint32_t v[32];
      for (int j = 0; j < ntiles; ++j) {
        ok = mbar_wait(smem_u32(&c.s_full[x]), sph);
        if (!ok) break;
        sph ^= 1;
        tc_fence_after();
        const int key0 = j * kBN;
        const bool masked = key0 + kBN > it.kv_len ||
                            (it.causal && it.kv_tok0 + key0 + kBN - 1 > it.tok0 + x * kTileM);
        const int lim = it.causal ? min(it.kv_len, qpos - it.kv_tok0 + 1) : it.kv_len;   // keys < lim are visible
        // pass 1: row maximum
        float mx = -INFINITY;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(tS + ch * 32, v);
          tmem_wait_ld();
          if (masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              mx = (key0 + ch * 32 + i < lim) ? fmaxf(mx, __uint_as_float(v[i])) : mx;
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
          }
        }
        const float m_new = fmaxf(m_ref, mx * sl2);
        const bool grow = m_new > m_ref + 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = (m_new == -INFINITY) ? 1.f : ex2(m_ref - m_new);
          if (j > 0) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              tmem_ld32(tO + ch * 32, v);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tmem_st32(tO + ch * 32, v);
            }
            tmem_wait_st();
          }
          l *= alpha;
          m_ref = m_new;
        }
        // pass 2: P = exp2(S * sl2 - m_ref), bf16, written over the first 64 columns of S
        const float neg_m = -m_ref;
        float rs = 0.f;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(tS + ch * 32, v);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float p0 = ex2(fmaf(__uint_as_float(v[2 * i]), sl2, neg_m));
            float p1 = ex2(fmaf(__uint_as_float(v[2 * i + 1]), sl2, neg_m));
            if (masked) {
              p0 = (key0 + ch * 32 + 2 * i < lim) ? p0 : 0.f;
              p1 = (key0 + ch * 32 + 2 * i + 1 < lim) ? p1 : 0.f;
            }
            rs += p0 + p1;
            pk[i] = pack_bf16(p0, p1);
          }
          tmem_st16(tS + ch * 16, pk);
        }
        l += rs;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&c.p_full[x]));
      }
      if (ok) ok = mbar_wait(smem_u32(&c.o_full[x]), oph);
      if (ok) {
        oph ^= 1;
        tc_fence_after();
        const int32_t e = c.entry[x * kTileM + row];
        const float inv = 1.f / l;
        float* dst = partial_out + (int64_t)(e >= 0 ? e : 0) * kHeadDim;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(tO + ch * 32, v);
          tmem_wait_ld();
          if (e >= 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(dst + ch * 32)[i] =
                  make_float4(__uint_as_float(v[4 * i]) * inv, __uint_as_float(v[4 * i + 1]) * inv,
                              __uint_as_float(v[4 * i + 2]) * inv, __uint_as_float(v[4 * i + 3]) * inv);
          }
        }
        if (e >= 0) partial_lse[e] = (m_ref + log2f(l)) * 0.6931471805599453f;
        tc_fence_before();
      } else {
        atomicExch(status, ST_SOFTMAX);
        c.abort = 1;
      }
    }
  }

  // teardown: all roles are past their last wait; give in-flight copies time to
  // land after an abort, then release tensor memory
  if (c.abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [T, Hkv, D] bf16 with element strides (st, sh, 1): boxes of 128 tokens x 1 head x 64 dims
bool make_kv_map(CUtensorMap* m, const __nv_bfloat16* base, int64_t T, int Hkv, int64_t st, int64_t sh) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)Hkv, (cuuint64_t)T};
  const cuuint64_t strides[2] = {(cuuint64_t)sh * 2, (cuuint64_t)st * 2};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)kBN};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_attend_tc5(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                              const __nv_bfloat16* v, const int32_t* cu, const int32_t* list_counts,
                              const int32_t* list_offsets, const int32_t* tile_prefix,
                              const int32_t* row_list, float* partial_out, float* partial_lse,
                              int32_t* work_counter, int32_t* status, cudaStream_t st) {
  CUtensorMap mk, mv;
  if (!make_kv_map(&mk, k, p.T, p.Hkv, p.sk_t, p.sk_h) || !make_kv_map(&mv, v, p.T, p.Hkv, p.sv_t, p.sv_h))
    return cudaErrorNotSupported;
  cudaError_t e = cudaFuncSetAttribute(attend_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  attend_tc5_kernel<<<sms, kThreads, kSmemBytes, st>>>(p, mk, mv, q, cu, list_counts, list_offsets, tile_prefix,
                                                      row_list, partial_out, partial_lse, work_counter, status);
  return cudaGetLastError();
}

}  // namespace moba
