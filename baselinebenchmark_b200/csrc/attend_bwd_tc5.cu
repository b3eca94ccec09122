// dQ of the MoBA dense stage on the Blackwell tensor path (tcgen05.mma, accumulators in
// tensor memory, K/V tiles staged by TMA).
//
// Replaces, for the training path of the reference, the dq kernel of
//   _triton_varlen_backward   backends/_mthreads/ops/moba/attention.py:163-369
// as called for both branches by MixedAttention.backward (parallel.py:171-236): with the
// merged LSE and delta_i = sum_d dO_id O_id of the merged output,
//   p_ij = exp(s_ij * scale - lse_i),  dS_ij = p_ij (dO_i . V_j - delta_i),
//   dQ_i = scale * sum_j dS_ij K_j.
//
// Work items are those of the forward's tcgen05 dense stage: up to 256 query rows (two
// 128-row MMA tiles, "A" and "B") against the keys of one chunk, visited in tiles of 64 keys.
// Per tile step and row tile X the tensor core computes
//   S_X  = Q_X . K^T     (128 x 64, operands in shared memory)
//   dP_X = dO_X . V^T    (128 x 64, operands in shared memory)
//   dQ_X += dS_X . K     (128 x D, dS read from tensor memory, K as the MN-major operand)
// and one thread per row turns S and dP into dS (input dtype) in between.  Each item writes
// scale * dQ as an fp32 partial into the row's slot (own chunk = 0, rank r = r + 1); a later
// kernel adds a row's slots.  No atomics: the result is bit-identical run to run.
//
// Warp roles (384 threads) as in the forward kernel: warp 0 TMA producer (K tiles in three
// stages, V tiles in two), warp 1 MMA issuer and owner of the TMEM allocation, warp 2 draws and resolves
// the next item, warps 4-7 / 8-11 the rows of tile A / B.
// TMEM columns of row tile X: S 128X..128X+63 (dS, 16-bit, overwrites the first 32),
// dP 128X+64..128X+127, dQ 256+128X..; 512 columns in all, which is why a key step is 64 wide.
// Every wait is bounded; a wait that gives up sets a status word that the summing kernel
// turns into NaN results.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace moba {

// defined with the forward kernel: tiled map of a [T, Hkv, D] tensor, boxes of `box_rows` x 1 x 64
bool make_kv_map(CUtensorMap* m, bool fp16, int D, const __nv_bfloat16* base, int64_t T, int Hkv, int64_t st,
                 int64_t sh, int box_rows);

namespace {

using namespace ptx;

constexpr int kThreads = 384;
constexpr int kTileM = 128;                 // rows per MMA tile
constexpr int kBN = 64;                     // keys per step
constexpr int kQBlockBytes = 128 * 64 * 2;  // one [128 rows][64 dims] swizzled block of Q or dO
constexpr int kQTileBytes = 2 * kQBlockBytes;
constexpr int kKvBlockBytes = kBN * 64 * 2; // one [64 keys][64 dims] swizzled block of K or V
constexpr int kKvTileBytes = 2 * kKvBlockBytes;
constexpr uint32_t kTmemCols = 512;
constexpr int kPrefixCache = 2048;          // ints of tile_prefix kept in shared memory
constexpr int kKStages = 3;                 // K tiles serve S (early) and dQ (late): three stages give the next one a full step of lead

template <bool kHalf> constexpr uint32_t kIdescS = idesc_16_f32(kHalf, 128, kBN, 0, 0);
template <bool kHalf, int D> constexpr uint32_t kIdescDQ = idesc_16_f32(kHalf, 128, D, 0, 1);

enum { ST_OK = 0, ST_PRODUCER = 11, ST_MMA = 12, ST_ROWS = 13 };

struct Ctrl {
  uint64_t k_full[kKStages], k_empty[kKStages], v_full[2], v_empty[2];
  uint64_t s_full[2], ds_full[2], dq_full[2];
  uint64_t item_ready[2];
  uint32_t tmem_slot;
  volatile int32_t abort;
  Item item[2];                              // slot (n & 1) holds item n, resolved one item ahead
  int32_t done[2];
  int64_t qoff[2][2 * kTileM];               // element offset of the row in q
  int32_t grow[2][2 * kTileM];               // row index t * Hq + h (dO, lse and delta are indexed by it)
  int32_t entry[2][2 * kTileM];              // partial slot of the row, -1: no row
  int32_t prefix_cache[kPrefixCache];
};

constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + 4 * kQTileBytes + (kKStages + 2) * kKvTileBytes + sizeof(Ctrl);
static_assert(kSmemBytes <= 232448, "shared memory of one CTA");

struct KernelArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* dout;                 // contiguous [T, Hq, D]
  const int32_t* cu;
  const int32_t* list_counts;
  const int32_t* list_offsets;
  const int32_t* tile_prefix;
  const int32_t* row_list;
  const float* lse2;                         // lse * log2(e), [rows]
  const float* delta;                        // [rows]
  float* partial_dq;
  int32_t* work_counter;
  int32_t* status;
};

// One spare warp, one item ahead of the others: draws the next item from the global queue,
// decodes it and resolves its rows into prefetch slot `slot`.
__device__ __forceinline__ void prefetch_item(const Params& p, const KernelArgs& a, Ctrl& c, int slot,
                                              int n_routed, int n_items) {
  const int lane = threadIdx.x & 31;
  Item it;
  it.valid = 0;
  int done = 0;
  for (;;) {
    int idx = 0;
    if (lane == 0) idx = c.abort ? 0x7fffffff : atomicAdd(a.work_counter, 1);
    idx = __shfl_sync(0xffffffffu, idx, 0);
    if (idx >= n_items) { done = 1; break; }
    it = decode_item(p, idx, n_routed, 2 * kTileM, a.cu, a.list_counts, a.list_offsets,
                     p.lists < kPrefixCache ? c.prefix_cache : a.tile_prefix);
    if (it.valid) break;
  }
  if (lane == 0) { c.item[slot] = it; c.done[slot] = done; }
  if (!done) {
    int32_t ent[2 * kTileM / 32];
#pragma unroll
    for (int u = 0; u < 2 * kTileM / 32; ++u) {
      const int r = lane + 32 * u;
      ent[u] = -1;
      if (r < it.nrows) {
        if (it.causal) ent[u] = (int32_t)(((int64_t)(it.tok0 - p.win_lo + r) * p.Hq + it.head) * p.NP);
        else ent[u] = __ldg(a.row_list + it.row_start + r);
      }
    }
#pragma unroll
    for (int u = 0; u < 2 * kTileM / 32; ++u) {
      const int r = lane + 32 * u;
      const int32_t e = ent[u];
      int64_t off = 0;
      int32_t row = 0;
      if (e >= 0) {
        row = e / p.NP;
        const int64_t t = row / p.Hq;
        off = t * p.sq_t + (row - t * p.Hq) * p.sq_h;
      }
      c.entry[slot][r] = e;
      c.qoff[slot][r] = off;
      c.grow[slot][r] = row;
      if (e >= 0) {                                            // the gather of the next item then hits L2
        const __nv_bfloat16* g = a.dout + (int64_t)row * p.D;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(g));
        if (p.D > 64) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + off + 64));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(g + 64));
        }
      }
    }
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(smem_u32(&c.item_ready[slot]));
}

// Common head of an item, executed by all 384 threads: take the prefetched item of slot
// `slot`; the 256 row threads (kGather) gather its Q and dO rows into 128-byte-swizzled
// tiles (Q tile A, Q tile B, dO tile A, dO tile B).  Returns false when the queue is empty.
template <bool kGather, int D>
__device__ __forceinline__ bool next_item(const KernelArgs& a, Ctrl& c, unsigned char* smem, int slot, Item& it) {
  __syncthreads();
  if (c.done[slot]) return false;
  it = c.item[slot];
  if (kGather) {
    const int32_t* entry = c.entry[slot];
    const int64_t* qoff = c.qoff[slot];
    const int32_t* grow = c.grow[slot];
    constexpr int kChunks = D / 8;                  // 16-byte pieces of a row
    const int t = threadIdx.x - 128;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      uint4 val[kChunks];
#pragma unroll
      for (int u = 0; u < kChunks; ++u) {
        const int i = t + u * 256;
        const int r = i / kChunks, ch = i % kChunks;
        val[u] = make_uint4(0, 0, 0, 0);
        if (entry[r] >= 0) {
          const __nv_bfloat16* src = which == 0 ? a.q + qoff[r] : a.dout + (int64_t)grow[r] * D;
          val[u] = __ldg(reinterpret_cast<const uint4*>(src + ch * 8));
        }
      }
#pragma unroll
      for (int u = 0; u < kChunks; ++u) {
        const int i = t + u * 256;
        const int r = i / kChunks, ch = i % kChunks;
        const uint32_t dst = (uint32_t)(which * 2 * kQTileBytes + (r >> 7) * kQTileBytes + (ch >> 3) * kQBlockBytes +
                                        (r & 127) * 128 + (((ch & 7) ^ (r & 7)) << 4));
        *reinterpret_cast<uint4*>(smem + dst) = val[u];
      }
    }
  }
  fence_proxy_async_smem();
  __syncthreads();
  return true;
}

// Exponentials evaluated with the cubic on the FMA pipe instead of the special-function
// unit: kPolyPairs of every 8 column pairs (never in masked steps, where a masked column must
// give exactly zero).
#ifndef MOBA_BWD_POLY_PAIRS
#define MOBA_BWD_POLY_PAIRS 2
#endif
constexpr int kPolyPairs = MOBA_BWD_POLY_PAIRS;

// One step of one row: S and dP (64 fp32 columns each of this thread's TMEM lane) -> dS in
// the input dtype, written over the first 32 columns of S.
//   p = 2^(s * scale * log2 e - lse * log2 e),  dS = p * (dP - delta)
// Rows that do not exist carry lse = +inf (p = 0) and zero Q / dO rows.
template <bool kMasked, bool kHalf>
__device__ __forceinline__ void ds_row(uint32_t tS, int key0, int lim, float sl2, float neg_lse2, float delta) {
  uint32_t s[64], g[64];
  tmem_ld64(tS, s);
  tmem_ld64(tS + 64, g);
  tmem_wait_ld();
  if (kMasked) {
#pragma unroll
    for (int i = 0; i < 64; ++i) s[i] = (key0 + i < lim) ? s[i] : 0xff800000u;   // -inf: p = 0
  }
  const uint64_t scale2 = pack2(sl2, sl2);
  const uint64_t nl2 = pack2(neg_lse2, neg_lse2);
  const uint64_t dl2 = pack2(delta, delta);
#pragma unroll
  for (int ch = 0; ch < 2; ++ch) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = ch * 32 + 2 * i;
      const uint64_t x = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, nl2);
      uint64_t pr;
      if (!kMasked && (i & 7) < kPolyPairs) pr = ex2_poly2(x);
      else pr = pack2(ex2_approx(lo2(x)), ex2_approx(hi2(x)));
      const uint64_t d = mul2(pr, sub2(pack2(__uint_as_float(g[e]), __uint_as_float(g[e + 1])), dl2));
      pk[i] = pack2_16<kHalf>(lo2(d), hi2(d));
    }
    tmem_st16(tS + ch * 16, pk);
  }
  tmem_wait_st();
}

// Shared-memory descriptor words (128-byte swizzle).  Low word: start address >> 4 |
// (leading byte offset >> 4) << 16; high word: stride byte offset 1024 >> 4 | version 1 << 14
// | SWIZZLE_128B (2) << 29.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);

// S_X = Q_X . K^T and dP_X = dO_X . V^T for one 64-key tile: D / 16 k-steps each; `dk`, `dv`:
// descriptor words of the K and V stage.
template <int X, bool kHalf, int D>
__device__ __forceinline__ void issue_s_dp(uint32_t tmem, uint32_t dq, uint32_t dg, uint32_t dk, uint32_t dv) {
  constexpr int kQBlock = kQBlockBytes >> 4, kQTile = kQTileBytes >> 4;
  constexpr int kKvBlock = kKvBlockBytes >> 4;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint32_t qo = (uint32_t)(X * kQTile + (ks >> 2) * kQBlock + (ks & 3) * 2);
    const uint32_t ko = (uint32_t)((ks >> 2) * kKvBlock + (ks & 3) * 2);
    mma_ss_lo<kDescHi>(tmem + X * 128, dq + qo, dk + ko, kIdescS<kHalf>, ks > 0);
  }
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint32_t qo = (uint32_t)(X * kQTile + (ks >> 2) * kQBlock + (ks & 3) * 2);
    const uint32_t ko = (uint32_t)((ks >> 2) * kKvBlock + (ks & 3) * 2);
    mma_ss_lo<kDescHi>(tmem + X * 128 + 64, dg + qo, dv + ko, kIdescS<kHalf>, ks > 0);
  }
}
// dQ_X (+)= dS_X . K for one 64-key tile: 4 k-steps of 16 keys, dS read from tensor memory,
// K read as the MN-major operand (`dkt`: descriptor word with the 64-dim block stride).
template <int X, bool kHalf, int D>
__device__ __forceinline__ void issue_dq(uint32_t tmem, uint32_t dkt, bool first) {
#pragma unroll
  for (int ks = 0; ks < kBN / 16; ++ks)
    mma_ts_lo<kDescHi>(tmem + 256 + X * 128, tmem + X * 128 + ks * 8,
                       dkt + ks * (2048 >> 4), kIdescDQ<kHalf, D>, (!first) || ks > 0);
}

template <bool kHalf, int D>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_tc5_kernel(const Params p, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const KernelArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sQ = smem_u32(smem);                       // Q tile A, Q tile B
  const uint32_t sG = sQ + 2 * kQTileBytes;                 // dO tile A, dO tile B
  const uint32_t sK = sG + 2 * kQTileBytes;                 // 3 stages
  const uint32_t sV = sK + kKStages * kKvTileBytes;         // 2 stages
  Ctrl& c = *reinterpret_cast<Ctrl*>(smem + 4 * kQTileBytes + (kKStages + 2) * kKvTileBytes);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kKStages; ++i) {
      mbar_init(smem_u32(&c.k_full[i]), 1);
      mbar_init(smem_u32(&c.k_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&c.v_full[i]), 1);
      mbar_init(smem_u32(&c.v_empty[i]), 1);
      mbar_init(smem_u32(&c.s_full[i]), 1);
      mbar_init(smem_u32(&c.ds_full[i]), kTileM);
      mbar_init(smem_u32(&c.dq_full[i]), 1);
      mbar_init(smem_u32(&c.item_ready[i]), 1);
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
  if (p.hist > 0 && p.lists < kPrefixCache)
    for (int i = threadIdx.x; i <= (int)p.lists; i += kThreads) c.prefix_cache[i] = a.tile_prefix[i];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c.tmem_slot;

  const int n_routed = p.hist > 0 ? a.tile_prefix[p.lists] : 0;
  const int n_items = n_routed + own_item_count(p.slots, p.Hq, p.C, 2 * kTileM);
  Item it;

  if (warp < 4) {
    // =============================================== warps 0-3: TMA producer, MMA issuer, item prefetch
    setmaxnreg_dec<72>();
    uint32_t g = 0;                        // K/V tiles produced (warp 0) or consumed (warp 1) so far
    uint32_t pph0 = 0, pph1 = 0;           // ds_full phases of tile A / B
    int pre = 0;                           // producer: tiles of the coming item already requested
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t dq = __shfl_sync(0xffffffffu, desc_lo(sQ, 16), 0);
    const uint32_t dg = __shfl_sync(0xffffffffu, desc_lo(sG, 16), 0);
    const uint32_t dk = __shfl_sync(0xffffffffu, desc_lo(sK, 16), 0);
    const uint32_t dv = __shfl_sync(0xffffffffu, desc_lo(sV, 16), 0);
    const uint32_t dkt = __shfl_sync(0xffffffffu, desc_lo(sK, kKvBlockBytes), 0);
    const uint32_t el = elect_one();
    for (int n = 0;; ++n) {
      if (warp == 2) prefetch_item(p, a, c, n & 1, n_routed, n_items);
      if (!next_item<false, D>(a, c, smem, n & 1, it)) break;
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      if (warp == 0 && lane == 0) {
        // K and V tile `j` of item `w` into the next stage; false after a timeout
        auto load_tile = [&](const Item& w, int j) -> bool {
          const int tok = w.kv_tok0 + j * kBN;
          {
            const uint32_t s = g % kKStages, par = ((g / kKStages) & 1) ^ 1;
            if (!mbar_wait(smem_u32(&c.k_empty[s]), par)) return false;
            const uint32_t bar = smem_u32(&c.k_full[s]);
            mbar_expect_tx(bar, ((D + 63) / 64) * kKvBlockBytes);
            tma_load_3d(sK + s * kKvTileBytes, &tmap_k, bar, 0, w.kv_head, tok);
            if (D > 64) tma_load_3d(sK + s * kKvTileBytes + kKvBlockBytes, &tmap_k, bar, 64, w.kv_head, tok);
          }
          {
            const uint32_t s = g & 1, par = ((g >> 1) & 1) ^ 1;
            if (!mbar_wait(smem_u32(&c.v_empty[s]), par)) return false;
            const uint32_t bar = smem_u32(&c.v_full[s]);
            mbar_expect_tx(bar, ((D + 63) / 64) * kKvBlockBytes);
            tma_load_3d(sV + s * kKvTileBytes, &tmap_v, bar, 0, w.kv_head, tok);
            if (D > 64) tma_load_3d(sV + s * kKvTileBytes + kKvBlockBytes, &tmap_v, bar, 64, w.kv_head, tok);
          }
          ++g;
          return true;
        };
        bool alive = true;
        for (int j = pre; alive && j < ntiles; ++j) alive = load_tile(it, j);
        pre = 0;
        // first tiles of the next item as soon as stages free up
        if (alive) {
          const int s1 = (n + 1) & 1;
          alive = mbar_wait(smem_u32(&c.item_ready[s1]), ((n + 1) >> 1) & 1);
          if (alive && !c.done[s1]) {
            const Item nx = c.item[s1];
            const int nt = min(2, (nx.kv_len + kBN - 1) / kBN);
            for (; alive && pre < nt; ++pre) alive = load_tile(nx, pre);
          }
        }
        if (!alive) { atomicExch(a.status, ST_PRODUCER); c.abort = 1; }
      } else if (warp == 1) {
        // MMA issuer: the whole warp runs convergent, one elected lane issues.
        bool ok = true;
        constexpr uint32_t kStageDesc = kKvTileBytes >> 4;
        tc_fence_after();
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.k_full[g % kKStages]), (g / kKStages) & 1));
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.v_full[g & 1]), (g >> 1) & 1));
        if (ok) {
          tc_fence_after();
          if (el) {
            const uint32_t ko = (g % kKStages) * kStageDesc, vo = (g & 1) * kStageDesc;
            issue_s_dp<0, kHalf, D>(tm, dq, dg, dk + ko, dv + vo);
            tc_commit(smem_u32(&c.s_full[0]));
            issue_s_dp<1, kHalf, D>(tm, dq, dg, dk + ko, dv + vo);
            tc_commit(smem_u32(&c.s_full[1]));
            tc_commit(smem_u32(&c.v_empty[g & 1]));
          }
          __syncwarp();
        }
        for (int j = 0; ok && j < ntiles; ++j) {
          const bool more = j + 1 < ntiles;
          const uint32_t kcur = g % kKStages, g1 = g + 1, knxt = g1 % kKStages, vnxt = g1 & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.ds_full[0]), pph0));
          if (!ok) break;
          pph0 ^= 1;
          tc_fence_after();
          if (el) issue_dq<0, kHalf, D>(tm, dkt + kcur * kStageDesc, j == 0);
          __syncwarp();
          if (more) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.k_full[knxt]), (g1 / kKStages) & 1));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.v_full[vnxt]), (g1 >> 1) & 1));
            if (!ok) break;
            tc_fence_after();
            if (el) {
              issue_s_dp<0, kHalf, D>(tm, dq, dg, dk + knxt * kStageDesc, dv + vnxt * kStageDesc);
              tc_commit(smem_u32(&c.s_full[0]));
            }
          } else if (el) {
            tc_commit(smem_u32(&c.dq_full[0]));
          }
          __syncwarp();
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.ds_full[1]), pph1));
          if (!ok) break;
          pph1 ^= 1;
          tc_fence_after();
          if (el) {
            issue_dq<1, kHalf, D>(tm, dkt + kcur * kStageDesc, j == 0);
            tc_commit(smem_u32(&c.k_empty[kcur]));
            if (more) {
              issue_s_dp<1, kHalf, D>(tm, dq, dg, dk + knxt * kStageDesc, dv + vnxt * kStageDesc);
              tc_commit(smem_u32(&c.s_full[1]));
              tc_commit(smem_u32(&c.v_empty[vnxt]));
            } else {
              tc_commit(smem_u32(&c.dq_full[1]));
            }
          }
          __syncwarp();
          ++g;
        }
        if (!ok && lane == 0) { atomicExch(a.status, ST_MMA); c.abort = 1; }
      }
      __syncwarp();
    }
  } else {
    // =============================================== warps 4-11: one thread per row
    setmaxnreg_inc<216>();
    const int x = (warp - 4) >> 2;                       // 0: tile A, 1: tile B
    const int row = (warp & 3) * 32 + lane;              // row inside the tile = TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_base + x * 128;
    const uint32_t tDQ = tmem + lane_base + 256 + x * 128;
    const float scale = rsqrtf((float)D);
    const float sl2 = scale * 1.4426950408889634f;
    uint32_t sph = 0, oph = 0;                           // s_full / dq_full phases of this tile
    for (int n = 0; next_item<true, D>(a, c, smem, n & 1, it); ++n) {
      const int32_t e = c.entry[n & 1][x * kTileM + row];
      float neg_lse2 = -INFINITY, delta = 0.f;
      if (e >= 0) {
        const int32_t gr = c.grow[n & 1][x * kTileM + row];
        neg_lse2 = -__ldg(a.lse2 + gr);
        delta = __ldg(a.delta + gr);
      }
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      const int qpos = it.tok0 + x * kTileM + row;
      const int lim = it.causal ? min(it.kv_len, qpos - it.kv_tok0 + 1) : it.kv_len;   // keys < lim are visible
      bool ok = true;
      for (int j = 0; ok && j < ntiles; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.s_full[x]), sph));   // warp-uniform exit
        if (!ok) break;
        sph ^= 1;
        tc_fence_after();
        const int key0 = j * kBN;
        const bool masked = key0 + kBN > it.kv_len ||
                            (it.causal && it.kv_tok0 + key0 + kBN - 1 > it.tok0 + x * kTileM);
        if (masked) ds_row<true, kHalf>(tS, key0, lim, sl2, neg_lse2, delta);
        else ds_row<false, kHalf>(tS, key0, lim, sl2, neg_lse2, delta);
        tc_fence_before();
        mbar_arrive(smem_u32(&c.ds_full[x]));
      }
      if (ok) ok = mbar_wait(smem_u32(&c.dq_full[x]), oph);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        oph ^= 1;
        tc_fence_after();
        // dQ rows go through this warp's 8 KB of the (now idle) Q tile so that every global
        // store writes whole 128-byte pieces of four rows: 32 columns at a time, rows 144
        // bytes apart in shared memory.
        unsigned char* stage = smem + x * kQTileBytes + (warp & 3) * 8192;
        uint32_t v[32];
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          tmem_ld32(tDQ + ch * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(stage + lane * 144 + i * 16) =
                make_float4(__uint_as_float(v[4 * i]) * scale, __uint_as_float(v[4 * i + 1]) * scale,
                            __uint_as_float(v[4 * i + 2]) * scale, __uint_as_float(v[4 * i + 3]) * scale);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3), c16 = lane & 7;
            const int32_t er = __shfl_sync(0xffffffffu, e, rl);
            const float4 val = *reinterpret_cast<const float4*>(stage + rl * 144 + c16 * 16);
            if (er >= 0) *reinterpret_cast<float4*>(a.partial_dq + (int64_t)er * D + ch * 32 + c16 * 4) = val;
          }
          __syncwarp();
        }
        tc_fence_before();
      } else {
        atomicExch(a.status, ST_ROWS);
        c.abort = 1;
      }
    }
  }

  // teardown: all roles are past their last wait; give in-flight copies time to land after
  // an abort, then release tensor memory
  if (c.abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

cudaError_t launch_bwd_dq_tc5(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                              const __nv_bfloat16* v, const __nv_bfloat16* dout, const int32_t* cu,
                              const int32_t* list_counts, const int32_t* list_offsets, const int32_t* tile_prefix,
                              const int32_t* row_list, const float* lse2, const float* delta, float* partial_dq,
                              int32_t* work_counter, int32_t* status, cudaStream_t st) {
  if (p.D != 64 && p.D != 96 && p.D != 128) return cudaErrorInvalidValue;
  CUtensorMap mk, mv;
  if (!make_kv_map(&mk, p.fp16 != 0, p.D, k, p.T, p.Hkv, p.sk_t, p.sk_h, kBN) ||
      !make_kv_map(&mv, p.fp16 != 0, p.D, v, p.T, p.Hkv, p.sv_t, p.sv_h, kBN))
    return cudaErrorNotSupported;
  auto kernel = p.D == 128 ? (p.fp16 ? bwd_dq_tc5_kernel<true, 128> : bwd_dq_tc5_kernel<false, 128>)
              : p.D == 96  ? (p.fp16 ? bwd_dq_tc5_kernel<true, 96> : bwd_dq_tc5_kernel<false, 96>)
                           : (p.fp16 ? bwd_dq_tc5_kernel<true, 64> : bwd_dq_tc5_kernel<false, 64>);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const KernelArgs args{q, dout, cu, list_counts, list_offsets, tile_prefix, row_list, lse2, delta, partial_dq,
                        work_counter, status};
  kernel<<<sms, kThreads, kSmemBytes, st>>>(p, mk, mv, args);
  return cudaGetLastError();
}

}  // namespace moba
