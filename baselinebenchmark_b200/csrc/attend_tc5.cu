// Dense stage of MoBA on the Blackwell tensor path: block-sparse flash-attention
// forward with tcgen05.mma, accumulators in tensor memory (TMEM) and K/V tiles
// staged by TMA.
//
// Replaces, for the inference path of the reference,
//   _varlen_attn_fwd_kernel        backends/_mthreads/ops/moba/attention.py:53-160  (own chunk, causal)
//   native_moba.routed / MATE FMHA backends/_mthreads/ops/moba/native_moba.py:120-135
//   _routed_gqa_attn_fwd_kernel    attention.py:610-707                           (selected chunks)
// Templated on the element type (bf16, fp16) and the head dim (64, 96, 128); buffer
// strides in shared memory and TMEM are those of head dim 128.  At head dim 96 the second
// 64-dim block of a K / V tile is half filled (TMA fills dims 96-127 with zeros), Q.K^T runs
// six 16-dim steps and P.V writes 96 accumulator columns.
// Numerics follow attention.py:116-155 (fp32 scores * D^-0.5 * log2 e, P rounded
// to the input dtype before P.V, fp32 accumulation, natural-log LSE); the running maximum is
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
//   warp 2      draws, decodes and resolves the next work item while the current one runs
//   warp 1      MMA issuer: S = Q.K^T into TMEM, O += P.V with P read from TMEM; the
//               warp runs convergent, one elected lane issues; owns the TMEM allocation
//   warps 4-7   softmax of tile A: one thread per row (TMEM lane)
//   warps 8-11  softmax of tile B
//   warps 4-11  also gather the Q rows into 128B-swizzled shared memory at the item start
// TMEM columns: S_A 0-127, S_B 128-255, O_A 256-383, O_B 384-511; the 16-bit P
// tile overwrites the first 64 columns of its S tile.
// The tensor core alternates  QK_A(j+1) | PV_B(j) | QK_B(j+1) | PV_A(j+1) ...
// so that the softmax of one tile runs while the MMAs of the other execute.
#include <mutex>

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

template <bool kHalf> constexpr uint32_t kIdescQK = idesc_16_f32(kHalf, 128, kBN, 0, 0);
template <bool kHalf, int D> constexpr uint32_t kIdescPV = idesc_16_f32(kHalf, 128, D, 0, 1);

constexpr int kPrefixCache = 6144;       // ints of tile_prefix kept in shared memory (24 KB)

enum { ST_OK = 0, ST_PRODUCER = 1, ST_MMA = 2, ST_SOFTMAX = 3 };

struct Ctrl {
  static constexpr int kPrefix = kPrefixCache;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint64_t item_ready[2];                  // slot filled by the prefetch warp (phase = fill count)
  uint32_t tmem_slot;
  volatile int32_t abort;
  int32_t n_routed, n_items;               // work items of the launch (routed tiles first), set by thread 0
  SlotRange own;                           // slots the own-chunk items run over
  // Work items are drawn and resolved one item ahead by a spare warp: slot (n & 1)
  // holds item n, its output entries and the offsets of its Q rows.
  Item item[2];
  int32_t done[2];
  int64_t qoff[2][2 * kTileM];
  int32_t entry[2][2 * kTileM];
  // tile_prefix sampled once per CTA (whole when it fits): decoding an item searches it, and with
  // short items (small chunks) eleven dependent global loads per item were the critical path
  int32_t prefix_cache[kPrefixCache];
  float row_inv[kTileM];                   // head dim 256: the row's factor (scale / row sum), handed to the warps that write the second half of O
};

constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + 6 * kTileBytes + sizeof(Ctrl);

// Pairs of score columns whose exponential is evaluated with the cubic on the
// FMA pipe instead of the special-function unit: kPolyPairs out of every 8.
// The special-function unit sustains 16 ex2 per clock and SM, which is exactly
// the rate two 128x128 MMAs per 1024 cycles would ask of it.
#ifndef MOBA_POLY_PAIRS
#define MOBA_POLY_PAIRS 2
#endif
constexpr int kPolyPairs = MOBA_POLY_PAIRS;

struct KernelArgs {
  const __nv_bfloat16* q;
  const int32_t* cu;
  const int32_t* list_counts;
  const int32_t* list_offsets;
  const int32_t* tile_prefix;
  const int32_t* row_list;
  __half* partial_out;                     // fp16 rows scaled by a power of two per row
  float2* partial_lse;                     // {natural-log LSE, 1 / scale}
  int32_t* work_counter;
  int32_t* status;
};

// tile_prefix is kept in shared memory sampled every 2^shift entries (shift 0: whole), so that
// finding the list of a routed item costs `shift` dependent global loads instead of log2(lists).
__host__ __device__ inline int prefix_shift(int64_t lists, int cache_entries) {
  int shift = 0;
  while ((lists >> shift) + 2 > cache_entries) ++shift;
  return shift;
}
template <typename CtrlT>
__device__ __forceinline__ void fill_prefix_cache(CtrlT& c, const int32_t* __restrict__ tile_prefix, int64_t lists,
                                                  int nthreads) {
  const int shift = prefix_shift(lists, CtrlT::kPrefix);
  const int n = (int)(lists >> shift) + 1;                   // samples 0, 2^shift, ..., the last one <= lists
  for (int i = threadIdx.x; i < n; i += nthreads) c.prefix_cache[i] = tile_prefix[(int64_t)i << shift];
}
// last l in [0, lists) with tile_prefix[l] <= i (i is a routed item: tile_prefix[lists] > i)
template <typename CtrlT>
__device__ __forceinline__ int find_list(const CtrlT& c, const int32_t* __restrict__ tile_prefix, int64_t lists, int i) {
  const int shift = prefix_shift(lists, CtrlT::kPrefix);
  int lo = 0, hi = (int)(lists >> shift) + 1;                // samples: last k with cache[k] <= i
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (c.prefix_cache[mid] <= i) lo = mid; else hi = mid;
  }
  int l = lo << shift;
  int r = min(l + (1 << shift), (int)lists);                 // tile_prefix[r] > i, or r == lists
  while (r - l > 1) {
    const int mid = (l + r) >> 1;
    if (__ldg(tile_prefix + mid) <= i) l = mid; else r = mid;
  }
  return l;
}

// Runs in one spare warp while the other warps work on the current item: draws the
// next item from the global queue (skipping empty own-chunk tiles), decodes it and
// resolves its rows (output entry and Q row offset) into prefetch slot `slot`.
template <int kItemRows, typename CtrlT>
__device__ __forceinline__ void prefetch_item(const Params& p, const KernelArgs& a, CtrlT& c, int slot) {
  const int lane = threadIdx.x & 31;
  const int n_routed = c.n_routed, n_items = c.n_items;
  const SlotRange own = c.own;
  Item it;
  it.valid = 0;
  int done = 0;
  for (;;) {
    int idx = 0;
    if (lane == 0) idx = c.abort ? 0x7fffffff : atomicAdd(a.work_counter, 1);
    idx = __shfl_sync(0xffffffffu, idx, 0);
    if (idx >= n_items) { done = 1; break; }
    it = decode_item(p, idx, n_routed, kItemRows, a.cu, a.list_counts, a.list_offsets, a.tile_prefix,
                     idx < n_routed ? find_list(c, a.tile_prefix, p.lists, idx) : 0, own);
    if (it.valid) break;
  }
  if (lane == 0) { c.item[slot] = it; c.done[slot] = done; }
  if (!done) {
    // the rows of a lane: all row_list loads in flight before any of them is used
    int32_t ent[kItemRows / 32];
#pragma unroll
    for (int u = 0; u < kItemRows / 32; ++u) {
      const int r = lane + 32 * u;
      ent[u] = -1;
      if (r < it.nrows) {
        if (!it.causal) ent[u] = __ldg(a.row_list + it.row_start + r);
        else if (r >= it.row_start)                            // rows before the query window stay absent
          ent[u] = (int32_t)(((int64_t)(it.tok0 - p.win_lo + r) * p.Hq + it.head) * p.NP);
      }
    }
#pragma unroll
    for (int u = 0; u < kItemRows / 32; ++u) {
      const int r = lane + 32 * u;
      const int32_t e = ent[u];
      int64_t off = 0;
      if (e >= 0) {
        // entries and rows fit 32 bits (checked on the host): unsigned 32-bit divisions, not the
        // 64-bit ones, which are a subroutine of a hundred instructions each
        const uint32_t row = (uint32_t)e / (uint32_t)p.NP;
        const uint32_t t = row / (uint32_t)p.Hq;
        off = (int64_t)t * p.sq_t + (int64_t)(row - t * (uint32_t)p.Hq) * p.sq_h;
      }
      c.entry[slot][r] = e;
      c.qoff[slot][r] = off;
      if (e >= 0) {                                            // the gather of the next item then hits L2
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + off));
        if (p.D > 64) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + off + 64));
        if (p.D > 128) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + off + 128));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + off + 192));
        }
      }
    }
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(smem_u32(&c.item_ready[slot]));   // the producer may look at the slot now
}

// Common head of an item, executed by all 384 threads: take the prefetched item
// of slot `slot`; the softmax warps (kGather) gather its Q rows into the two swizzled Q tiles.  Returns
// false when the queue is empty (or the kernel is aborting).
template <bool kGather, int D, int kItemRows = 2 * kTileM>
__device__ __forceinline__ bool next_item(const KernelArgs& a, Ctrl& c, unsigned char* smem, int slot, Item& it) {
  __syncthreads();                         // every role has finished the previous item; slot is filled
  if (c.done[slot]) return false;
  it = c.item[slot];
  const int32_t* entry = c.entry[slot];
  const int64_t* qoff = c.qoff[slot];
  // gather Q rows into two tiles of D/64 [128][64] blocks with the 128-byte swizzle TMA would
  // produce; the 256 softmax threads do it, each with its D/8 loads in flight at once
  if (kGather) {
    constexpr int kChunks = D / 8;                  // 16-byte pieces of a row
    constexpr int kPieces = kItemRows * kChunks / 256;   // pieces per thread
    const int t = threadIdx.x - 128;
    uint4 val[kPieces];
#pragma unroll
    for (int u = 0; u < kPieces; ++u) {
      const int i = t + u * 256;
      const int r = i / kChunks, ch = i % kChunks;
      val[u] = make_uint4(0, 0, 0, 0);
      if (entry[r] >= 0) val[u] = __ldg(reinterpret_cast<const uint4*>(a.q + qoff[r] + ch * 8));
    }
#pragma unroll
    for (int u = 0; u < kPieces; ++u) {
      const int i = t + u * 256;
      const int r = i / kChunks, ch = i % kChunks;
      const uint32_t dst = (uint32_t)((r >> 7) * kTileBytes + (ch >> 3) * kHalfBytes + (r & 127) * 128 +
                                      (((ch & 7) ^ (r & 7)) << 4));
      *reinterpret_cast<uint4*>(smem + dst) = val[u];
    }
  }
  fence_proxy_async_smem();
  __syncthreads();
  return true;
}

// One softmax step of one row: S (128 fp32 columns of this thread's TMEM lane)
// -> P (bf16, written over the first 64 columns), running max / sum updated.
// `before_rescale` runs (warp-uniformly) before the accumulator O is rescaled: a kernel whose
// previous P.V may still be executing at that point waits for it there.
template <bool kMasked, bool kHalf, int D, typename F>
__device__ __forceinline__ void softmax_row(uint32_t tS, uint32_t tO, int j, int key0, int lim, float sl2,
                                            float& m_ref, float& l, F&& before_rescale) {
  uint32_t v[128];
  tmem_ld128(tS, v);
  tmem_wait_ld();
  if (kMasked) {
#pragma unroll
    for (int i = 0; i < 128; ++i) v[i] = (key0 + i < lim) ? v[i] : 0xff800000u;   // -inf
  }
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 128; i += 8) {
    mx0 = max3(mx0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
    mx1 = max3(mx1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
    mx2 = max3(mx2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
    mx3 = max3(mx3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
  }
  const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
  const float m_new = fmaxf(m_ref, mx * sl2);
  if (__any_sync(0xffffffffu, m_new > m_ref + 8.f)) {
    const float alpha = (m_new == -INFINITY) ? 1.f : ex2_approx(m_ref - m_new);
    if (j > 0) {
      before_rescale();
      uint32_t o[32];
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        tmem_ld32(tO + ch * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st32(tO + ch * 32, o);
      }
    }
    l *= alpha;
    m_ref = m_new;
  }
  const uint64_t scale2 = pack2(sl2, sl2);
  const uint64_t negm2 = pack2(-m_ref, -m_ref);
  uint64_t sum_a = 0, sum_b = 0;           // two packed accumulators = four running sums
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = ch * 32 + 2 * i;
      const uint64_t x = fma2(pack2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])), scale2, negm2);
      uint64_t pr;
      if ((i & 7) < kPolyPairs) {
        pr = ex2_poly2(x);
      } else {
        pr = pack2(ex2_approx(lo2(x)), ex2_approx(hi2(x)));
      }
      if (i & 1) sum_b = add2(sum_b, pr); else sum_a = add2(sum_a, pr);
      pk[i] = pack2_16<kHalf>(lo2(pr), hi2(pr));
    }
    tmem_st16(tS + ch * 16, pk);
  }
  const uint64_t sum = add2(sum_a, sum_b);
  l += lo2(sum) + hi2(sum);
  tmem_wait_st();
}

// Descriptor words.  Low word: start address >> 4 | (leading byte offset >> 4) << 16;
// high word (constant): stride byte offset 1024 >> 4 | version 1 << 14 | SWIZZLE_128B (2) << 29.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint64_t desc64(uint32_t lo) { return ((uint64_t)kDescHi << 32) | lo; }

// S_X = Q_X . K^T for one K tile: 8 k-steps of 16 dims; X and STAGE are compile-time
// so every descriptor is the base word plus an immediate.
template <int X, int STAGE, bool kHalf, int D>
__device__ __forceinline__ void issue_qk(uint32_t tmem, uint32_t dq, uint32_t dk) {
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    constexpr int kBlock = kHalfBytes >> 4, kTile = kTileBytes >> 4;
    const uint32_t koff = (uint32_t)((ks >> 2) * kBlock + (ks & 3) * 2);
    mma_ss(tmem + X * kBN, desc64(dq + X * kTile + koff), desc64(dk + STAGE * kTile + koff), kIdescQK<kHalf>, ks > 0);
  }
}
// O_X (+)= P_X . V for one V tile: 8 k-steps of 16 keys, P read from tensor memory.
template <int X, int STAGE, bool kHalf, int D>
__device__ __forceinline__ void issue_pv(uint32_t tmem, uint32_t dv, bool first) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    mma_ts(tmem + 256 + X * 128, tmem + X * kBN + ks * 8,
           desc64(dv + STAGE * (kTileBytes >> 4) + ks * (2048 >> 4)), kIdescPV<kHalf, D>, (!first) || ks > 0);
}

template <bool kHalf, int D>
__global__ void __launch_bounds__(kThreads, 1)
attend_tc5_kernel(const Params p, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const KernelArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sQ = smem_u32(smem);                       // tile A, tile B
  const uint32_t sK = sQ + 2 * kTileBytes;                  // 2 stages
  const uint32_t sV = sK + 2 * kTileBytes;                  // 2 stages
  Ctrl& c = *reinterpret_cast<Ctrl*>(smem + 6 * kTileBytes);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;   // warp index, uniform

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&c.k_full[i]), 1);
      mbar_init(smem_u32(&c.k_empty[i]), 1);
      mbar_init(smem_u32(&c.v_full[i]), 1);
      mbar_init(smem_u32(&c.v_empty[i]), 1);
      mbar_init(smem_u32(&c.s_full[i]), 1);
      mbar_init(smem_u32(&c.p_full[i]), kTileM);
      mbar_init(smem_u32(&c.o_full[i]), 1);
      mbar_init(smem_u32(&c.item_ready[i]), 1);
    }
    c.abort = 0;
    c.n_routed = p.hist > 0 ? a.tile_prefix[p.lists] : 0;
    c.own = own_slot_range(p, a.cu);
    c.n_items = c.n_routed + own_item_count(c.own.n, p.Hq, p.C, 2 * kTileM);
    fence_barrier_init();
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&c.tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (p.hist > 0) fill_prefix_cache(c, a.tile_prefix, p.lists, kThreads);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c.tmem_slot;
  Item it;

  if (warp < 4) {
    // =============================================== warps 0-3: TMA producer, MMA issuer, two spare warps
    setmaxnreg_dec<72>();
    uint32_t kc = 0, vc = 0;               // K / V tiles produced (warp 0) or consumed (warp 1) so far
    uint32_t pph0 = 0, pph1 = 0;           // p_full phases of tile A / B
    int pre = 0;                           // producer: tiles of the coming item already requested
    // warp-uniform copies of the TMEM base and of the low words of the shared-memory
    // descriptors of the first Q / K / V block (every other block or k-step is a
    // compile-time offset from these), and the lane that issues
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t dq = __shfl_sync(0xffffffffu, desc_lo(sQ, 16), 0);
    const uint32_t dk = __shfl_sync(0xffffffffu, desc_lo(sK, 16), 0);
    const uint32_t dv = __shfl_sync(0xffffffffu, desc_lo(sV, kHalfBytes), 0);
    const uint32_t el = elect_one();
    for (int n = 0;; ++n) {
      // warp 2 runs one item ahead: it fills slot n & 1 while the others still work on item n - 1
      if (warp == 2) prefetch_item<2 * kTileM>(p, a, c, n & 1);
      if (!next_item<false, D>(a, c, smem, n & 1, it)) break;
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      if (warp == 0 && lane == 0) {
        // K and V tile `j` of item `w` into the next free stages; false after a timeout
        auto load_tile = [&](const Item& w, int j) -> bool {
          const int tok = w.kv_tok0 + j * kBN;
          {
            const uint32_t s = kc & 1;
            if (!mbar_wait(smem_u32(&c.k_empty[s]), ((kc >> 1) & 1) ^ 1)) return false;
            const uint32_t bar = smem_u32(&c.k_full[s]);
            mbar_expect_tx(bar, ((D + 63) / 64) * kHalfBytes);
            tma_load_3d(sK + s * kTileBytes, &tmap_k, bar, 0, w.kv_head, tok);
            if (D > 64) tma_load_3d(sK + s * kTileBytes + kHalfBytes, &tmap_k, bar, 64, w.kv_head, tok);
            ++kc;
          }
          {
            const uint32_t s = vc & 1;
            if (!mbar_wait(smem_u32(&c.v_empty[s]), ((vc >> 1) & 1) ^ 1)) return false;
            const uint32_t bar = smem_u32(&c.v_full[s]);
            mbar_expect_tx(bar, ((D + 63) / 64) * kHalfBytes);
            tma_load_3d(sV + s * kTileBytes, &tmap_v, bar, 0, w.kv_head, tok);
            if (D > 64) tma_load_3d(sV + s * kTileBytes + kHalfBytes, &tmap_v, bar, 64, w.kv_head, tok);
            ++vc;
          }
          return true;
        };
        bool alive = true;
        for (int j = pre; alive && j < ntiles; ++j) alive = load_tile(it, j);
        pre = 0;
        // The first tiles of the next item are requested as soon as stages free up, while the
        // tail of this item still computes: the prefetch warp has the next item ready by then.
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
        // MMA issuer.  The whole warp runs this code so that addresses and descriptors
        // stay warp-uniform (uniform registers); one elected lane executes the
        // tcgen05 instructions.  Issued from a single-lane branch instead, every MMA
        // costs a dozen dependent vector instructions and the issuer starves for
        // issue slots next to the softmax warps of its scheduler partition.
        bool ok = true;
        tc_fence_after();
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.k_full[kc & 1]), (kc >> 1) & 1));
        if (ok) {
          tc_fence_after();
          if (el) {
            if (kc & 1) { issue_qk<0, 1, kHalf, D>(tm, dq, dk); tc_commit(smem_u32(&c.s_full[0])); issue_qk<1, 1, kHalf, D>(tm, dq, dk); }
            else        { issue_qk<0, 0, kHalf, D>(tm, dq, dk); tc_commit(smem_u32(&c.s_full[0])); issue_qk<1, 0, kHalf, D>(tm, dq, dk); }
            tc_commit(smem_u32(&c.s_full[1]));
            tc_commit(smem_u32(&c.k_empty[kc & 1]));
          }
          __syncwarp();
          ++kc;
        }
        // K tile j+1 and V tile j always sit in opposite stages (kc == vc + 1 here)
        for (int j = 0; ok && j < ntiles; ++j) {
          const bool more = j + 1 < ntiles;
          const uint32_t vs = vc & 1, ks = vs ^ 1;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.v_full[vs]), (vc >> 1) & 1));
          if (!ok) break;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.p_full[0]), pph0));
          if (!ok) break;
          pph0 ^= 1;
          tc_fence_after();
          if (el) { if (vs) issue_pv<0, 1, kHalf, D>(tm, dv, j == 0); else issue_pv<0, 0, kHalf, D>(tm, dv, j == 0); }
          __syncwarp();
          if (more) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.k_full[ks]), (kc >> 1) & 1));
            if (!ok) break;
            tc_fence_after();
            if (el) {
              if (ks) issue_qk<0, 1, kHalf, D>(tm, dq, dk); else issue_qk<0, 0, kHalf, D>(tm, dq, dk);
              tc_commit(smem_u32(&c.s_full[0]));
            }
          } else if (el) {
            tc_commit(smem_u32(&c.o_full[0]));
          }
          __syncwarp();
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.p_full[1]), pph1));
          if (!ok) break;
          pph1 ^= 1;
          tc_fence_after();
          if (el) {
            if (vs) issue_pv<1, 1, kHalf, D>(tm, dv, j == 0); else issue_pv<1, 0, kHalf, D>(tm, dv, j == 0);
            tc_commit(smem_u32(&c.v_empty[vs]));
            if (more) {
              if (ks) issue_qk<1, 1, kHalf, D>(tm, dq, dk); else issue_qk<1, 0, kHalf, D>(tm, dq, dk);
              tc_commit(smem_u32(&c.s_full[1]));
              tc_commit(smem_u32(&c.k_empty[ks]));
            } else {
              tc_commit(smem_u32(&c.o_full[1]));
            }
          }
          __syncwarp();
          ++vc;
          if (more) ++kc;
        }
        if (!ok && lane == 0) { atomicExch(a.status, ST_MMA); c.abort = 1; }
      }
      __syncwarp();
    }
  } else {
    // =============================================== warps 4-11: softmax + epilogue, one thread per row
    setmaxnreg_inc<216>();
    const int x = (warp - 4) >> 2;                       // 0: tile A, 1: tile B
    const int row = (warp & 3) * 32 + lane;              // row inside the tile = TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_base + x * kBN;
    const uint32_t tO = tmem + lane_base + 256 + x * 128;
    const float sl2 = rsqrtf((float)D) * 1.4426950408889634f;
    uint32_t sph = 0, oph = 0;                           // s_full / o_full phases of this tile
    for (int n = 0; next_item<true, D>(a, c, smem, n & 1, it); ++n) {
      const int32_t* entries = c.entry[n & 1];
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      const int qpos = it.tok0 + x * kTileM + row;
      const int lim = it.causal ? min(it.kv_len, qpos - it.kv_tok0 + 1) : it.kv_len;   // keys < lim are visible
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; ok && j < ntiles; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.s_full[x]), sph));   // warp-uniform exit
        if (!ok) break;
        sph ^= 1;
        tc_fence_after();
        const int key0 = j * kBN;
        const bool masked = key0 + kBN > it.kv_len ||
                            (it.causal && it.kv_tok0 + key0 + kBN - 1 > it.tok0 + x * kTileM);
        // S of the next step is only computed after this tile's P.V: O is quiet here
        if (masked) softmax_row<true, kHalf, D>(tS, tO, j, key0, lim, sl2, m_ref, l, [] {});
        else softmax_row<false, kHalf, D>(tS, tO, j, key0, lim, sl2, m_ref, l, [] {});
        tc_fence_before();
        mbar_arrive(smem_u32(&c.p_full[x]));
      }
      if (ok) ok = mbar_wait(smem_u32(&c.o_full[x]), oph);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        oph ^= 1;
        tc_fence_after();
        const int32_t e = entries[x * kTileM + row];
        // the row's largest magnitude decides the power of two its fp16 copy is scaled by
        uint32_t v0[32], v1[32];
        float amax = 0.f;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          tmem_ld32(tO + ch * 32, v0);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            amax = max3(amax, fabsf(__uint_as_float(v0[i])), fabsf(__uint_as_float(v0[i + 1])));
        }
        const float inv = 1.f / l;
        const PartialScale ps = partial_scale(amax * inv);
        const float mul = inv * ps.scale;
        // O rows go through this warp's 8 KB of the (now idle) Q tile so that every global
        // store instruction writes whole 128-byte pieces of four rows: 64 columns at a
        // time, rows 144 bytes apart in shared memory (conflict-free both ways).
        unsigned char* stage = smem + x * kTileBytes + (warp & 3) * 8192;
#pragma unroll
        for (int ch = 0; ch < (D + 63) / 64; ++ch) {
          constexpr int kLast = D % 64 == 0 ? 64 : D % 64;      // columns of the last piece (head dim 96: 32)
          const int cols = ch == (D + 63) / 64 - 1 ? kLast : 64;
          tmem_ld32(tO + ch * 64, v0);
          if (cols > 32) tmem_ld32(tO + ch * 64 + 32, v1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (i * 8 < cols) {
              const uint32_t* s8 = i < 4 ? v0 + 8 * i : v1 + 8 * (i - 4);
              *reinterpret_cast<uint4*>(stage + lane * 144 + i * 16) =
                  make_uint4(pack2_half(__uint_as_float(s8[0]) * mul, __uint_as_float(s8[1]) * mul),
                             pack2_half(__uint_as_float(s8[2]) * mul, __uint_as_float(s8[3]) * mul),
                             pack2_half(__uint_as_float(s8[4]) * mul, __uint_as_float(s8[5]) * mul),
                             pack2_half(__uint_as_float(s8[6]) * mul, __uint_as_float(s8[7]) * mul));
            }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3), c16 = lane & 7;
            const int32_t er = __shfl_sync(0xffffffffu, e, rl);
            const uint4 val = *reinterpret_cast<const uint4*>(stage + rl * 144 + c16 * 16);
            if (er >= 0 && c16 * 8 < cols)
              __stcs(reinterpret_cast<uint4*>(a.partial_out + (int64_t)er * D + ch * 64 + c16 * 8), val);
          }
          __syncwarp();
        }
        if (e >= 0) a.partial_lse[e] = make_float2((m_ref + log2f(l)) * 0.6931471805599453f, ps.inv);
        tc_fence_before();
      } else {
        atomicExch(a.status, ST_SOFTMAX);
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

// ---------------------------------------------------------------------------
// head dim 256
//
// One 128-row tile per work item.  Operands keep the shapes of the kernel above: Q, K and V are
// handled as two 128-dim halves ("lo", "hi"); S = Q_lo.K_lo^T + Q_hi.K_hi^T (16 k-steps into one
// accumulator), O_lo += P.V_lo and O_hi += P.V_hi (two 128-column accumulators).
// TMEM columns: S buffers 0-127 and 128-255 (tile g of the CTA uses buffer g & 1), O 256-511.
// Shared memory: Q 64 KB (lo, hi), the K halves in two 32 KB slots, the V halves in two.
// With S double-buffered Q.K^T of tile j+1 runs while the softmax of tile j does.  Per tile the
// tensor core has 2048 cycles of MMAs against about 1700 of softmax, so one softmax warpgroup
// keeps it busy.  Order on the tensor core: QK(0) QK(1) PV(0) QK(2) PV(1) ...; the producer
// requests K and V in that order.  The P.V of a tile may still be executing when the softmax
// of the next tile wants to rescale O: that (rare) path waits for it first.
// Warps 8-11 take no part in the softmax: they gather Q rows and write the hi half of O.
// ---------------------------------------------------------------------------
template <int SB, int H, bool kHalf>
__device__ __forceinline__ void issue_qk_wide(uint32_t tmem, uint32_t dq, uint32_t dk) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    constexpr int kBlock = kHalfBytes >> 4, kTile = kTileBytes >> 4;
    const uint32_t koff = (uint32_t)(H * kTile + (ks >> 2) * kBlock + (ks & 3) * 2);
    mma_ss(tmem + SB * kBN, desc64(dq + koff), desc64(dk + koff), kIdescQK<kHalf>, (H | ks) > 0);
  }
}
template <int SB, int H, bool kHalf>
__device__ __forceinline__ void issue_pv_wide(uint32_t tmem, uint32_t dv, bool first) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    mma_ts(tmem + 256 + H * 128, tmem + SB * kBN + ks * 8,
           desc64(dv + H * (kTileBytes >> 4) + ks * (2048 >> 4)), kIdescPV<kHalf, 128>, (!first) || ks > 0);
}

__device__ __forceinline__ void bar_sync_256() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <bool kHalf>
__global__ void __launch_bounds__(kThreads, 1)
attend_tc5_wide_kernel(const Params p, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const KernelArgs a) {
  constexpr int D = 256;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sQ = smem_u32(smem);                       // lo, hi
  const uint32_t sK = sQ + 2 * kTileBytes;                  // lo, hi
  const uint32_t sV = sK + 2 * kTileBytes;                  // lo, hi
  Ctrl& c = *reinterpret_cast<Ctrl*>(smem + 6 * kTileBytes);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&c.k_full[i]), 1);
      mbar_init(smem_u32(&c.k_empty[i]), 1);
      mbar_init(smem_u32(&c.v_full[i]), 1);
      mbar_init(smem_u32(&c.v_empty[i]), 1);
      mbar_init(smem_u32(&c.s_full[i]), 1);
      mbar_init(smem_u32(&c.p_full[i]), kTileM);
      mbar_init(smem_u32(&c.o_full[i]), 1);
      mbar_init(smem_u32(&c.item_ready[i]), 1);
    }
    c.abort = 0;
    c.n_routed = p.hist > 0 ? a.tile_prefix[p.lists] : 0;
    c.own = own_slot_range(p, a.cu);
    c.n_items = c.n_routed + own_item_count(c.own.n, p.Hq, p.C, kTileM);
    fence_barrier_init();
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&c.tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (p.hist > 0) fill_prefix_cache(c, a.tile_prefix, p.lists, kThreads);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c.tmem_slot;
  Item it;
  // c.o_full[0] completes once per tile, when its P.V has executed; "tile g" counts the CTA's tiles

  if (warp < 4) {
    setmaxnreg_dec<72>();
    uint32_t kt = 0, vt = 0;               // K / V tiles produced (warp 0) or consumed (warp 1) so far
    uint32_t g = 0, gp = 0;                // tiles whose Q.K^T / P.V has been issued (warp 1)
    bool pre_k0 = false, pre_v0 = false;   // producer: K(0) / V(0) of the coming item already requested
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t dq = __shfl_sync(0xffffffffu, desc_lo(sQ, 16), 0);
    const uint32_t dk = __shfl_sync(0xffffffffu, desc_lo(sK, 16), 0);
    const uint32_t dv = __shfl_sync(0xffffffffu, desc_lo(sV, kHalfBytes), 0);
    const uint32_t el = elect_one();
    for (int n = 0;; ++n) {
      if (warp == 2) prefetch_item<kTileM>(p, a, c, n & 1);
      if (!next_item<false, D, kTileM>(a, c, smem, n & 1, it)) break;
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      if (warp == 0 && lane == 0) {
        // both halves of K (V) tile `j` of item `w`, each into its slot; false after a timeout
        auto load_k = [&](const Item& w, int j) -> bool {
          const int tok = w.kv_tok0 + j * kBN;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (!mbar_wait(smem_u32(&c.k_empty[h]), (kt & 1) ^ 1)) return false;
            const uint32_t bar = smem_u32(&c.k_full[h]);
            mbar_expect_tx(bar, kTileBytes);
            tma_load_3d(sK + h * kTileBytes, &tmap_k, bar, h * 128, w.kv_head, tok);
            tma_load_3d(sK + h * kTileBytes + kHalfBytes, &tmap_k, bar, h * 128 + 64, w.kv_head, tok);
          }
          ++kt;
          return true;
        };
        auto load_v = [&](const Item& w, int j) -> bool {
          const int tok = w.kv_tok0 + j * kBN;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (!mbar_wait(smem_u32(&c.v_empty[h]), (vt & 1) ^ 1)) return false;
            const uint32_t bar = smem_u32(&c.v_full[h]);
            mbar_expect_tx(bar, kTileBytes);
            tma_load_3d(sV + h * kTileBytes, &tmap_v, bar, h * 128, w.kv_head, tok);
            tma_load_3d(sV + h * kTileBytes + kHalfBytes, &tmap_v, bar, h * 128 + 64, w.kv_head, tok);
          }
          ++vt;
          return true;
        };
        // in the order the tensor core consumes them: K(0), then K(j + 1), V(j) for every tile j
        bool alive = pre_k0 ? true : load_k(it, 0);
        for (int j = 0; alive && j < ntiles; ++j) {
          if (j + 1 < ntiles) alive = load_k(it, j + 1);
          if (alive && !(j == 0 && pre_v0)) alive = load_v(it, j);
        }
        pre_k0 = pre_v0 = false;
        // K(0) and V(0) of the next item go into the slots the tail of this item frees (K(1)
        // would need a slot that only the next item's own first MMAs free: not before it starts)
        if (alive) {
          const int s1 = (n + 1) & 1;
          alive = mbar_wait(smem_u32(&c.item_ready[s1]), ((n + 1) >> 1) & 1);
          if (alive && !c.done[s1]) {
            const Item nx = c.item[s1];
            alive = load_k(nx, 0);
            pre_k0 = alive;
            if (alive) { alive = load_v(nx, 0); pre_v0 = alive; }
          }
        }
        if (!alive) { atomicExch(a.status, ST_PRODUCER); c.abort = 1; }
      } else if (warp == 1) {
        bool ok = true;
        tc_fence_after();
        // S(g & 1) = Q.K^T for the next K tile
        auto qk = [&]() -> bool {
          if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&c.k_full[0]), kt & 1))) return false;
          tc_fence_after();
          if (el) {
            if (g & 1) issue_qk_wide<1, 0, kHalf>(tm, dq, dk); else issue_qk_wide<0, 0, kHalf>(tm, dq, dk);
            tc_commit(smem_u32(&c.k_empty[0]));
          }
          __syncwarp();
          if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&c.k_full[1]), kt & 1))) return false;
          tc_fence_after();
          if (el) {
            if (g & 1) issue_qk_wide<1, 1, kHalf>(tm, dq, dk); else issue_qk_wide<0, 1, kHalf>(tm, dq, dk);
            tc_commit(smem_u32(&c.k_empty[1]));
            tc_commit(smem_u32(&c.s_full[g & 1]));
          }
          __syncwarp();
          ++kt;
          ++g;
          return true;
        };
        ok = qk();
        if (ok && ntiles > 1) ok = qk();
        for (int j = 0; ok && j < ntiles; ++j) {
          // O += P.V: P of tile gp sits in S buffer gp & 1
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.v_full[0]), vt & 1));
          if (!ok) break;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.p_full[0]), gp & 1));
          if (!ok) break;
          tc_fence_after();
          if (el) {
            if (gp & 1) issue_pv_wide<1, 0, kHalf>(tm, dv, j == 0); else issue_pv_wide<0, 0, kHalf>(tm, dv, j == 0);
            tc_commit(smem_u32(&c.v_empty[0]));
          }
          __syncwarp();
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.v_full[1]), vt & 1));
          if (!ok) break;
          tc_fence_after();
          if (el) {
            if (gp & 1) issue_pv_wide<1, 1, kHalf>(tm, dv, j == 0); else issue_pv_wide<0, 1, kHalf>(tm, dv, j == 0);
            tc_commit(smem_u32(&c.v_empty[1]));
            tc_commit(smem_u32(&c.o_full[0]));
          }
          __syncwarp();
          ++vt;
          ++gp;
          if (j + 2 < ntiles) ok = qk();
        }
        if (!ok && lane == 0) { atomicExch(a.status, ST_MMA); c.abort = 1; }
      }
      __syncwarp();
    }
  } else {
    setmaxnreg_inc<216>();
    const int xg = (warp - 4) >> 2;                      // 0: softmax + lo half of O, 1: hi half of O
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tO = tmem + lane_base + 256;
    const float sl2 = rsqrtf((float)D) * 1.4426950408889634f;
    uint32_t g = 0;                                      // tiles of this CTA before the current one
    for (int n = 0; next_item<true, D, kTileM>(a, c, smem, n & 1, it); ++n) {
      const int32_t* entries = c.entry[n & 1];
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      if (xg == 0) {
        const int qpos = it.tok0 + row;
        const int lim = it.causal ? min(it.kv_len, qpos - it.kv_tok0 + 1) : it.kv_len;
        for (int j = 0; ok && j < ntiles; ++j, ++g) {
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.s_full[g & 1]), (g >> 1) & 1));
          if (!ok) break;
          tc_fence_after();
          const uint32_t tS = tmem + lane_base + (g & 1) * kBN;
          const int key0 = j * kBN;
          const bool masked = key0 + kBN > it.kv_len || (it.causal && it.kv_tok0 + key0 + kBN - 1 > it.tok0);
          // the P.V of tile g - 1 must have executed before O is touched (tile g - 2 is known to have)
          auto wait_pv = [&] {
            if (!mbar_wait(smem_u32(&c.o_full[0]), (g - 1) & 1)) ok = false;
            tc_fence_after();
          };
          if (masked) softmax_row<true, kHalf, D>(tS, tO, j, key0, lim, sl2, m_ref, l, wait_pv);
          else softmax_row<false, kHalf, D>(tS, tO, j, key0, lim, sl2, m_ref, l, wait_pv);
          // keeps the completions of o_full at most one behind, so that a wait on the parity of a
          // tile index can never be answered by an older phase
          if (j > 0 && !mbar_wait(smem_u32(&c.o_full[0]), (g - 1) & 1)) ok = false;
          ok = __all_sync(0xffffffffu, ok);
          tc_fence_before();
          mbar_arrive(smem_u32(&c.p_full[0]));
        }
      } else {
        g += (uint32_t)ntiles;
      }
      bar_sync_256();                                    // the last P has been published
      if (ok) ok = mbar_wait(smem_u32(&c.o_full[0]), (g - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      const int32_t e = entries[row];
      uint32_t v0[32], v1[32];
      if (ok) tc_fence_after();
      if (ok && xg == 0) {
        // the row's largest magnitude over all 256 dims decides the power of two of its fp16 copy
        float amax = 0.f;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          tmem_ld32(tO + ch * 32, v0);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            amax = max3(amax, fabsf(__uint_as_float(v0[i])), fabsf(__uint_as_float(v0[i + 1])));
        }
        const float inv = 1.f / l;
        const PartialScale ps = partial_scale(amax * inv);
        c.row_inv[row] = inv * ps.scale;
        if (e >= 0) a.partial_lse[e] = make_float2((m_ref + log2f(l)) * 0.6931471805599453f, ps.inv);
      }
      bar_sync_256();                                    // the rows' factors are visible to warps 8-11
      if (ok) {
        const float mul = c.row_inv[row];
        // as above: O rows pass through this warp's 8 KB of the idle Q tile; warps 4-7 write
        // dims 0-127, warps 8-11 dims 128-255
        unsigned char* stage = smem + xg * kTileBytes + (warp & 3) * 8192;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          tmem_ld32(tO + xg * 128 + ch * 64, v0);
          tmem_ld32(tO + xg * 128 + ch * 64 + 32, v1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t* s8 = i < 4 ? v0 + 8 * i : v1 + 8 * (i - 4);
            *reinterpret_cast<uint4*>(stage + lane * 144 + i * 16) =
                make_uint4(pack2_half(__uint_as_float(s8[0]) * mul, __uint_as_float(s8[1]) * mul),
                           pack2_half(__uint_as_float(s8[2]) * mul, __uint_as_float(s8[3]) * mul),
                           pack2_half(__uint_as_float(s8[4]) * mul, __uint_as_float(s8[5]) * mul),
                           pack2_half(__uint_as_float(s8[6]) * mul, __uint_as_float(s8[7]) * mul));
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3), c16 = lane & 7;
            const int32_t er = __shfl_sync(0xffffffffu, e, rl);
            const uint4 val = *reinterpret_cast<const uint4*>(stage + rl * 144 + c16 * 16);
            if (er >= 0)
              __stcs(reinterpret_cast<uint4*>(a.partial_out + (int64_t)er * D + xg * 128 + ch * 64 + c16 * 8), val);
          }
          __syncwarp();
        }
        tc_fence_before();
      } else {
        atomicExch(a.status, ST_SOFTMAX);
        c.abort = 1;
      }
    }
  }

  if (c.abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// ---------------------------------------------------------------------------
// small chunks (at most kSmallChunk keys): one 128-row tile per work item, two CTAs per SM
//
// With one or two key tiles per item the kernels above spend most of an item on its hand-over
// (description, Q gather, epilogue: 13-19 thousand cycles for 2-3 thousand of MMA), during which the
// tensor pipe idles.  This variant halves every per-CTA resource - 192 threads (one softmax
// warpgroup, warps 0-3; warp 4 describes the next item and requests K/V tiles, warp 5 issues the
// MMAs), one Q tile, one K and one V stage, 256 TMEM columns (S 0-127, O 128-255), about 110 KB
// of shared memory, 168 registers per thread - so that two CTAs share an SM and one works while
// the other changes items.  Per tile: QK -> softmax -> PV in sequence (S is single-buffered; P
// overwrites it), K(j+1) is requested when QK(j) has executed, V(j+1) when PV(j) has.
// ---------------------------------------------------------------------------
constexpr int kSmallThreads = 192;
constexpr int kSmallPrefix = 2048;

struct SmallCtrl {
  static constexpr int kPrefix = kSmallPrefix;
  uint64_t k_full, k_empty, v_full, v_empty, s_full, p_full, o_full;
  uint64_t item_ready[2];
  uint32_t tmem_slot;
  volatile int32_t abort;
  int32_t n_routed, n_items;
  SlotRange own;
  Item item[2];
  int32_t done[2];
  int64_t qoff[2][kTileM];
  int32_t entry[2][kTileM];
  int32_t prefix_cache[kSmallPrefix];
};
constexpr size_t kSmallSmemBytes = 1024 + 3 * kTileBytes + sizeof(SmallCtrl);
static_assert(2 * (kSmallSmemBytes + 1024) <= 232448, "two CTAs per SM");

template <bool kHalf, int D>
__global__ void __launch_bounds__(kSmallThreads, 2)
attend_tc5_small_kernel(const Params p, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const KernelArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + kTileBytes;
  const uint32_t sV = sK + kTileBytes;
  SmallCtrl& c = *reinterpret_cast<SmallCtrl*>(smem + 3 * kTileBytes);
  constexpr uint32_t kCols = 256;

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&c.k_full), 1);
    mbar_init(smem_u32(&c.k_empty), 1);
    mbar_init(smem_u32(&c.v_full), 1);
    mbar_init(smem_u32(&c.v_empty), 1);
    mbar_init(smem_u32(&c.s_full), 1);
    mbar_init(smem_u32(&c.p_full), kTileM);
    mbar_init(smem_u32(&c.o_full), 1);
    mbar_init(smem_u32(&c.item_ready[0]), 1);
    mbar_init(smem_u32(&c.item_ready[1]), 1);
    c.abort = 0;
    c.n_routed = p.hist > 0 ? a.tile_prefix[p.lists] : 0;
    c.own = own_slot_range(p, a.cu);
    c.n_items = c.n_routed + own_item_count(c.own.n, p.Hq, p.C, kTileM);
    fence_barrier_init();
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&c.tmem_slot), kCols);
    tmem_relinquish();
  }
  if (p.hist > 0) fill_prefix_cache(c, a.tile_prefix, p.lists, kSmallThreads);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c.tmem_slot;

  // Head of item n for every thread: the slot filled by warp 4; warps 0-3 gather the Q rows.  Warp 4
  // does not wait for the gather: it goes on to describe item n + 1 at once (its chain of
  // dependent global loads is as long as an item).
  auto next_item = [&](int n, Item& it) -> bool {
    const int slot = n & 1;
    __syncthreads();
    if (c.done[slot]) return false;
    it = c.item[slot];
    if (warp < 4) {
      constexpr int kChunks = D / 8;
      const int32_t* entry = c.entry[slot];
      const int64_t* qoff = c.qoff[slot];
      const int t = threadIdx.x;
      uint4 val[kChunks];
#pragma unroll
      for (int u = 0; u < kChunks; ++u) {
        const int i = t + u * 128;
        const int r = i / kChunks, ch = i % kChunks;
        val[u] = make_uint4(0, 0, 0, 0);
        if (entry[r] >= 0) val[u] = __ldg(reinterpret_cast<const uint4*>(a.q + qoff[r] + ch * 8));
      }
#pragma unroll
      for (int u = 0; u < kChunks; ++u) {
        const int i = t + u * 128;
        const int r = i / kChunks, ch = i % kChunks;
        const uint32_t dst = (uint32_t)((ch >> 3) * kHalfBytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4));
        *reinterpret_cast<uint4*>(smem + dst) = val[u];
      }
    }
    fence_proxy_async_smem();
    if (warp != 4) asm volatile("bar.sync 1, 160;" ::: "memory");
    return true;
  };
  Item it;

  if (warp >= 4) {
    uint32_t kt = 0, vt = 0;               // K / V tiles produced (warp 4) or consumed (warp 5) so far
    uint32_t pph = 0;                      // p_full phase
    int pre = 0;                           // warp 4: 1 when K(0) and V(0) of the coming item are requested
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t dq = __shfl_sync(0xffffffffu, desc_lo(sQ, 16), 0);
    const uint32_t dk = __shfl_sync(0xffffffffu, desc_lo(sK, 16), 0);
    const uint32_t dv = __shfl_sync(0xffffffffu, desc_lo(sV, kHalfBytes), 0);
    const uint32_t el = elect_one();
    if (warp == 4) prefetch_item<kTileM>(p, a, c, 0);
    for (int n = 0;; ++n) {
      if (!next_item(n, it)) break;
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      if (warp == 4) {
        // K and V tile `j` of item `w`; false after a timeout (lane 0 only)
        auto load_tile = [&](const Item& w, int j) -> bool {
          const int tok = w.kv_tok0 + j * kBN;
          if (!mbar_wait(smem_u32(&c.k_empty), (kt & 1) ^ 1)) return false;
          uint32_t bar = smem_u32(&c.k_full);
          mbar_expect_tx(bar, ((D + 63) / 64) * kHalfBytes);
          tma_load_3d(sK, &tmap_k, bar, 0, w.kv_head, tok);
          if (D > 64) tma_load_3d(sK + kHalfBytes, &tmap_k, bar, 64, w.kv_head, tok);
          ++kt;
          if (!mbar_wait(smem_u32(&c.v_empty), (vt & 1) ^ 1)) return false;
          bar = smem_u32(&c.v_full);
          mbar_expect_tx(bar, ((D + 63) / 64) * kHalfBytes);
          tma_load_3d(sV, &tmap_v, bar, 0, w.kv_head, tok);
          if (D > 64) tma_load_3d(sV + kHalfBytes, &tmap_v, bar, 64, w.kv_head, tok);
          ++vt;
          return true;
        };
        bool alive = true;
        if (lane == 0)
          for (int j = pre; alive && j < ntiles; ++j) alive = load_tile(it, j);
        pre = 0;
        __syncwarp();
        // the next item: described by the whole warp, its first tiles requested as soon as the
        // stages free up
        const int s1 = (n + 1) & 1;
        prefetch_item<kTileM>(p, a, c, s1);
        if (lane == 0 && alive && !c.done[s1]) {
          const Item nx = c.item[s1];
          alive = load_tile(nx, 0);
          pre = alive ? 1 : 0;
        }
        pre = __shfl_sync(0xffffffffu, pre, 0);
        if (lane == 0 && !alive) { atomicExch(a.status, ST_PRODUCER); c.abort = 1; }
      } else {
        bool ok = true;
        tc_fence_after();
        for (int j = 0; ok && j < ntiles; ++j) {
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.k_full), kt & 1));
          if (!ok) break;
          tc_fence_after();
          if (el) {
            issue_qk<0, 0, kHalf, D>(tm, dq, dk);
            tc_commit(smem_u32(&c.s_full));
            tc_commit(smem_u32(&c.k_empty));
          }
          __syncwarp();
          ++kt;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.v_full), vt & 1));
          if (!ok) break;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.p_full), pph));
          if (!ok) break;
          pph ^= 1;
          tc_fence_after();
          if (el) {
            // O in columns 128-255: the P.V of the kernels above with the accumulator moved
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              mma_ts(tm + 128, tm + ks * 8, desc64(dv + ks * (2048 >> 4)), kIdescPV<kHalf, D>, j > 0 || ks > 0);
            tc_commit(smem_u32(&c.v_empty));
            if (j + 1 == ntiles) tc_commit(smem_u32(&c.o_full));
          }
          __syncwarp();
          ++vt;
        }
        if (!ok && lane == 0) { atomicExch(a.status, ST_MMA); c.abort = 1; }
      }
      __syncwarp();
    }
  } else {
    const int row = warp * 32 + lane;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const uint32_t tS = tmem + lane_base;
    const uint32_t tO = tmem + lane_base + 128;
    const float sl2 = rsqrtf((float)D) * 1.4426950408889634f;
    uint32_t sph = 0, oph = 0;
    for (int n = 0; next_item(n, it); ++n) {
      const int32_t* entries = c.entry[n & 1];
      const int ntiles = (it.kv_len + kBN - 1) / kBN;
      const int qpos = it.tok0 + row;
      const int lim = it.causal ? min(it.kv_len, qpos - it.kv_tok0 + 1) : it.kv_len;
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; ok && j < ntiles; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.s_full), sph));
        if (!ok) break;
        sph ^= 1;
        tc_fence_after();
        const int key0 = j * kBN;
        const bool masked = key0 + kBN > it.kv_len || (it.causal && it.kv_tok0 + key0 + kBN - 1 > it.tok0);
        if (masked) softmax_row<true, kHalf, D>(tS, tO, j, key0, lim, sl2, m_ref, l, [] {});
        else softmax_row<false, kHalf, D>(tS, tO, j, key0, lim, sl2, m_ref, l, [] {});
        tc_fence_before();
        mbar_arrive(smem_u32(&c.p_full));
      }
      if (ok) ok = mbar_wait(smem_u32(&c.o_full), oph);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        oph ^= 1;
        tc_fence_after();
        const int32_t e = entries[row];
        uint32_t v0[32], v1[32];
        float amax = 0.f;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          tmem_ld32(tO + ch * 32, v0);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            amax = max3(amax, fabsf(__uint_as_float(v0[i])), fabsf(__uint_as_float(v0[i + 1])));
        }
        const float inv = 1.f / l;
        const PartialScale ps = partial_scale(amax * inv);
        const float mul = inv * ps.scale;
        unsigned char* stage = smem + warp * 8192;            // this warp's part of the idle Q tile
#pragma unroll
        for (int ch = 0; ch < (D + 63) / 64; ++ch) {
          constexpr int kLast = D % 64 == 0 ? 64 : D % 64;
          const int cols = ch == (D + 63) / 64 - 1 ? kLast : 64;
          tmem_ld32(tO + ch * 64, v0);
          if (cols > 32) tmem_ld32(tO + ch * 64 + 32, v1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (i * 8 < cols) {
              const uint32_t* s8 = i < 4 ? v0 + 8 * i : v1 + 8 * (i - 4);
              *reinterpret_cast<uint4*>(stage + lane * 144 + i * 16) =
                  make_uint4(pack2_half(__uint_as_float(s8[0]) * mul, __uint_as_float(s8[1]) * mul),
                             pack2_half(__uint_as_float(s8[2]) * mul, __uint_as_float(s8[3]) * mul),
                             pack2_half(__uint_as_float(s8[4]) * mul, __uint_as_float(s8[5]) * mul),
                             pack2_half(__uint_as_float(s8[6]) * mul, __uint_as_float(s8[7]) * mul));
            }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3), c16 = lane & 7;
            const int32_t er = __shfl_sync(0xffffffffu, e, rl);
            const uint4 val = *reinterpret_cast<const uint4*>(stage + rl * 144 + c16 * 16);
            if (er >= 0 && c16 * 8 < cols)
              __stcs(reinterpret_cast<uint4*>(a.partial_out + (int64_t)er * D + ch * 64 + c16 * 8), val);
          }
          __syncwarp();
        }
        if (e >= 0) a.partial_lse[e] = make_float2((m_ref + log2f(l)) * 0.6931471805599453f, ps.inv);
        tc_fence_before();
      } else {
        atomicExch(a.status, ST_SOFTMAX);
        c.abort = 1;
      }
    }
  }

  if (c.abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, kCols);
}

// One warp waits, with the same bounded wait every role of the dense stage uses, on a barrier
// nobody ever arrives on: the wait gives up after `limit_ns`, the status word is set like the
// kernel would set it, and the warp returns.  Lets a test see the give-up path without a fault.
__global__ void bounded_wait_probe_kernel(int32_t* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (!mbar_wait(smem_u32(&bar), 0, limit_ns) && threadIdx.x == 0) atomicExch(status, ST_SOFTMAX);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

}  // namespace

// [T, H, D] 16-bit tensor with element strides (st, sh, 1): boxes of `box_rows` tokens x `box_heads` heads x
// 64 dims, 128-byte swizzle; elements outside the tensor read as zero
bool make_tile_map(CUtensorMap* m, bool fp16, int D, const __nv_bfloat16* base, int64_t T, int H, int64_t st,
                   int64_t sh, int box_heads, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T};
  const cuuint64_t strides[2] = {(cuuint64_t)sh * 2, (cuuint64_t)st * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool make_kv_map(CUtensorMap* m, bool fp16, int D, const __nv_bfloat16* base, int64_t T, int Hkv, int64_t st, int64_t sh,
                 int box_rows) {
  return make_tile_map(m, fp16, D, base, T, Hkv, st, sh, 1, box_rows);
}

cudaError_t launch_bounded_wait_probe(int32_t* status, unsigned long long limit_ns, cudaStream_t st) {
  bounded_wait_probe_kernel<<<1, 32, 0, st>>>(status, limit_ns);
  return cudaGetLastError();
}

cudaError_t launch_attend_tc5(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                              const __nv_bfloat16* v, const int32_t* cu, const int32_t* list_counts,
                              const int32_t* list_offsets, const int32_t* tile_prefix,
                              const int32_t* row_list, __half* partial_out, float2* partial_lse,
                              int32_t* work_counter, int32_t* status, cudaStream_t st) {
  CUtensorMap mk, mv;
  if (!make_kv_map(&mk, p.fp16 != 0, p.D, k, p.T, p.Hkv, p.sk_t, p.sk_h, kBN) || !make_kv_map(&mv, p.fp16 != 0, p.D, v, p.T, p.Hkv, p.sv_t, p.sv_h, kBN))
    return cudaErrorNotSupported;
  if (p.D != 64 && p.D != 96 && p.D != 128 && p.D != 256) return cudaErrorInvalidValue;
  auto kernel = p.D == 256 ? (p.fp16 ? attend_tc5_wide_kernel<true> : attend_tc5_wide_kernel<false>)
              : p.D == 128 ? (p.fp16 ? attend_tc5_kernel<true, 128> : attend_tc5_kernel<false, 128>)
              : p.D == 96  ? (p.fp16 ? attend_tc5_kernel<true, 96> : attend_tc5_kernel<false, 96>)
                           : (p.fp16 ? attend_tc5_kernel<true, 64> : attend_tc5_kernel<false, 64>);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const KernelArgs args{q, cu, list_counts, list_offsets, tile_prefix, row_list, partial_out, partial_lse,
                        work_counter, status};
  if (tc5_small_items(p.D, p.C)) {
    auto small = p.D == 128 ? (p.fp16 ? attend_tc5_small_kernel<true, 128> : attend_tc5_small_kernel<false, 128>)
               : p.D == 96  ? (p.fp16 ? attend_tc5_small_kernel<true, 96> : attend_tc5_small_kernel<false, 96>)
                            : (p.fp16 ? attend_tc5_small_kernel<true, 64> : attend_tc5_small_kernel<false, 64>);
    e = cudaFuncSetAttribute(small, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmallSmemBytes);
    if (e != cudaSuccess) return e;
    small<<<2 * sms, kSmallThreads, kSmallSmemBytes, st>>>(p, mk, mv, args);
    return cudaGetLastError();
  }
  kernel<<<sms, kThreads, kSmemBytes, st>>>(p, mk, mv, args);
  return cudaGetLastError();
}

}  // namespace moba
