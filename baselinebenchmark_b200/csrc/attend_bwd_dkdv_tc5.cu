// dK and dV of the MoBA dense stage on the Blackwell tensor path (tcgen05.mma, accumulators
// in tensor memory).
//
// Replaces, for the training path of the reference, the dk/dv kernel of
//   _triton_varlen_backward   backends/_mthreads/ops/moba/attention.py:163-369
// and the scatter of routed gradients (routing.py:1776-1896), as called for both branches by
// MixedAttention.backward (parallel.py:171-236):
//   p_ij = exp(s_ij * scale - lse_i),  dS_ij = p_ij (dO_i . V_j - delta_i),
//   dV_j = sum_i p_ij dO_i,  dK_j = scale * sum_i dS_ij Q_i
// over the (query, key) pairs the forward attends.
//
// Key-stationary: a unit is 128 keys of one (chunk, kv head); its K and V tiles stay in shared
// memory (TMA) and dK, dV stay in tensor memory while the CTA visits every query row that
// attends the keys - the routed list of the chunk, then the chunk's own rows of every query
// head of the group - in steps of 64 rows brought into a four-stage ring.  A step of own-chunk
// rows is a 64-token box of q / dO (TMA).  The rows of a routed list are scattered over q and
// dO and are read once per 128-key tile of the chunk: with chunks of kPackMinTiles tiles or
// more a pre-pass (pack_rows_kernel) copies them, in list order, into two packed arrays
// [entries, D] and a step is a 64-row box of those (gathered with cp.async every time, the
// 16-byte copies kept the load/store pipe busier than the tensor pipe); with shorter chunks the
// copy would cost more than it saves and the rows are gathered with cp.async.  Per step
//   S^T  = K . Q^T      (128 keys x 64 rows, operands in shared memory)
//   dP^T = V . dO^T     (128 x 64)
//   one thread per key turns them into P^T and dS^T (input dtype) in tensor memory
//   dV  += P^T . dO     (128 x D, P^T read from tensor memory, dO as the MN-major operand)
//   dK  += dS^T . Q     (128 x D)
// No atomics: a key's gradient is written once.  The order of the rows of a routed list is
// the compaction's (unspecified), so dK and dV vary in their last bits from run to run.
//
// Warp roles (384 threads): warp 0 lane 0 loads K/V by TMA, warp 1 issues the MMAs and owns
// the TMEM allocation, warps 2-3 describe the rows of the coming steps (LSE, delta, token), warps
// 4-7 handle the even steps (S buffer 0) and write dK, warps 8-11 the odd steps (S buffer 1) and
// write dV; after a step the group brings in the Q / dO rows of the step three ahead (one thread
// requests the boxes, or all 128 gather).
// TMEM columns: buffer X: S^T 128X..+63 (P^T, 16-bit, over the first 32), dP^T 128X+64..+127
// (dS^T over its first 32); dK 256.., dV 384...
// Every wait is bounded; a wait that gives up sets a status word, the CTAs stop drawing units
// and a small kernel launched behind this one overwrites dK and dV with NaN.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace moba {

bool make_kv_map(CUtensorMap* m, bool fp16, int D, const __nv_bfloat16* base, int64_t T, int Hkv, int64_t st,
                 int64_t sh, int box_rows);
bool make_tile_map(CUtensorMap* m, bool fp16, int D, const __nv_bfloat16* base, int64_t T, int H, int64_t st,
                   int64_t sh, int box_heads, int box_rows);

namespace {

using namespace ptx;

constexpr int kThreads = 384;
constexpr int kKeys = 128;                    // keys per unit
constexpr int kStep = 64;                     // rows per step
constexpr int kStages = 4;
// Chunks of at least this many 128-key tiles have their routed rows packed.  Measured backward of
// 32768 tokens x 32/8 heads, packed against gathered: 4 tiles 21.7 / 20.1 ms, 8 tiles 17.0 / 17.2,
// 16 tiles 26.1 / 27.3, 32 tiles (config 2) 33.5 / 35.8.
constexpr int kPackMinTiles = 8;
constexpr int kKvBlockBytes = kKeys * 64 * 2; // [128 keys][64 dims]
constexpr int kKvTileBytes = 2 * kKvBlockBytes;
constexpr int kRowBlockBytes = kStep * 64 * 2;  // [64 rows][64 dims]
constexpr int kRowTileBytes = 2 * kRowBlockBytes;
constexpr uint32_t kTmemCols = 512;

template <bool kHalf> constexpr uint32_t kIdescST = idesc_16_f32(kHalf, 128, kStep, 0, 0);
template <bool kHalf, int D> constexpr uint32_t kIdescAcc = idesc_16_f32(kHalf, 128, D, 0, 1);
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);

enum { ST_PRODUCER = 21, ST_MMA = 22, ST_ROWS = 23, ST_GATHER = 24 };

struct Ctrl {
  uint64_t kv_full, acc_full;
  uint64_t row_full[kStages], row_empty[kStages], meta_full[kStages];
  uint64_t s_full[2], p_full[2];
  uint32_t tmem_slot;
  volatile int32_t abort;
  int32_t unit;
  alignas(16) float2 meta[kStages][kStep];     // {lse * log2 e, delta} of the row; {0, 0}: no row
  alignas(16) int32_t tok[kStages][kStep];                 // query token of an own-chunk row (causal limit), else INT_MAX
  int32_t ent[4][kStep];                       // routed-list entries of the steps ahead (0: no row)
  int64_t qoff[kStages][kStep];                // gathered routed rows: element offset of the row in q, -1: no row
  int32_t grow[kStages][kStep];                // ... and row index t * Hq + h
};

constexpr size_t kSmemBytes = 1024 + 2 * kKvTileBytes + kStages * 2 * kRowTileBytes + sizeof(Ctrl);
static_assert(kSmemBytes <= 232448, "shared memory of one CTA");

struct KernelArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* dout;                   // contiguous [T, Hq, D]
  const int32_t* cu;
  const int32_t* list_counts;
  const int32_t* list_offsets;
  const int32_t* row_list;
  const float* lse2;
  const float* delta;
  __nv_bfloat16* dk;                           // contiguous [T, Hkv, D]
  __nv_bfloat16* dv;
  int32_t* work_counter;
  int32_t* status;
  int packed;                                  // routed rows come from the packed arrays (TMA), else gathered
};

// What every thread derives from the unit index.
struct Unit {
  int l, kvh, key0, nkeys, end;                // list, kv head, first key token, keys in the tile, chunk end
  int n_routed, routed_steps, own_steps, steps;
  int64_t list_off;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool pred) {
  const int n = pred ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
// arrives on the mbarrier once every cp.async this thread has issued so far has landed
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Row `r` of own-chunk step `i` of the unit: the global row index t * Hq + h (or -1) and its
// token, which limits the keys it sees.
__device__ __forceinline__ void own_row(const Params& p, const Unit& u, int i, int r, int& row, int& tokq) {
  const int o = i - u.routed_steps;
  const int hl = o / u.own_steps, ot = o - hl * u.own_steps;
  const int tok = u.key0 + ot * kStep + r;
  row = -1;
  tokq = 0x7fffffff;
  if (tok < u.end) { row = (tok - p.win_lo) * p.Hq + (u.kvh * p.G + hl); tokq = tok; }
}

// Optional cycle accounting (build with -DMOBA_DKDV_TRACE): sums over all CTAs are added to
// 64-bit counters at status + 64 ints; status must then be followed by zeroed memory.
#ifdef MOBA_DKDV_TRACE
#define TR_T0(var) const long long var = clock64()
#define TR_BASE(args) reinterpret_cast<unsigned long long*>(((uintptr_t)((args).status + 64) + 7) & ~(uintptr_t)7)
#define TR_ADD(args, slot, t0) atomicAdd(TR_BASE(args) + (slot), (unsigned long long)(clock64() - (t0)))
#define TR_COUNT(args, slot, n) atomicAdd(TR_BASE(args) + (slot), (unsigned long long)(n))
#else
#define TR_T0(var)
#define TR_ADD(args, slot, t0)
#define TR_COUNT(args, slot, n)
#endif

#ifndef MOBA_BWD_POLY_PAIRS
#define MOBA_BWD_POLY_PAIRS 2
#endif
constexpr int kPolyPairs = MOBA_BWD_POLY_PAIRS;

// One step of one key: S^T and dP^T (64 fp32 columns each, one per query row of the step) ->
// P^T over the first 32 columns of S^T, dS^T over the first 32 columns of dP^T (input dtype).
//   p = 2^(s * scale * log2 e - lse_row * log2 e),  dS = p * (dP - delta_row)
// `meta[row]` = {lse * log2 e, delta}.  Rows that do not exist carry {0, 0} and zero Q / dO rows:
// their p is 1 but multiplies a zero dO row, their dS is 1 * (0 - 0).  Masked steps (own-chunk
// rows around the diagonal) also compare the key token with the row's token.
template <bool kMasked, bool kHalf>
__device__ __forceinline__ void ps_row(uint32_t tS, const float2* meta, const int32_t* tok, int key_tok, bool key_ok,
                                       float sl2) {
  uint32_t s[64], g[64];
  tmem_ld64(tS, s);
  tmem_ld64(tS + 64, g);
  tmem_wait_ld();
  const uint64_t scale2 = pack2(sl2, sl2);
#pragma unroll
  for (int ch = 0; ch < 2; ++ch) {
    uint32_t pp[16], pd[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = ch * 32 + 2 * i;
      const float4 m = *reinterpret_cast<const float4*>(meta + e);      // {-lse2, delta} of rows e, e + 1
      uint64_t x = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2,
                        pack2(m.x, m.z) ^ 0x8000000080000000ull);
      uint64_t pr;
      if (kMasked) {
        const int2 t = *reinterpret_cast<const int2*>(tok + e);
        const float x0 = key_tok <= t.x ? lo2(x) : -INFINITY, x1 = key_tok <= t.y ? hi2(x) : -INFINITY;
        pr = pack2(ex2_approx(x0), ex2_approx(x1));
      } else if ((i & 7) < kPolyPairs) {
        pr = ex2_poly2(x);
      } else {
        pr = pack2(ex2_approx(lo2(x)), ex2_approx(hi2(x)));
      }
      const uint64_t d = mul2(pr, sub2(pack2(__uint_as_float(g[e]), __uint_as_float(g[e + 1])), pack2(m.y, m.w)));
      pp[i] = key_ok ? pack2_16<kHalf>(lo2(pr), hi2(pr)) : 0u;
      pd[i] = key_ok ? pack2_16<kHalf>(lo2(d), hi2(d)) : 0u;
    }
    tmem_st16(tS + ch * 16, pp);
    tmem_st16(tS + 64 + ch * 16, pd);
  }
  tmem_wait_st();
}

// Low word of a shared-memory descriptor (128-byte swizzle): start address >> 4 | (leading
// byte offset >> 4) << 16; the high word is kDescHi.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}

// S^T = K . Q^T and dP^T = V . dO^T of one step into S buffer column `xcol`; `dqs`, `dgs`: the
// stage's Q and dO tiles as K-major operands.
template <bool kHalf, int D>
__device__ __forceinline__ void issue_st(uint32_t tm, uint32_t xcol, uint32_t dk, uint32_t dv, uint32_t dqs,
                                         uint32_t dgs) {
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint32_t ao = (uint32_t)((ks >> 2) * (kKvBlockBytes >> 4) + (ks & 3) * 2);
    const uint32_t bo = (uint32_t)((ks >> 2) * (kRowBlockBytes >> 4) + (ks & 3) * 2);
    mma_ss_lo<kDescHi>(tm + xcol, dk + ao, dqs + bo, kIdescST<kHalf>, ks > 0);
  }
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint32_t ao = (uint32_t)((ks >> 2) * (kKvBlockBytes >> 4) + (ks & 3) * 2);
    const uint32_t bo = (uint32_t)((ks >> 2) * (kRowBlockBytes >> 4) + (ks & 3) * 2);
    mma_ss_lo<kDescHi>(tm + xcol + 64, dv + ao, dgs + bo, kIdescST<kHalf>, ks > 0);
  }
}
// dV += P^T . dO and dK += dS^T . Q of one step; `dgt`, `dqt`: the stage's dO and Q tiles as
// MN-major operands (64-dim blocks 8 KB apart, 16 rows per k-step).
template <bool kHalf, int D>
__device__ __forceinline__ void issue_acc(uint32_t tm, uint32_t xcol, uint32_t dgt, uint32_t dqt, bool first) {
#pragma unroll
  for (int ks = 0; ks < kStep / 16; ++ks) {
    mma_ts_lo<kDescHi>(tm + 384, tm + xcol + ks * 8, dgt + ks * (2048 >> 4), kIdescAcc<kHalf, D>, (!first) || ks > 0);
    mma_ts_lo<kDescHi>(tm + 256, tm + xcol + 64 + ks * 8, dqt + ks * (2048 >> 4), kIdescAcc<kHalf, D>,
                       (!first) || ks > 0);
  }
}

// Draws units until one has keys (all threads take part: two block barriers per draw).
// Returns false when the queue is empty or the kernel is aborting.
__device__ __forceinline__ bool next_unit(const Params& p, const KernelArgs& a, Ctrl& c, int key_tiles,
                                          int64_t n_units, Unit& u) {
  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) c.unit = c.abort ? 0x7fffffff : atomicAdd(a.work_counter, 1);
    __syncthreads();
    const int64_t idx = c.unit;
    if (idx >= n_units) return false;
    u.l = (int)(idx / key_tiles);
    const int kt = (int)(idx - (int64_t)u.l * key_tiles);
    const int slot = u.l / p.Hkv;
    u.kvh = u.l - slot * p.Hkv;
    const int b = slot / p.mc, jc = slot - b * p.mc;
    const Slot sl = slot_of(a.cu, b, jc, p.C);
    u.key0 = sl.start + kt * kKeys;
    u.end = sl.end;
    if (u.key0 >= sl.end) continue;
    u.nkeys = min(kKeys, sl.end - u.key0);
    u.n_routed = p.hist > 0 ? a.list_counts[u.l] : 0;
    u.list_off = p.hist > 0 ? a.list_offsets[u.l] : 0;
    u.routed_steps = (u.n_routed + kStep - 1) / kStep;
    u.own_steps = (sl.end - u.key0 + kStep - 1) / kStep;       // tokens key0 .. end see at least one key
    u.steps = u.routed_steps + u.own_steps * p.G;
    return true;
  }
}

template <bool kHalf, int D>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dkdv_tc5_kernel(const Params p, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_g, const __grid_constant__ CUtensorMap tmap_qp,
                    const __grid_constant__ CUtensorMap tmap_gp, const KernelArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sK = smem_u32(smem);
  const uint32_t sV = sK + kKvTileBytes;
  const uint32_t sRows = sV + kKvTileBytes;                 // stage s: Q tile, dO tile
  Ctrl& c = *reinterpret_cast<Ctrl*>(smem + 2 * kKvTileBytes + kStages * 2 * kRowTileBytes);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&c.kv_full), 1);
    mbar_init(smem_u32(&c.acc_full), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&c.row_full[i]), 64 + kKeys);     // lse / delta of 64 rows + the 128 threads of the group that copies
      mbar_init(smem_u32(&c.row_empty[i]), 1);
      mbar_init(smem_u32(&c.meta_full[i]), 64);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&c.s_full[i]), 1);
      mbar_init(smem_u32(&c.p_full[i]), kKeys);
    }
    c.abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_g);
    prefetch_tmap(&tmap_qp);
    prefetch_tmap(&tmap_gp);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&c.tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c.tmem_slot;

  const int key_tiles = (p.C + kKeys - 1) / kKeys;
  const int64_t n_units = p.lists * key_tiles;
  const float scale = rsqrtf((float)D);
  const float sl2 = scale * 1.4426950408889634f;
  TR_T0(t_kernel);
  if (warp < 4) {
    setmaxnreg_dec<72>();
    uint32_t g0 = 0;                       // steps of the units this CTA has finished
    uint32_t nu = 0;                       // units this CTA has finished
    Unit u;
    while (next_unit(p, a, c, key_tiles, n_units, u)) {
    if (warp == 0) {
      // ------------------------------------------------ K and V of the unit
      if (lane == 0) {
        const uint32_t bar = smem_u32(&c.kv_full);
        mbar_expect_tx(bar, 2 * ((D + 63) / 64) * kKvBlockBytes);
        tma_load_3d(sK, &tmap_k, bar, 0, u.kvh, u.key0);
        if (D > 64) tma_load_3d(sK + kKvBlockBytes, &tmap_k, bar, 64, u.kvh, u.key0);
        tma_load_3d(sV, &tmap_v, bar, 0, u.kvh, u.key0);
        if (D > 64) tma_load_3d(sV + kKvBlockBytes, &tmap_v, bar, 64, u.kvh, u.key0);
      }
    } else if (warp == 1) {
      // ------------------------------------------------ MMA issuer (warp convergent, one lane issues)
      const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
      const uint32_t dk = __shfl_sync(0xffffffffu, desc_lo(sK, 16), 0);
      const uint32_t dv = __shfl_sync(0xffffffffu, desc_lo(sV, 16), 0);
      const uint32_t dq = __shfl_sync(0xffffffffu, desc_lo(sRows, 16), 0);                      // K-major views
      const uint32_t dg = __shfl_sync(0xffffffffu, desc_lo(sRows + kRowTileBytes, 16), 0);
      const uint32_t dqt = __shfl_sync(0xffffffffu, desc_lo(sRows, kRowBlockBytes), 0);         // MN-major views
      const uint32_t dgt = __shfl_sync(0xffffffffu, desc_lo(sRows + kRowTileBytes, kRowBlockBytes), 0);
      const uint32_t el = elect_one();
      constexpr uint32_t kStageDesc = (2 * kRowTileBytes) >> 4;
      bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.kv_full), nu & 1));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.row_full[g0 & 3]), (g0 >> 2) & 1));
      if (ok) {
        fence_proxy_async_smem();
        tc_fence_after();
        if (el) {
          issue_st<kHalf, D>(tm, (g0 & 1) * 128, dk, dv, dq + (g0 & 3) * kStageDesc, dg + (g0 & 3) * kStageDesc);
          tc_commit(smem_u32(&c.s_full[g0 & 1]));
        }
        __syncwarp();
      }
      for (int i = 0; ok && i < u.steps; ++i) {
        const uint32_t gi = g0 + i, g1 = gi + 1;
        if (i + 1 < u.steps) {
          TR_T0(t_r);
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.row_full[g1 & 3]), (g1 >> 2) & 1));
          if (!ok) break;
          if (lane == 0) TR_ADD(a, 0, t_r);
          fence_proxy_async_smem();
          tc_fence_after();
          if (el) {
            issue_st<kHalf, D>(tm, (g1 & 1) * 128, dk, dv, dq + (g1 & 3) * kStageDesc, dg + (g1 & 3) * kStageDesc);
            tc_commit(smem_u32(&c.s_full[g1 & 1]));
          }
          __syncwarp();
        }
        TR_T0(t_p);
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.p_full[gi & 1]), (gi >> 1) & 1));
        if (!ok) break;
        if (lane == 0) TR_ADD(a, 1, t_p);
        tc_fence_after();
        if (el) {
          issue_acc<kHalf, D>(tm, (gi & 1) * 128, dgt + (gi & 3) * kStageDesc, dqt + (gi & 3) * kStageDesc, i == 0);
          tc_commit(smem_u32(&c.row_empty[gi & 3]));
          if (i + 1 == u.steps) tc_commit(smem_u32(&c.acc_full));
        }
        __syncwarp();
      }
      if (!ok && lane == 0) { atomicExch(a.status, ST_MMA); c.abort = 1; }
      if (lane == 0) TR_COUNT(a, 6, u.steps);
    } else {
      // ------------------------------------------------ warps 2-3: describe the rows of each step (32 rows each)
      const int w = warp - 2, r = w * 32 + lane;
      // Nothing in the loop waits for a global load: the list entries of step i + 3 travel into a
      // small ring with the copies of step i (cp.async), the LSE and delta of a row go straight
      // into the stage's meta array the same way.  A routed entry is row * NP + rank + 1, never 0:
      // the zero a predicated-off copy leaves means "no row".
      auto request_entries = [&](int i) {
        if (i < u.routed_steps) {
          const int j = i * kStep + r;
          const bool in = j < u.n_routed;
          cp_async4(smem_u32(&c.ent[i & 3][r]), a.row_list + u.list_off + (in ? j : 0), in);
        }
      };
      request_entries(0);
      request_entries(1);
      request_entries(2);
      cp_async_commit();
      cp_async_wait<0>();
      bool ok = true;
      for (int i = 0; i < u.steps; ++i) {
        TR_T0(t_c);
        cp_async_wait<2>();                          // group i - 3 has landed: the entries of step i
        if (threadIdx.x == 64) TR_ADD(a, 5, t_c);
        int row = -1, tokq = 0x7fffffff;
        if (i < u.routed_steps) {
          const int ent = c.ent[i & 3][r];
          if (ent > 0) row = ent / p.NP;
        } else {
          own_row(p, u, i, r, row, tokq);
        }
        const uint32_t gi = g0 + i, st = gi & 3;
        TR_T0(t_e);
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.row_empty[st]), ((gi >> 2) & 1) ^ 1));
        if (!ok) break;
        if (threadIdx.x == 64) TR_ADD(a, 4, t_e);
        TR_T0(t_i);
        {
          c.tok[st][r] = tokq;
          if (!a.packed && i < u.routed_steps) {
            int64_t off = -1;
            if (row >= 0) {
              const int t = row / p.Hq;
              off = (int64_t)t * p.sq_t + (int64_t)(row - t * p.Hq) * p.sq_h;
            }
            c.qoff[st][r] = off;
            c.grow[st][r] = row;
          }
          // A place of the step without a row still holds data in the stage (the box goes on into
          // the next list, the next chunk, or the zero rows behind the last list): an LSE of
          // +inf makes its p = 2^(s - inf) = 0, and with it its share of dV and dS.
          if (row >= 0) {
            cp_async4(smem_u32(&c.meta[st][r].x), a.lse2 + row, true);
            cp_async4(smem_u32(&c.meta[st][r].y), a.delta + row, true);
          } else {
            c.meta[st][r] = make_float2(INFINITY, 0.f);
          }
        }
        // lse and delta travel asynchronously and count on the stage's barrier when they land;
        // the offsets are there now: the row threads may start copying the rows
        mbar_arrive(smem_u32(&c.meta_full[st]));
        cp_async_arrive(smem_u32(&c.row_full[st]));
        request_entries(i + 3);
        cp_async_commit();
        if (threadIdx.x == 64) TR_ADD(a, 9, t_i);
      }
      cp_async_wait<0>();
      if (!ok && lane == 0) { atomicExch(a.status, ST_GATHER); c.abort = 1; }
    }
      g0 += (uint32_t)u.steps;
      ++nu;
    }
  } else {
    setmaxnreg_inc<216>();
    uint32_t g0 = 0, nu = 0;
    Unit u;
    while (next_unit(p, a, c, key_tiles, n_units, u)) {
      // ------------------------------------------------ warps 4-11: one thread per key
      const int x = (warp - 4) >> 2;                       // S buffer and parity of the steps handled
      const int key = (warp & 3) * 32 + lane;              // key inside the tile = TMEM lane
      const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
      const uint32_t tS = tmem + lane_base + x * 128;
      const bool key_ok = key < u.nkeys;
      const int key_tok = u.key0 + key;
      bool ok = true;
      // The Q and dO rows of step j: 64-row boxes requested by one thread of the group.  It first
      // waits for the step's description, which the describing warps only write once the stage
      // is free again.
      auto copy_rows = [&](int j) -> bool {
        if (j >= u.steps) return true;
        const uint32_t gj = g0 + j, sj = gj & 3;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&c.meta_full[sj]), (gj >> 2) & 1))) return false;
        if (!a.packed && j < u.routed_steps) {
          // a warp takes 16 rows of Q and the same 16 rows of dO; an instruction covers whole rows
          // (D / 8 lanes per row), so every 32-byte sector it asks for is used in full
          constexpr int kChunks = D / 8, kRowsPerInstr = 32 / kChunks;
          const int ch = lane % kChunks;
          const uint32_t qb = sRows + sj * 2 * kRowTileBytes + (ch >> 3) * kRowBlockBytes, gb = qb + kRowTileBytes;
          if (lane / kChunks < kRowsPerInstr) {                // head dim 96: 24 of the 32 lanes copy
#pragma unroll
            for (int it = 0; it < 16 / kRowsPerInstr; ++it) {
              const int rr = (warp & 3) * 16 + it * kRowsPerInstr + lane / kChunks;
              const int64_t off = c.qoff[sj][rr];
              const bool valid = off >= 0;
              const uint32_t dst = (uint32_t)(rr * 128 + (((ch & 7) ^ (rr & 7)) << 4));
              cp_async16(qb + dst, a.q + (valid ? off : 0) + ch * 8, valid);
              cp_async16(gb + dst, a.dout + (valid ? (int64_t)c.grow[sj][rr] * D : 0) + ch * 8, valid);
            }
          }
          cp_async_arrive(smem_u32(&c.row_full[sj]));
        } else if ((warp & 3) != 0 || lane != 0) {
          mbar_arrive(smem_u32(&c.row_full[sj]));
        } else {
          const uint32_t bar = smem_u32(&c.row_full[sj]);
          const uint32_t qb = sRows + sj * 2 * kRowTileBytes, gb = qb + kRowTileBytes;
          mbar_expect_tx(bar, 2 * ((D + 63) / 64) * kRowBlockBytes);
          if (j < u.routed_steps) {
            const int pos = (int)u.list_off + j * kStep;
#pragma unroll
            for (int blk = 0; blk < (D + 63) / 64; ++blk) {
              tma_load_3d(qb + blk * kRowBlockBytes, &tmap_qp, bar, blk * 64, 0, pos);
              tma_load_3d(gb + blk * kRowBlockBytes, &tmap_gp, bar, blk * 64, 0, pos);
            }
          } else {
            const int o = j - u.routed_steps;
            const int hl = o / u.own_steps, ot = o - hl * u.own_steps;
            const int tok = u.key0 + ot * kStep, head = u.kvh * p.G + hl;
#pragma unroll
            for (int blk = 0; blk < (D + 63) / 64; ++blk) {
              tma_load_3d(qb + blk * kRowBlockBytes, &tmap_q, bar, blk * 64, head, tok);
              tma_load_3d(gb + blk * kRowBlockBytes, &tmap_g, bar, blk * 64, head, tok);
            }
          }
        }
        return true;
      };
      const int first = ((g0 & 1) == (uint32_t)x) ? 0 : 1;
      {
        TR_T0(t_w);
        ok = copy_rows(first);                     // steps 0, 1, 2 before the loop: 0 and 2 by the group of step 0
        if (ok && first == 0) ok = copy_rows(2);
        if (threadIdx.x == 128) TR_ADD(a, 10, t_w);
      }
      for (int i = first; ok && i < u.steps; i += 2) {
        const uint32_t gi = g0 + i, st = gi & 3;
        TR_T0(t_s);
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.row_full[st]), (gi >> 2) & 1));   // row data of the stage
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&c.s_full[x]), (gi >> 1) & 1));
        if (!ok) break;
        if (threadIdx.x == 128) TR_ADD(a, 2, t_s);
        TR_T0(t_x);
        tc_fence_after();
        bool masked = false;
        if (i >= u.routed_steps) {
          const int o = i - u.routed_steps;
          const int ot = o - (o / u.own_steps) * u.own_steps;
          masked = ot * kStep < kKeys - 1;                 // rows whose token lies inside the key tile
        }
        if (masked) ps_row<true, kHalf>(tS, c.meta[st], c.tok[st], key_tok, key_ok, sl2);
        else ps_row<false, kHalf>(tS, c.meta[st], c.tok[st], key_tok, key_ok, sl2);
        tc_fence_before();
        mbar_arrive(smem_u32(&c.p_full[x]));
        if (threadIdx.x == 128) TR_ADD(a, 3, t_x);
        TR_T0(t_w);
        ok = copy_rows(i + 3);
        if (threadIdx.x == 128) TR_ADD(a, 10, t_w);
      }
      cp_async_wait_all();
      TR_T0(t_a);
      if (ok) ok = mbar_wait(smem_u32(&c.acc_full), nu & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        // warps 4-7 write dK (scaled), warps 8-11 dV: a thread owns the D values of its key
        const uint32_t tA = tmem + lane_base + 256 + x * 128;
        const float f = x == 0 ? scale : 1.f;
        __nv_bfloat16* dst = (x == 0 ? a.dk : a.dv) + ((int64_t)key_tok * p.Hkv + u.kvh) * D;
        uint32_t v[32];
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          tmem_ld32(tA + ch * 32, v);
          tmem_wait_ld();
          if (key_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o;
              o.x = pack2_16<kHalf>(__uint_as_float(v[8 * i]) * f, __uint_as_float(v[8 * i + 1]) * f);
              o.y = pack2_16<kHalf>(__uint_as_float(v[8 * i + 2]) * f, __uint_as_float(v[8 * i + 3]) * f);
              o.z = pack2_16<kHalf>(__uint_as_float(v[8 * i + 4]) * f, __uint_as_float(v[8 * i + 5]) * f);
              o.w = pack2_16<kHalf>(__uint_as_float(v[8 * i + 6]) * f, __uint_as_float(v[8 * i + 7]) * f);
              *reinterpret_cast<uint4*>(dst + ch * 32 + i * 8) = o;
            }
          }
        }
        tc_fence_before();
        if (threadIdx.x == 128) TR_ADD(a, 8, t_a);
      } else {
        atomicExch(a.status, ST_ROWS);
        c.abort = 1;
      }
      g0 += (uint32_t)u.steps;
      ++nu;
    }
  }

  if (threadIdx.x == 0) TR_ADD(a, 7, t_kernel);
  if (c.abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// Pre-pass: the Q and dO rows of every routed list, in list order, into qp / gp [entries, D];
// 64 rows of zeros behind the last list (a 64-row box may reach past it).  One 16-byte piece per
// thread and tensor: a warp copies whole rows.
template <int D>
__global__ void __launch_bounds__(256)
pack_rows_kernel(Params p, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ dout,
                 const int32_t* __restrict__ list_offsets, const int32_t* __restrict__ row_list,
                 __nv_bfloat16* __restrict__ qp, __nv_bfloat16* __restrict__ gp) {
  constexpr int kChunks = D / 8;
  const int64_t total = list_offsets[p.lists];
  const int64_t pieces = (total + kStep) * kChunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t pos = i / kChunks;
    const int ch = (int)(i - pos * kChunks);
    uint4 vq = make_uint4(0, 0, 0, 0), vg = vq;
    if (pos < total) {
      const uint32_t row = (uint32_t)row_list[pos] / (uint32_t)p.NP;
      const uint32_t t = row / (uint32_t)p.Hq;
      vq = __ldg(reinterpret_cast<const uint4*>(q + (int64_t)t * p.sq_t + (int64_t)(row - t * (uint32_t)p.Hq) * p.sq_h) + ch);
      vg = __ldg(reinterpret_cast<const uint4*>(dout + (int64_t)row * D) + ch);
    }
    reinterpret_cast<uint4*>(qp + pos * D)[ch] = vq;
    reinterpret_cast<uint4*>(gp + pos * D)[ch] = vg;
  }
}

// dk, dv <- NaN when a kernel of the call gave up on a wait
__global__ void poison_kernel(const int32_t* __restrict__ status, uint32_t* dk, uint32_t* dv, int64_t words) {
  if (*status == 0) return;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (int64_t)gridDim.x * blockDim.x) {
    dk[i] = 0x7fc07fc0u;       // NaN in bf16; NaN in fp16 as well (exponent all ones, mantissa non-zero)
    dv[i] = 0x7fc07fc0u;
  }
}

}  // namespace

cudaError_t launch_bwd_dkdv_tc5(const Params& p, const __nv_bfloat16* q, const __nv_bfloat16* k,
                                const __nv_bfloat16* v, const __nv_bfloat16* dout, const int32_t* cu,
                                const int32_t* list_counts, const int32_t* list_offsets, const int32_t* row_list,
                                const float* lse2, const float* delta, __nv_bfloat16* dk, __nv_bfloat16* dv,
                                __nv_bfloat16* packed, int32_t* work_counter, int32_t* status, cudaStream_t st) {
  if (p.D != 64 && p.D != 96 && p.D != 128) return cudaErrorInvalidValue;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // packed rows of the routed lists: qp, then gp, each [hist * rows + 64, D]
  const int64_t cap = (int64_t)p.hist * p.rows + kStep;
  __nv_bfloat16* qp = packed;
  __nv_bfloat16* gp = packed + cap * p.D;
  // chunks of at least this many 128-key tiles: their lists are read often enough to pay for packing
  const int use_packed = (p.C + kKeys - 1) / kKeys >= kPackMinTiles ? 1 : 0;
  if (p.hist > 0 && use_packed) {
    if (p.D == 128) pack_rows_kernel<128><<<sms * 8, 256, 0, st>>>(p, q, dout, list_offsets, row_list, qp, gp);
    else if (p.D == 96) pack_rows_kernel<96><<<sms * 8, 256, 0, st>>>(p, q, dout, list_offsets, row_list, qp, gp);
    else pack_rows_kernel<64><<<sms * 8, 256, 0, st>>>(p, q, dout, list_offsets, row_list, qp, gp);
    const cudaError_t pe = cudaGetLastError();
    if (pe != cudaSuccess) return pe;
  }
  CUtensorMap mk, mv, mq, mg, mqp, mgp;
  const bool half = p.fp16 != 0;
  if (!make_kv_map(&mk, half, p.D, k, p.T, p.Hkv, p.sk_t, p.sk_h, kKeys) ||
      !make_kv_map(&mv, half, p.D, v, p.T, p.Hkv, p.sv_t, p.sv_h, kKeys) ||
      !make_tile_map(&mq, half, p.D, q, p.T, p.Hq, p.sq_t, p.sq_h, 1, kStep) ||
      !make_tile_map(&mg, half, p.D, dout, p.T, p.Hq, (int64_t)p.Hq * p.D, p.D, 1, kStep) ||
      !make_tile_map(&mqp, half, p.D, qp, cap, 1, p.D, p.D, 1, kStep) ||
      !make_tile_map(&mgp, half, p.D, gp, cap, 1, p.D, p.D, 1, kStep))
    return cudaErrorNotSupported;
  auto kernel = p.D == 128 ? (p.fp16 ? bwd_dkdv_tc5_kernel<true, 128> : bwd_dkdv_tc5_kernel<false, 128>)
              : p.D == 96  ? (p.fp16 ? bwd_dkdv_tc5_kernel<true, 96> : bwd_dkdv_tc5_kernel<false, 96>)
                           : (p.fp16 ? bwd_dkdv_tc5_kernel<true, 64> : bwd_dkdv_tc5_kernel<false, 64>);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  const KernelArgs args{q, dout, cu, list_counts, list_offsets, row_list, lse2, delta, dk, dv, work_counter, status,
                        use_packed};
  kernel<<<sms, kThreads, kSmemBytes, st>>>(p, mk, mv, mq, mg, mqp, mgp, args);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  poison_kernel<<<sms, 256, 0, st>>>(status, reinterpret_cast<uint32_t*>(dk), reinterpret_cast<uint32_t*>(dv),
                                     (int64_t)p.T * p.Hkv * p.D / 2);
  return cudaGetLastError();
}

}  // namespace moba
