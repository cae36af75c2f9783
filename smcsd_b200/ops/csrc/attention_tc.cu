// Shared-prefix attention pass on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// All particles of an SMC group share the prompt's KV pages, so the attention of their new tokens over the prompt
// can be computed from ONE stream of those keys: up to 128 query rows (tokens x query heads of one kv head, several
// particles at a time) form the M = 128 operand of tcgen05.mma.  Per 128-key tile:
//     S = Q K^T        UMMA 128 x 128 x D, bf16 in, fp32 accumulator in tensor memory (two S buffers)
//     softmax          four warps, one query row per thread: one batched tcgen05.ld of the row's scores, running sum,
//                      P = exp2(S - m_ref) as bf16 written into a SWIZZLE_128B shared-memory tile
//     O += P V         UMMA 128 x D x 128 accumulating in tensor memory, V taken as an MN-major operand straight from
//                      its [key][dim] tile
// The exponent reference m_ref of a row only moves when the row's maximum has grown by more than 2^8 (P stays within
// bf16 / fp32 range); only then is the row's O rescaled in tensor memory (tcgen05.ld / st), which after the first few
// tiles is rare.  O is read back once, at the end.
// K/V rows live one page per token.  A tile whose 64 pages are consecutive, in ascending or descending order (what the
// allocator hands a prompt on a fresh or lightly fragmented pool), is fetched with one TMA box per 64-column panel; a scattered tile is gathered by the
// four loader warps with 16-byte cp.async copies into the same swizzled layout (a warp owns 16 keys and passes page
// ids by shuffle).  Page ids are fetched four tiles ahead.  The pass has no causal limit
// (every prompt key precedes every new token) and no new-token handling; it parks the unnormalised state
// (D values, running max, running sum) per (token, head), which the per-particle pass of attention_fused.cu folds
// in.  Key ranges can be split over several CTAs; each split parks its own state.
//
// Replaces the group pass of the mma.sync kernel for long prompts (what the reference's Triton verify kernel and its
// unmerged cascade kernel do with tl.dot: smcsd/core/kernels/verify_attention.py:56-273, docs/smc/performance.md:116-128).
// Every mbarrier wait is bounded; a timeout raises a status bit and every role unwinds.
#include "common.cuh"
#include "tmap_host.h"

#include <mutex>
#include <unordered_map>

namespace smc {

constexpr int TC_MAX_STAGES = 8;
// Keys per tile and ring depth by head size, within 227 KB of shared memory next to the Q tile and the two P tiles.
template <int D> struct TcCfg;
// Warps 0..3 run the softmax, warp 4 issues the MMAs, warps 5.. gather K/V.  Registers are granted per four warps:
// nine warps leave 168 per thread (enough for 64 scores per row), seven leave 255 (needed for 128 scores per row).
template <> struct TcCfg<128> { static constexpr int BK = 64, STAGES = 5, LOADERS = 4; };
template <> struct TcCfg<64> { static constexpr int BK = 64, STAGES = 8, LOADERS = 4; };

struct TcAttnParams {
  const __nv_bfloat16* q;        // rotated queries [T, Hq * D]; null: rotate the fp32 projections below in the kernel
  const float* qkv;              // [T, ld_qkv] fp32 projections, query heads at q_off
  const int* positions;          // [T]
  const float* rope;             // [max_pos, rd] cos | sin (rotary pairs i, i + rd / 2; dims beyond rd pass through)
  int ld_qkv, q_off, rd;
  int pdl;                       // launched with programmatic stream serialisation: wait for the previous grid here
  const __nv_bfloat16* k_pool;   // [pages + 1, Hkv * D]
  const __nv_bfloat16* v_pool;
  const int* block_table;
  const int* rows;               // [n_seq] block-table row of each (super-)sequence
  const int* key_count;          // [n_seq] keys [0, key_count) are attended
  float* part_out;               // [KS, T, Hq, D + 2]
  int bt_stride, n_pages, E, Hq, Hkv, KS, T;
  int use_tma;                   // 0: always gather with cp.async
  float scale_log2;              // softmax scale * log2(e)
  int* status;
  long long* trace;              // optional [CTAs][12] cycles: softmax {s_full wait, score load, P-buffer wait, exp + store, total},
                                 //   MMA {K/V wait, score-buffer wait, P wait}, first loader {stage wait, copy issue, landing wait, total}
};

struct TcShared {
  uint64_t kv_full[TC_MAX_STAGES], kv_empty[TC_MAX_STAGES], s_full[2], s_empty[2], p_full[2], p_empty[2];
  uint32_t tmem_slot;
  volatile int abort;
};

__device__ __forceinline__ bool tc_wait(TcShared& S, int* status, uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  if (S.abort) return false;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (S.abort) return false;
    if (clock64() - t0 > SMC_SPIN_CYCLES) {
      atomicOr(status, SMC_ERR_BARRIER_TIMEOUT);
      S.abort = 1;
      return false;
    }
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cp_async16_tc(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}

template <int D>
__global__ void __launch_bounds__((5 + TcCfg<D>::LOADERS) * 32, 1) attn_prefix_tc_kernel(const TcAttnParams p, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV) {
  constexpr int TC_BK = TcCfg<D>::BK, TC_STAGES = TcCfg<D>::STAGES, LOADERS = TcCfg<D>::LOADERS;
  constexpr int TC_THREADS = (5 + LOADERS) * 32;
  static_assert(TC_BK == 64 && LOADERS == 4, "the loaders assume 64-key tiles, 16 keys per warp");
  constexpr int KPW = TC_BK / LOADERS;                // keys of a scattered tile gathered by one loader warp
  constexpr int NPAN = D / 64;                        // 64-element (128-byte) panels along the head dimension
  constexpr int PANEL_Q = 128 * 128;                  // bytes of one [128 rows][128 B] panel
  constexpr int PANEL_KV = TC_BK * 128;
  constexpr int Q_BYTES = NPAN * PANEL_Q;
  constexpr int KV_BYTES = NPAN * PANEL_KV;           // one of K or V of a stage
  constexpr int P_BYTES = (TC_BK / 64) * PANEL_Q;
  constexpr int CPR = D / 8;                          // 16-byte chunks per K/V row
  extern __shared__ uint8_t tc_smem_raw[];
  __shared__ TcShared S;
  const uint32_t raw = smem_u32(tc_smem_raw);
  uint8_t* smem = tc_smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* q_s = smem;
  uint8_t* kv_s = q_s + Q_BYTES;                      // [stage][K | V]
  uint8_t* p_s = kv_s + TC_STAGES * 2 * KV_BYTES;     // two P tiles (tile j uses buffer j & 1)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv, R = p.E * G, MT = (R + 127) >> 7;       // the R query rows take MT tiles of 128
  const int mt = blockIdx.x % MT, kvh = (blockIdx.x / MT) % p.Hkv, seq = blockIdx.x / (MT * p.Hkv), ks = blockIdx.y;
  const int hbase = kvh * G, row0 = mt * 128;
  const int n_keys = p.key_count[seq];
  int per = (n_keys + p.KS - 1) / p.KS;
  per = (per + TC_BK - 1) / TC_BK * TC_BK;
  const int kb = ks * per, ke = min(n_keys, kb + per);
  const int n_tiles = ke > kb ? (ke - kb + TC_BK - 1) / TC_BK : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&S.kv_full[s], LOADERS);
      mbar_init(&S.kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&S.s_full[i], 1);
      mbar_init(&S.s_empty[i], 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&S.p_full[i], 4);
      mbar_init(&S.p_empty[i], 1);
    }
    S.abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 4) {
    tmem_alloc(&S.tmem_slot, 512);
    tmem_relinquish();
  }
  // everything above overlaps the previous kernel; the query projections are its output
  if (p.pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  // ---- Q tile: rows r = e * G + gq of this (super-)sequence, zero padded to 128, swizzled K-major panels ----------
  for (int idx = threadIdx.x; idx < 128 * CPR; idx += TC_THREADS) {
    const int r = idx / CPR, c = idx % CPR;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row0 + r < R) {
      const int e = (row0 + r) / G, gq = (row0 + r) % G, tkn = seq * p.E + e;
      if (p.q != nullptr) {
        v = *reinterpret_cast<const uint4*>(p.q + ((size_t)tkn * p.Hq + hbase + gq) * D + c * 8);
      } else {
        // rotate this 8-element chunk of the fp32 query row: element i pairs with i + half inside the rotary span
        const float* src = p.qkv + (size_t)tkn * p.ld_qkv + p.q_off + (size_t)(hbase + gq) * D;
        const int half = p.rd >> 1, i0 = c * 8;
        float x[8];
        *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(src + i0);
        *reinterpret_cast<float4*>(x + 4) = *reinterpret_cast<const float4*>(src + i0 + 4);
        if (i0 < p.rd) {
          const bool lo = i0 < half;
          const int j0 = lo ? i0 : i0 - half;                 // index into the cos / sin halves
          const float* cs = p.rope + (size_t)p.positions[tkn] * p.rd;
          float y[8], cv[8], sv[8];
          *reinterpret_cast<float4*>(y) = *reinterpret_cast<const float4*>(src + (lo ? i0 + half : j0));
          *reinterpret_cast<float4*>(y + 4) = *reinterpret_cast<const float4*>(src + (lo ? i0 + half : j0) + 4);
          *reinterpret_cast<float4*>(cv) = *reinterpret_cast<const float4*>(cs + j0);
          *reinterpret_cast<float4*>(cv + 4) = *reinterpret_cast<const float4*>(cs + j0 + 4);
          *reinterpret_cast<float4*>(sv) = *reinterpret_cast<const float4*>(cs + half + j0);
          *reinterpret_cast<float4*>(sv + 4) = *reinterpret_cast<const float4*>(cs + half + j0 + 4);
#pragma unroll
          for (int u = 0; u < 8; ++u) x[u] = lo ? x[u] * cv[u] - y[u] * sv[u] : x[u] * cv[u] + y[u] * sv[u];
        }
        v = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
      }
    }
    const int pan = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(q_s + pan * PANEL_Q + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async();                               // generic-proxy writes of Q before the tensor core reads them
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_slot;
  const uint32_t tO = tmem_base + 256u;              // scores live in columns [0, BK) and [128, 128 + BK)

  if (warp >= 5) {
    // ================================================================= loaders
    const int lw = warp - 5;
    const int* bt = p.block_table + (size_t)p.rows[seq] * p.bt_stride;
    const size_t kv_row = (size_t)p.Hkv * D;
    // every loader warp reads all 64 page ids of a tile (lane l: keys l and l + 32), so that all of them take the same
    // decision between the TMA and the gather path without talking to one another
    auto page_of = [&](int tile, int half) {
      const int key = kb + tile * TC_BK + half * 32 + lane;
      int page = 0;
      if (tile < n_tiles && key < ke) {
        page = bt[key];
        if (page < 0 || page > p.n_pages) { atomicOr(p.status, SMC_ERR_BOUNDS); page = 0; }
      }
      return page;
    };
    // LAG + 1 tiles of copies stay in flight per warp: a gathered tile is handed over once LAG later tiles have been
    // requested.  The page ids are a dependent global load in front of every tile's copies, so they are fetched PD tiles
    // ahead (a register ring, statically indexed by unrolling the tile loop PD times).
    constexpr int LAG = TC_STAGES - 2, PD = 4;
    static_assert(LAG < 32, "the per-tile mode history is a 32-bit mask");
    int issued = 0;
    uint32_t gathered = 0;                           // bit (j & 31): tile j went through cp.async (arrival still owed)
    int pg[PD][2];
#pragma unroll
    for (int u = 0; u < PD; ++u) {
      pg[u][0] = page_of(u, 0);
      pg[u][1] = page_of(u, 1);
    }
    bool go = true;
    const bool tr = p.trace != nullptr && warp == 5 && lane == 0;
    long long tl[3] = {0, 0, 0}, t_begin = tr ? clock64() : 0, t_mark = t_begin;
    auto lap = [&](int slot) {
      if (tr) {
        const long long now = clock64();
        tl[slot] += now - t_mark;
        t_mark = now;
      }
    };
    const uint64_t pol = l2_policy_evict_last();     // the other row tiles of this KV head read the same keys
    for (int j0 = 0; go && j0 < n_tiles; j0 += PD) {
#pragma unroll
      for (int u = 0; u < PD; ++u) {
        const int j = j0 + u;
        if (j >= n_tiles) break;
        const int st = j % TC_STAGES, use = j / TC_STAGES;
        const bool ok = use < 1 || tc_wait(S, p.status, &S.kv_empty[st], (uint32_t)(use - 1) & 1u);
        if (!__all_sync(0xffffffffu, ok)) { go = false; break; }
        lap(0);
        const int pa = pg[u][0], pb = pg[u][1];
        pg[u][0] = page_of(j + PD, 0);
        pg[u][1] = page_of(j + PD, 1);
        // 64 consecutive pages, ascending or descending (pages popped from a free stack come out either way; the pass
        // has no causal limit, so the order of the keys inside a tile does not matter)
        const int base = __shfl_sync(0xffffffffu, pa, 0);
        const bool full_tile = kb + (j + 1) * TC_BK <= ke;
        const bool asc = __all_sync(0xffffffffu, pa == base + lane && pb == base + 32 + lane);
        const bool desc = __all_sync(0xffffffffu, pa == base - lane && pb == base - 32 - lane) && base >= TC_BK;
        const bool run = p.use_tma && full_tile && base >= 1 && (asc || desc);
        const int first_page = asc ? base : base - (TC_BK - 1);
        uint8_t* k_ptr = kv_s + (size_t)st * 2 * KV_BYTES;
        if (run) {
          // 64 consecutive pages: one TMA box per 64-column panel of K and of V; every warp owes the barrier one arrival
          if (lane == 0) {
            if (lw == 0) {
              mbar_expect_tx(&S.kv_full[st], 2 * KV_BYTES);
#pragma unroll
              for (int pan = 0; pan < NPAN; ++pan) {
                tma_load_2d(k_ptr + pan * PANEL_KV, &tmK, &S.kv_full[st], kvh * D + pan * 64, first_page, pol);
                tma_load_2d(k_ptr + KV_BYTES + pan * PANEL_KV, &tmV, &S.kv_full[st], kvh * D + pan * 64, first_page, pol);
              }
            } else {
              mbar_arrive(&S.kv_full[st]);
            }
          }
          gathered &= ~(1u << (j & 31));
        } else {
          const uint32_t k_t = smem_u32(k_ptr), v_t = k_t + KV_BYTES;
          const int mine = lw < 2 ? pa : pb;         // this warp's 16 keys sit in lanes (lw & 1) * 16 ..
#pragma unroll 4
          for (int idx = lane; idx < KPW * CPR; idx += 32) {
            const int kl = idx / CPR, c = idx % CPR, key = lw * KPW + kl;
            const int pgi = __shfl_sync(0xffffffffu, mine, (lw & 1) * 16 + kl);
            const size_t off = (size_t)pgi * kv_row + (size_t)kvh * D + c * 8;
            const uint32_t dst = (uint32_t)((c >> 3) * PANEL_KV + key * 128 + (((c & 7) ^ (key & 7)) << 4));
            cp_async16_tc(k_t + dst, p.k_pool + off);
            cp_async16_tc(v_t + dst, p.v_pool + off);
          }
          gathered |= 1u << (j & 31);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // one group per tile (empty for a TMA tile)
        lap(1);
        if (j >= LAG && ((gathered >> ((j - LAG) & 31)) & 1u)) {  // gathered tile j - LAG has landed: hand it over
          asm volatile("cp.async.wait_group %0;" ::"n"(LAG) : "memory");
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&S.kv_full[(j - LAG) % TC_STAGES]);
        }
        lap(2);
        ++issued;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    fence_proxy_async();
    __syncwarp();
    if (lane == 0)
      for (int t = max(0, issued - LAG); t < issued; ++t)
        if ((gathered >> (t & 31)) & 1u) mbar_arrive(&S.kv_full[t % TC_STAGES]);
    if (tr) {
      long long* t = p.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 12;
      t[8] = tl[0]; t[9] = tl[1]; t[10] = tl[2]; t[11] = clock64() - t_begin;
    }
  } else if (warp == 4) {
    // ================================================================= MMA issuer (one thread)
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, TC_BK);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, D) | (1u << 16);       // B operand (V) is MN-major
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      const bool tr = p.trace != nullptr;
      long long tm[3] = {0, 0, 0};
      auto issue_s = [&](int j) -> bool {
        const int st = j % TC_STAGES;
        long long t0 = tr ? clock64() : 0;
        if (!tc_wait(S, p.status, &S.kv_full[st], (uint32_t)(j / TC_STAGES) & 1u)) return false;
        if (tr) { const long long t1 = clock64(); tm[0] += t1 - t0; t0 = t1; }
        if (j >= 2 && !tc_wait(S, p.status, &S.s_empty[j & 1], (uint32_t)((j >> 1) - 1) & 1u)) return false;
        if (tr) tm[1] += clock64() - t0;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(kv_s + (size_t)st * 2 * KV_BYTES);
#pragma unroll
        for (int pan = 0; pan < NPAN; ++pan)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + (uint32_t)(j & 1) * 128u, umma_desc_k_sw128(q_addr + pan * PANEL_Q) + 2 * k,
                         umma_desc_k_sw128(k_addr + pan * PANEL_KV) + 2 * k, idesc_s, (pan | k) ? 1u : 0u);
        umma_commit(&S.s_full[j & 1]);
        return true;
      };
      bool ok = n_tiles > 0 && issue_s(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles && !issue_s(j + 1)) break;                 // next tile's scores overlap this tile's softmax
        const long long t0 = tr ? clock64() : 0;
        if (!tc_wait(S, p.status, &S.p_full[j & 1], (uint32_t)(j >> 1) & 1u)) break;
        if (tr) tm[2] += clock64() - t0;
        tc_fence_after();
        const int st = j % TC_STAGES;
        const uint32_t pj_addr = p_addr + (uint32_t)(j & 1) * P_BYTES;
        const uint32_t v_addr = smem_u32(kv_s + (size_t)st * 2 * KV_BYTES + KV_BYTES);
#pragma unroll
        for (int kp = 0; kp < TC_BK / 64; ++kp)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tO, umma_desc_k_sw128(pj_addr + kp * PANEL_Q) + 2 * k,
                         umma_desc_mn_sw128(v_addr + kp * 8192 + k * 2048, PANEL_KV), idesc_o, (j | kp | k) ? 1u : 0u);
        umma_commit(&S.kv_empty[st]);
        umma_commit(&S.p_empty[j & 1]);              // also: O holds the sum over tiles 0..j
      }
      if (tr) {
        long long* t = p.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 12;
        t[5] = tm[0]; t[6] = tm[1]; t[7] = tm[2];
      }
    }
    __syncwarp();
  } else {
    // ================================================================= softmax (one query row per thread)
    const int r = warp * 32 + lane;
    const uint32_t lane_off = ((uint32_t)(warp * 32)) << 16;
    float m_ref = -INFINITY, l = 0.f;                // exponent reference (log2 domain) and running sum of the row
    bool alive = true;
    const bool tr = p.trace != nullptr && threadIdx.x == 0;
    long long tw[4] = {0, 0, 0, 0}, t_begin = tr ? clock64() : 0, t_mark = t_begin;
    auto lap = [&](int slot) {
      if (tr) {
        const long long now = clock64();
        tw[slot] += now - t_mark;
        t_mark = now;
      }
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int nvalid = min(TC_BK, ke - kb - j * TC_BK);
      if (!__all_sync(0xffffffffu, tc_wait(S, p.status, &S.s_full[j & 1], (uint32_t)(j >> 1) & 1u))) { alive = false; break; }
      lap(0);
      tc_fence_after();
      const uint32_t ts = tmem_base + (uint32_t)(j & 1) * 128u + lane_off;
      uint32_t x[TC_BK];
#pragma unroll
      for (int c0 = 0; c0 < TC_BK; c0 += 16) tmem_ld_32x32b_x16(ts + c0, *reinterpret_cast<uint32_t(*)[16]>(&x[c0]));
      tmem_ld_wait();
      tc_fence_before();                             // the scores are in registers: the buffer can take tile j + 2
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.s_empty[j & 1]);
      lap(1);
      const bool full = nvalid == TC_BK;
      float mx = -INFINITY;
      if (full) {
#pragma unroll
        for (int i = 0; i < TC_BK; ++i) mx = fmaxf(mx, __uint_as_float(x[i]));
      } else {
#pragma unroll
        for (int i = 0; i < TC_BK; ++i)
          if (i < nvalid) mx = fmaxf(mx, __uint_as_float(x[i]));
      }
      mx *= p.scale_log2;
      const bool grow = mx > m_ref + 8.f;            // also true on the first tile (m_ref = -inf)
      if (j >= 1 && __any_sync(0xffffffffu, grow)) {
        // rare after the first tiles: PV of tile j - 1 must have completed before O is rescaled in tensor memory
        if (!__all_sync(0xffffffffu, tc_wait(S, p.status, &S.p_empty[(j - 1) & 1], (uint32_t)((j - 1) >> 1) & 1u))) { alive = false; break; }
        tc_fence_after();
        const float alpha = grow ? exp2f(m_ref - mx) : 1.f;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 16) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tO + lane_off + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x16(tO + lane_off + c0, o);
        }
        tmem_st_wait();
        l *= alpha;
      }
      if (grow) m_ref = mx;
      // P buffer j & 1 was last read by PV of tile j - 2
      if (!__all_sync(0xffffffffu, j < 2 || tc_wait(S, p.status, &S.p_empty[j & 1], (uint32_t)((j - 2) >> 1) & 1u))) { alive = false; break; }
      lap(2);
      float sum0 = 0.f, sum1 = 0.f;
      uint8_t* pbuf = p_s + (j & 1) * P_BYTES;
#pragma unroll
      for (int c0 = 0; c0 < TC_BK; c0 += 16) {
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(x[c0 + i]), p.scale_log2, -m_ref));
          float p1 = ex2_approx(fmaf(__uint_as_float(x[c0 + i + 1]), p.scale_log2, -m_ref));
          if (!full) {
            p0 = c0 + i < nvalid ? p0 : 0.f;
            p1 = c0 + i + 1 < nvalid ? p1 : 0.f;
          }
          sum0 += p0;
          sum1 += p1;
          const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        const int pan = c0 >> 6, cc = (c0 & 63) >> 3;           // two 16-byte chunks of this row's 128-byte panel row
        uint8_t* prow = pbuf + pan * PANEL_Q + r * 128;
        *reinterpret_cast<uint4*>(prow + ((cc ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        *reinterpret_cast<uint4*>(prow + (((cc + 1) ^ (r & 7)) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
      l += sum0 + sum1;
      tc_fence_before();
      fence_proxy_async();                           // P must be visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.p_full[j & 1]);
      lap(3);
    }
    if (tr) {
      long long* t = p.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 12;
      t[0] = tw[0]; t[1] = tw[1]; t[2] = tw[2]; t[3] = tw[3]; t[4] = clock64() - t_begin;
    }
    // the last PV has completed when its P buffer is released: read the accumulated O once
    if (alive && n_tiles > 0)
      alive = __all_sync(0xffffffffu, tc_wait(S, p.status, &S.p_empty[(n_tiles - 1) & 1], (uint32_t)((n_tiles - 1) >> 1) & 1u));
    tc_fence_after();
    const bool write = row0 + r < R && alive && !S.abort;
    const int e = row0 + r < R ? (row0 + r) / G : 0, gq = (row0 + r) % G, tkn = seq * p.E + e, head = hbase + gq;
    float* so = p.part_out + (((size_t)ks * p.T + tkn) * p.Hq + head) * (D + 2);
    if (n_tiles > 0 && alive) {
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 16) {
        uint32_t o[16];
        tmem_ld_32x32b_x16(tO + lane_off + c0, o);
        tmem_ld_wait();
        if (write) {
#pragma unroll
          for (int i = 0; i < 16; i += 2)             // rows are D + 2 floats apart: 8-byte, not 16-byte, aligned
            *reinterpret_cast<float2*>(so + c0 + i) = make_float2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
        }
      }
    } else if (write) {
      for (int i = 0; i < D; ++i) so[i] = 0.f;
    }
    if (write) {
      so[D] = m_ref == -INFINITY ? -INFINITY : m_ref * 0.6931471805599453f;      // reference exponent in natural-log units
      so[D + 1] = l;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, 512);
}

template <int D>
static size_t tc_smem_bytes() {
  constexpr int BK = TcCfg<D>::BK, ST = TcCfg<D>::STAGES;
  return (size_t)(D / 64) * 128 * 128 + (size_t)ST * 2 * (D / 64) * BK * 128 + (size_t)2 * (BK / 64) * 128 * 128 + 1024;
}

// Tensor maps of the K / V pools ([pages + 1, Hkv * D] bf16, box = 64 columns x 64 pages), cached per pool.
struct PoolMapKey {
  const void* base; long long rows, cols;
  bool operator==(const PoolMapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols; }
};
struct PoolMapHash {
  size_t operator()(const PoolMapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<long long>()(k.rows) * 1315423911u) ^ std::hash<long long>()(k.cols);
  }
};
static int pool_tmap(CUtensorMap* tm, const void* base, long long rows, long long cols) {
  static std::unordered_map<PoolMapKey, CUtensorMap, PoolMapHash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const PoolMapKey key{base, rows, cols};
  auto it = cache.find(key);
  if (it != cache.end()) { *tm = it->second; return 0; }
  const int rc = make_tmap(tm, base, rows, cols, cols, 64);
  if (rc == 0) {
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *tm);
  }
  return rc;
}

}  // namespace smc

// Key-range splits for n_seq (super-)sequences of `rows` query rows (tokens x query heads per KV head) and about `keys`
// shared keys: one wave of CTAs, at least 256 keys per split.
SMC_API int smc_attention_tc_splits(int n_seq, int Hkv, int keys, int rows) {
  const long long base = (long long)n_seq * Hkv * ((rows + 127) / 128);
  int ks = (int)(148 / (base > 0 ? base : 1));
  ks = ks < 1 ? 1 : ks > 8 ? 8 : ks;
  while (ks > 1 && keys / ks < 256) --ks;
  return ks;
}

// q: rotated bf16 queries [T, Hq * D]; every (super-)sequence s has E consecutive tokens, block-table row rows[s] and
// attends keys [0, key_count[s]) without a causal limit; the E * Hq / Hkv query rows of a KV head take tiles of 128.  part_out [KS, T, Hq, D + 2] fp32 receives
// the unnormalised state of every key split (D values, running max in natural-log units, running sum).
// q may be null: then qkv (fp32 [T, ld_qkv], query heads at q_off), positions [T] and the rope table [max_pos, rd] are
// given and the kernel rotates the queries itself (rd and rd / 2 multiples of 8, rd <= D).
SMC_API int smc_attention_prefix_tc(const void* q, const void* k_pool, const void* v_pool, int n_pages,
                                    const int* block_table, int bt_stride, const int* rows, const int* key_count,
                                    float* part_out, int n_seq, int E, int T, int Hq, int Hkv, int D, int KS, float scale,
                                    int* status, long long* trace, int use_tma, const float* qkv, int ld_qkv, int q_off,
                                    const int* positions, const float* rope, int rd, int pdl, cudaStream_t st) {
  using namespace smc;
  if (n_seq <= 0) return 0;
  if (q == nullptr && (qkv == nullptr || positions == nullptr || rope == nullptr || (rd & 15) || rd > D ||
                       (ld_qkv & 3) || (q_off & 3)))
    return -82;
  if (Hq % Hkv || E < 1 || KS < 1 || KS > 8) return -80;
  TcAttnParams p;
  p.pdl = pdl;
  p.qkv = qkv; p.positions = positions; p.rope = rope; p.ld_qkv = ld_qkv; p.q_off = q_off; p.rd = rd;
  p.q = (const __nv_bfloat16*)q; p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
  p.block_table = block_table; p.rows = rows; p.key_count = key_count; p.part_out = part_out;
  p.bt_stride = bt_stride; p.n_pages = n_pages; p.E = E; p.Hq = Hq; p.Hkv = Hkv; p.KS = KS; p.T = T;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.trace = trace;
  p.use_tma = use_tma && ((size_t)Hkv * D) % 8 == 0;
  CUtensorMap tmK, tmV;
  int rc = pool_tmap(&tmK, k_pool, (long long)n_pages + 1, (long long)Hkv * D);
  if (rc == 0) rc = pool_tmap(&tmV, v_pool, (long long)n_pages + 1, (long long)Hkv * D);
  if (rc) return rc;
  void (*kern)(const TcAttnParams, const CUtensorMap, const CUtensorMap) = nullptr;
  size_t smem = 0;
  int threads = 0;
  if (D == 128) { kern = attn_prefix_tc_kernel<128>; smem = tc_smem_bytes<128>(); threads = (5 + TcCfg<128>::LOADERS) * 32; }
  else if (D == 64) { kern = attn_prefix_tc_kernel<64>; smem = tc_smem_bytes<64>(); threads = (5 + TcCfg<64>::LOADERS) * 32; }
  else return -81;
  CUDA_CHECK_RET(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(n_seq * Hkv * ((E * (Hq / Hkv) + 127) / 128)), (unsigned)KS);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, kern, p, tmK, tmV));
  return (int)cudaGetLastError();
}
