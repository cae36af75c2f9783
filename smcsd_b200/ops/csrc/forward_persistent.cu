// One launch per model forward: a persistent kernel (one CTA per SM) that walks every layer of a dense
// Llama-style decoder for a few-token batch and ends with the lm_head fused with sampling / scoring.
//
// Why: at 8..80 token rows a decoder layer is five dependent kernels whose fixed hand-off latency (a few
// microseconds each) is as long as the time their weights need to stream from HBM.  Here the hand-offs become
// grid-wide barriers inside one kernel and, more importantly, the weight stream never stops: a producer thread
// per CTA keeps a shared-memory ring full of weight tiles of the *following* phases (weights do not depend on
// activations), so HBM stays busy while a phase drains, synchronises and the next one starts.  (How much that buys
// is bounded by the ring: about 13 MB of prefetch on the whole GPU.  Measured, a K-split phase here costs 6-8 us
// against 4.7-5.4 us for the stand-alone GEMM kernels, so the kernel is an option of the runner, not its default.)
//
// Phases (all CTAs walk the same list):
//   embed                       ids -> fp32 residual h, bf16 copy hb, per-128-column sums of squares
//   per layer: QKV GEMM         qkv = (hb W^T) * rstd                (RMSNorm folded into W; rstd from the sums of squares)
//              attention        rope + bf16 + KV page write of the new tokens, GQA-packed causal attention over the
//                               paged cache (mma.sync tiles, key-ways merged in the CTA, key splits merged by the
//                               last CTA to arrive through a global workspace)
//              o-proj GEMM      h += attn W^T ; hb ; sums of squares
//              gate/up GEMM     act = silu(g * rstd) * (u * rstd)
//              down GEMM        h += act W^T ; hb ; sums of squares
//   lm_head GEMM                the epilogue reduces every 128-row vocabulary slab to (max, sum-exp, Gumbel candidate,
//                               chosen logit) per row: logits never reach memory
//   merge                       per row: token, log-probability, logZ
//
// GEMMs are tcgen05 with swapped operands (a 128-row weight slab is the M operand, the tokens are N, fp32
// accumulator in tensor memory, two accumulators so the epilogue of one unit overlaps the MMAs of the next).  The grid
// is made of thread-block clusters of eight CTAs.  Matrices with few slabs (QKV, o-proj, down) are split along K
// over the CTAs of a cluster: each parks its fp32 tile in shared memory, signals its seven peers through an
// mbarrier, and every CTA then sums its share of the token columns over all eight tiles through distributed shared
// memory in a fixed order (deterministic, nothing visits HBM; a reduction through an L2 workspace measured about
// 7 us per phase, this one about 1.5).  Matrices with many slabs (gate/up, lm_head) are dealt as whole slabs.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer, 4..7 = epilogue (TMEM lanes 32 * (warp % 4)), 2..7 = attention.
// Every wait is bounded; a timeout raises a status bit and an abort flag that short-circuits all later waits.
#include <string.h>

#include "attn_core.cuh"
#include "common.cuh"
#include "sample_core.cuh"
#include "tmap_host.h"

namespace smc {

constexpr int PF_THREADS = 256;
constexpr int PF_MAX_STAGES = 12;
constexpr int PF_RANGE = 512;             // page ids staged per attention pass
constexpr int PF_A_BYTES = 128 * 64 * 2;  // one weight tile: 128 rows x 64 k
constexpr int PF_TMEM_COLS = 256;         // two accumulators of up to 128 columns

enum { PF_EPI_QKV = 0, PF_EPI_RESID = 1, PF_EPI_SWIGLU = 2, PF_EPI_LMHEAD = 3 };
enum { PF_SYNC_BARRIER = 0, PF_SYNC_EXIT = 1, PF_SYNC_ABORT = 2 };

struct PfParams {
  // ---- model
  int L, d, Hq, Hkv, D, ffn, V, nqkv;
  int rd, max_pos, n_pages, bt_stride;
  float rms_eps, softcap, scale, pad0;
  const CUtensorMap* maps;       // device array: [4 l + {qkv, o, gate/up, down}], lm_head at 4L, then hb, attn, act, hb rows of the lm_head
  const __nv_bfloat16* embed;
  const float* rope;
  __nv_bfloat16* k_pool;         // [L][n_pages + 1][Hkv * D]
  __nv_bfloat16* v_pool;
  long long kv_layer_stride;     // elements between layers
  const int* block_table;
  // ---- batch
  int bs, E, M, BN;
  int KS, lm_rows, n_mt, n_kw;
  int att_stg, stages, ring_bytes, att_bytes;
  int lm_row_off, lm_row_step;   // sampled row i is token row lm_row_off + i * lm_row_step
  const int* ids;
  const int* positions;
  const int* cache_locs;
  const int* rows;
  const int* prefix_lens;
  // ---- activations
  float* h;                      // [M, d] fp32 residual stream
  __nv_bfloat16* hb;             // [M, d] bf16 copy
  float* ssq;                    // [d / 128, ssq_ld] sums of squares per 128-column part
  float* qkv;                    // [M, nqkv]
  __nv_bfloat16* attn;           // [M, Hq * D]
  __nv_bfloat16* act;            // [M, ffn]
  int ssq_ld, pad1;
  // ---- workspaces
  float* att_part;               // [bs * Hkv * KS][n_mt][16 D + 64] key-split partial states
  int* att_ctr;                  // [bs * Hkv]
  // ---- sampling
  float inv_temp, alpha;
  const int* tokens_in;          // per row: >= 0 score that token, < 0 sample (null: all rows sample)
  unsigned long long seed;
  const long long* cycle_counter;
  int call_id, pad2;
  RowPartial* sparts;            // [lm_rows][ctas]
  int* tok_out;
  float* logp_out;
  float* logz_out;
  // ---- synchronisation
  unsigned int* sync;            // [0] phase arrivals, [1] exit arrivals, [2] abort flag
  int* status;
  long long* trace;              // optional [phases][ctas][8] nanosecond stamps: 0 inputs seen ready, 1 phase work done, 2.. detail
};

struct PfShared {
  uint64_t full[PF_MAX_STAGES], empty[PF_MAX_STAGES], acc_full[2], acc_empty[2];
  uint64_t red_full, red_done;    // cluster reduction: all eight tiles parked / all eight CTAs done reading this one
  uint32_t tmem_slot;
  volatile int abort, issued, consumed;
  int flag, pad;
  volatile int open_upto;         // highest phase whose inputs this CTA's leader has seen ready
  int pad2;
  int pos[16];
  float xcol[2][4][64];           // up-channel values handed to the gate rows (split gate/up reduction)
  float rstd[128];
  float ssq[2][4][16];
  RowPartial rp[128];
};

struct PfCtx {
  volatile int* sh_abort;
  volatile unsigned int* g_abort;
  int* status;
};

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void pf_raise(const PfCtx& c, int code) {
  atomicOr(c.status, code);
  *c.sh_abort = 1;
  *c.g_abort = 1u;
  __threadfence();
}
// Bounded mbarrier wait that gives up at once when the kernel has been aborted.
__device__ __forceinline__ bool pf_mbar_wait(const PfCtx& c, uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*c.sh_abort) return false;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*c.sh_abort || *c.g_abort) {
      *c.sh_abort = 1;
      return false;
    }
    if (clock64() - t0 > SMC_SPIN_CYCLES) {
      pf_raise(c, SMC_ERR_BARRIER_TIMEOUT);
      return false;
    }
  }
}
// Bounded wait until the phase counter reaches `want` (all CTAs have finished the phases before).
__device__ __forceinline__ bool pf_wait_counter(const PfCtx& c, const unsigned int* ctr, unsigned int want) {
  if (ld_acquire_gpu_u32(ctr) >= want) return true;
  if (*c.sh_abort) return false;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 32; ++i) {
      __nanosleep(40);                 // hundreds of pollers share one L2 line with the arriving atomics
      if (ld_acquire_gpu_u32(ctr) >= want) return true;
    }
    if (*c.sh_abort || *c.g_abort) {
      *c.sh_abort = 1;
      return false;
    }
    if (clock64() - t0 > SMC_SPIN_CYCLES) {
      pf_raise(c, SMC_ERR_BARRIER_TIMEOUT);
      return false;
    }
  }
}
// The leader's wait for a phase, published to the producer of the same CTA.
__device__ __forceinline__ void pf_leader_wait(const PfParams& p, const PfCtx& c, volatile int* open_upto, int ph,
                                               int ncta) {
  pf_wait_counter(c, p.sync + PF_SYNC_BARRIER, (unsigned int)ph * (unsigned int)ncta);
  __threadfence();
  *open_upto = ph;
}
__device__ __forceinline__ void bar_epi() { group_barrier(1, 128); }     // warps 4..7
__device__ __forceinline__ void bar_att() { group_barrier(2, 192); }     // warps 2..7

constexpr int PF_CLUSTER = 8;
// arrive on the mbarrier at the same shared-memory offset in CTA `rank` of this cluster; earlier writes of the
// arriving thread (and, through a preceding CTA barrier, of its CTA) are visible to whoever waits with acquire
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(dsmem_map(smem_u32(bar), rank))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool pf_mbar_wait_cluster(const PfCtx& c, uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  if (*c.sh_abort) return false;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*c.sh_abort || *c.g_abort) {
      *c.sh_abort = 1;
      return false;
    }
    if (clock64() - t0 > SMC_SPIN_CYCLES) {
      pf_raise(c, SMC_ERR_BARRIER_TIMEOUT);
      return false;
    }
  }
}

// ---------------------------------------------------------------- phase list and work shares
struct GemmDesc {
  int N, K, n_slabs, kblocks, split, wmap, xmap, epi;
};

__device__ __forceinline__ int pf_num_phases(const PfParams& p) { return 1 + 5 * p.L + (p.lm_rows > 0 ? 2 : 0); }

__device__ __forceinline__ bool pf_gemm_desc(const PfParams& p, int ph, GemmDesc& g) {
  const int L5 = 5 * p.L;
  bool lm = false;
  if (ph >= 1 && ph <= L5) {
    const int l = (ph - 1) / 5, j = (ph - 1) % 5;
    const int xbase = 4 * p.L + 1;
    if (j == 0) { g.N = p.nqkv; g.K = p.d; g.wmap = 4 * l; g.xmap = xbase; g.epi = PF_EPI_QKV; }
    else if (j == 2) { g.N = p.d; g.K = p.Hq * p.D; g.wmap = 4 * l + 1; g.xmap = xbase + 1; g.epi = PF_EPI_RESID; }
    else if (j == 3) { g.N = 2 * p.ffn; g.K = p.d; g.wmap = 4 * l + 2; g.xmap = xbase; g.epi = PF_EPI_SWIGLU; }
    else if (j == 4) { g.N = p.d; g.K = p.ffn; g.wmap = 4 * l + 3; g.xmap = xbase + 2; g.epi = PF_EPI_RESID; }
    else return false;
  } else if (ph == L5 + 1 && p.lm_rows > 0) {
    g.N = p.V; g.K = p.d; g.wmap = 4 * p.L; g.xmap = 4 * p.L + 4; g.epi = PF_EPI_LMHEAD;
    lm = true;
  } else {
    return false;
  }
  g.n_slabs = (g.N + 127) >> 7;
  g.kblocks = (g.K + 63) >> 6;
  // few slabs and a reduction long enough to cut in eight: split along K inside the clusters; otherwise whole slabs
  g.split = (!lm && g.kblocks >= PF_CLUSTER && g.n_slabs * 3 < (int)gridDim.x * 2) ? 1 : 0;
  return true;
}

// Work units of a GEMM phase.  Split phases: slab (cluster + i * clusters), k-blocks cut evenly over the eight ranks.
// Whole phases: consecutive slabs per CTA over the full reduction.
__device__ __forceinline__ int pf_units(const GemmDesc& g, int cta, int ncta) {
  if (g.split) {
    const int cl = cta / PF_CLUSTER, ncl = ncta / PF_CLUSTER;
    return cl < g.n_slabs ? (g.n_slabs - cl + ncl - 1) / ncl : 0;
  }
  const unsigned int ns = (unsigned int)g.n_slabs, un = (unsigned int)ncta;
  return (int)(ns * (unsigned int)(cta + 1) / un) - (int)(ns * (unsigned int)cta / un);
}
__device__ __forceinline__ void pf_unit(const GemmDesc& g, int cta, int ncta, int i, int& slab, int& kb0, int& kb1) {
  if (g.split) {
    const int cl = cta / PF_CLUSTER, ncl = ncta / PF_CLUSTER, r = cta % PF_CLUSTER;
    slab = cl + i * ncl;
    kb0 = g.kblocks * r / PF_CLUSTER;
    kb1 = g.kblocks * (r + 1) / PF_CLUSTER;
  } else {
    slab = (int)((unsigned int)g.n_slabs * (unsigned int)cta / (unsigned int)ncta) + i;
    kb0 = 0;
    kb1 = g.kblocks;
  }
}

struct PfCursor {
  int ph, i, n, slab, kb, kb_end;
  GemmDesc g;
  // position on the first k-block of the first unit of the first GEMM phase >= from_ph in which this CTA has work
  __device__ __forceinline__ bool seek(const PfParams& p, int from_ph, int cta, int ncta, int n_phases) {
    for (ph = from_ph; ph < n_phases; ++ph) {
      if (!pf_gemm_desc(p, ph, g)) continue;
      n = pf_units(g, cta, ncta);
      if (n > 0) {
        i = 0;
        pf_unit(g, cta, ncta, 0, slab, kb, kb_end);
        return true;
      }
    }
    return false;
  }
  // next k-block (of this unit, the next unit or the next phase); false at the end of the program
  __device__ __forceinline__ bool step(const PfParams& p, int cta, int ncta, int n_phases) {
    if (++kb < kb_end) return true;
    if (++i < n) {
      pf_unit(g, cta, ncta, i, slab, kb, kb_end);
      return true;
    }
    return seek(p, ph + 1, cta, ncta, n_phases);
  }
};

__device__ __forceinline__ long long pf_now_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void pf_stamp(const PfParams& p, int ph, int which) {
  if (p.trace != nullptr) p.trace[((size_t)ph * gridDim.x + blockIdx.x) * 8 + which] = pf_now_ns();
}
__device__ __forceinline__ void pf_arrive(const PfParams& p, int ph) {
  pf_stamp(p, ph, 1);
  __threadfence();
  atomicAdd(p.sync + PF_SYNC_BARRIER, 1u);
}

// ---------------------------------------------------------------- producer (one thread)
__device__ void pf_producer(const PfParams& p, const PfCtx& ctx, PfShared& S, uint8_t* ring, int cta, int ncta) {
  const int n_phases = pf_num_phases(p);
  const int nst = p.stages;
  const int stage_bytes = PF_A_BYTES + p.BN * 128;
  const uint64_t pol_w = l2_policy_evict_first();
  const uint64_t pol_x = l2_policy_evict_last();
  PfCursor W, X;
  bool wv = W.seek(p, 1, cta, ncta, n_phases);
  bool xv = X.seek(p, 1, cta, ncta, n_phases);
  int wi = 0, xi = 0;                    // stages whose weight tile / activation tile has been requested
  int wslot = 0, wuse = 0, xslot = 0;
  unsigned int open_upto = 0;            // phases 0..open_upto may read their inputs
  long long t_idle = clock64();
  while (xv) {
    bool progressed = false;
    // weight tiles first: every free slot of the ring is refilled before the (slow) look at the phase counter
    while (wv && (wuse == 0 || mbar_test_wait(&S.empty[wslot], (uint32_t)(wuse - 1) & 1u))) {
      mbar_expect_tx(&S.full[wslot], (uint32_t)stage_bytes);
      tma_load_2d(ring + (size_t)wslot * stage_bytes, p.maps + W.g.wmap, &S.full[wslot], W.kb * 64, W.slab * 128,
                  pol_w);
      ++wi;
      S.issued = wi;
      if (++wslot == nst) { wslot = 0; ++wuse; }
      wv = W.step(p, cta, ncta, n_phases);
      progressed = true;
    }
    // activation tiles of every stage whose phase is open
    while (xi < wi) {
      if ((unsigned int)X.ph > open_upto) {
        // the epilogue leader of this CTA watches the phase counter and publishes what it saw: no global
        // polling here, so refilling the ring is never held up by a round trip to L2
        const unsigned int done = (unsigned int)S.open_upto;
        if (done > open_upto) {
          __threadfence();
          open_upto = done;
          fence_proxy_async_all();       // activations were written with ordinary stores by other CTAs
        }
        if ((unsigned int)X.ph > open_upto) break;
      }
      tma_load_2d(ring + (size_t)xslot * stage_bytes + PF_A_BYTES, p.maps + X.g.xmap, &S.full[xslot], X.kb * 64, 0,
                  pol_x);
      ++xi;
      if (++xslot == nst) xslot = 0;
      xv = X.step(p, cta, ncta, n_phases);
      progressed = true;
    }
    if (progressed) {
      t_idle = clock64();
    } else {
      if (*ctx.sh_abort || *ctx.g_abort) { *ctx.sh_abort = 1; break; }
      if (clock64() - t_idle > SMC_SPIN_CYCLES) { pf_raise(ctx, SMC_ERR_BARRIER_TIMEOUT); break; }
    }
  }
}

// ---------------------------------------------------------------- MMA issuer (one thread)
__device__ void pf_mma(const PfParams& p, const PfCtx& ctx, PfShared& S, uint8_t* ring, uint32_t tmem_base, int cta,
                       int ncta) {
  const int n_phases = pf_num_phases(p);
  const int nst = p.stages;
  const int stage_bytes = PF_A_BYTES + p.BN * 128;
  const uint32_t idesc = umma_idesc_bf16(128, p.BN);
  PfCursor C;
  bool v = C.seek(p, 1, cta, ncta, n_phases);
  int slot = 0, unit = 0, consumed = 0;
  uint32_t fph = 0u;
  while (v) {
    const int a = unit & 1, use = unit >> 1;
    if (use >= 1 && !pf_mbar_wait(ctx, &S.acc_empty[a], (uint32_t)(use - 1) & 1u)) return;
    tc_fence_after();
    const uint32_t tacc = tmem_base + (uint32_t)a * 128u;
    const int nkb = C.kb_end - C.kb;
    for (int j = 0; j < nkb; ++j) {
      if (!pf_mbar_wait(ctx, &S.full[slot], fph)) return;
      tc_fence_after();
      const uint32_t a_addr = smem_u32(ring + (size_t)slot * stage_bytes);
      const uint64_t adesc = umma_desc_k_sw128(a_addr);
      const uint64_t bdesc = umma_desc_k_sw128(a_addr + PF_A_BYTES);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16_ss(tacc, adesc + 2 * k, bdesc + 2 * k, idesc, (j == 0 && k == 0) ? 0u : 1u);
      umma_commit(&S.empty[slot]);
      S.consumed = ++consumed;
      if (++slot == nst) { slot = 0; fph ^= 1u; }
    }
    umma_commit(&S.acc_full[a]);
    ++unit;
    C.kb = C.kb_end - 1;                 // on to the next unit
    v = C.step(p, cta, ncta, n_phases);
  }
}

// ---------------------------------------------------------------- epilogues
// One chunk of 16 token columns of a 128-row slab; `v` holds this thread's row (t = 0..127 of the slab).
// All 128 epilogue threads call this together (it contains group barriers).
__device__ __forceinline__ void pf_epi_chunk(const PfParams& p, const GemmDesc& g, PfShared& S, float* scratch, int slab,
                                             int c0, const float (&v)[16], int t, int parity) {
  const int warp_e = t >> 5, lane = t & 31;
  const int n = slab * 128 + t;
  if (g.epi == PF_EPI_QKV) {
    if (n < g.N) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int m = c0 + j;
        if (m < p.M) p.qkv[(size_t)m * p.nqkv + n] = v[j] * S.rstd[m];
      }
    }
  } else if (g.epi == PF_EPI_RESID) {
    float sq[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int m = c0 + j;
      float hv = 0.f;
      if (m < p.M && n < g.N) {
        hv = __ldcg(p.h + (size_t)m * p.d + n) + v[j];
        p.h[(size_t)m * p.d + n] = hv;
        p.hb[(size_t)m * p.d + n] = __float2bfloat16(hv);
      }
      sq[j] = hv * hv;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float s = warp_sum(sq[j]);
      if (lane == 0) S.ssq[parity][warp_e][j] = s;
    }
    bar_epi();
    if (t < 16 && c0 + t < p.M)
      p.ssq[(size_t)slab * p.ssq_ld + c0 + t] =
          S.ssq[parity][0][t] + S.ssq[parity][1][t] + S.ssq[parity][2][t] + S.ssq[parity][3][t];
  } else if (g.epi == PF_EPI_SWIGLU) {
    // rows 0..63 of a slab are gate channels, rows 64..127 the matching up channels
    float* xch = scratch + parity * (64 * 17);
    if (t >= 64) {
#pragma unroll
      for (int j = 0; j < 16; ++j) xch[(t - 64) * 17 + j] = v[j];
    }
    bar_epi();
    if (t < 64) {
      const int ch = slab * 64 + t;
      if (ch * 2 < g.N) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = c0 + j;
          if (m < p.M) {
            const float r = S.rstd[m];
            const float gt = v[j] * r, up = xch[t * 17 + j] * r;
            p.act[(size_t)m * p.ffn + ch] = __float2bfloat16(gt / (1.0f + __expf(-gt)) * up);
          }
        }
      }
    }
  } else {
    // lm_head: transpose the chunk through shared memory, then 8 threads share one token column (16 rows each)
    float* tr = scratch + parity * (16 * 129);
#pragma unroll
    for (int j = 0; j < 16; ++j) tr[j * 129 + t] = v[j] * S.rstd[min(c0 + j, 127)];
    bar_epi();
    SampleArgs sa;
    sa.inv_temp = p.inv_temp; sa.alpha = p.alpha; sa.softcap = p.softcap; sa.V = p.V; sa.rows = p.lm_rows;
    sa.call_id = p.call_id; sa.tokens_in = p.tokens_in; sa.seed = p.seed; sa.cycle_counter = p.cycle_counter;
    lm_reduce_chunk(sa, tr, slab * 128, c0, 0, t, S.rp);
  }
}

// One token column m of a slab after the cluster reduction; `v` is this thread's row (t = 0..127 of the slab).
// All 128 epilogue threads call this together (it contains group barriers for two of the epilogues).
__device__ __forceinline__ void pf_epi_col(const PfParams& p, const GemmDesc& g, PfShared& S, int slab, int m, float v,
                                           int t, int parity, int u) {
  const int warp_e = t >> 5, lane = t & 31;
  const int n = slab * 128 + t;
  if (g.epi == PF_EPI_QKV) {
    if (n < g.N) p.qkv[(size_t)m * p.nqkv + n] = v * S.rstd[m];
  } else if (g.epi == PF_EPI_RESID) {
    float hv = 0.f;
    if (n < g.N) {
      hv = __ldcg(p.h + (size_t)m * p.d + n) + v;
      p.h[(size_t)m * p.d + n] = hv;
      p.hb[(size_t)m * p.d + n] = __float2bfloat16(hv);
    }
    const float sq = warp_sum(hv * hv);
    if (lane == 0) S.ssq[parity][warp_e][u] = sq;
  } else {
    // gate/up cut along K: rows 64..127 hand their sums to the gate rows 0..63
    if (t >= 64) S.xcol[parity][u][t - 64] = v;
  }
}
// second half of pf_epi_col for the epilogues that exchange through shared memory (after a group barrier)
__device__ __forceinline__ void pf_epi_col_finish(const PfParams& p, const GemmDesc& g, PfShared& S, int slab, int m,
                                                  float v, int t, int parity, int u) {
  if (g.epi == PF_EPI_RESID) {
    if (t == u)
      p.ssq[(size_t)slab * p.ssq_ld + m] =
          S.ssq[parity][0][u] + S.ssq[parity][1][u] + S.ssq[parity][2][u] + S.ssq[parity][3][u];
  } else if (g.epi == PF_EPI_SWIGLU) {
    const int ch = slab * 64 + t;
    if (t < 64 && ch * 2 < g.N) {
      const float r = S.rstd[m];
      const float gt = v * r, up = S.xcol[parity][u][t] * r;
      p.act[(size_t)m * p.ffn + ch] = __float2bfloat16(gt / (1.0f + __expf(-gt)) * up);
    }
  }
}

// Epilogue of one GEMM phase for warps 4..7 (t = 0..127).  `red_use` counts the cluster reductions this CTA has taken
// part in (all CTAs of a cluster walk the same units, so the counts agree); `red_pending` is set while peers may
// still be reading this CTA's parked tile.
__device__ void pf_gemm_epilogue(const PfParams& p, const PfCtx& ctx, PfShared& S, float* scratch, uint32_t tmem_base,
                                 const GemmDesc& g, int ph, int cta, int ncta, int t, int& unit, int& red_use,
                                 int& red_pending) {
  const int warp_e = t >> 5, lane = t & 31;
  // the inputs of this phase (sums of squares for the folded norm) are ready once every CTA has left the phase before
  if (t == 0) {
    pf_leader_wait(p, ctx, &S.open_upto, ph, ncta);
    pf_stamp(p, ph, 0);
  }
  bar_epi();
  const int cols = g.epi == PF_EPI_LMHEAD ? p.lm_rows : p.M;
  if (g.epi != PF_EPI_RESID) {
    const int parts = p.d >> 7;
    if (t < cols) {
      // column t of the lm_head accumulator is token row lm_row_off + t * lm_row_step
      const int col = g.epi == PF_EPI_LMHEAD ? (p.lm_row_off + t * p.lm_row_step) : t;
      float ss = 0.f;
      for (int q = 0; q < parts; ++q) ss += __ldcg(p.ssq + (size_t)q * p.ssq_ld + col);
      S.rstd[t] = rsqrtf(ss / (float)p.d + p.rms_eps);
    }
    if (g.epi == PF_EPI_LMHEAD) S.rp[t] = row_partial_neutral();
    bar_epi();
  }
  const int n_units = pf_units(g, cta, ncta);
  const uint32_t lane_off = ((uint32_t)(warp_e * 32)) << 16;
  const uint32_t rank = (uint32_t)(cta % PF_CLUSTER);
  int parity = 0;
  for (int i = 0; i < n_units; ++i) {
    int slab, kb0, kb1;
    pf_unit(g, cta, ncta, i, slab, kb0, kb1);
    const int a = unit & 1, use = unit >> 1;
    pf_mbar_wait(ctx, &S.acc_full[a], (uint32_t)use & 1u);
    if (t == 0 && i == 0) pf_stamp(p, ph, 2);
    tc_fence_after();
    const uint32_t taddr = tmem_base + (uint32_t)a * 128u + lane_off;
    if (!g.split) {
      for (int c0 = 0; c0 < cols; c0 += 16) {
        uint32_t r[16];
        float v[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
        if (c0 + 16 >= cols) {           // accumulator fully read: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&S.acc_empty[a]);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        pf_epi_chunk(p, g, S, scratch, slab, c0, v, t, parity);
        parity ^= 1;
      }
    } else {
      // ---- cluster reduction: park this CTA's tile, wait for all eight, sum this rank's columns ------------
      float* park = scratch;             // [cols][128] fp32
      if (red_pending) {                 // peers may still be reading the tile parked for the previous unit
        pf_mbar_wait_cluster(ctx, &S.red_done, (uint32_t)(red_use - 1) & 1u);
        red_pending = 0;
      }
      for (int c0 = 0; c0 < cols; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) park[(c0 + j) * 128 + t] = __uint_as_float(r[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.acc_empty[a]);
      bar_epi();
      if (t < PF_CLUSTER) mbar_arrive_remote(&S.red_full, (uint32_t)t);
      if (t == 0) pf_stamp(p, ph, 3);
      pf_mbar_wait_cluster(ctx, &S.red_full, (uint32_t)red_use & 1u);
      if (t == 0) pf_stamp(p, ph, 4);
      uint32_t rbase[PF_CLUSTER];
#pragma unroll
      for (uint32_t q = 0; q < PF_CLUSTER; ++q) rbase[q] = dsmem_map(smem_u32(park) + (uint32_t)t * 4u, q);
      constexpr int UN = 4;
      for (int cb = (int)rank; cb < cols; cb += PF_CLUSTER * UN) {
        float x[UN][PF_CLUSTER];
        // all remote loads of a batch of columns are issued before the first add
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int c = cb + u * PF_CLUSTER;
#pragma unroll
          for (uint32_t q = 0; q < PF_CLUSTER; ++q)
            x[u][q] = c < cols ? ld_dsmem_f32_at(rbase[q] + (uint32_t)c * 512u) : 0.f;
        }
        float v[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          float acc = 0.f;
#pragma unroll
          for (uint32_t q = 0; q < PF_CLUSTER; ++q) acc += x[u][q];
          v[u] = acc;
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int c = cb + u * PF_CLUSTER;
          if (c < cols) pf_epi_col(p, g, S, slab, c, v[u], t, parity, u);
        }
        if (g.epi != PF_EPI_QKV) {
          bar_epi();
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            const int c = cb + u * PF_CLUSTER;
            if (c < cols) pf_epi_col_finish(p, g, S, slab, c, v[u], t, parity, u);
          }
          parity ^= 1;
        }
      }
      if (t == 0) pf_stamp(p, ph, 5);
      bar_epi();                         // every thread of this CTA has finished its remote reads
      if (t < PF_CLUSTER) mbar_arrive_remote(&S.red_done, (uint32_t)t);
      ++red_use;
      red_pending = 1;
    }
    ++unit;
  }
  if (red_pending) {                     // the staging region is reused by the next phase
    pf_mbar_wait_cluster(ctx, &S.red_done, (uint32_t)(red_use - 1) & 1u);
    red_pending = 0;
  }
  if (g.epi == PF_EPI_LMHEAD) {
    bar_epi();
    if (t < p.lm_rows) p.sparts[(size_t)t * ncta + cta] = S.rp[t];
  }
  bar_epi();
  if (t == 0) pf_arrive(p, ph);
}

// Last phase: merge the per-CTA partials of every sampled / scored row.
__device__ void pf_sample_merge(const PfParams& p, int cta, int ncta, int t) {
  if (t >= 32) return;
  SampleArgs sa;
  sa.inv_temp = p.inv_temp; sa.alpha = p.alpha; sa.softcap = p.softcap; sa.V = p.V; sa.rows = p.lm_rows;
  sa.call_id = p.call_id; sa.tokens_in = p.tokens_in; sa.seed = p.seed; sa.cycle_counter = p.cycle_counter;
  for (int row = cta; row < p.lm_rows; row += ncta)
    sample_merge_row(sa, p.sparts + (size_t)row * ncta, ncta, 1, row, t, p.tok_out, p.logp_out, p.logz_out);
}

// ---------------------------------------------------------------- embedding phase (warps 2..7)
__device__ void pf_embed_phase(const PfParams& p, int cta, int ncta, int ta) {
  const int warp_a = ta >> 5, lane = ta & 31;
  const int parts = p.d >> 7;
  const int total = p.M * parts;
  for (int it = cta * 6 + warp_a; it < total; it += ncta * 6) {
    const int m = it / parts, part = it - m * parts;
    int id = p.ids[m];
    if (id < 0 || id >= p.V) {
      if (lane == 0) atomicOr(p.status, SMC_ERR_BOUNDS);
      id = 0;
    }
    const int col = part * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(p.embed + (size_t)id * p.d + col);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float4 a = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
    *reinterpret_cast<float4*>(p.h + (size_t)m * p.d + col) = a;
    *reinterpret_cast<uint2*>(p.hb + (size_t)m * p.d + col) = raw;
    const float ss = warp_sum(a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w);
    if (lane == 0) p.ssq[(size_t)part * p.ssq_ld + m] = ss;
  }
}

// ---------------------------------------------------------------- attention phase (warps 2..7, ta = 0..191)
template <int D>
__device__ void pf_attention_phase(const PfParams& p, const PfCtx& ctx, PfShared& S, uint8_t* att_smem, int layer, int cta,
                                   int ncta, int ta) {
  constexpr int LD = D + 8;
  constexpr int TILE = TK * LD;
  constexpr int CPR = D / 8;
  constexpr bool Q_REGS = D <= 128;
  const int warp_a = ta >> 5, lane = ta & 31;
  const int n_mt = p.n_mt, n_kw = p.n_kw, stg = p.att_stg;
  const int G = p.Hq / p.Hkv, R = p.E * G, Rpad = n_mt * 16;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(att_smem);            // [Rpad][LD]
  __nv_bfloat16* Kn = Qs + (size_t)Rpad * LD;                                 // [16][LD]
  __nv_bfloat16* Vn = Kn + 16 * LD;                                           // [16][LD]
  int* pg = reinterpret_cast<int*>(Vn + 16 * LD);                             // [PF_RANGE]
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(pg + PF_RANGE);     // [n_kw][stg][K|V][TK][LD]
  float* marea = reinterpret_cast<float*>(tiles);
  const int slot_floats = 16 * D + 64;
  const bool active = warp_a < n_mt * n_kw;
  const int mt = active ? warp_a % n_mt : 0, kw = active ? warp_a / n_mt : 0;
  const int g = lane >> 2, t = lane & 3;
  const int gsize = 32 * n_mt, gt = mt * 32 + lane;
  __nv_bfloat16* k_pool = p.k_pool + (size_t)layer * p.kv_layer_stride;
  __nv_bfloat16* v_pool = p.v_pool + (size_t)layer * p.kv_layer_stride;
  const size_t kv_row = (size_t)p.Hkv * D;
  __nv_bfloat16* my_tiles = tiles + (size_t)kw * stg * 2 * TILE;
  const int n_items = p.bs * p.Hkv * p.KS;

  for (int item = cta; item < n_items; item += ncta) {
    const int ks = item % p.KS, bk = item / p.KS, kvh = bk % p.Hkv, b = bk / p.Hkv;
    const int hbase = kvh * G;
    bar_att();                                     // the shared memory of the previous item is free
    const int prefix = p.prefix_lens[b];
    int per = (prefix + p.KS - 1) / p.KS;
    per = (per + TK - 1) / TK * TK;
    const int kb = ks * per, ke = min(prefix, kb + per);
    const int* bt = p.block_table + (size_t)p.rows[b] * p.bt_stride;

    auto load_pages = [&](int r0, int r1) {
      for (int i = ta; i < r1 - r0; i += 192) {
        int page = bt[r0 + i];
        if (page < 0 || page > p.n_pages) { atomicOr(p.status, SMC_ERR_BOUNDS); page = 0; }
        pg[i] = page;
      }
    };
    auto issue = [&](int r0, int r1, int tile, int stage) {
      __nv_bfloat16* Kt = my_tiles + (size_t)stage * 2 * TILE;
      __nv_bfloat16* Vt = Kt + TILE;
      const int k0 = tile * TK;
      for (int c = gt; c < TK * CPR; c += gsize) {
        const int key = c / CPR, col = c % CPR;
        const int page = (r0 + k0 + key < r1) ? pg[k0 + key] : 0;
        const size_t off = (size_t)page * kv_row + (size_t)kvh * D + col * 8;
        cp_async16(Kt + key * LD + col * 8, k_pool + off);
        cp_async16(Vt + key * LD + col * 8, v_pool + off);
      }
    };
    auto prologue = [&](int r0, int r1) {
      const int nt_r = (r1 - r0 + TK - 1) / TK;
      for (int j = 0; j < stg - 1; ++j) {
        if (active && kw + j * n_kw < nt_r) issue(r0, r1, kw + j * n_kw, j);
        cp_async_commit();
      }
    };
    if (ta < 16) {
      int pos = 0;
      if (ta < p.E) {
        pos = p.positions[b * p.E + ta];
        if (pos < 0 || pos >= p.max_pos) {
          atomicOr(p.status, SMC_ERR_BOUNDS);
          pos = pos < 0 ? 0 : p.max_pos - 1;
        }
      }
      S.pos[ta] = pos;
    }
    if (kb < ke) load_pages(kb, min(ke, kb + PF_RANGE));
    bar_att();
    if (kb < ke) prologue(kb, min(ke, kb + PF_RANGE));

    // ---- q / k / v of the new tokens: rotary embedding, bf16 ---------------------------------------
    {
      const int half = p.rd >> 1;
      auto real_row = [&](int j, __nv_bfloat16*& dst, const float*& src, int& pos) {
        if (j < R) {
          const int e = j / G, gq = j % G;
          dst = Qs + (size_t)j * LD;
          src = p.qkv + (size_t)(b * p.E + e) * p.nqkv + (size_t)(hbase + gq) * D;
          pos = S.pos[e];
        } else {
          const bool is_k = j < R + p.E;
          const int e = is_k ? j - R : j - R - p.E;
          dst = (is_k ? Kn : Vn) + (size_t)e * LD;
          src = p.qkv + (size_t)(b * p.E + e) * p.nqkv + (size_t)(p.Hq + (is_k ? 0 : p.Hkv)) * D + (size_t)kvh * D;
          pos = S.pos[e];
        }
      };
      auto store4 = [](__nv_bfloat16* dst, float4 v) {
        uint2 o;
        o.x = pack_bf16(v.x, v.y);
        o.y = pack_bf16(v.z, v.w);
        *reinterpret_cast<uint2*>(dst) = o;
      };
      for (int idx = ta; idx < (Rpad - R) * (D / 8); idx += 192)
        *reinterpret_cast<uint4*>(Qs + (size_t)(R + idx / (D / 8)) * LD + (idx % (D / 8)) * 8) = make_uint4(0u, 0u, 0u, 0u);
      for (int idx = ta; idx < 2 * (16 - p.E) * (D / 8); idx += 192) {
        const int rr = idx / (D / 8), c = idx % (D / 8);
        __nv_bfloat16* base = rr < 16 - p.E ? Kn + (size_t)(p.E + rr) * LD : Vn + (size_t)(p.E + rr - (16 - p.E)) * LD;
        *reinterpret_cast<uint4*>(base + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
      const int hq = half >> 2;
      for (int idx = ta; idx < (R + p.E) * hq; idx += 192) {       // rotated part of q and k rows
        const int j = idx / hq, i4 = (idx % hq) * 4;
        __nv_bfloat16* dst; const float* src; int pos;
        real_row(j, dst, src, pos);
        const float* cs = p.rope + (size_t)pos * p.rd;
        const float4 a = __ldcg(reinterpret_cast<const float4*>(src + i4));
        const float4 bb = __ldcg(reinterpret_cast<const float4*>(src + half + i4));
        const float4 c = *reinterpret_cast<const float4*>(cs + i4);
        const float4 sn = *reinterpret_cast<const float4*>(cs + half + i4);
        store4(dst + i4, make_float4(a.x * c.x - bb.x * sn.x, a.y * c.y - bb.y * sn.y, a.z * c.z - bb.z * sn.z,
                                     a.w * c.w - bb.w * sn.w));
        store4(dst + half + i4, make_float4(bb.x * c.x + a.x * sn.x, bb.y * c.y + a.y * sn.y, bb.z * c.z + a.z * sn.z,
                                            bb.w * c.w + a.w * sn.w));
      }
      const int pq = (D - p.rd) >> 2;                               // pass-through dims of q and k rows
      for (int idx = ta; idx < (R + p.E) * pq; idx += 192) {
        const int j = idx / pq, i4 = p.rd + (idx % pq) * 4;
        __nv_bfloat16* dst; const float* src; int pos;
        real_row(j, dst, src, pos);
        store4(dst + i4, __ldcg(reinterpret_cast<const float4*>(src + i4)));
      }
      for (int idx = ta; idx < p.E * (D / 4); idx += 192) {         // value rows
        const int j = R + p.E + idx / (D / 4), i4 = (idx % (D / 4)) * 4;
        __nv_bfloat16* dst; const float* src; int pos;
        real_row(j, dst, src, pos);
        store4(dst + i4, __ldcg(reinterpret_cast<const float4*>(src + i4)));
      }
    }
    bar_att();
    // new K/V rows go to their pages (the last key split of every (sequence, kv head) writes them)
    if (ks == p.KS - 1) {
      for (int c = ta; c < p.E * CPR * 2; c += 192) {
        const bool is_v = c >= p.E * CPR;
        const int cc = is_v ? c - p.E * CPR : c;
        const int e = cc / CPR, col = cc % CPR;
        int loc = p.cache_locs[b * p.E + e];
        if (loc < 0 || loc > p.n_pages) { atomicOr(p.status, SMC_ERR_BOUNDS); loc = 0; }
        const uint4 v = *reinterpret_cast<const uint4*>((is_v ? Vn : Kn) + (size_t)e * LD + col * 8);
        *reinterpret_cast<uint4*>((is_v ? v_pool : k_pool) + (size_t)loc * kv_row + (size_t)kvh * D + col * 8) = v;
      }
    }

    // ---- query fragments, then the cached prefix in 32-key tiles -----------------------------------
    const __nv_bfloat16* Qs_mt = Qs + (size_t)mt * 16 * LD;
    uint32_t qa[Q_REGS ? D / 16 : 1][4];
    if constexpr (Q_REGS) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        qa[kk][0] = *reinterpret_cast<const uint32_t*>(Qs_mt + g * LD + kk * 16 + 2 * t);
        qa[kk][1] = *reinterpret_cast<const uint32_t*>(Qs_mt + (g + 8) * LD + kk * 16 + 2 * t);
        qa[kk][2] = *reinterpret_cast<const uint32_t*>(Qs_mt + g * LD + kk * 16 + 2 * t + 8);
        qa[kk][3] = *reinterpret_cast<const uint32_t*>(Qs_mt + (g + 8) * LD + kk * 16 + 2 * t + 8);
      }
    }
    const int e_row0 = (mt * 16 + g) / G, e_row1 = (mt * 16 + g + 8) / G;
    WarpState<D> st;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) st.o[nt][0] = st.o[nt][1] = st.o[nt][2] = st.o[nt][3] = 0.f;

    for (int r0 = kb; r0 < ke; r0 += PF_RANGE) {
      const int r1 = min(ke, r0 + PF_RANGE);
      const int ntiles = (r1 - r0 + TK - 1) / TK;
      if (r0 != kb) {
        cp_async_wait<0>();
        bar_att();
        load_pages(r0, r1);
        bar_att();
        prologue(r0, r1);
      }
      if (active) {
        int j = 0;
        for (int tile = kw; tile < ntiles; tile += n_kw, ++j) {
          cp_async_wait_dyn(stg - 2);
          group_barrier(3 + kw, gsize);
          const int jn = j + stg - 1;
          if (kw + jn * n_kw < ntiles) issue(r0, r1, kw + jn * n_kw, jn % stg);
          cp_async_commit();
          const int nvalid = min(TK, r1 - r0 - tile * TK);
          const __nv_bfloat16* Kt = my_tiles + (size_t)(j % stg) * 2 * TILE;
          const int key0 = r0 + tile * TK;
          process_tile<D, TK / 8, Q_REGS>(Kt, Kt + TILE, qa, Qs_mt, p.scale, st, nvalid, prefix + e_row0 - key0,
                                          prefix + e_row1 - key0);
        }
      }
    }
    cp_async_wait<0>();
    if (active && ks == p.KS - 1 && kw == 0)
      process_tile<D, 2, Q_REGS>(Kn, Vn, qa, Qs_mt, p.scale, st, p.E, e_row0, e_row1);
    st.l0 += __shfl_xor_sync(0xffffffffu, st.l0, 1);
    st.l0 += __shfl_xor_sync(0xffffffffu, st.l0, 2);
    st.l1 += __shfl_xor_sync(0xffffffffu, st.l1, 1);
    st.l1 += __shfl_xor_sync(0xffffffffu, st.l1, 2);

    // ---- merge the key-ways of this CTA in a fixed order ------------------------------------------
    auto park = [&](float* slot) {
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        *reinterpret_cast<float2*>(slot + g * D + nt * 8 + 2 * t) = make_float2(st.o[nt][0], st.o[nt][1]);
        *reinterpret_cast<float2*>(slot + (g + 8) * D + nt * 8 + 2 * t) = make_float2(st.o[nt][2], st.o[nt][3]);
      }
      if (t == 0) {
        slot[16 * D + g] = st.m0; slot[16 * D + 8 + g] = st.m1;
        slot[16 * D + 16 + g] = st.l0; slot[16 * D + 24 + g] = st.l1;
      }
    };
    auto absorb = [&](const float* slot, bool global) {
      auto ld1 = [&](const float* q) { return global ? __ldcg(q) : *q; };
      auto ld2 = [&](const float* q) { return global ? __ldcg(reinterpret_cast<const float2*>(q)) : *reinterpret_cast<const float2*>(q); };
      const float m0b = ld1(slot + 16 * D + g), m1b = ld1(slot + 16 * D + 8 + g);
      const float l0b = ld1(slot + 16 * D + 16 + g), l1b = ld1(slot + 16 * D + 24 + g);
      const float M0 = fmaxf(st.m0, m0b), M1 = fmaxf(st.m1, m1b);
      const float a0 = M0 == -INFINITY ? 1.f : __expf(st.m0 - M0), b0 = M0 == -INFINITY ? 0.f : __expf(m0b - M0);
      const float a1 = M1 == -INFINITY ? 1.f : __expf(st.m1 - M1), b1 = M1 == -INFINITY ? 0.f : __expf(m1b - M1);
      st.l0 = st.l0 * a0 + l0b * b0; st.l1 = st.l1 * a1 + l1b * b1;
      st.m0 = M0; st.m1 = M1;
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        const float2 x0 = ld2(slot + g * D + nt * 8 + 2 * t);
        const float2 x1 = ld2(slot + (g + 8) * D + nt * 8 + 2 * t);
        st.o[nt][0] = st.o[nt][0] * a0 + x0.x * b0; st.o[nt][1] = st.o[nt][1] * a0 + x0.y * b0;
        st.o[nt][2] = st.o[nt][2] * a1 + x1.x * b1; st.o[nt][3] = st.o[nt][3] * a1 + x1.y * b1;
      }
    };
    bar_att();                                       // every tile has been consumed: the tile area becomes the merge area
    if (active && kw > 0) park(marea + (size_t)((kw - 1) * n_mt + mt) * slot_floats);
    bar_att();
    if (active && kw == 0)
      for (int k2 = 1; k2 < n_kw; ++k2) absorb(marea + (size_t)((k2 - 1) * n_mt + mt) * slot_floats, false);

    // ---- merge the key splits: the last CTA to arrive reduces all of them in split order ------------
    bool writer = true;
    if (p.KS > 1) {
      float* mine = p.att_part + ((size_t)item * n_mt) * slot_floats;
      if (active && kw == 0) {
        float* slot = mine + (size_t)mt * slot_floats;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
          __stcg(reinterpret_cast<float2*>(slot + g * D + nt * 8 + 2 * t), make_float2(st.o[nt][0], st.o[nt][1]));
          __stcg(reinterpret_cast<float2*>(slot + (g + 8) * D + nt * 8 + 2 * t), make_float2(st.o[nt][2], st.o[nt][3]));
        }
        if (t == 0) {
          __stcg(slot + 16 * D + g, st.m0); __stcg(slot + 16 * D + 8 + g, st.m1);
          __stcg(slot + 16 * D + 16 + g, st.l0); __stcg(slot + 16 * D + 24 + g, st.l1);
        }
      }
      bar_att();
      if (ta == 64) {
        __threadfence();
        const int old = atomicAdd(p.att_ctr + bk, 1);
        const int last = old == p.KS - 1;
        if (last) {
          p.att_ctr[bk] = 0;
          __threadfence();
        }
        S.flag = last;
      }
      bar_att();
      writer = S.flag != 0;
      if (writer && active && kw == 0) {
        st.m0 = st.m1 = -INFINITY;
        st.l0 = st.l1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) st.o[nt][0] = st.o[nt][1] = st.o[nt][2] = st.o[nt][3] = 0.f;
        for (int s2 = 0; s2 < p.KS; ++s2)
          absorb(p.att_part + ((size_t)(bk * p.KS + s2) * n_mt + mt) * slot_floats, true);
      }
    }
    if (writer && active && kw == 0) {
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const int r = mt * 16 + g + 8 * hrow;
        if (r >= R) continue;
        const int e = r / G, gq = r % G, tkn = b * p.E + e, head = hbase + gq;
        const float l = hrow ? st.l1 : st.l0;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.attn + ((size_t)tkn * p.Hq + head) * D;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt)
          *reinterpret_cast<uint32_t*>(orow + nt * 8 + 2 * t) =
              pack_bf16(st.o[nt][2 * hrow] * inv, st.o[nt][2 * hrow + 1] * inv);
      }
    }
  }
}

// ---------------------------------------------------------------- the kernel
template <int D>
__global__ void __launch_bounds__(PF_THREADS, 1) pf_forward_kernel(const PfParams p) {
  extern __shared__ uint8_t pf_smem_raw[];
  __shared__ PfShared S;
  const uint32_t raw = smem_u32(pf_smem_raw);
  uint8_t* ring = pf_smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* att_smem = ring + p.ring_bytes;
  const int cta = blockIdx.x, ncta = gridDim.x;
  const int warp = threadIdx.x >> 5;
  PfCtx ctx{&S.abort, p.sync + PF_SYNC_ABORT, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < PF_MAX_STAGES; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&S.acc_full[a], 1);
      mbar_init(&S.acc_empty[a], 4);
    }
    mbar_init(&S.red_full, PF_CLUSTER);
    mbar_init(&S.red_done, PF_CLUSTER);
    S.abort = 0;
    S.open_upto = 0;
    S.issued = 0;
    S.consumed = 0;
    S.flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_slot, PF_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync();                        // every CTA of the cluster has initialised the barriers its peers arrive on
  const uint32_t tmem_base = S.tmem_slot;
  const int n_phases = pf_num_phases(p);

  if (warp == 0) {
    if (elect_one()) pf_producer(p, ctx, S, ring, cta, ncta);
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) pf_mma(p, ctx, S, ring, tmem_base, cta, ncta);
    __syncwarp();
  } else {
    const int ta = (int)threadIdx.x - 64;          // attention-group thread (warps 2..7)
    const int t = (int)threadIdx.x - 128;          // epilogue-group thread (warps 4..7); negative for warps 2, 3
    float* scratch = reinterpret_cast<float*>(att_smem);
    int unit = 0, red_use = 0, red_pending = 0;
    for (int ph = 0; ph < n_phases; ++ph) {
      GemmDesc g;
      if (ph == 0) {
        if (t == 0) pf_stamp(p, ph, 0);
        pf_embed_phase(p, cta, ncta, ta);
        bar_att();
        if (t == 0) pf_arrive(p, ph);
      } else if (pf_gemm_desc(p, ph, g)) {
        if (t >= 0) pf_gemm_epilogue(p, ctx, S, scratch, tmem_base, g, ph, cta, ncta, t, unit, red_use, red_pending);
      } else if (ph <= 5 * p.L) {
        if (t == 0) {
          pf_leader_wait(p, ctx, &S.open_upto, ph, ncta);
          pf_stamp(p, ph, 0);
        }
        bar_att();
        pf_attention_phase<D>(p, ctx, S, att_smem, (ph - 1) / 5, cta, ncta, ta);
        bar_att();
        if (t == 0) pf_arrive(p, ph);
      } else {
        if (t >= 0) {
          if (t == 0) {
            pf_leader_wait(p, ctx, &S.open_upto, ph, ncta);
            pf_stamp(p, ph, 0);
          }
          bar_epi();
          pf_sample_merge(p, cta, ncta, t);
          if (t == 0) pf_stamp(p, ph, 1);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();                        // no CTA leaves while a peer could still touch its shared memory
  if (warp == 1) tmem_dealloc(tmem_base, PF_TMEM_COLS);
  if (threadIdx.x == 0) {
    if (S.abort) {
      // let copies that were requested but never consumed land before the shared memory goes away
      const int issued = S.issued, consumed = S.consumed, nst = p.stages;
      for (int i = consumed; i < issued; ++i) (void)mbar_wait(&S.full[i % nst], (uint32_t)(i / nst) & 1u);
    } else {
      const unsigned int old = atomicAdd(p.sync + PF_SYNC_EXIT, 1u);
      if (old == (unsigned int)ncta - 1u) {          // nobody polls any more: rearm the counters for the next launch
        p.sync[PF_SYNC_BARRIER] = 0u;
        p.sync[PF_SYNC_EXIT] = 0u;
        __threadfence();
      }
    }
  }
}

// shared memory of the attention phase for head size D, n_mt query tiles, n_kw key-ways and stg ring stages
static size_t pf_att_bytes(int D, int n_mt, int n_kw, int stg) {
  const size_t LD = D + 8;
  const size_t base = ((size_t)n_mt * 16 + 32) * LD * 2 + PF_RANGE * 4;
  const size_t tiles = (size_t)n_kw * stg * 2 * TK * LD * 2;
  const size_t merge = (size_t)(n_kw > 1 ? (n_kw - 1) * n_mt : 0) * (16 * D + 64) * 4;
  const size_t epi = 2 * 16 * 129 * 4;             // the GEMM epilogues stage through the same region
  size_t b = base + (tiles > merge ? tiles : merge);
  return b > epi ? b : epi;
}

}  // namespace smc

SMC_API int smc_pf_params_size() { return (int)sizeof(smc::PfParams); }

namespace smc {
static void (*pf_kernel_for(int D))(const PfParams) {
  if (D == 64) return pf_forward_kernel<64>;
  if (D == 128) return pf_forward_kernel<128>;
  return nullptr;
}
static const int PF_DYN_SMEM_MAX = 232448 - (int)sizeof(PfShared) - 512;

// Grid of the persistent kernel: as many clusters of eight CTAs (one CTA per SM) as the device can hold at once.
static int pf_grid(int D) {
  static int cached[2] = {0, 0};
  const int ki = D == 64 ? 0 : 1;
  if (cached[ki] > 0) return cached[ki];
  auto kern = pf_kernel_for(D);
  if (!kern) return -101;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_DYN_SMEM_MAX) != cudaSuccess) return -108;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(PF_CLUSTER);
  cfg.blockDim = dim3(PF_THREADS);
  cfg.dynamicSmemBytes = (size_t)PF_DYN_SMEM_MAX;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PF_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) return -109;
  cached[ki] = n * PF_CLUSTER;
  return cached[ki];
}
}  // namespace smc

// CTAs the persistent kernel is launched with for head size D (a multiple of the cluster size).
SMC_API int smc_pf_num_ctas(int D) { return smc::pf_grid(D); }

// Writes one 128-byte tensor map for a bf16 matrix [rows, cols] of pitch ld (elements) with a [box_rows, 64] box
// into host memory at dst (the caller copies the table to the device).
SMC_API int smc_pf_encode_map(void* dst, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  CUtensorMap tm;
  const int rc = smc::make_tmap(&tm, base, rows, cols, ld, box_rows);
  if (rc) return rc;
  memcpy(dst, &tm, sizeof(tm));
  return 0;
}

// Shapes the attention phase and the weight ring for a batch geometry.  Outputs: query tiles, key-ways, ring depth of
// the K/V tiles, bytes of the attention region, stages and bytes of the weight ring.  Returns 0, or a negative code
// when the geometry is not supported by the persistent kernel.
SMC_API int smc_pf_plan(int D, int E, int G, int BN, int* n_mt, int* n_kw, int* att_stg, int* att_bytes, int* stages,
                        int* ring_bytes) {
  using namespace smc;
  if (!(D == 64 || D == 128)) return -101;
  if (E < 1 || E > 16 || G < 1) return -102;
  if (BN < 16 || BN > 128 || (BN % 16) != 0) return -103;
  const int R = E * G, mt = (R + 15) / 16;
  if (mt > 6) return -104;
  int kw = 6 / mt;
  if (kw > 4) kw = 4;
  int stg = 2;
  while (stg < 4 && pf_att_bytes(D, mt, kw, stg + 1) <= 72 * 1024) ++stg;
  while (kw > 1 && pf_att_bytes(D, mt, kw, stg) > 96 * 1024) --kw;
  size_t att_raw = pf_att_bytes(D, mt, kw, stg);
  if (att_raw < (size_t)BN * 512) att_raw = (size_t)BN * 512;      // the cluster reduction parks a [BN][128] fp32 tile there
  const int att = (int)((att_raw + 1023) / 1024 * 1024);
  const int stage_bytes = PF_A_BYTES + BN * 128;
  const int budget = PF_DYN_SMEM_MAX - 1024 - att;
  int st = budget / stage_bytes;
  if (st > PF_MAX_STAGES) st = PF_MAX_STAGES;
  if (st < 3) return -105;
  *n_mt = mt; *n_kw = kw; *att_stg = stg; *att_bytes = att; *stages = st; *ring_bytes = st * stage_bytes;
  return 0;
}

// Launches one forward on a grid of clusters of eight CTAs, one CTA per SM.  `coop` adds the cooperative-launch
// attribute (all CTAs guaranteed co-resident); without it co-residency relies on the stream being otherwise idle,
// and every wait in the kernel is bounded either way.
SMC_API int smc_pf_forward(const smc::PfParams* p, int coop, cudaStream_t st) {
  using namespace smc;
  auto kern = pf_kernel_for(p->D);
  if (!kern) return -101;
  if (p->M < 1 || p->M > p->BN || p->lm_rows > p->BN || (p->d % 128) != 0 || p->stages < 3 ||
      p->stages > PF_MAX_STAGES || p->Hq % p->Hkv || (p->rd & 7) || p->rd > p->D || ((p->D - p->rd) & 3))
    return -106;
  const int smem = p->ring_bytes + p->att_bytes + 1024;
  if (smem > PF_DYN_SMEM_MAX || p->att_bytes < p->BN * 512) return -110;
  const int ncta = pf_grid(p->D);
  if (ncta <= 0) return ncta < 0 ? ncta : -107;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ncta);
  cfg.blockDim = dim3(PF_THREADS);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PF_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = coop ? 2 : 1;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, kern, *p));
  return 0;
}
