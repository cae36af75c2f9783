// Weight-streaming GEMM for few-token batches on sm_100a:  Y[m, n] = sum_k X[m, k] * W[n, k].
//
// Decode-time SMC batches have 8..72 token rows, so the product is bound by reading W once.
// The operands are swapped for the 5th-generation tensor cores: a 128-row slab of W is the
// M operand of tcgen05.mma, the token rows are the N operand (16..256 wide), and the fp32
// accumulator tile [128 weight rows x tokens] lives in tensor memory.  One CTA streams one
// slab over one K range through a multi-stage TMA -> shared-memory ring (SWIZZLE_128B tiles,
// consumed directly by UMMA descriptors); split-K ranges fill all 148 SMs when a matrix has
// few slabs.  Warp 0 is the TMA producer, warp 1 issues the MMAs, all four warps run the
// epilogue straight out of tensor memory.
//
// Split-K reduction happens on chip: the CTAs of one slab form a thread-block cluster along K,
// park their fp32 tiles in shared memory and sum them in a fixed order through distributed
// shared memory, so the result is deterministic and no partial sums visit HBM.
//
// Epilogues: fp32 store, fp32 accumulate into the residual stream (h += X W^T), fp32 split-K
// partials in global memory (oracle / fallback), bf16 store, and a fused SwiGLU for gate/up
// matrices whose rows are interleaved in blocks of 64 channels.
//
// FP8 (W8A8): with `fp8` set both operands are e4m3 bytes (128 per 128-byte tile row), the MMAs are issued as
// tcgen05.mma.kind::f8f6f4 (K = 32 per instruction, fp32 accumulation) and the epilogues scale every value by the
// weight row's scale and the token's activation scale.  Tiles, ring and descriptors are the same bytes as for bf16.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises a status bit, drains its
// outstanding copies, frees its tensor memory and returns.
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "sample_core.cuh"
#include "tmap_host.h"

namespace smc {

enum { EPI_PARTIAL_F32 = 0, EPI_BF16 = 1, EPI_SWIGLU_BF16 = 2, EPI_STORE_F32 = 3, EPI_RESID_F32 = 4, EPI_RS_F32 = 5,
       EPI_SWIGLU_SPLIT = 6,     // 6: SwiGLU after a split-K reduction inside the cluster
       EPI_LMHEAD = 7 };         // 7: lm_head: every slab is reduced to per-row sampling partials, logits are not stored

// Tensor-parallel links of one GEMM.  Consumer side (all-gather -> GEMM): peers store their
// activation rows into this GPU's buffer and bump a counter here; the TMA producer waits for the
// counter before it fetches activations from local memory.  Producer side (GEMM -> reduce-scatter):
// the epilogue stores each reduced token row straight into the owning rank's receive buffer over
// NVLink (plain peer stores) and bumps that rank's counter.  Counters only grow; the value to wait
// for is derived from a device-resident epoch so captured graphs work unchanged on every replay.
struct TpLink {
  const unsigned long long* ag_flag;   // null: no all-gather wait
  const long long* epoch;              // device epoch, first use has epoch 1
  long long ag_uses, ag_idx, ag_inc;   // wait for ((epoch-1)*uses + idx + 1) * inc
  unsigned long long peer_base[8];     // symmetric-heap base address on every rank
  long long rs_off, rs_flag_off;       // byte offsets of the receive buffer / its counter in the heap
  int tp, rank, rows_per_rank, pad;
  int* arrive;                         // local arrival counter of this call site (self-resetting)
};

struct GemmParams {
  int N, K, M;          // weight rows, reduction length, token rows
  int kblocks;          // ceil(K / 64)
  int m_tiles;          // token tiles (grid x = weight slabs * m_tiles)
  int stages;           // 3 selects the lean build of the 128-token tile (host-side choice only)
  int splits;
  void* out;            // fp32 [splits, M, N] | bf16 [M, ldo]
  int ldo;
  int* status;
  int pdl;              // 1: wait for the previous grid only before touching activations
  TpLink tp;
  // RMSNorm folded into the GEMMs (norm weights are pre-multiplied into W):
  //   consumer side: the activation operand is the raw bf16 residual stream; every output column (token) is scaled
  //     by rstd = rsqrt(sum_p ssq_in[p, m] / norm_d + eps) in the epilogue;
  //   producer side (residual epilogue): besides h += X W^T it writes the bf16 copy of the new rows and the
  //     sum of squares of its 128 columns per token into ssq_out[n_tile, m], summed later in a fixed order.
  const float* ssq_in;
  int ssq_parts, ssq_ld, ssq_mstride;     // token of output row m is ssq column m * ssq_mstride
  float norm_inv_d, norm_eps;
  float* ssq_out;
  __nv_bfloat16* hb_out;
  int hb_ld;
  // lm_head with fused sampling / scoring (EPI_LMHEAD): out = RowPartial [M, slabs]
  SampleArgs samp;
  // FP8 operands: e4m3 bytes, value = byte * scale; w_scale per weight row, x_scale per token row (null: 1)
  int fp8;
  const float* w_scale;
  const float* x_scale;
};

template <int BN, int EPI, bool LEAN>
struct GemmCfg {
  static constexpr int BM = 128, BK = 64;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // Ring depth.  128-token tiles come in two builds: LEAN keeps three 32 KB stages so that two CTAs share an SM
  // (chosen for the split-K epilogues: 8B down at 1152 tokens 193 -> 149 us, and for multi-wave gate/up grids:
  // 325 -> 262 us at 1152 tokens); single-wave gate/up grids keep four (three measured 22 -> 28 us there).
  static constexpr int STAGES = BN <= 32 ? 5 : ((BN == 128 && LEAN) ? 3 : 4);
  static constexpr int TMEM_COLS = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, int EPI, bool LEAN, bool FP8>
__global__ void __launch_bounds__(128) gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW,
                                                         const __grid_constant__ CUtensorMap tmX,
                                                         const GemmParams p) {
  using C = GemmCfg<BN, EPI, LEAN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  constexpr int nst = C::STAGES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + nst * C::STAGE_BYTES);
  uint64_t* empty = full + nst;
  uint64_t* accum = empty + nst;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* sh_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sh_issued = sh_abort + 1;
  volatile int* sh_consumed = sh_abort + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // token tiles of one weight slab are neighbours in launch order, so the slab is fetched from HBM once and
  // the other token tiles find it in L2
  const int n_tile = blockIdx.x / p.m_tiles, split = blockIdx.y, m_tile = blockIdx.x % p.m_tiles;
  // Let the next kernel of the stream start its prologue (and its weight prefetch) right away;
  // it still waits for this grid to finish before it touches anything this grid writes.
  if (p.pdl) pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    *sh_abort = 0;
    *sh_issued = 0;
    *sh_consumed = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // balanced K partition
  const int kb_begin = (int)(((long long)p.kblocks * split) / p.splits);
  const int kb_end = (int)(((long long)p.kblocks * (split + 1)) / p.splits);
  const int nkb = kb_end - kb_begin;

  __shared__ float s_rstd[BN];
  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      constexpr int bk = FP8 ? 2 * C::BK : C::BK;    // elements per 128-byte tile row
      // Weights do not depend on the previous kernel: start streaming them before the
      // programmatic-dependency wait, then fetch the activations.
      const int pre = nkb < nst ? nkb : nst;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], C::STAGE_BYTES);
        tma_load_2d(smem + i * C::STAGE_BYTES, &tmW, &full[i], (kb_begin + i) * bk, n_tile * C::BM, pol_w);
      }
      if (p.pdl) pdl_wait_prior_grid();
      if (p.tp.ag_flag != nullptr) {
        // activations are being pushed by the peers: wait (bounded) for all of their rows
        const unsigned long long want =
            (unsigned long long)(((*p.tp.epoch - 1) * p.tp.ag_uses + p.tp.ag_idx + 1) * p.tp.ag_inc);
        if (!wait_counter_sys(p.tp.ag_flag, want)) {
          atomicOr(p.status, SMC_ERR_PEER_TIMEOUT);
          *sh_abort = 1;
        }
        fence_proxy_async_all();
      }
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem + i * C::STAGE_BYTES + C::A_BYTES, &tmX, &full[i], (kb_begin + i) * bk, m_tile * BN,
                    pol_x);
      *sh_issued = pre;
      // stage index and phase advance by counting (the ring depth is a launch parameter: no division per k-block)
      int s = pre == nst ? 0 : pre;
      uint32_t ph = pre == nst ? 1u : 0u;
      for (int i = pre; i < nkb; ++i, ++s) {
        if (s == nst) { s = 0; ph ^= 1u; }
        if (*sh_abort || !mbar_wait(&empty[s], ph ^ 1u)) {
          *sh_abort = 1;
          break;
        }
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
        tma_load_2d(smem + s * C::STAGE_BYTES, &tmW, &full[s], (kb_begin + i) * bk, n_tile * C::BM, pol_w);
        tma_load_2d(smem + s * C::STAGE_BYTES + C::A_BYTES, &tmX, &full[s], (kb_begin + i) * bk, m_tile * BN,
                    pol_x);
        *sh_issued = i + 1;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(C::BM, BN);
      constexpr uint32_t idesc8 = umma_idesc_e4m3(C::BM, BN);
      int s = 0;
      uint32_t ph = 0u;
      for (int i = 0; i < nkb; ++i, ++s) {
        if (s == nst) { s = 0; ph ^= 1u; }
        if (*sh_abort || !mbar_wait(&full[s], ph)) {
          *sh_abort = 1;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
        const uint64_t adesc = umma_desc_k_sw128(a_addr);
        const uint64_t bdesc = umma_desc_k_sw128(a_addr + C::A_BYTES);
#pragma unroll
        for (int k = 0; k < C::BK / 16; ++k) {   // advance 32 bytes (16 bf16 or 32 e4m3) inside the swizzle atom
          if constexpr (FP8) umma_f8_ss(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc8, (i | k) ? 1u : 0u);
          else umma_bf16_ss(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
        *sh_consumed = i + 1;
      }
      if (!*sh_abort) umma_commit(accum);
    }
    __syncwarp();
  } else {
    // warps 2 and 3 are idle until the epilogue: they turn the per-slab sums of squares of the activation rows
    // into the per-token 1/rms factors while the weight stream runs
    const int tid2 = threadIdx.x - 64;
    if (p.ssq_in != nullptr) {
      if (p.pdl) pdl_wait_prior_grid();
      for (int c = tid2; c < BN; c += 64) {
        const int m = m_tile * BN + c;
        float ss = 0.f;
        if (m < p.M)
          for (int q = 0; q < p.ssq_parts; ++q) ss += p.ssq_in[(size_t)q * p.ssq_ld + (size_t)m * p.ssq_mstride];
        s_rstd[c] = rsqrtf(ss * p.norm_inv_d + p.norm_eps);
      }
    } else if (FP8 && p.x_scale != nullptr) {
      if (p.pdl) pdl_wait_prior_grid();
      for (int c = tid2; c < BN; c += 64) {
        const int m = m_tile * BN + c;
        s_rstd[c] = m < p.M ? p.x_scale[(size_t)m * p.ssq_mstride] : 1.f;
      }
    } else {
      for (int c = tid2; c < BN; c += 64) s_rstd[c] = 1.f;
    }
  }

  // ---- wait for the accumulator (all threads), bounded ------------------------------------
  bool ok = nkb > 0;
  if (ok && !mbar_try_wait(accum, 0)) {
    const long long t0 = clock64();
    for (;;) {
      if (mbar_try_wait(accum, 0)) break;
      if (*sh_abort || clock64() - t0 > SMC_SPIN_CYCLES) {
        ok = false;
        break;
      }
    }
  }
  const int failed = __syncthreads_or(ok ? 0 : 1);
  tc_fence_after();

  if (!failed) {
    const int row_in_tile = warp * 32 + lane;
    const int n = n_tile * C::BM + row_in_tile;
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
    const int m_base = m_tile * BN;
    float wsc = 1.f;                                   // FP8: scale of this weight row
    if constexpr (FP8) wsc = n < p.N ? p.w_scale[n] : 1.f;
    if constexpr (EPI == EPI_SWIGLU_BF16) {
      // rows 0..63 of the slab are gate channels, rows 64..127 the matching up channels
      float* sbuf = reinterpret_cast<float*>(smem);      // the ring is idle: every MMA has completed
      constexpr int LD = BN + 1;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
        if (warp >= 2) {
#pragma unroll
          for (int j = 0; j < 16; ++j) sbuf[(row_in_tile - 64) * LD + c0 + j] = __uint_as_float(r[j]) * wsc;
        }
        __syncthreads();
        if (warp < 2) {
          const int ch = n_tile * 64 + row_in_tile;
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m_base + c0 + j;
            if (m < p.M && ch * 2 < p.N) {
              const float g = __uint_as_float(r[j]) * wsc * s_rstd[c0 + j];
              const float u = sbuf[row_in_tile * LD + c0 + j] * s_rstd[c0 + j];
              out[(size_t)m * p.ldo + ch] = __float2bfloat16(g / (1.0f + __expf(-g)) * u);
            }
          }
        }
        __syncthreads();
      }
    } else if constexpr (EPI == EPI_STORE_F32 || EPI == EPI_RESID_F32 || EPI == EPI_RS_F32 || EPI == EPI_SWIGLU_SPLIT) {
      // park this CTA's tile as sbuf[token][128 weight rows]; the cluster reduces it below
      float* sbuf = reinterpret_cast<float*>(smem);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) sbuf[(c0 + j) * C::BM + row_in_tile] = __uint_as_float(r[j]) * wsc;
      }
    } else if constexpr (EPI == EPI_LMHEAD) {
      // Sampling / scoring straight out of tensor memory: the slab's 128 vocabulary rows are reduced per token to
      // (max, sum-exp, best Gumbel candidate, chosen logit); a small merge kernel combines the slabs.
      float* tr = reinterpret_cast<float*>(smem);        // [2][16][129]; the ring is idle: every MMA has completed
      __shared__ RowPartial s_rp[BN];
      for (int c = threadIdx.x; c < BN; c += 128) s_rp[c] = row_partial_neutral();
      __syncthreads();
      int parity = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN && m_base + c0 < p.M; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
        float* trp = tr + parity * (16 * 129);
#pragma unroll
        for (int j = 0; j < 16; ++j) trp[j * 129 + row_in_tile] = __uint_as_float(r[j]) * wsc * s_rstd[c0 + j];
        __syncthreads();
        lm_reduce_chunk(p.samp, trp, n_tile * C::BM, c0, m_base, (int)threadIdx.x, s_rp);
        parity ^= 1;
      }
      __syncthreads();
      RowPartial* parts = reinterpret_cast<RowPartial*>(p.out);
      const int n_slabs = (p.N + C::BM - 1) / C::BM;
      for (int c = threadIdx.x; c < BN; c += 128)
        if (m_base + c < p.M) parts[(size_t)(m_base + c) * n_slabs + n_tile] = s_rp[c];
    } else {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m_base + c0 + j;
            if (m < p.M) {
              if constexpr (EPI == EPI_PARTIAL_F32) {
                reinterpret_cast<float*>(p.out)[((size_t)split * p.M + m) * p.N + n] =
                    __uint_as_float(r[j]) * wsc * s_rstd[c0 + j];
              } else {
                reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] =
                    __float2bfloat16(__uint_as_float(r[j]) * wsc * s_rstd[c0 + j]);
              }
            }
          }
        }
      }
    }
  } else if (threadIdx.x == 0) {
    if (nkb > 0) atomicOr(p.status, SMC_ERR_BARRIER_TIMEOUT);
    // drain copies that were issued but never consumed, so none lands after the CTA is gone
    const int issued = *sh_issued, consumed = *sh_consumed;
    for (int i = consumed; i < issued; ++i)
      (void)mbar_wait(&full[i % nst], (uint32_t)(i / nst) & 1u);
  }

  if constexpr (EPI == EPI_STORE_F32 || EPI == EPI_RESID_F32 || EPI == EPI_RS_F32 || EPI == EPI_SWIGLU_SPLIT) {
    // ---- on-chip split-K reduction across the cluster (CTA rank == split index) --------------
    // Both cluster barriers are unconditional so that a CTA that gave up still releases its peers.
    __shared__ int sh_failed;
    __shared__ float s_red[4][4];
    __shared__ float s_pair[4][64];      // SwiGLU after the reduction: up rows hand their sums to the gate rows
    if (threadIdx.x == 0) sh_failed = failed;
    cluster_sync();
    const uint32_t S = (uint32_t)p.splits;
    // one thread per rank fetches that rank's flag, so the remote reads overlap instead of queueing up
    int peer_failed = 0;
    if (threadIdx.x < S) peer_failed = ld_dsmem_u32(smem_u32(&sh_failed), threadIdx.x) != 0;
    const bool any_failed = __syncthreads_or(peer_failed) != 0;
    if (!any_failed) {
      const float* sbuf = reinterpret_cast<const float*>(smem);
      const int n = n_tile * C::BM + (int)threadIdx.x;
      const int m_base = m_tile * BN;
      float* out = reinterpret_cast<float*>(p.out);
      // tokens are dealt round-robin to the CTAs of the cluster; ranks are summed in a fixed order.
      // All remote loads of a batch of tokens are issued before the first add, so their
      // latencies overlap instead of queueing up behind one another.
      uint32_t rbase[8];
#pragma unroll
      for (uint32_t s = 0; s < 8; ++s) rbase[s] = s < S ? dsmem_map(smem_u32(sbuf) + threadIdx.x * 4u, s) : 0u;
      constexpr int UN = 4;
      for (int c0 = split; c0 < BN && m_base + c0 < p.M; c0 += (int)S * UN) {
        float v[UN][8];
        float prev[UN];
        float sq[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) sq[u] = 0.f;
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int c = c0 + u * (int)S;
          const bool live = c < BN && m_base + c < p.M;
#pragma unroll
          for (uint32_t s = 0; s < 8; ++s)
            v[u][s] = (live && s < S) ? ld_dsmem_f32_at(rbase[s] + (uint32_t)c * (C::BM * 4u)) : 0.f;
          prev[u] = 0.f;
          if constexpr (EPI == EPI_RESID_F32) {
            if (live && n < p.N) prev[u] = out[(size_t)(m_base + c) * p.ldo + n];
          }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int c = c0 + u * (int)S;
          if (c < BN && m_base + c < p.M && n < p.N) {
            float acc = 0.f;
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) acc += v[u][s];
            acc *= s_rstd[c];
            if constexpr (EPI == EPI_SWIGLU_SPLIT) {
              prev[u] = acc;               // paired below: rows 0..63 are gate channels, 64..127 the matching up channels
            } else if constexpr (EPI == EPI_RS_F32) {
              // reduce-scatter: the token row belongs to rank `owner`; store into its receive buffer
              const int m = m_base + c, owner = m / p.tp.rows_per_rank, ml = m - owner * p.tp.rows_per_rank;
              float* dst = reinterpret_cast<float*>(p.tp.peer_base[owner] + p.tp.rs_off) +
                           ((size_t)p.tp.rank * p.tp.rows_per_rank + ml) * p.ldo + n;
              *dst = acc;
            } else {
              const float hv = prev[u] + acc;
              out[(size_t)(m_base + c) * p.ldo + n] = hv;
              if constexpr (EPI == EPI_RESID_F32) {
                if (p.hb_out != nullptr) p.hb_out[(size_t)(m_base + c) * p.hb_ld + n] = __float2bfloat16(hv);
                sq[u] = hv * hv;
              }
            }
          }
        }
        if constexpr (EPI == EPI_SWIGLU_SPLIT) {
          if (warp >= 2) {
#pragma unroll
            for (int u = 0; u < UN; ++u) s_pair[u][threadIdx.x - 64] = prev[u];
          }
          __syncthreads();
          if (warp < 2) {
            const int ch = n_tile * 64 + (int)threadIdx.x;
            __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
            for (int u = 0; u < UN; ++u) {
              const int c = c0 + u * (int)S;
              if (c < BN && m_base + c < p.M && ch * 2 < p.N) {
                const float g = prev[u], up = s_pair[u][threadIdx.x];
                ob[(size_t)(m_base + c) * p.ldo + ch] = __float2bfloat16(g / (1.0f + __expf(-g)) * up);
              }
            }
          }
          __syncthreads();
        }
        if constexpr (EPI == EPI_RESID_F32) {
          if (p.ssq_out != nullptr) {
            // sum of squares of this slab's 128 columns for each token this CTA owns (block reduction, fixed order)
#pragma unroll
            for (int u = 0; u < UN; ++u) {
              float v = warp_sum(sq[u]);
              if (lane == 0) s_red[u][warp] = v;
            }
            __syncthreads();
            if (threadIdx.x < UN) {
              const int c = c0 + (int)threadIdx.x * (int)S;
              if (c < BN && m_base + c < p.M)
                p.ssq_out[(size_t)n_tile * p.ssq_ld + m_base + c] =
                    s_red[threadIdx.x][0] + s_red[threadIdx.x][1] + s_red[threadIdx.x][2] + s_red[threadIdx.x][3];
            }
            __syncthreads();
          }
        }
      }
    }
    if constexpr (EPI == EPI_RS_F32) {
      // publish: every CTA makes its peer stores visible system-wide and checks in; the last CTA of
      // the grid bumps every rank's counter once, so the counters advance by `tp` per GEMM whatever
      // the batch size is
      // the CTA barrier orders every thread's peer stores before thread 0's fence, and the fence is cumulative, so
      // one system-scope fence per CTA publishes them all
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        const int total = (int)(gridDim.x * gridDim.y * gridDim.z);
        if (atomicAdd(p.tp.arrive, 1) == total - 1) {
          *p.tp.arrive = 0;
          __threadfence_system();
          for (int o = 0; o < p.tp.tp; ++o)
            atomicAdd_system(reinterpret_cast<unsigned long long*>(p.tp.peer_base[o] + p.tp.rs_flag_off), 1ull);
        }
      }
    }
    cluster_sync();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------- host side
template <int BN, int EPI, bool LEAN = false, bool FP8 = false>
static int launch(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, dim3 grid, cudaStream_t st) {
  using C = GemmCfg<BN, EPI, LEAN>;
  static bool configured = false;
  auto kern = gemm_skinny_kernel<BN, EPI, LEAN, FP8>;
  if (!configured) {
    CUDA_CHECK_RET(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (EPI == EPI_STORE_F32 || EPI == EPI_RESID_F32 || EPI == EPI_RS_F32 || EPI == EPI_SWIGLU_SPLIT) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = (unsigned)p.splits;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p));
  return 0;
}

// e4m3 operands: the epilogues the quantised layer chain uses
template <int EPI>
static int dispatch_bn_fp8(int bn, const CUtensorMap& a, const CUtensorMap& b, const GemmParams& p, dim3 g,
                           cudaStream_t st) {
  switch (bn) {
    case 16: return launch<16, EPI, false, true>(a, b, p, g, st);
    case 32: return launch<32, EPI, false, true>(a, b, p, g, st);
    case 64: return launch<64, EPI, false, true>(a, b, p, g, st);
    case 80: return launch<80, EPI, false, true>(a, b, p, g, st);
    case 128: return p.stages == 3 ? launch<128, EPI, true, true>(a, b, p, g, st) : launch<128, EPI, false, true>(a, b, p, g, st);
    case 256: return launch<256, EPI, false, true>(a, b, p, g, st);
  }
  return -10;
}

template <int EPI>
static int dispatch_bn(int bn, const CUtensorMap& a, const CUtensorMap& b, const GemmParams& p, dim3 g, cudaStream_t st) {
  switch (bn) {
    case 16: return launch<16, EPI>(a, b, p, g, st);
    case 32: return launch<32, EPI>(a, b, p, g, st);
    case 64: return launch<64, EPI>(a, b, p, g, st);
    case 80: return launch<80, EPI>(a, b, p, g, st);
    case 128: return p.stages == 3 ? launch<128, EPI, true>(a, b, p, g, st) : launch<128, EPI, false>(a, b, p, g, st);
    case 256: return launch<256, EPI>(a, b, p, g, st);
  }
  return -10;
}

}  // namespace smc

// Token-tile width used for a batch of M rows.
SMC_API int smc_gemm_bn_for(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 80) return 80;
  if (M <= 128) return 128;
  return 256;
}

// Token-tile width for a weight matrix of N rows.  Up to 128 tokens one tile covers the batch.  Beyond that every
// CTA is bound by the bytes it pulls through its SM (a 128-row weight slab plus BN activation rows per k-block),
// so the width is the one that minimises waves x bytes per CTA: e.g. 1152 tokens on 32 slabs run as 288 tiles of
// 128 tokens (two full waves) rather than 160 tiles of 256 (one full wave and a nearly empty one).
static int bn_for(int M, int N, bool clustered) {
  // 65..128 tokens on a gate/up-sized grid: two 64-token tiles per slab (two CTAs per SM, up to 296 in one wave)
  // instead of one 128-token tile per SM (1B gate/up at 128 tokens: 22.0 -> 18.1 us)
  if (!clustered && M > 80 && M <= 128 && N > 0 && ((N + 127) / 128) * 2 <= 296)
    return 64;
  // 81..128 tokens on the split-K epilogues: two 64-token tiles as well (1B down at 128 tokens: 15.3 -> 13.1 us);
  // up to 80 tokens the single 80-token tile of the verify pass stays
  if (clustered && M > 80 && M <= 128 && N > 0) return 64;
  if (M <= 128 || N <= 0) return smc_gemm_bn_for(M);
  const long long n_tiles = (N + 127) / 128;
  long long best_cost = 0;
  int best = 256;
  for (int bn = 256; bn >= 128; bn -= 128) {
    const long long tiles = n_tiles * ((M + bn - 1) / bn);
    const long long slots = bn == 128 ? 296 : 148;      // 128-token tiles run two CTAs per SM (three-stage ring)
    const long long waves = (tiles + slots - 1) / slots;
    const long long cost = waves * (128 + bn);
    if (best_cost == 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

// Split-K factor that gives every SM about two resident CTAs while keeping >= 4 k-blocks per CTA.
SMC_API int smc_gemm_default_splits(int N, int K, int M) {
  const int n_tiles = (N + 127) / 128;
  const int bn = bn_for(M, N, false);
  const int m_tiles = (M + bn - 1) / bn;
  const int kblocks = (K + 63) / 64;
  int s = (296 + n_tiles * m_tiles - 1) / (n_tiles * m_tiles);
  int cap = kblocks / 4;
  if (cap < 1) cap = 1;
  if (s > cap) s = cap;
  if (s > 32) s = 32;
  if (s < 1) s = 1;
  return s;
}

// Cluster size for the on-chip split-K epilogues: the largest power of two that keeps the grid within about two
// CTAs per SM and leaves every CTA at least two k-blocks.  The kernel accepts any size from 1 to 8, but sizes that
// are not powers of two measured clearly slower on B200 (8B QKV, 48 slabs: 3 -> 17.0 us, 4 -> 15.7 us, 6 -> 22.0 us).
SMC_API int smc_gemm_cluster_splits(int N, int K, int M) {
  const int n_tiles = (N + 127) / 128;
  const int bn = bn_for(M, N, true);
  const int m_tiles = (M + bn - 1) / bn;
  const int kblocks = (K + 63) / 64;
  int s = 1;
  while (s < 8 && n_tiles * m_tiles * s * 2 <= 256 && kblocks / (s * 2) >= 2) s *= 2;
  return s;
}

// W [N, K] bf16 row-major, X [M, ldx] bf16 row-major (ldx >= K).
// epi 3: out = fp32 [M, ldo] = X W^T;  epi 4: out (fp32 [M, ldo]) += X W^T.  Both reduce split-K inside a
// thread-block cluster, so splits must be 1..8.
// epi 0: out = fp32 [splits, M, N] partials; epi 1: out = bf16 [M, ldo] (splits must be 1);
// epi 2: out = bf16 [M, ldo] holding SwiGLU(gate, up) for N/2 channels (N % 128 == 0; splits > 1 reduce split-K
//        inside a cluster first).
struct NormLink {            // host-side description of the folded RMSNorm (all fields optional)
  const float* ssq_in; int ssq_parts; int ssq_ld; int norm_d; float norm_eps; float* ssq_out; void* hb_out; int hb_ld;
  int ssq_mstride;
};

// Encoded tensor maps are cached per (base, shape, pitch, box): an encode costs a driver call, and eager chains
// (prompt passes, batches beyond the graph caps) issue two per GEMM with the same few operands over and over.
struct TmapKey {
  const void* base; long long rows, cols, ld; int box, es;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box && es == o.es;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    h = h * 1000003u ^ std::hash<long long>()(k.rows * 131 + k.box * 2 + k.es);
    h = h * 1000003u ^ std::hash<long long>()(k.cols * 8191 + k.ld);
    return h;
  }
};
static int cached_tmap(CUtensorMap* tm, const void* base, long long rows, long long cols, long long ld, int box,
                       int es = 2) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  const TmapKey key{base, rows, cols, ld, box, es};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *tm = it->second; return 0; }
  const int rc = es == 1 ? smc::make_tmap_u8(tm, base, rows, cols, ld, box) : smc::make_tmap(tm, base, rows, cols, ld, box);
  if (rc == 0) {
    if (cache.size() > 65536) cache.clear();
    cache.emplace(key, *tm);
  }
  return rc;
}

struct Fp8Link { const float* w_scale; const float* x_scale; };      // e4m3 operands with their dequantisation scales

static int gemm_entry(const void* W, const void* X, void* out, int N, int K, int M, int ldx, int ldo, int splits,
                      int epi, int* status, int pdl, const smc::TpLink* tp, const NormLink* nl, cudaStream_t stream,
                      const smc::SampleArgs* samp = nullptr, const Fp8Link* f8 = nullptr) {
  using namespace smc;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int es = f8 != nullptr ? 1 : 2;                 // element size in bytes
  if ((K * es) % 16 != 0 || (ldx * es) % 16 != 0) return -20;       // row pitch must be a multiple of 16 bytes
  if (f8 != nullptr && nl != nullptr) return -28;
  if (epi == EPI_SWIGLU_BF16 && splits > 1) epi = EPI_SWIGLU_SPLIT;      // split-K reduced in the cluster, then SwiGLU
  const bool clustered = epi == EPI_STORE_F32 || epi == EPI_RESID_F32 || epi == EPI_RS_F32 || epi == EPI_SWIGLU_SPLIT;
  if (!clustered && epi != EPI_PARTIAL_F32 && splits != 1) return -21;
  if (clustered && (splits < 1 || splits > 8)) return -23;
  if ((epi == EPI_SWIGLU_BF16 || epi == EPI_SWIGLU_SPLIT) && (N % 128) != 0) return -22;
  if (epi == EPI_RS_F32 && (tp == nullptr || tp->tp < 1 || tp->tp > 8 || tp->rows_per_rank < 1)) return -24;
  if (epi == EPI_LMHEAD && (samp == nullptr || splits != 1 || M > 256)) return -26;
  const int bn = bn_for(M, N, clustered);
  GemmParams p;
  p.N = N; p.K = K; p.M = M;
  p.kblocks = f8 != nullptr ? (K + 127) / 128 : (K + 63) / 64;
  p.fp8 = f8 != nullptr; p.w_scale = f8 ? f8->w_scale : nullptr; p.x_scale = f8 ? f8->x_scale : nullptr;
  p.splits = splits < 1 ? 1 : (splits > p.kblocks ? p.kblocks : splits);
  p.out = out; p.ldo = ldo; p.status = status; p.pdl = pdl;
  if (tp != nullptr) p.tp = *tp; else memset(&p.tp, 0, sizeof(p.tp));
  p.ssq_mstride = 1;
  p.ssq_in = nullptr; p.ssq_parts = 0; p.ssq_ld = 0; p.norm_inv_d = 0.f; p.norm_eps = 0.f; p.ssq_out = nullptr;
  p.hb_out = nullptr; p.hb_ld = 0;
  memset(&p.samp, 0, sizeof(p.samp));
  if (samp != nullptr) p.samp = *samp;
  if (nl != nullptr) {
    p.ssq_in = nl->ssq_in; p.ssq_parts = nl->ssq_parts; p.ssq_ld = nl->ssq_ld;
    p.norm_inv_d = nl->norm_d > 0 ? 1.0f / (float)nl->norm_d : 0.f; p.norm_eps = nl->norm_eps;
    p.ssq_out = nl->ssq_out; p.hb_out = (__nv_bfloat16*)nl->hb_out; p.hb_ld = nl->hb_ld;
    p.ssq_mstride = nl->ssq_mstride > 0 ? nl->ssq_mstride : 1;
    if (p.ssq_out != nullptr && epi != EPI_RESID_F32) return -25;
  }
  CUtensorMap tmW, tmX;
  int rc = cached_tmap(&tmW, W, N, K, K, 128, es);
  if (rc) return rc;
  rc = cached_tmap(&tmX, X, M, K, ldx, bn, es);
  if (rc) return rc;
  p.m_tiles = (M + bn - 1) / bn;
  {
    // ring depth: 128-token tiles drop to three stages where two CTAs per SM pay off (see GemmCfg)
    const long long tiles = (long long)((N + 127) / 128) * p.m_tiles * p.splits;
    p.stages = bn <= 32 ? 5 : 4;
    if (bn == 128 && (clustered || tiles > 148)) p.stages = 3;
  }
  dim3 grid(((N + 127) / 128) * p.m_tiles, p.splits, 1);
  if (p.fp8) {
    switch (epi) {
      case EPI_BF16: return dispatch_bn_fp8<EPI_BF16>(bn, tmW, tmX, p, grid, stream);
      case EPI_SWIGLU_BF16: return dispatch_bn_fp8<EPI_SWIGLU_BF16>(bn, tmW, tmX, p, grid, stream);
      case EPI_STORE_F32: return dispatch_bn_fp8<EPI_STORE_F32>(bn, tmW, tmX, p, grid, stream);
      case EPI_RESID_F32: return dispatch_bn_fp8<EPI_RESID_F32>(bn, tmW, tmX, p, grid, stream);
      case EPI_SWIGLU_SPLIT: return dispatch_bn_fp8<EPI_SWIGLU_SPLIT>(bn, tmW, tmX, p, grid, stream);
    }
    return -30;
  }
  switch (epi) {
    case EPI_PARTIAL_F32: return dispatch_bn<EPI_PARTIAL_F32>(bn, tmW, tmX, p, grid, stream);
    case EPI_BF16: return dispatch_bn<EPI_BF16>(bn, tmW, tmX, p, grid, stream);
    case EPI_SWIGLU_BF16: return dispatch_bn<EPI_SWIGLU_BF16>(bn, tmW, tmX, p, grid, stream);
    case EPI_STORE_F32: return dispatch_bn<EPI_STORE_F32>(bn, tmW, tmX, p, grid, stream);
    case EPI_RESID_F32: return dispatch_bn<EPI_RESID_F32>(bn, tmW, tmX, p, grid, stream);
    case EPI_RS_F32: return dispatch_bn<EPI_RS_F32>(bn, tmW, tmX, p, grid, stream);
    case EPI_SWIGLU_SPLIT: return dispatch_bn<EPI_SWIGLU_SPLIT>(bn, tmW, tmX, p, grid, stream);
    case EPI_LMHEAD: return dispatch_bn<EPI_LMHEAD>(bn, tmW, tmX, p, grid, stream);
  }
  return -11;
}

SMC_API int smc_gemm_skinny(const void* W, const void* X, void* out, int N, int K, int M, int ldx, int ldo,
                            int splits, int epi, int* status, int pdl, cudaStream_t stream) {
  return gemm_entry(W, X, out, N, K, M, ldx, ldo, splits, epi, status, pdl, nullptr, nullptr, stream);
}

// FP8 variant (W8A8): W [N, K] and X [M, ldx] hold e4m3 bytes; w_scale [N] and x_scale [M] (fp32) are the per-row
// dequantisation scales applied in the epilogue (x_scale may be null).  K and ldx must be multiples of 16.
SMC_API int smc_gemm_skinny_fp8(const void* W, const void* X, void* out, int N, int K, int M, int ldx, int ldo,
                                int splits, int epi, const float* w_scale, const float* x_scale, int* status, int pdl,
                                cudaStream_t stream) {
  if (w_scale == nullptr) return -29;
  Fp8Link f8 = {w_scale, x_scale};
  return gemm_entry(W, X, out, N, K, M, ldx, ldo, splits, epi, status, pdl, nullptr, nullptr, stream, nullptr, &f8);
}

// Tensor-parallel variant: `tp` describes the all-gather wait of the activation operand and / or the
// reduce-scatter target of the output (epi 5: reduced token rows are stored into the owning rank's
// receive buffer [src_rank, rows_per_rank, ldo] fp32 and that rank's counter is bumped).
SMC_API int smc_gemm_skinny_tp(const void* W, const void* X, void* out, int N, int K, int M, int ldx, int ldo,
                               int splits, int epi, int* status, int pdl, const smc::TpLink* tp,
                               cudaStream_t stream) {
  return gemm_entry(W, X, out, N, K, M, ldx, ldo, splits, epi, status, pdl, tp, nullptr, stream);
}

// GEMM with the RMSNorm folded in.  ssq_in [ssq_parts, ssq_ld] fp32: per-token partial sums of squares of the
// activation rows (null: no scaling); outputs are scaled per token by rsqrt(sum / norm_d + eps).  With epi 4 and
// ssq_out / hb_out given, the residual epilogue also emits the bf16 copy of the updated rows and their per-slab
// sums of squares ssq_out[n_tile, m] for the next consumer.
SMC_API int smc_gemm_skinny_norm(const void* W, const void* X, void* out, int N, int K, int M, int ldx, int ldo,
                                 int splits, int epi, int* status, int pdl, const float* ssq_in, int ssq_parts,
                                 int ssq_ld, int norm_d, float norm_eps, float* ssq_out, void* hb_out, int hb_ld,
                                 int ssq_mstride, cudaStream_t stream) {
  NormLink nl = {ssq_in, ssq_parts, ssq_ld, norm_d, norm_eps, ssq_out, hb_out, hb_ld, ssq_mstride};
  return gemm_entry(W, X, out, N, K, M, ldx, ldo, splits, epi, status, pdl, nullptr, &nl, stream);
}

namespace smc {
__global__ void __launch_bounds__(32) lm_sample_merge_kernel(SampleArgs a, const RowPartial* __restrict__ parts,
                                                            int n_slabs, int* tok_out, float* logp_out,
                                                            float* logz_out, int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int row = blockIdx.x;
  sample_merge_row(a, parts + (size_t)row * n_slabs, n_slabs, 1, row, (int)threadIdx.x, tok_out, logp_out, logz_out);
}
}  // namespace smc

SMC_API int smc_lm_parts_bytes(int rows, int V) { return rows * ((V + 127) / 128) * (int)sizeof(smc::RowPartial); }

// lm_head fused with sampling / scoring: logits = (X W^T) * rstd are reduced per 128-row vocabulary slab inside the
// GEMM epilogue (they never reach memory), then one warp per row merges the slabs.  Rows choose their mode through
// tokens_in (>= 0: score that token, < 0 or null: sample from softmax(alpha * x / T)); same outputs and the same
// noise stream as smc_sample_or_score on stored logits.  parts: scratch of smc_lm_parts_bytes(M, V) bytes.
SMC_API int smc_lm_head_sample(const void* W, const void* X, int V, int K, int M, int ldx, int* status, int pdl,
                               const float* ssq_in, int ssq_parts, int ssq_ld, int norm_d, float norm_eps,
                               int ssq_mstride, float temperature, float alpha, float softcap, const int* tokens_in,
                               unsigned long long seed, const long long* cycle_counter, int call_id, void* parts,
                               int* tok_out, float* logp_out, float* logz_out, cudaStream_t stream) {
  using namespace smc;
  if (M <= 0) return 0;
  if (temperature <= 0.f || parts == nullptr || cycle_counter == nullptr) return -27;
  SampleArgs a;
  a.inv_temp = 1.0f / temperature; a.alpha = alpha; a.softcap = softcap; a.V = V; a.rows = M; a.call_id = call_id;
  a.tokens_in = tokens_in; a.seed = seed; a.cycle_counter = cycle_counter;
  NormLink nl = {ssq_in, ssq_parts, ssq_ld, norm_d, norm_eps, nullptr, nullptr, 0, ssq_mstride};
  int rc = gemm_entry(W, X, parts, V, K, M, ldx, 0, 1, EPI_LMHEAD, status, pdl, nullptr, &nl, stream, &a);
  if (rc) return rc;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)M);
  cfg.blockDim = dim3(32);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, lm_sample_merge_kernel, a, (const RowPartial*)parts, (V + 127) / 128, tok_out,
                                    logp_out, logz_out, pdl));
  return 0;
}

SMC_API int smc_tp_link_size() { return (int)sizeof(smc::TpLink); }
