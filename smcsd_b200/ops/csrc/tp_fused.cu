// Tensor-parallel glue kernels over NVLink peer memory (no NCCL on these paths).
//
// Activations between the sharded GEMMs are token-row sharded: rank r owns rows
// [r * rows_per_rank, (r+1) * rows_per_rank) of the residual stream.
//
//   tp_norm_allgather   consumer of GEMM -> reduce-scatter and producer of all-gather -> GEMM:
//                       waits (bounded) for every rank's partial rows, h += sum of partials
//                       (or h = embedding row), RMSNorm, then stores the bf16 row into EVERY rank's
//                       full activation buffer and bumps their counters.
//   tp_sample_stage1/2  vocab-parallel lm_head epilogue: each rank scans its vocabulary shard once
//                       (max / sum-exp / Gumbel-argmax candidate / chosen-token logit), stores the
//                       per-chunk partials into every rank's gather buffer, and each rank merges all
//                       shards in a fixed order, so every rank draws the same token and computes the
//                       same log-probabilities without an all-gather of logits.
//
// All cross-GPU waits are bounded and report SMC_ERR_PEER_TIMEOUT through the status word.
#include "common.cuh"

namespace smc {

struct TpPeers {
  unsigned long long base[8];
  int tp, rank;
};

constexpr int TPN_THREADS = 256;
constexpr int TPN_MAXV = 8;

// grid = rows owned by this rank.  rs_buf [tp, rows_per_rank, d] fp32 (local), h_local [rows_per_rank, d].
__global__ void __launch_bounds__(TPN_THREADS)
tp_norm_allgather_kernel(TpPeers peers, float* __restrict__ h_local, const float* __restrict__ rs_buf,
                         const unsigned long long* __restrict__ rs_flag, long long rs_uses, long long rs_idx,
                         long long rs_inc, const long long* __restrict__ epoch, const int* __restrict__ ids,
                         const __nv_bfloat16* __restrict__ embed, const __nv_bfloat16* __restrict__ w,
                         long long xn_off, long long ag_flag_off, int rows_per_rank, int my_rows, int d, float eps,
                         int plus_one, int* arrive, int* status, int pdl) {
  __shared__ float red[32];
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int row = blockIdx.x;
  if (my_rows == 0) {
    // a rank that owns no rows of this batch still takes part in the handshake
    if (threadIdx.x == 0) {
      if (rs_buf != nullptr) {
        const unsigned long long want = (unsigned long long)(((*epoch - 1) * rs_uses + rs_idx + 1) * rs_inc);
        if (!wait_counter_sys(rs_flag, want)) atomicOr(status, SMC_ERR_PEER_TIMEOUT);
      }
      for (int pr = 0; pr < peers.tp; ++pr)
        atomicAdd_system(reinterpret_cast<unsigned long long*>(peers.base[pr] + ag_flag_off), 1ull);
    }
    return;
  }
  if (row >= my_rows) return;
  if (rs_buf != nullptr && threadIdx.x == 0) {
    const unsigned long long want = (unsigned long long)(((*epoch - 1) * rs_uses + rs_idx + 1) * rs_inc);
    if (!wait_counter_sys(rs_flag, want)) atomicOr(status, SMC_ERR_PEER_TIMEOUT);
  }
  __syncthreads();
  const int nvec = d >> 2;
  const int grow = peers.rank * rows_per_rank + row;     // global token row
  float4 v[TPN_MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < TPN_MAXV; ++i) {
    const int c = threadIdx.x + i * TPN_THREADS;
    if (c < nvec) {
      float4 a;
      if (ids != nullptr) {
        const uint2 raw = *reinterpret_cast<const uint2*>(embed + (size_t)ids[grow] * d + c * 4);
        const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        a = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
      } else {
        a = reinterpret_cast<const float4*>(h_local + (size_t)row * d)[c];
      }
      if (rs_buf != nullptr) {
        for (int s = 0; s < peers.tp; ++s) {     // fixed order: identical on every replay
          const float4 b = reinterpret_cast<const float4*>(rs_buf + ((size_t)s * rows_per_rank + row) * d)[c];
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
      }
      v[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = (threadIdx.x & 31) < (TPN_THREADS >> 5) ? red[threadIdx.x & 31] : 0.f;
  tot = warp_sum(tot);
  const float inv = rsqrtf(tot / (float)d + eps);
#pragma unroll
  for (int i = 0; i < TPN_MAXV; ++i) {
    const int c = threadIdx.x + i * TPN_THREADS;
    if (c < nvec) {
      reinterpret_cast<float4*>(h_local + (size_t)row * d)[c] = v[i];
      const uint2 wr = *reinterpret_cast<const uint2*>(w + c * 4);
      const __nv_bfloat162 w0 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x);
      const __nv_bfloat162 w1 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
      const float add = plus_one ? 1.f : 0.f;
      __nv_bfloat162 o0 = __floats2bfloat162_rn(v[i].x * inv * (__low2float(w0) + add),
                                                v[i].y * inv * (__high2float(w0) + add));
      __nv_bfloat162 o1 = __floats2bfloat162_rn(v[i].z * inv * (__low2float(w1) + add),
                                                v[i].w * inv * (__high2float(w1) + add));
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&o0);
      o.y = *reinterpret_cast<uint32_t*>(&o1);
      // all-gather by peer stores: the row lands in every rank's full activation buffer
      for (int pr = 0; pr < peers.tp; ++pr) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peers.base[pr] + xn_off) + (size_t)grow * d + c * 4;
        *reinterpret_cast<uint2*>(dst) = o;
      }
    }
  }
  // the last row of this rank to finish tells every peer that this rank's rows have landed
  // one cumulative system-scope fence per CTA (after the CTA barrier) publishes every thread's peer stores
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
  if (threadIdx.x == 0 && atomicAdd(arrive, 1) == my_rows - 1) {
    *arrive = 0;
    __threadfence_system();
    for (int pr = 0; pr < peers.tp; ++pr)
      atomicAdd_system(reinterpret_cast<unsigned long long*>(peers.base[pr] + ag_flag_off), 1ull);
  }
}

// ---------------------------------------------------------------------------------------------------
struct RowPartialTP {
  float max_s, sum_s, max_b, sum_b, best, best_scaled;
  int best_idx;      // global vocabulary index
  float given;       // scaled-by-1/T logit of the given token if it lies in this shard, else -inf
};

__device__ __forceinline__ void lse_merge2(float& m, float& s, float m2, float s2) {
  const float M = fmaxf(m, m2);
  if (M == -INFINITY) { m = M; s = 0.f; return; }
  s = s * __expf(m - M) + s2 * __expf(m2 - M);
  m = M;
}

constexpr int TS_THREADS = 256;

// grid (rows, nchunks).  logits: this rank's shard [rows(row_stride), Vshard] fp32; v0 = first global index.
__global__ void __launch_bounds__(TS_THREADS)
tp_sample_stage1_kernel(TpPeers peers, const float* __restrict__ logits, long long row_stride, int Vshard, int v0,
                        int Vtotal, float inv_temp, float alpha, const int* __restrict__ tokens_in, uint64_t seed,
                        const long long* __restrict__ cycle_counter, int call_id, float softcap, long long gather_off,
                        long long flag_off, int rows, int* arrive, int* status, int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int row = blockIdx.x, chunk = blockIdx.y, nchunks = gridDim.y;
  const int per = (((Vshard + nchunks - 1) / nchunks) + 3) & ~3;
  const int c_begin = chunk * per, c_end = min(min(Vshard, Vtotal - v0), c_begin + per);
  const int given_tok = tokens_in ? tokens_in[row] : -1;
  const bool sampling = given_tok < 0;
  const float* base = logits + (size_t)row * row_stride;
  const Philox rng(seed);
  const uint32_t ctr_lo = (uint32_t)(*cycle_counter), ctr_hi = (uint32_t)((*cycle_counter) >> 32);
  float max_s = -INFINITY, sum_s = 0.f, max_b = -INFINITY, sum_b = 0.f, best = -INFINITY, best_scaled = 0.f;
  float given = -INFINITY;
  int best_idx = v0 + (c_begin < Vshard ? c_begin : 0);
  for (int c = c_begin + threadIdx.x * 4; c < c_end; c += TS_THREADS * 4) {
    float x[4];
    if (c + 3 < c_end) {
      const float4 a = *reinterpret_cast<const float4*>(base + c);
      x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    } else {
      for (int j = 0; j < 4; ++j) x[j] = (c + j < c_end) ? base[c + j] : -INFINITY;
    }
    uint32_t rnd[4] = {0, 0, 0, 0};
    // the counter uses the GLOBAL column, so the draw does not depend on how the vocabulary is sharded
    if (sampling) rng.run((uint32_t)((v0 + c) >> 2), (uint32_t)row, (uint32_t)call_id ^ (ctr_hi << 8), ctr_lo, rnd);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (c + j >= c_end) continue;
      float v = x[j];
      if (softcap > 0.f) v = tanhf(v / softcap) * softcap;
      const float b = v * inv_temp;
      const float sc = b * alpha;
      if (sc > max_s) { sum_s = sum_s * __expf(max_s - sc) + 1.f; max_s = sc; } else { sum_s += __expf(sc - max_s); }
      if (alpha != 1.f) {
        if (b > max_b) { sum_b = sum_b * __expf(max_b - b) + 1.f; max_b = b; } else { sum_b += __expf(b - max_b); }
      }
      if (sampling) {
        const float u = u32_to_unit(rnd[j]);
        const float pert = sc - __logf(-__logf(u));
        if (pert > best) { best = pert; best_scaled = sc; best_idx = v0 + c + j; }
      } else if (v0 + c + j == given_tok) {
        given = b;
      }
    }
  }
  __shared__ RowPartialTP red[TS_THREADS / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lse_merge2(max_s, sum_s, __shfl_xor_sync(0xffffffffu, max_s, o), __shfl_xor_sync(0xffffffffu, sum_s, o));
    lse_merge2(max_b, sum_b, __shfl_xor_sync(0xffffffffu, max_b, o), __shfl_xor_sync(0xffffffffu, sum_b, o));
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o), bs2 = __shfl_xor_sync(0xffffffffu, best_scaled, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_idx, o);
    if (b2 > best || (b2 == best && i2 < best_idx)) { best = b2; best_scaled = bs2; best_idx = i2; }
    given = fmaxf(given, __shfl_xor_sync(0xffffffffu, given, o));
  }
  if (lane == 0) red[warp] = RowPartialTP{max_s, sum_s, max_b, sum_b, best, best_scaled, best_idx, given};
  __syncthreads();
  if (threadIdx.x == 0) {
    RowPartialTP a = red[0];
    for (int w = 1; w < TS_THREADS / 32; ++w) {
      const RowPartialTP b2 = red[w];
      lse_merge2(a.max_s, a.sum_s, b2.max_s, b2.sum_s);
      lse_merge2(a.max_b, a.sum_b, b2.max_b, b2.sum_b);
      if (b2.best > a.best || (b2.best == a.best && b2.best_idx < a.best_idx)) {
        a.best = b2.best; a.best_scaled = b2.best_scaled; a.best_idx = b2.best_idx;
      }
      a.given = fmaxf(a.given, b2.given);
    }
    // gather buffer on every rank: [tp, rows, nchunks] records; exchange by peer stores
    const size_t slot = ((size_t)peers.rank * rows + row) * nchunks + chunk;
    for (int pr = 0; pr < peers.tp; ++pr) {
      RowPartialTP* dst = reinterpret_cast<RowPartialTP*>(peers.base[pr] + gather_off) + slot;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&a);
      *(reinterpret_cast<uint4*>(dst) + 1) = *(reinterpret_cast<const uint4*>(&a) + 1);
    }
    __threadfence_system();
    if (atomicAdd(arrive, 1) == (int)(gridDim.x * gridDim.y) - 1) {
      *arrive = 0;
      __threadfence_system();
      for (int pr = 0; pr < peers.tp; ++pr)
        atomicAdd_system(reinterpret_cast<unsigned long long*>(peers.base[pr] + flag_off), 1ull);
    }
  }
}

__global__ void tp_sample_stage2_kernel(const RowPartialTP* __restrict__ gather, int tp, int nchunks, int rows,
                                        const unsigned long long* __restrict__ flag, long long uses, long long idx,
                                        const long long* __restrict__ epoch, float alpha,
                                        const int* __restrict__ tokens_in, int* __restrict__ tok_out,
                                        float* __restrict__ logp_out, float* __restrict__ logz_out, int* status,
                                        int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  __shared__ int ok;
  if (threadIdx.x == 0) {
    const unsigned long long want =
        (unsigned long long)(((*epoch - 1) * uses + idx + 1) * (long long)tp);
    ok = wait_counter_sys(flag, want) ? 1 : 0;
    if (!ok) atomicOr(status, SMC_ERR_PEER_TIMEOUT);
  }
  __syncthreads();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  RowPartialTP a = gather[(size_t)row * nchunks];
  for (int s = 0; s < tp; ++s)
    for (int c = (s == 0 ? 1 : 0); c < nchunks; ++c) {
      const RowPartialTP b2 = gather[((size_t)s * rows + row) * nchunks + c];
      lse_merge2(a.max_s, a.sum_s, b2.max_s, b2.sum_s);
      lse_merge2(a.max_b, a.sum_b, b2.max_b, b2.sum_b);
      if (b2.best > a.best || (b2.best == a.best && b2.best_idx < a.best_idx)) {
        a.best = b2.best; a.best_scaled = b2.best_scaled; a.best_idx = b2.best_idx;
      }
      a.given = fmaxf(a.given, b2.given);
    }
  const float lse_s = a.max_s + __logf(a.sum_s);
  const int given = tokens_in ? tokens_in[row] : -1;
  if (given >= 0) {
    const float lse_b = (alpha != 1.f) ? a.max_b + __logf(a.sum_b) : lse_s;
    tok_out[row] = given;
    logp_out[row] = a.given - lse_b;
    if (logz_out) logz_out[row] = 0.f;
  } else {
    tok_out[row] = a.best_idx;
    logp_out[row] = a.best_scaled - lse_s;
    if (logz_out) logz_out[row] = (alpha != 1.f) ? lse_s - alpha * (a.max_b + __logf(a.sum_b)) : 0.f;
  }
}

// Test helper: one "peer" increments a counter; used to exercise the bounded-wait timeout path on a
// single GPU by simply not running it.
__global__ void tp_bump_counter_kernel(unsigned long long* flag, unsigned long long by) {
  if (threadIdx.x == 0 && blockIdx.x == 0) atomicAdd_system(flag, by);
}

// Waits for a counter with the library's bounded spin and records the outcome (1 reached, 0 timeout).
__global__ void tp_wait_counter_kernel(const unsigned long long* flag, unsigned long long want, int* outcome,
                                       int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const bool ok = wait_counter_sys(flag, want);
    *outcome = ok ? 1 : 0;
    if (!ok) atomicOr(status, SMC_ERR_PEER_TIMEOUT);
  }
}

static void set_pdl(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int pdl) {
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
}

}  // namespace smc

SMC_API int smc_tp_peers_size() { return (int)sizeof(smc::TpPeers); }
SMC_API int smc_tp_partial_bytes() { return (int)sizeof(smc::RowPartialTP); }

SMC_API int smc_tp_norm_allgather(const smc::TpPeers* peers, float* h_local, const float* rs_buf,
                                  const unsigned long long* rs_flag, long long rs_uses, long long rs_idx,
                                  long long rs_inc, const long long* epoch, const int* ids, const void* embed,
                                  const void* w, long long xn_off, long long ag_flag_off, int rows_per_rank,
                                  int my_rows, int d, float eps, int plus_one, int* arrive, int* status, int pdl,
                                  cudaStream_t st) {
  using namespace smc;
  if (my_rows < 0) return 0;
  if ((d & 3) || d > TPN_THREADS * 4 * TPN_MAXV) return -80;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  cfg.gridDim = dim3(my_rows > 0 ? my_rows : 1);
  cfg.blockDim = dim3(TPN_THREADS);
  cfg.stream = st;
  set_pdl(cfg, attr, pdl);
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, tp_norm_allgather_kernel, *peers, h_local, rs_buf, rs_flag, rs_uses, rs_idx,
                                    rs_inc, epoch, ids, (const __nv_bfloat16*)embed, (const __nv_bfloat16*)w, xn_off,
                                    ag_flag_off, rows_per_rank, my_rows, d, eps, plus_one, arrive, status, pdl));
  return 0;
}

SMC_API int smc_tp_sample_or_score(const smc::TpPeers* peers, const float* logits, long long row_stride, int rows,
                                   int Vshard, int v0, int Vtotal, float temperature, float alpha, float softcap,
                                   const int* tokens_in, unsigned long long seed, const long long* cycle_counter,
                                   int call_id, long long gather_off, const void* gather_local, long long flag_off,
                                   const unsigned long long* flag_local, long long uses, long long idx,
                                   const long long* epoch, int nchunks, int* tok_out, float* logp_out,
                                   float* logz_out, int* arrive, int* status, int pdl, int phase, cudaStream_t st) {
  // phase 0: both stages; 1: scan + exchange only; 2: merge only (used by single-GPU multi-rank emulation)
  using namespace smc;
  if (rows <= 0) return 0;
  if ((row_stride & 3) || (v0 & 3)) return -81;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  cfg.gridDim = dim3(rows, nchunks);
  cfg.blockDim = dim3(TS_THREADS);
  cfg.stream = st;
  set_pdl(cfg, attr, pdl);
  if (phase != 2)
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, tp_sample_stage1_kernel, *peers, logits, row_stride, Vshard, v0, Vtotal,
                                    1.0f / temperature, alpha, tokens_in, (uint64_t)seed, cycle_counter, call_id,
                                    softcap, gather_off, flag_off, rows, arrive, status, pdl));
  cfg.gridDim = dim3((rows + 63) / 64);
  cfg.blockDim = dim3(64);
  if (phase != 1)
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, tp_sample_stage2_kernel, (const RowPartialTP*)gather_local, peers->tp,
                                    nchunks, rows, flag_local, uses, idx, epoch, alpha, tokens_in, tok_out, logp_out,
                                    logz_out, status, pdl));
  return 0;
}

SMC_API int smc_tp_bump_counter(unsigned long long* flag, unsigned long long by, cudaStream_t st) {
  smc::tp_bump_counter_kernel<<<1, 32, 0, st>>>(flag, by);
  return (int)cudaGetLastError();
}

SMC_API int smc_tp_wait_counter(const unsigned long long* flag, unsigned long long want, int* outcome, int* status,
                                cudaStream_t st) {
  smc::tp_wait_counter_kernel<<<1, 32, 0, st>>>(flag, want, outcome, status);
  return (int)cudaGetLastError();
}
