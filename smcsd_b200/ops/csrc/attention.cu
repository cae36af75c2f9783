// Causal "extend" attention over a token-granular paged KV cache, for uniform extend length E:
// E = 1 (draft decode), E = 2 (draft head), E = gamma + 1 (target verify).  Every sequence row
// has `prefix` cached tokens plus E new ones whose K/V were already written to their pages, so
// all keys are fetched through the block table and query e sees keys 0 .. prefix + e.
//
// GQA packing: the E * G query rows that share one KV head are processed against each key once.
// Split-KV: grid.y splits the key range; each warp owns up to RW query rows of one
// (sequence, kv head, split) and keeps flash-style (max, sum, acc) state in registers:
//   scores  : lane = key   (each lane dots its key row against the warp's query rows in smem)
//   values  : lane = slice of head_dim (probabilities broadcast by shuffle)
// A second kernel merges the splits.
#include "common.cuh"

namespace smc {

struct AttnParams {
  const __nv_bfloat16* q;        // [bs * E, Hq, D]
  const __nv_bfloat16* k_pool;   // [pages, Hkv * D]
  const __nv_bfloat16* v_pool;
  const int* block_table;        // [rows, bt_stride]
  const int* rows;               // [bs] block-table row per sequence
  const int* prefix_lens;        // [bs]
  float* part_acc;               // [bs * E * Hq, splits, D]
  float* part_ml;                // [bs * E * Hq, splits, 2]
  int bt_stride, n_pages;
  int E, Hq, Hkv, splits;
  float scale;
  int* status;
  int pdl;
};

__device__ __forceinline__ void bf16x8_to_float(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p[i]);
    f[2 * i + 1] = __high2float(p[i]);
  }
}

template <int D, int RW>
__global__ void __launch_bounds__(32 * 8) attn_extend_kernel(const AttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_attn[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_attn);   // [R, D]
  constexpr int DPL = D / 32;   // head-dim elements per lane in the value phase
  const int G = p.Hq / p.Hkv;
  const int R = p.E * G;
  const int b = blockIdx.x / p.Hkv, kvh = blockIdx.x % p.Hkv;
  const int split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (p.pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }

  // stage this CTA's query rows: row r = e * G + g  ->  token b * E + e, head kvh * G + g
  for (int idx = threadIdx.x; idx < R * (D / 8); idx += blockDim.x) {
    const int r = idx / (D / 8), c = idx % (D / 8);
    const int e = r / G, g = r % G;
    const uint4 v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(b * p.E + e) * p.Hq + kvh * G + g) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + (size_t)r * D + c * 8) = v;
  }
  __syncthreads();

  const int r0 = warp * RW;
  if (r0 >= R) return;
  const int nr = min(RW, R - r0);
  const int prefix = p.prefix_lens[b];
  const int L = prefix + p.E;
  int chunk = (L + p.splits - 1) / p.splits;
  chunk = (chunk + 31) & ~31;
  const int k_begin = split * chunk;
  const int k_end = min(L, k_begin + chunk);
  const int* bt = p.block_table + (size_t)p.rows[b] * p.bt_stride;
  const size_t kv_row = (size_t)p.Hkv * D;

  float m_run[RW], l_run[RW], acc[RW][DPL];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[r][d] = 0.f;
  }

  for (int kb = k_begin; kb < k_end; kb += 32) {
    const int key = kb + lane;
    const bool valid = key < k_end;
    int page = valid ? bt[key] : 0;
    if (page < 0 || page > p.n_pages) {
      atomicOr(p.status, SMC_ERR_BOUNDS);
      page = 0;
    }
    // ---- scores: this lane's key against the warp's rows
    float s[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) s[r] = 0.f;
    const __nv_bfloat16* kp = p.k_pool + (size_t)page * kv_row + (size_t)kvh * D;
#pragma unroll 4
    for (int d0 = 0; d0 < D; d0 += 8) {
      float kf[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(kp + d0), kf);
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        if (r < nr) {
          float qf[8];
          bf16x8_to_float(*reinterpret_cast<const uint4*>(q_s + (size_t)(r0 + r) * D + d0), qf);
#pragma unroll
          for (int j = 0; j < 8; ++j) s[r] = fmaf(qf[j], kf[j], s[r]);
        }
      }
    }
    // ---- online softmax update per row
    float pr[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const int e = (r0 + r) / G;
      const bool vis = valid && (r < nr) && (key <= prefix + e);
      const float sv = vis ? s[r] * p.scale : -INFINITY;
      const float mx = warp_max(sv);
      const float m_new = fmaxf(m_run[r], mx);
      const float corr = (m_new == -INFINITY) ? 1.f : __expf(m_run[r] - m_new);
      pr[r] = vis ? __expf(sv - m_new) : 0.f;
      l_run[r] = l_run[r] * corr + pr[r];
      m_run[r] = m_new;
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[r][d] *= corr;
    }
    // ---- values: lane owns DPL consecutive dims
    const int nk = min(32, k_end - kb);
    for (int kk = 0; kk < nk; ++kk) {
      const int pg = __shfl_sync(0xffffffffu, page, kk);
      const __nv_bfloat16* vp = p.v_pool + (size_t)pg * kv_row + (size_t)kvh * D + lane * DPL;
      float vf[DPL];
      if constexpr (DPL == 8) {
        bf16x8_to_float(*reinterpret_cast<const uint4*>(vp), vf);
      } else if constexpr (DPL == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vp);
        const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        vf[0] = __low2float(q2[0]); vf[1] = __high2float(q2[0]);
        vf[2] = __low2float(q2[1]); vf[3] = __high2float(q2[1]);
      } else {
        const __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162*>(vp);
        vf[0] = __low2float(q2); vf[1] = __high2float(q2);
      }
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float w = __shfl_sync(0xffffffffu, pr[r], kk);
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[r][d] = fmaf(w, vf[d], acc[r][d]);
      }
    }
  }
  // ---- write this split's partial state
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    if (r < nr) {
      const int e = (r0 + r) / G, g = (r0 + r) % G;
      const size_t qrow = (size_t)(b * p.E + e) * p.Hq + kvh * G + g;
      const float l_tot = warp_sum(l_run[r]);
      float* pa = p.part_acc + (qrow * p.splits + split) * D + lane * DPL;
#pragma unroll
      for (int d = 0; d < DPL; ++d) pa[d] = acc[r][d];
      if (lane == 0) {
        p.part_ml[(qrow * p.splits + split) * 2] = m_run[r];
        p.part_ml[(qrow * p.splits + split) * 2 + 1] = l_tot;
      }
    }
  }
}

// out[qrow, :] = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M)
__global__ void attn_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                  __nv_bfloat16* __restrict__ out, int splits, int D, int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const size_t qrow = blockIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(qrow * splits + s) * 2]);
  float denom = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = part_ml[(qrow * splits + s) * 2];
    if (m != -INFINITY) denom += part_ml[(qrow * splits + s) * 2 + 1] * __expf(m - M);
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = part_ml[(qrow * splits + s) * 2];
      if (m != -INFINITY) a += part_acc[(qrow * splits + s) * D + d] * __expf(m - M);
    }
    out[qrow * D + d] = __float2bfloat16(a * inv);
  }
}

template <int D, int RW>
static int launch_attn(const AttnParams& p, int bs, cudaStream_t st) {
  const int G = p.Hq / p.Hkv, R = p.E * G;
  const int warps = (R + RW - 1) / RW;
  if (warps > 8) return -41;
  const size_t smem = (size_t)R * D * 2;
  auto kern = attn_extend_kernel<D, RW>;
  if (smem > 48 * 1024) CUDA_CHECK_RET(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(bs * p.Hkv, p.splits);
  cfg.blockDim = dim3(32 * warps);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, kern, p));
  return 0;
}

template <int D>
static int dispatch_rw(const AttnParams& p, int bs, cudaStream_t st) {
  const int R = p.E * (p.Hq / p.Hkv);
  if (R <= 4) return launch_attn<D, 4>(p, bs, st);
  if (R <= 8) return launch_attn<D, 8>(p, bs, st);
  return launch_attn<D, 12>(p, bs, st);
}

}  // namespace smc

// q [bs*E, Hq, D] bf16 -> out [bs*E, Hq*D] bf16.  part_acc / part_ml are caller-provided scratch of
// bs*E*Hq*splits*D and bs*E*Hq*splits*2 floats.
SMC_API int smc_attention_extend(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                 int bt_stride, int n_pages, const int* rows, const int* prefix_lens, float* part_acc,
                                 float* part_ml, void* out, int bs, int E, int Hq, int Hkv, int D, int splits,
                                 float scale, int* status, int pdl, cudaStream_t st) {
  using namespace smc;
  if (bs <= 0) return 0;
  if (Hq % Hkv) return -40;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
  p.block_table = block_table; p.rows = rows; p.prefix_lens = prefix_lens;
  p.part_acc = part_acc; p.part_ml = part_ml;
  p.bt_stride = bt_stride; p.n_pages = n_pages; p.E = E; p.Hq = Hq; p.Hkv = Hkv; p.splits = splits;
  p.scale = scale; p.status = status; p.pdl = pdl;
  int rc;
  if (D == 64) rc = dispatch_rw<64>(p, bs, st);
  else if (D == 128) rc = dispatch_rw<128>(p, bs, st);
  else if (D == 256) rc = dispatch_rw<256>(p, bs, st);
  else return -42;
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(bs * E * Hq);
  cfg.blockDim = dim3(D < 128 ? 64 : 128);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, attn_merge_kernel, (const float*)part_acc, (const float*)part_ml,
                                    (__nv_bfloat16*)out, splits, D, pdl));
  return 0;
}
