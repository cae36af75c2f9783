// Small fused kernels around the GEMMs: each one also performs the split-K reduction of the
// GEMM that feeds it, so partial sums never make an extra trip through memory.
//   embed_rmsnorm      token ids -> residual stream (fp32) + normalised bf16 activations
//   add_rmsnorm        residual += sum_s partials ; normalised bf16 activations
//   rope_kv_write      sum_s qkv partials -> rotated q (bf16) ; rotated k and v into the paged cache
//   swiglu_partials    sum_s gate/up partials -> silu(gate) * up (bf16)
#include <cuda_fp8.h>

#include "common.cuh"

namespace smc {

template <int VEC_ITERS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// One block per token row.  d <= 256 * 4 * MAXV.
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 8;   // float4 per thread -> d up to 8192

__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ partials, int splits, long long split_stride,
                   const int* __restrict__ ids, const __nv_bfloat16* __restrict__ embed,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ xn, int ldx, int d, float eps,
                   int plus_one, __nv_bfloat16* __restrict__ hb, float* __restrict__ ssq, uint8_t* __restrict__ q8,
                   int ldq, float* __restrict__ qscale, int pdl) {
  __shared__ float red[32];
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int m = blockIdx.x;
  const int nvec = d >> 2;
  float4 v[NORM_MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float4 a;
      if (ids != nullptr) {
        const __nv_bfloat16* e = embed + (size_t)ids[m] * d + c * 4;
        const uint2 raw = *reinterpret_cast<const uint2*>(e);
        const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        a = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
      } else {
        a = reinterpret_cast<const float4*>(h + (size_t)m * d)[c];
      }
      for (int s = 0; s < splits; ++s) {
        const float4 b = reinterpret_cast<const float4*>(partials + (size_t)s * split_stride + (size_t)m * d)[c];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      v[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  const float tot = block_sum<0>(ss, red);
  const float inv = rsqrtf(tot / (float)d + eps);
  if (ssq != nullptr && threadIdx.x == 0) ssq[m] = tot;     // for GEMMs that apply the norm in their epilogue
  // optional e4m3 copy of the normalised row (W8A8 consumers): per-row scale = max|xn| / 448 over the bf16-rounded values
  float q_inv = 0.f;
  if (q8 != nullptr) {
    float amax = 0.f;
    const float add = plus_one ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        const uint2 wr = *reinterpret_cast<const uint2*>(w + c * 4);
        const __nv_bfloat162 w0 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x);
        const __nv_bfloat162 w1 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x * inv * (__low2float(w0) + add)), fabsf(v[i].y * inv * (__high2float(w0) + add))),
                                 fmaxf(fabsf(v[i].z * inv * (__low2float(w1) + add)), fabsf(v[i].w * inv * (__high2float(w1) + add)))));
      }
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    float t = (threadIdx.x & 31) < (NORM_THREADS >> 5) ? red[threadIdx.x & 31] : 0.f;
    t = warp_max(t);                     // every warp reduces the eight partial maxima itself
    __syncthreads();
    // scale taken over the bf16-rounded maximum, as a separate quantisation pass over xn would see it
    const float sc = fmaxf(__bfloat162float(__float2bfloat16(t)), 1e-12f) * (1.f / 448.f);
    q_inv = 1.f / sc;
    if (threadIdx.x == 0) qscale[m] = sc;
  }
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      reinterpret_cast<float4*>(h + (size_t)m * d)[c] = v[i];
      if (hb != nullptr) {
        __nv_bfloat162 r0 = __floats2bfloat162_rn(v[i].x, v[i].y), r1 = __floats2bfloat162_rn(v[i].z, v[i].w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&r0);
        o.y = *reinterpret_cast<uint32_t*>(&r1);
        *reinterpret_cast<uint2*>(hb + (size_t)m * d + c * 4) = o;
      }
      if (xn != nullptr) {
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
        *reinterpret_cast<uint2*>(xn + (size_t)m * ldx + c * 4) = o;
        if (q8 != nullptr) {
          const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(
              make_float2(__low2float(o0) * q_inv, __high2float(o0) * q_inv), __NV_SATFINITE, __NV_E4M3);
          const __nv_fp8x2_storage_t b2 = __nv_cvt_float2_to_fp8x2(
              make_float2(__low2float(o1) * q_inv, __high2float(o1) * q_inv), __NV_SATFINITE, __NV_E4M3);
          *reinterpret_cast<uint32_t*>(q8 + (size_t)m * ldq + c * 4) = (uint32_t)a | ((uint32_t)b2 << 16);
        }
      }
    }
  }
}

// One block per token.  qkv partials [splits, M, (Hq + 2 Hkv) * D]; rope table [max_pos, rd] = cos | sin.
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(const float* __restrict__ partials, int splits, long long split_stride,
                     const int* __restrict__ positions, const int* __restrict__ cache_locs,
                     const float* __restrict__ rope, int rd, int max_pos, __nv_bfloat16* __restrict__ q_out,
                     __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int n_pages, int Hq,
                     int Hkv, int D, int* status, int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int m = blockIdx.x;
  const int nq = Hq * D, nk = Hkv * D, ntot = nq + 2 * nk;
  int pos = positions[m];
  int loc = cache_locs[m];
  if (pos < 0 || pos >= max_pos || loc < 0 || loc > n_pages) {
    if (threadIdx.x == 0) atomicOr(status, SMC_ERR_BOUNDS);
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    loc = 0;
  }
  const float* row = partials + (size_t)m * ntot;
  const float* cs = rope + (size_t)pos * rd;
  const int half = rd >> 1;
  // rotated pairs of q and k heads
  const int pairs_per_head = D >> 1;
  const int n_rot_heads = Hq + Hkv;
  for (int idx = threadIdx.x; idx < n_rot_heads * pairs_per_head; idx += blockDim.x) {
    const int head = idx / pairs_per_head, i = idx % pairs_per_head;
    // element i pairs with i + half inside the rotary span; dims beyond rd pass through
    const int base = head * D;
    float x1 = 0.f, x2 = 0.f;
    int i1, i2;
    bool rot;
    if (i < half) { i1 = i; i2 = i + half; rot = true; }
    else { const int j = i - half; i1 = rd + 2 * j; i2 = rd + 2 * j + 1; rot = false; }
    for (int s = 0; s < splits; ++s) {
      const float* r = row + (size_t)s * split_stride;
      x1 += r[base + i1];
      x2 += r[base + i2];
    }
    float o1 = x1, o2 = x2;
    if (rot) {
      const float c = cs[i], sn = cs[half + i];
      o1 = x1 * c - x2 * sn;
      o2 = x2 * c + x1 * sn;
    }
    if (head < Hq) {
      q_out[(size_t)m * nq + base + i1] = __float2bfloat16(o1);
      q_out[(size_t)m * nq + base + i2] = __float2bfloat16(o2);
    } else {
      const int kb = (head - Hq) * D;
      k_pool[(size_t)loc * nk + kb + i1] = __float2bfloat16(o1);
      k_pool[(size_t)loc * nk + kb + i2] = __float2bfloat16(o2);
    }
  }
  for (int idx = threadIdx.x; idx < nk; idx += blockDim.x) {
    float x = 0.f;
    for (int s = 0; s < splits; ++s) x += row[(size_t)s * split_stride + nq + nk + idx];
    v_pool[(size_t)loc * nk + idx] = __float2bfloat16(x);
  }
}

// General form of the new-token stage for prompt passes: one block per token, one warp per head row.
// qkv fp32 [M, ld] holds q heads at q_off, k heads at k_off, v heads at v_off (other columns, e.g. an output
// gate, are ignored).  Optional per-head RMSNorm of q and k (weights [D], optionally stored as w - 1), rotary
// over the first rd dims (pairs i, i + rd/2), bf16 rounding; q -> q_out [M, Hq*D], k/v -> their cache pages.
__global__ void __launch_bounds__(256)
rope_kv_write_heads_kernel(const float* __restrict__ qkv, int ld, int q_off, int k_off, int v_off,
                           const int* __restrict__ positions, const int* __restrict__ cache_locs,
                           const float* __restrict__ rope, int rd, int max_pos,
                           const __nv_bfloat16* __restrict__ qn_w, const __nv_bfloat16* __restrict__ kn_w, float eps,
                           int plus_one, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool,
                           __nv_bfloat16* __restrict__ v_pool, int n_pages, int Hq, int Hkv, int D, int* status,
                           int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  int pos = positions[m];
  int loc = cache_locs[m];
  if (pos < 0 || pos >= max_pos || loc < 0 || loc > n_pages) {
    if (threadIdx.x == 0) atomicOr(status, SMC_ERR_BOUNDS);
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    loc = 0;
  }
  const float* cs = rope + (size_t)pos * rd;
  const int half = rd >> 1;
  const float add = plus_one ? 1.f : 0.f;
  const size_t kv_row = (size_t)Hkv * D;
  for (int j = warp; j < Hq + 2 * Hkv; j += nwarps) {
    const bool is_q = j < Hq, is_v = j >= Hq + Hkv;
    const int hd = is_q ? j : (is_v ? j - Hq - Hkv : j - Hq);
    const float* src = qkv + (size_t)m * ld + (is_q ? q_off : (is_v ? v_off : k_off)) + (size_t)hd * D;
    __nv_bfloat16* dst = is_q ? q_out + ((size_t)m * Hq + hd) * D
                              : (is_v ? v_pool : k_pool) + (size_t)loc * kv_row + (size_t)hd * D;
    const __nv_bfloat16* nw = is_v ? nullptr : (is_q ? qn_w : kn_w);
    float rstd = 1.f;
    if (nw != nullptr) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) ss += src[i] * src[i];
      rstd = rsqrtf(warp_sum(ss) / (float)D + eps);
    }
    for (int i = lane; i < D / 2; i += 32) {
      int i1, i2;
      bool rot;
      if (i < half) { i1 = i; i2 = i + half; rot = !is_v; }
      else { const int jj = i - half; i1 = rd + 2 * jj; i2 = i1 + 1; rot = false; }
      float x1 = src[i1], x2 = src[i2];
      if (nw != nullptr) {
        x1 *= rstd * (__bfloat162float(nw[i1]) + add);
        x2 *= rstd * (__bfloat162float(nw[i2]) + add);
      }
      if (rot) {
        const float c = cs[i], sn = cs[half + i];
        const float y1 = x1 * c - x2 * sn, y2 = x2 * c + x1 * sn;
        x1 = y1; x2 = y2;
      }
      dst[i1] = __float2bfloat16(x1);
      dst[i2] = __float2bfloat16(x2);
    }
  }
}

// act[m, c] = silu(gate) * up with gate/up interleaved in blocks of `blk` channels.
__global__ void __launch_bounds__(256)
swiglu_partials_kernel(const float* __restrict__ partials, int splits, long long split_stride,
                       __nv_bfloat16* __restrict__ act, int M, int ffn, int blk, int ldo, int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const long long total = (long long)M * ffn;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(idx / ffn), c = (int)(idx % ffn);
    const int gi = (c / blk) * 2 * blk + (c % blk);
    float g = 0.f, u = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* r = partials + (size_t)s * split_stride + (size_t)m * 2 * ffn;
      g += r[gi];
      u += r[gi + blk];
    }
    act[(size_t)m * ldo + c] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
  }
}

template <typename K, typename... Args>
static int launch_pdl(K kern, dim3 grid, dim3 block, cudaStream_t st, int pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, kern, args...));
  return 0;
}

}  // namespace smc

namespace smc {
// Per-row dynamic quantisation of bf16 activations to e4m3: scale[m] = max|x| / 448, q = x / scale (saturating).
// One block per row; the row is read twice (second time from L1 / L2).
__global__ void __launch_bounds__(256) quant_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                              uint8_t* __restrict__ q, int ldq,
                                                              float* __restrict__ scale, int K, int pdl) {
  __shared__ float red[32];
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int m = blockIdx.x;
  const __nv_bfloat16* xr = x + (size_t)m * ldx;
  float amax = 0.f;
  for (int c = threadIdx.x * 8; c < K; c += blockDim.x * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(__low2float(h2[i])), fabsf(__high2float(h2[i]))));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_max(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  const float sc = fmaxf(red[0], 1e-12f) * (1.f / 448.f), inv = 1.f / sc;
  if (threadIdx.x == 0) scale[m] = sc;
  uint8_t* qr = q + (size_t)m * ldq;
  for (int c = threadIdx.x * 8; c < K; c += blockDim.x * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint32_t o[2];
#pragma unroll
    for (int i = 0; i < 4; i += 2) {
      const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(
          make_float2(__low2float(h2[i]) * inv, __high2float(h2[i]) * inv), __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t b = __nv_cvt_float2_to_fp8x2(
          make_float2(__low2float(h2[i + 1]) * inv, __high2float(h2[i + 1]) * inv), __NV_SATFINITE, __NV_E4M3);
      o[i >> 1] = (uint32_t)a | ((uint32_t)b << 16);
    }
    *reinterpret_cast<uint2*>(qr + c) = make_uint2(o[0], o[1]);
  }
}
}  // namespace smc

namespace smc {
// Rotated K / V rows (bf16, [M, Hkv * D]) -> the e4m3 cache: one warp per (token, kv head, K | V) row; the row's scale
// max|x| / 448 goes behind the value bytes of its page row.
__global__ void __launch_bounds__(256) kv_store_e4m3_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                            int M, const int* __restrict__ cache_locs,
                                                            uint8_t* __restrict__ k_pool, uint8_t* __restrict__ v_pool,
                                                            int n_pages, int Hkv, int D, int row_bytes, int* status,
                                                            int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= M * Hkv * 2) return;
  const int is_v = warp & 1, kvh = (warp >> 1) % Hkv, m = (warp >> 1) / Hkv;
  int loc = cache_locs[m];
  if (loc < 0 || loc > n_pages) { if (lane == 0) atomicOr(status, SMC_ERR_BOUNDS); loc = 0; }
  const __nv_bfloat16* src = (is_v ? v : k) + (size_t)m * Hkv * D + (size_t)kvh * D;
  float amax = 0.f;
  for (int i = lane; i < D; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[i])));
  amax = warp_max(amax);
  const float sc = fmaxf(amax, 1e-12f) * (1.f / 448.f), inv = 1.f / sc;
  uint8_t* dst = (is_v ? v_pool : k_pool) + (size_t)loc * row_bytes;
  for (int i = lane * 2; i < D; i += 64) {
    const __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(
        make_float2(__bfloat162float(src[i]) * inv, __bfloat162float(src[i + 1]) * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint16_t*>(dst + (size_t)kvh * D + i) = (uint16_t)q;
  }
  if (lane == 0) *reinterpret_cast<float*>(dst + (size_t)Hkv * D + kvh * 4) = sc;
}
}  // namespace smc

SMC_API int smc_kv_store_e4m3(const void* k, const void* v, int M, const int* cache_locs, void* k_pool, void* v_pool,
                              int n_pages, int Hkv, int D, int row_bytes, int* status, int pdl, cudaStream_t st) {
  using namespace smc;
  if (M <= 0) return 0;
  if ((D & 1) || row_bytes < Hkv * D + Hkv * 4) return -34;
  const long long warps = (long long)M * Hkv * 2;
  return launch_pdl(kv_store_e4m3_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), st, pdl,
                    (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, M, cache_locs, (uint8_t*)k_pool, (uint8_t*)v_pool,
                    n_pages, Hkv, D, row_bytes, status, pdl);
}

// x [M, ldx] bf16 -> q [M, ldq] e4m3 bytes + scale [M] fp32 (x ~ q * scale).  K, ldx and ldq multiples of 8.
SMC_API int smc_quant_rows_e4m3(const void* x, int ldx, void* q, int ldq, float* scale, int M, int K, int pdl,
                                cudaStream_t st) {
  using namespace smc;
  if (M <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldq & 7)) return -33;
  return launch_pdl(quant_rows_e4m3_kernel, dim3(M), dim3(256), st, pdl, (const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq,
                    scale, K, pdl);
}

// h [M, d] fp32 in/out.  With ids != null the row is first loaded from the embedding table
// (h's previous content is ignored); partials may be null (splits = 0).
SMC_API int smc_add_rmsnorm(float* h, const float* partials, int splits, long long split_stride, const int* ids,
                            const void* embed, const void* w, void* xn, int ldx, int M, int d, float eps,
                            int plus_one, void* hb, float* ssq, int pdl, cudaStream_t st) {
  using namespace smc;
  if (M <= 0) return 0;
  if ((d & 3) || d > NORM_THREADS * 4 * NORM_MAXV) return -30;
  return launch_pdl(add_rmsnorm_kernel, dim3(M), dim3(NORM_THREADS), st, pdl, h, partials, splits, split_stride, ids,
                    (const __nv_bfloat16*)embed, (const __nv_bfloat16*)w, (__nv_bfloat16*)xn, ldx, d, eps, plus_one,
                    (__nv_bfloat16*)hb, ssq, (uint8_t*)nullptr, 0, (float*)nullptr, pdl);
}

// Same, also emitting the e4m3 copy of the normalised rows (q8 [M, ldq] bytes, qscale [M]) for W8A8 consumers; xn is
// required (the scale is taken over its bf16 values).
SMC_API int smc_add_rmsnorm_q8(float* h, const int* ids, const void* embed, const void* w, void* xn, int ldx, int M, int d,
                               float eps, int plus_one, void* q8, int ldq, float* qscale, int pdl, cudaStream_t st) {
  using namespace smc;
  if (M <= 0) return 0;
  if ((d & 3) || d > NORM_THREADS * 4 * NORM_MAXV || xn == nullptr || q8 == nullptr || qscale == nullptr || (ldq & 3))
    return -30;
  return launch_pdl(add_rmsnorm_kernel, dim3(M), dim3(NORM_THREADS), st, pdl, h, (const float*)nullptr, 0, 0ll, ids,
                    (const __nv_bfloat16*)embed, (const __nv_bfloat16*)w, (__nv_bfloat16*)xn, ldx, d, eps, plus_one,
                    (__nv_bfloat16*)nullptr, (float*)nullptr, (uint8_t*)q8, ldq, qscale, pdl);
}

SMC_API int smc_rope_kv_write(const float* partials, int splits, long long split_stride, const int* positions,
                              const int* cache_locs, const float* rope, int rd, int max_pos, void* q_out, void* k_pool,
                              void* v_pool, int n_pages, int M, int Hq, int Hkv, int D, int* status, int pdl,
                              cudaStream_t st) {
  using namespace smc;
  if (M <= 0) return 0;
  if (rd > D || (rd & 1) || (D & 1)) return -31;
  return launch_pdl(rope_kv_write_kernel, dim3(M), dim3(256), st, pdl, partials, splits, split_stride, positions,
                    cache_locs, rope, rd, max_pos, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                    (__nv_bfloat16*)v_pool, n_pages, Hq, Hkv, D, status, pdl);
}

SMC_API int smc_rope_kv_write_heads(const float* qkv, int ld, int q_off, int k_off, int v_off, const int* positions,
                                    const int* cache_locs, const float* rope, int rd, int max_pos, const void* qn_w,
                                    const void* kn_w, float eps, int plus_one, void* q_out, void* k_pool,
                                    void* v_pool, int n_pages, int M, int Hq, int Hkv, int D, int* status, int pdl,
                                    cudaStream_t st) {
  using namespace smc;
  if (M <= 0) return 0;
  if (rd > D || (rd & 1) || (D & 1)) return -32;
  return launch_pdl(rope_kv_write_heads_kernel, dim3(M), dim3(256), st, pdl, qkv, ld, q_off, k_off, v_off, positions,
                    cache_locs, rope, rd, max_pos, (const __nv_bfloat16*)qn_w, (const __nv_bfloat16*)kn_w, eps,
                    plus_one, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_pages, Hq, Hkv,
                    D, status, pdl);
}

SMC_API int smc_swiglu_partials(const float* partials, int splits, long long split_stride, void* act, int M, int ffn,
                                int blk, int ldo, int pdl, cudaStream_t st) {
  using namespace smc;
  if (M <= 0) return 0;
  long long total = (long long)M * ffn;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch_pdl(swiglu_partials_kernel, dim3(blocks), dim3(256), st, pdl, partials, splits, split_stride,
                    (__nv_bfloat16*)act, M, ffn, blk, ldo, pdl);
}
