// Gated DeltaNet (linear attention) step kernels for E new tokens per sequence row (E = 1 draft
// decode, 2 draft head, gamma+1 target verify).  SMC accepts every token, so the recurrent state is
// advanced in place through all E tokens.
//   gdn_conv      depthwise causal conv (width W) + SiLU over the mixed q|k|v channels, one thread per
//                 (row, channel); also rolls the conv window kept in the state pool
//   gdn_recurrent one CTA per (row, value head); thread j owns column j of the state S [dk, dv] in
//                 registers, so the delta-rule update and the read-out are thread-local:
//                     S *= exp(g);  kv = S^T k;  delta = (v - kv) * beta;  S += k (x) delta;  o = S^T q
//                 followed by the gated RMSNorm of the head output (norm, weight, * silu(z)) -> bf16
#include "common.cuh"

namespace smc {

// proj: fp32 [T, ldp] = mixed (conv_dim) | z (value_dim) | b (Hv) | a (Hv).
// WT: the conv width as a compile-time constant (window arrays stay in registers); 0 takes it from the argument.
template <int WT>
__global__ void gdn_conv_kernel(const float* __restrict__ proj, int ldp, float* __restrict__ conv_state,
                                const int* __restrict__ state_rows, const __nv_bfloat16* __restrict__ conv_w,
                                float* __restrict__ conv_out, int bs, int E, int conv_dim, int W_rt,
                                const int* __restrict__ tok_off, const int* __restrict__ tok_len, int pdl) {
  const int W = WT ? WT : W_rt;
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= bs * conv_dim) return;
  const int b = idx / conv_dim, ch = idx % conv_dim;
  const size_t t0 = tok_off ? (size_t)tok_off[b] : (size_t)b * E;
  if (tok_len) E = tok_len[b];
  float* win = conv_state + ((size_t)state_rows[b] * conv_dim + ch) * (W - 1);
  float hist[8];
  float w[8];
  for (int i = 0; i < W - 1; ++i) hist[i] = win[i];
  for (int i = 0; i < W; ++i) w[i] = __bfloat162float(conv_w[ch * W + i]);
  for (int e = 0; e < E; ++e) {
    const float x = proj[(t0 + e) * ldp + ch];
    float acc = w[W - 1] * x;
    for (int i = 0; i < W - 1; ++i) acc += w[i] * hist[i];
    for (int i = 0; i + 1 < W - 1; ++i) hist[i] = hist[i + 1];
    hist[W - 2] = x;
    conv_out[(t0 + e) * conv_dim + ch] = acc / (1.f + __expf(-acc));
  }
  for (int i = 0; i < W - 1; ++i) win[i] = hist[i];
}

// Prompt-pass form of the conv: the output at token t only needs inputs t-W+1 .. t, so tokens are processed in
// parallel, CONV_TILE per thread.  grid.x covers the channels, grid.y the row's token tiles, grid.z the rows.  The thread
// of a row's first tile is the only one that touches the row's window in the state pool: it reads the old window and
// writes the new one (the row's last W-1 inputs).
constexpr int CONV_TILE = 16;
// WT: the conv width as a compile-time constant (window arrays stay in registers); 0 takes it from the argument.
template <int WT>
__global__ void gdn_conv_prefill_kernel(const float* __restrict__ proj, int ldp, float* __restrict__ conv_state,
                                        const int* __restrict__ state_rows, const __nv_bfloat16* __restrict__ conv_w,
                                        float* __restrict__ conv_out, int conv_dim, int W_rt,
                                        const int* __restrict__ tok_off, const int* __restrict__ tok_len, int pdl) {
  const int W = WT ? WT : W_rt;
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int ch = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.z;
  const int len = tok_len[b], e0 = blockIdx.y * CONV_TILE;
  if (ch >= conv_dim || e0 >= len) return;
  const size_t t0 = (size_t)tok_off[b];
  float* win = conv_state + ((size_t)state_rows[b] * conv_dim + ch) * (W - 1);
  float w[8], hist[8];
  for (int i = 0; i < W; ++i) w[i] = __bfloat162float(conv_w[ch * W + i]);
  // inputs e0-W+1 .. e0-1: from the row itself, or from the old window for tokens before the row's first
  for (int i = 0; i < W - 1; ++i) {
    const int e = e0 - (W - 1) + i;
    hist[i] = e >= 0 ? proj[(t0 + e) * ldp + ch] : win[W - 1 + e];
  }
  if (e0 == 0) {
    // new window = inputs len-W+1 .. len-1 (old window entries where the row is shorter than the window)
    float nw[8];
    for (int i = 0; i < W - 1; ++i) {
      const int e = len - (W - 1) + i;
      nw[i] = e >= 0 ? proj[(t0 + e) * ldp + ch] : win[W - 1 + e];
    }
    for (int i = 0; i < W - 1; ++i) win[i] = nw[i];
  }
  // all of the tile's inputs first (independent loads in flight together), then the window arithmetic
  float xin[CONV_TILE];
#pragma unroll
  for (int u = 0; u < CONV_TILE; ++u) xin[u] = e0 + u < len ? proj[(t0 + e0 + u) * ldp + ch] : 0.f;
#pragma unroll
  for (int u = 0; u < CONV_TILE; ++u) {
    const float x = xin[u];
    float acc = w[W - 1] * x;
    for (int i = 0; i < W - 1; ++i) acc += w[i] * hist[i];
    for (int i = 0; i + 1 < W - 1; ++i) hist[i] = hist[i + 1];
    hist[W - 2] = x;
    if (e0 + u < len) conv_out[(t0 + e0 + u) * conv_dim + ch] = acc / (1.f + __expf(-acc));
  }
}

template <int DK>
__global__ void gdn_recurrent_kernel(const float* __restrict__ conv_out, const float* __restrict__ proj, int ldp,
                                     float* __restrict__ temporal, const int* __restrict__ state_rows,
                                     const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                     const __nv_bfloat16* __restrict__ gnorm_w, __nv_bfloat16* __restrict__ out,
                                     int E, int Hk, int Hv, int dv, int conv_dim, float eps,
                                     const int* __restrict__ tok_off, const int* __restrict__ tok_len, int pdl) {
  __shared__ __align__(16) float q_s[DK], k_s[DK];
  __shared__ float red[8];
  __shared__ float scal[4];
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int b = blockIdx.x, vh = blockIdx.y, kh = vh / (Hv / Hk);
  const size_t t0 = tok_off ? (size_t)tok_off[b] : (size_t)b * E;
  if (tok_len) E = tok_len[b];
  const int j = threadIdx.x;              // value-dim column owned by this thread (j < dv does real work)
  const int key_dim = Hk * DK, value_dim = Hv * dv;
  const bool live = j < dv;
  float* Sg = temporal + (((size_t)state_rows[b] * Hv + vh) * DK) * dv;
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = live ? Sg[(size_t)i * dv + j] : 0.f;
  const float wj = live ? __bfloat162float(gnorm_w[j]) : 0.f;
  const int nwarps = (blockDim.x + 31) >> 5;
  for (int e = 0; e < E; ++e) {
    const size_t t = t0 + e;
    const float* co = conv_out + t * conv_dim;
    // l2-normalised q (scaled by dk^-1/2) and k of this key head
    float qv = 0.f, kv_ = 0.f;
    if (j < DK) { qv = co[kh * DK + j]; kv_ = co[key_dim + kh * DK + j]; }
    float sq = warp_sum(qv * qv), sk = warp_sum(kv_ * kv_);
    if ((j & 31) == 0) { red[j >> 5] = sq; red[4 + (j >> 5)] = sk; }
    __syncthreads();
    if (j == 0) {
      float a = 0.f, c = 0.f;
      for (int w = 0; w < nwarps; ++w) { a += red[w]; c += red[4 + w]; }
      scal[0] = rsqrtf(a + 1e-6f) * rsqrtf((float)DK);
      scal[1] = rsqrtf(c + 1e-6f);
      const float av = proj[t * ldp + conv_dim + value_dim + Hv + vh];
      const float bv = proj[t * ldp + conv_dim + value_dim + vh];
      const float x = av + dt_bias[vh];
      const float sp = x > 20.f ? x : log1pf(__expf(x));
      scal[2] = __expf(-__expf(A_log[vh]) * sp);          // exp(g)
      scal[3] = 1.f / (1.f + __expf(-bv));                // beta
    }
    __syncthreads();
    if (j < DK) { q_s[j] = qv * scal[0]; k_s[j] = kv_ * scal[1]; }
    __syncthreads();
    const float decay = scal[2], beta = scal[3];
    const float v = live ? co[2 * key_dim + vh * dv + j] : 0.f;
    // four independent partial sums per dot product (a single chain of DK dependent FMAs would set the pace),
    // key / query values fetched four at a time
    float kv4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < DK; i += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(&k_s[i]);
      S[i] *= decay; S[i + 1] *= decay; S[i + 2] *= decay; S[i + 3] *= decay;
      kv4[0] = fmaf(S[i], kk.x, kv4[0]); kv4[1] = fmaf(S[i + 1], kk.y, kv4[1]);
      kv4[2] = fmaf(S[i + 2], kk.z, kv4[2]); kv4[3] = fmaf(S[i + 3], kk.w, kv4[3]);
    }
    const float kvm = (kv4[0] + kv4[1]) + (kv4[2] + kv4[3]);
    const float delta = (v - kvm) * beta;
    float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < DK; i += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(&k_s[i]);
      const float4 qq = *reinterpret_cast<const float4*>(&q_s[i]);
      S[i] = fmaf(kk.x, delta, S[i]); S[i + 1] = fmaf(kk.y, delta, S[i + 1]);
      S[i + 2] = fmaf(kk.z, delta, S[i + 2]); S[i + 3] = fmaf(kk.w, delta, S[i + 3]);
      o4[0] = fmaf(S[i], qq.x, o4[0]); o4[1] = fmaf(S[i + 1], qq.y, o4[1]);
      o4[2] = fmaf(S[i + 2], qq.z, o4[2]); o4[3] = fmaf(S[i + 3], qq.w, o4[3]);
    }
    float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    // gated RMSNorm over the head's dv outputs
    float so = warp_sum(live ? o * o : 0.f);
    __syncthreads();
    if ((j & 31) == 0) red[j >> 5] = so;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < nwarps; ++w) tot += red[w];
    if (live) {
      const float y = __bfloat162float(__float2bfloat16(o * rsqrtf(tot / (float)dv + eps)));
      const float z = proj[t * ldp + conv_dim + vh * dv + j];
      out[t * value_dim + vh * dv + j] = __float2bfloat16(y * wj * (z / (1.f + __expf(-z))));
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DK; ++i) Sg[(size_t)i * dv + j] = S[i];
  }
}

}  // namespace smc

// Conv + SiLU pass alone (rows as in smc_gdn_varlen); the chunk-parallel delta-rule kernel consumes conv_out.
// max_len: upper bound of tok_len known on the host (0 = unknown): rows longer than two token tiles use the
// token-parallel conv kernel.
SMC_API int smc_gdn_conv(const float* proj, int ldp, float* conv_state, const int* state_rows, const void* conv_w,
                         float* conv_out, int bs, int E, const int* tok_off, const int* tok_len, int conv_dim, int W,
                         int max_len, int pdl, cudaStream_t st) {
  using namespace smc;
  if ((tok_off == nullptr) != (tok_len == nullptr)) return -103;
  if (bs <= 0) return 0;
  if (W < 2 || W > 8) return -100;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  if (tok_len != nullptr && max_len > 2 * CONV_TILE && bs <= 65535) {
    // long rows: token-parallel form
    cfg.gridDim = dim3((conv_dim + 255) / 256, (max_len + CONV_TILE - 1) / CONV_TILE, bs);
    cfg.blockDim = dim3(256);
    if (W == 4)
      CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, gdn_conv_prefill_kernel<4>, proj, ldp, conv_state, state_rows,
                                        (const __nv_bfloat16*)conv_w, conv_out, conv_dim, W, tok_off, tok_len, pdl));
    else
      CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, gdn_conv_prefill_kernel<0>, proj, ldp, conv_state, state_rows,
                                        (const __nv_bfloat16*)conv_w, conv_out, conv_dim, W, tok_off, tok_len, pdl));
    return 0;
  }
  cfg.gridDim = dim3((bs * conv_dim + 255) / 256);
  cfg.blockDim = dim3(256);
  if (W == 4)
    CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, gdn_conv_kernel<4>, proj, ldp, conv_state, state_rows,
                                      (const __nv_bfloat16*)conv_w, conv_out, bs, E, conv_dim, W, tok_off, tok_len, pdl));
  else
    CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, gdn_conv_kernel<0>, proj, ldp, conv_state, state_rows,
                                      (const __nv_bfloat16*)conv_w, conv_out, bs, E, conv_dim, W, tok_off, tok_len, pdl));
  return 0;
}

// Rows of variable length (prompt passes): row b covers tokens [tok_off[b], tok_off[b] + tok_len[b]) of the
// token-major buffers.  With tok_off == tok_len == null every row has E tokens laid out back to back.
SMC_API int smc_gdn_varlen(const float* proj, int ldp, float* conv_state, float* temporal, const int* state_rows,
                           const void* conv_w, const float* dt_bias, const float* A_log, const void* gnorm_w,
                           float* conv_out, void* out, int bs, int E, const int* tok_off, const int* tok_len, int Hk,
                           int Hv, int dk, int dv, int W, float eps, int pdl, cudaStream_t st) {
  using namespace smc;
  if ((tok_off == nullptr) != (tok_len == nullptr)) return -103;
  if (bs <= 0) return 0;
  if (W < 2 || W > 8 || Hv % Hk || dv > 256 || dk > 256) return -100;
  const int conv_dim = 2 * Hk * dk + Hv * dv;
  {
    const int rc = smc_gdn_conv(proj, ldp, conv_state, state_rows, conv_w, conv_out, bs, E, tok_off, tok_len, conv_dim,
                                W, 0, pdl, st);
    if (rc) return rc;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  int threads = dv > dk ? dv : dk;
  threads = (threads + 31) / 32 * 32;
  if (threads > 128) return -101;
  cfg.gridDim = dim3(bs, Hv);
  cfg.blockDim = dim3(threads);
#define GDN_LAUNCH(DKV)                                                                                           \
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, gdn_recurrent_kernel<DKV>, (const float*)conv_out, proj, ldp, temporal, \
                                    state_rows, dt_bias, A_log, (const __nv_bfloat16*)gnorm_w,                    \
                                    (__nv_bfloat16*)out, E, Hk, Hv, dv, conv_dim, eps, tok_off, tok_len, pdl))
  switch (dk) {
    case 128: GDN_LAUNCH(128); break;
    case 64: GDN_LAUNCH(64); break;
    case 32: GDN_LAUNCH(32); break;
    case 16: GDN_LAUNCH(16); break;
    default: return -102;
  }
#undef GDN_LAUNCH
  return 0;
}

SMC_API int smc_gdn_step(const float* proj, int ldp, float* conv_state, float* temporal, const int* state_rows,
                         const void* conv_w, const float* dt_bias, const float* A_log, const void* gnorm_w,
                         float* conv_out, void* out, int bs, int E, int Hk, int Hv, int dk, int dv, int W, float eps,
                         int pdl, cudaStream_t st) {
  return smc_gdn_varlen(proj, ldp, conv_state, temporal, state_rows, conv_w, dt_bias, A_log, gnorm_w, conv_out, out, bs,
                        E, nullptr, nullptr, Hk, Hv, dk, dv, W, eps, pdl, st);
}
