// Chunk-parallel gated delta rule for prompt passes on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// One CTA per (sequence row, value head) walks the row's tokens in chunks of 64 instead of one by one.  With
// gc = cumsum(g) inside the chunk, decay[i][j] = exp(gc_i - gc_j), L = strict_lower((K beta) K^T * decay) and
// Tm = (I + L)^-1 (the WY / UT transform of the delta rule), the chunk needs
//     v_w   = Tm (V beta)                 k_cum = Tm (K beta e^gc)
//     v_new = v_w - k_cum S               out   = (Q e^gc) S + lower((Q K^T) * decay) v_new
//     S    <- S e^gc_last + (K e^(gc_last - gc))^T v_new
// Every product runs as tcgen05.mma with M = 128 by keeping the head dimension on the accumulator rows (the state is
// held transposed, S^T [dv][dk], in 128 columns of tensor memory for the whole row):
//     G     [128 x 64]  = [K beta ; Q] K^T                (rows 0..63 feed L, rows 64..127 the local attention)
//     v_w^T [dv x 64]   = (V beta)^T Tm^T                 k_cum^T [dk x 64] = (K beta e^gc)^T Tm^T
//     D1    [dv x 64]   = S^T k_cum^T                     out^T   [dv x 64] = S^T (Q e^gc)^T + v_new^T local^T
//     S^T   [dv x dk]  += v_new^T (K e^(gc_last - gc))    (B operand MN-major, straight from its [token][dk] tile)
// Operands are bf16 tiles in the 128-byte-swizzled layouts the MMA descriptors expect, written by the 128 threads
// (thread = accumulator row); accumulation and the state are fp32.  Tm is obtained exactly, in fp32: thread j solves
// (I + L) x = e_j by forward substitution with its column in registers and L broadcast from shared memory.
// The gated RMSNorm (norm over dv, weight, * silu(z)) is applied to every chunk's output before it is stored.
//
// Math: Qwen3.5 / Qwen3-Next gated delta net (transformers models/qwen3_5/modeling_qwen3_5.py:
// torch_chunk_gated_delta_rule); the reference serves it through its hybrid linear-attention backend
// (smcsd/core/hybrid_multistep_backend.py:47-222).  Built for dk = dv = 128; other head sizes keep the token-serial
// kernel of gdn.cu.  Every mbarrier wait is bounded; a timeout raises a status bit and the CTA unwinds.
#include "common.cuh"

namespace smc {

constexpr int GC = 64;      // tokens per chunk
constexpr int GD = 128;     // dk == dv

struct GdnChunkParams {
  const float* conv_out;      // [T][conv_dim] q | k | v channels after conv + SiLU
  const float* proj;          // [T][ldp] mixed | z | b | a
  float* temporal;            // [rows][Hv][dk][dv]
  const int* state_rows;
  const int* tok_off;         // optional (with tok_len): first token and token count of every row
  const int* tok_len;
  const float* dt_bias;
  const float* A_log;
  const __nv_bfloat16* gnorm_w;
  __nv_bfloat16* out;         // [T][Hv * dv]
  int conv_dim, ldp, E, Hk, Hv;
  float eps;
  int* status;
  int pdl;
  long long* trace;           // optional [10]: cycles CTA (0, 0) spent per phase, summed over its chunks (see lap() calls)
};

// shared-memory tiles (byte offsets from a 1024-byte aligned base)
constexpr int G_X1 = 0;                     // [2 panels][128 rows][128 B]  rows 0..63 K beta, 64..127 Q   (later: out staging)
constexpr int G_KT = G_X1 + 32768;          // [2][64][128]   K                      (K-major B)
constexpr int G_KD = G_KT + 16384;          // [2][64][128]   K e^(gc_last - gc)     (MN-major B)
constexpr int G_QG = G_KD + 16384;          // [2][64][128]   Q e^gc                 (K-major B)
constexpr int G_VBT = G_QG + 16384;         // [128][128 B]   (V beta)^T             (K-major A)
constexpr int G_KBGT = G_VBT + 16384;       // [128][128 B]   (K beta e^gc)^T        (K-major A)
constexpr int G_TM = G_KBGT + 16384;        // [64][128 B]    Tm                     (K-major B)
constexpr int G_LOC = G_TM + 8192;          // [64][128 B]    lower((Q K^T) decay)   (K-major B)
constexpr int G_KC = G_LOC + 8192;          // [2][64][128]   k_cum                  (K-major B)
constexpr int G_SB = G_KC + 16384;          // [2][128][128]  S^T as bf16            (K-major A)
constexpr int G_VNT = G_SB + 32768;         // [128][128 B]   v_new^T                (K-major A); before that: L fp32 [64][64]
constexpr int G_SMEM = G_VNT + 16384;
// tensor-memory columns
constexpr uint32_t T_S = 0, T_G = 128, T_VW = 192, T_KC = 256, T_D1 = 320, T_O = 384;

struct GdnShared {
  uint64_t bar;
  uint32_t tmem_slot;
  int abort;
  float g[GC], beta[GC], gc[GC];
};

// byte offset of bf16 element `e` of row `r` in a swizzled tile whose 64-element panels hold `rows` rows each
__device__ __forceinline__ uint32_t sw_off(int rows, int r, int e) {
  return (uint32_t)((e >> 6) * rows * 128 + r * 128 + ((((e & 63) >> 3) ^ (r & 7)) << 4) + (e & 7) * 2);
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// eight consecutive elements (one 16-byte chunk) of a row
__device__ __forceinline__ void store8(uint8_t* tile, int rows, int r, int e0, const float* v, float s) {
  *reinterpret_cast<uint4*>(tile + sw_off(rows, r, e0)) =
      make_uint4(pack_bf16(v[0] * s, v[1] * s), pack_bf16(v[2] * s, v[3] * s), pack_bf16(v[4] * s, v[5] * s),
                 pack_bf16(v[6] * s, v[7] * s));
}

__device__ __forceinline__ void prefetch_l2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

__device__ __forceinline__ bool gdn_wait(GdnShared& S, int* status, uint32_t parity) {
  if (mbar_try_wait(&S.bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(&S.bar, parity)) return true;
    if (S.abort) return false;
    if (clock64() - t0 > SMC_SPIN_CYCLES) {
      atomicOr(status, SMC_ERR_BARRIER_TIMEOUT);
      S.abort = 1;
      return false;
    }
  }
}

__global__ void __launch_bounds__(128, 1) gdn_chunk_kernel(const GdnChunkParams p) {
  extern __shared__ uint8_t gdn_smem_raw[];
  __shared__ GdnShared S;
  const uint32_t raw = smem_u32(gdn_smem_raw);
  uint8_t* sm = gdn_smem_raw + (((raw + 1023u) & ~1023u) - raw);
  if (p.pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x, vh = blockIdx.y, kh = vh / (p.Hv / p.Hk);
  const size_t t0 = p.tok_off ? (size_t)p.tok_off[b] : (size_t)b * p.E;
  const int len = p.tok_len ? p.tok_len[b] : p.E;
  if (len <= 0) return;
  const int key_dim = p.Hk * GD, value_dim = p.Hv * GD;
  const int n_chunks = (len + GC - 1) / GC;

  if (tid == 0) {
    mbar_init(&S.bar, 1);
    S.abort = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&S.tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = S.tmem_slot;
  const uint32_t lane_off = ((uint32_t)(warp * 32)) << 16;
  uint32_t phase = 0;

  // ---- state in: thread d owns row d of S^T (column d of S [dk][dv]) ------------------------------------------------
  float* Sg = p.temporal + (((size_t)p.state_rows[b] * p.Hv + vh) * GD) * GD;
#pragma unroll 1
  for (int c0 = 0; c0 < GD; c0 += 16) {
    uint32_t r[16];
    float f[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      f[i] = Sg[(size_t)(c0 + i) * GD + tid];
      r[i] = __float_as_uint(f[i]);
    }
    tmem_st_32x32b_x16(tm + T_S + lane_off + c0, r);
    store8(sm + G_SB, 128, tid, c0, f, 1.f);
    store8(sm + G_SB, 128, tid, c0 + 8, f + 8, 1.f);
  }
  tmem_st_wait();

  const float a_neg = -__expf(p.A_log[vh]), dtb = p.dt_bias[vh];
  const float wj[4] = {__bfloat162float(p.gnorm_w[lane * 4]), __bfloat162float(p.gnorm_w[lane * 4 + 1]),
                       __bfloat162float(p.gnorm_w[lane * 4 + 2]), __bfloat162float(p.gnorm_w[lane * 4 + 3])};
  constexpr uint32_t idesc64 = umma_idesc_bf16(128, 64);
  constexpr uint32_t idesc128mn = umma_idesc_bf16(128, 128) | (1u << 16);
  const uint32_t sb = smem_u32(sm);
  bool alive = true;
  // phase timing of CTA (0, 0): 0 gates + operand tiles, 1 G MMA, 2 L / local tiles, 3 triangular solve, 4 v_w / k_cum
  // MMAs, 5 k_cum scatter, 6 D1 / out MMAs, 7 v_new + state decay, 8 out / state MMAs, 9 outputs
  const bool tr = p.trace != nullptr && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0;
  long long t_mark = tr ? clock64() : 0;
  auto lap = [&](int slot) {
    if (tr) {
      const long long now = clock64();
      p.trace[slot] += now - t_mark;
      t_mark = now;
    }
  };

#pragma unroll 1
  for (int ch = 0; ch < n_chunks && alive; ++ch) {
    const int n = min(GC, len - ch * GC);
    const size_t tc0 = t0 + (size_t)ch * GC;
    // ---- gates: g_j, beta_j, gc = cumsum(g) (padding tokens: g = 0, beta = 0, all operands zero) ------------------
    if (tid < GC) {
      float g = 0.f, be = 0.f;
      if (tid < n) {
        const float* pr = p.proj + (tc0 + tid) * p.ldp + p.conv_dim + value_dim;
        const float x = pr[p.Hv + vh] + dtb;
        const float sp = x > 20.f ? x : log1pf(__expf(x));
        g = a_neg * sp;
        be = 1.f / (1.f + __expf(-pr[vh]));
      }
      S.beta[tid] = be;
      // inclusive scan over 64 tokens: two warps, then the second adds the first one's total
      float v = g;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      S.gc[tid] = v;
    }
    __syncthreads();
    if (tid >= 32 && tid < GC) S.gc[tid] += S.gc[31];
    __syncthreads();
    const float gl = S.gc[GC - 1];
    {
      // the output phase reads this chunk's gate rows z (512 bytes per token and head): start them towards L2 now
      const int jz = tid >> 1;
      if (jz < n) {
        const float* zr = p.proj + (tc0 + jz) * p.ldp + p.conv_dim + vh * GD + (tid & 1) * 64;
        prefetch_l2(zr);
        prefetch_l2(zr + 32);
      }
    }
    if (ch + 1 < n_chunks) {
      // pull the next chunk's q / k / v rows and gate values towards L2 while this chunk computes
      const int jn = tid >> 1, hfn = tid & 1;
      if ((ch + 1) * GC + jn < len) {
        const float* nrow = p.conv_out + (tc0 + GC + jn) * p.conv_dim;
        prefetch_l2(nrow + kh * GD + hfn * 64);
        prefetch_l2(nrow + kh * GD + hfn * 64 + 32);
        prefetch_l2(nrow + key_dim + kh * GD + hfn * 64);
        prefetch_l2(nrow + key_dim + kh * GD + hfn * 64 + 32);
        prefetch_l2(nrow + 2 * key_dim + vh * GD + hfn * 64);
        prefetch_l2(nrow + 2 * key_dim + vh * GD + hfn * 64 + 32);
        if (hfn == 0) prefetch_l2(p.proj + (tc0 + GC + jn) * p.ldp + p.conv_dim + value_dim + vh);
      }
    }
    {
      // ---- operands: thread (token j, half hf) normalises its 64 q / k elements and scatters them into the tiles ----
      const int j = tid >> 1, hf = tid & 1;
      const bool valid = j < n;
      const float* row = p.conv_out + (tc0 + j) * p.conv_dim;
      const float bj = S.beta[j], gcj = S.gc[j];
      const float egc = __expf(gcj), egl = __expf(gl - gcj);
      float qv[64], kv[64];
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), c = a;
        if (valid) {
          a = *reinterpret_cast<const float4*>(row + kh * GD + hf * 64 + i);
          c = *reinterpret_cast<const float4*>(row + key_dim + kh * GD + hf * 64 + i);
        }
        qv[i] = a.x; qv[i + 1] = a.y; qv[i + 2] = a.z; qv[i + 3] = a.w;
        kv[i] = c.x; kv[i + 1] = c.y; kv[i + 2] = c.z; kv[i + 3] = c.w;
        sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        sk += c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w;
      }
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      sk += __shfl_xor_sync(0xffffffffu, sk, 1);
      const float qn = rsqrtf(sq + 1e-6f) * rsqrtf((float)GD), kn = rsqrtf(sk + 1e-6f);
#pragma unroll
      for (int i = 0; i < 64; i += 8) {
        const int e0 = hf * 64 + i;
        store8(sm + G_X1, 128, j, e0, kv + i, kn * bj);
        store8(sm + G_X1, 128, 64 + j, e0, qv + i, qn);
        store8(sm + G_KT, 64, j, e0, kv + i, kn);
        store8(sm + G_KD, 64, j, e0, kv + i, kn * egl);
        store8(sm + G_QG, 64, j, e0, qv + i, qn * egc);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<__nv_bfloat16*>(sm + G_KBGT + sw_off(128, e0 + u, j)) =
              __float2bfloat16(kv[i + u] * kn * bj * egc);
      }
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid) a = *reinterpret_cast<const float4*>(row + 2 * key_dim + vh * GD + hf * 64 + i);
        const int d = hf * 64 + i;
        *reinterpret_cast<__nv_bfloat16*>(sm + G_VBT + sw_off(128, d, j)) = __float2bfloat16(a.x * bj);
        *reinterpret_cast<__nv_bfloat16*>(sm + G_VBT + sw_off(128, d + 1, j)) = __float2bfloat16(a.y * bj);
        *reinterpret_cast<__nv_bfloat16*>(sm + G_VBT + sw_off(128, d + 2, j)) = __float2bfloat16(a.z * bj);
        *reinterpret_cast<__nv_bfloat16*>(sm + G_VBT + sw_off(128, d + 3, j)) = __float2bfloat16(a.w * bj);
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    lap(0);
    // ---- G = [K beta ; Q] K^T ---------------------------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int pan = 0; pan < 2; ++pan)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tm + T_G, umma_desc_k_sw128(sb + G_X1 + pan * 16384) + 2 * k,
                       umma_desc_k_sw128(sb + G_KT + pan * 8192) + 2 * k, idesc64, (pan | k) ? 1u : 0u);
      umma_commit(&S.bar);
    }
    alive = !__syncthreads_or(!gdn_wait(S, p.status, phase));
    phase ^= 1u;
    if (!alive) break;
    tc_fence_after();
    lap(1);
    {
      // rows 0..63: L[i][j] = G decay below the diagonal (fp32, for the solve); rows 64..127: local attention tile
      const int i = tid & 63;
      const float gci = S.gc[i];
      float* Lf = reinterpret_cast<float*>(sm + G_VNT);
#pragma unroll
      for (int c0 = 0; c0 < GC; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(tm + T_G + lane_off + c0, r);
        tmem_ld_wait();
        float f[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int j = c0 + u;
          const float v = __uint_as_float(r[u]) * __expf(gci - S.gc[j]);
          f[u] = tid < 64 ? (j < i ? v : 0.f) : (j <= i ? v : 0.f);
        }
        if (tid < 64) {
#pragma unroll
          for (int u = 0; u < 16; u += 4)
            *reinterpret_cast<float4*>(Lf + i * GC + c0 + u) = make_float4(f[u], f[u + 1], f[u + 2], f[u + 3]);
        } else {
          store8(sm + G_LOC, 64, i, c0, f, 1.f);
          store8(sm + G_LOC, 64, i, c0 + 8, f + 8, 1.f);
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    lap(2);
    {
      // ---- Tm = (I + L)^-1, in 32 x 32 blocks: [[A, 0], [C, B]]^-1 = [[A^-1, 0], [-B^-1 C A^-1, B^-1]] --------------
      // (1) threads 0..63 solve the two diagonal blocks by forward substitution, one column per thread (fp32, exact);
      // (2) all threads form M = C A^-1, (3) X21 = -B^-1 M; (4) Tm is written as bf16 rows.  Xf (fp32 [64][64]) lives
      // in the k_cum tile, which is not live yet; M is parked in its unused upper-right quadrant.
      const float* Lf = reinterpret_cast<const float*>(sm + G_VNT);
      float* Xf = reinterpret_cast<float*>(sm + G_KC);
      constexpr int HB = GC / 2;
      if (tid < GC) {
        const int blk = tid >> 5, j = tid & 31, o = blk * HB;      // column j of diagonal block blk
        float x[HB];
#pragma unroll
        for (int i = 0; i < HB; ++i) {
          float a0 = (i == j) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
          const float* Li = Lf + (o + i) * GC + o;
#pragma unroll
          for (int k = 0; k + 3 < i; k += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(Li + k);
            a0 = fmaf(-l4.x, x[k], a0);
            a1 = fmaf(-l4.y, x[k + 1], a1);
            a2 = fmaf(-l4.z, x[k + 2], a2);
            a3 = fmaf(-l4.w, x[k + 3], a3);
          }
#pragma unroll
          for (int k = i & ~3; k < i; ++k) a0 = fmaf(-Li[k], x[k], a0);
          x[i] = (a0 + a1) + (a2 + a3);
        }
#pragma unroll
        for (int i = 0; i < HB; ++i) Xf[(o + i) * GC + o + j] = x[i];
      }
      __syncthreads();
      const int r = tid >> 2, c0 = (tid & 3) * 8;                  // every thread: row r, 8 columns of a 32 x 32 product
      {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const float* Cr = Lf + (HB + r) * GC;                      // row r of C = L[32.., 0..32)
#pragma unroll 8
        for (int k = 0; k < HB; ++k) {
          const float c = Cr[k];
          const float4 a0 = *reinterpret_cast<const float4*>(Xf + k * GC + c0);
          const float4 a1 = *reinterpret_cast<const float4*>(Xf + k * GC + c0 + 4);
          acc[0] = fmaf(c, a0.x, acc[0]); acc[1] = fmaf(c, a0.y, acc[1]); acc[2] = fmaf(c, a0.z, acc[2]);
          acc[3] = fmaf(c, a0.w, acc[3]); acc[4] = fmaf(c, a1.x, acc[4]); acc[5] = fmaf(c, a1.y, acc[5]);
          acc[6] = fmaf(c, a1.z, acc[6]); acc[7] = fmaf(c, a1.w, acc[7]);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) Xf[r * GC + HB + c0 + u] = acc[u];          // M[r][c0 + u], parked upper right
      }
      __syncthreads();
      {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const float* Br = Xf + (HB + r) * GC + HB;                 // row r of B^-1 (lower triangular)
#pragma unroll 8
        for (int k = 0; k < HB; ++k) {
          const float bv = Br[k];
          const float4 m0 = *reinterpret_cast<const float4*>(Xf + k * GC + HB + c0);
          const float4 m1 = *reinterpret_cast<const float4*>(Xf + k * GC + HB + c0 + 4);
          acc[0] = fmaf(bv, m0.x, acc[0]); acc[1] = fmaf(bv, m0.y, acc[1]); acc[2] = fmaf(bv, m0.z, acc[2]);
          acc[3] = fmaf(bv, m0.w, acc[3]); acc[4] = fmaf(bv, m1.x, acc[4]); acc[5] = fmaf(bv, m1.y, acc[5]);
          acc[6] = fmaf(bv, m1.z, acc[6]); acc[7] = fmaf(bv, m1.w, acc[7]);
        }
        __syncthreads();                                           // every read of M is done before it is overwritten
#pragma unroll
        for (int u = 0; u < 8; ++u) Xf[(HB + r) * GC + c0 + u] = -acc[u];       // X21
      }
      __syncthreads();
      {
        // Tm rows as bf16: thread (row i, half h) stores 32 columns; the upper-right quadrant is zero
        const int i = tid >> 1, h = tid & 1;
        float f[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) f[u] = (i < HB && h == 1) ? 0.f : Xf[i * GC + h * 32 + u];
#pragma unroll
        for (int u = 0; u < 32; u += 8) store8(sm + G_TM, 64, i, h * 32 + u, f + u, 1.f);
      }
    }
    fence_proxy_async();
    __syncthreads();
    lap(3);
    // ---- v_w^T = (V beta)^T Tm^T, k_cum^T = (K beta e^gc)^T Tm^T ----------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16_ss(tm + T_VW, umma_desc_k_sw128(sb + G_VBT) + 2 * k, umma_desc_k_sw128(sb + G_TM) + 2 * k, idesc64,
                     k ? 1u : 0u);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16_ss(tm + T_KC, umma_desc_k_sw128(sb + G_KBGT) + 2 * k, umma_desc_k_sw128(sb + G_TM) + 2 * k, idesc64,
                     k ? 1u : 0u);
      umma_commit(&S.bar);
    }
    alive = !__syncthreads_or(!gdn_wait(S, p.status, phase));
    phase ^= 1u;
    if (!alive) break;
    tc_fence_after();
    lap(4);
    // k_cum [token][dk]: thread d (= dk index) scatters its row of k_cum^T
#pragma unroll
    for (int c0 = 0; c0 < GC; c0 += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(tm + T_KC + lane_off + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 16; ++u)
        *reinterpret_cast<__nv_bfloat16*>(sm + G_KC + sw_off(64, c0 + u, tid)) = __float2bfloat16(__uint_as_float(r[u]));
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    lap(5);
    // ---- D1 = S^T k_cum^T, out^T = S^T (Q e^gc)^T -------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int pan = 0; pan < 2; ++pan)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tm + T_D1, umma_desc_k_sw128(sb + G_SB + pan * 16384) + 2 * k,
                       umma_desc_k_sw128(sb + G_KC + pan * 8192) + 2 * k, idesc64, (pan | k) ? 1u : 0u);
#pragma unroll
      for (int pan = 0; pan < 2; ++pan)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tm + T_O, umma_desc_k_sw128(sb + G_SB + pan * 16384) + 2 * k,
                       umma_desc_k_sw128(sb + G_QG + pan * 8192) + 2 * k, idesc64, (pan | k) ? 1u : 0u);
      umma_commit(&S.bar);
    }
    alive = !__syncthreads_or(!gdn_wait(S, p.status, phase));
    phase ^= 1u;
    if (!alive) break;
    tc_fence_after();
    lap(6);
    // v_new^T = v_w^T - D1 (bf16 operand tile, row d); S^T *= e^gc_last in tensor memory
#pragma unroll
    for (int c0 = 0; c0 < GC; c0 += 16) {
      uint32_t rv[16], rd[16];
      tmem_ld_32x32b_x16(tm + T_VW + lane_off + c0, rv);
      tmem_ld_32x32b_x16(tm + T_D1 + lane_off + c0, rd);
      tmem_ld_wait();
      float f[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) f[u] = __uint_as_float(rv[u]) - __uint_as_float(rd[u]);
      store8(sm + G_VNT, 128, tid, c0, f, 1.f);
      store8(sm + G_VNT, 128, tid, c0 + 8, f + 8, 1.f);
    }
    {
      const float dl = __expf(gl);
#pragma unroll 1
      for (int c0 = 0; c0 < GD; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(tm + T_S + lane_off + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 16; ++u) r[u] = __float_as_uint(__uint_as_float(r[u]) * dl);
        tmem_st_32x32b_x16(tm + T_S + lane_off + c0, r);
      }
      tmem_st_wait();
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    lap(7);
    // ---- out^T += v_new^T local^T;  S^T += v_new^T (K e^(gc_last - gc)) ---------------------------------------------
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16_ss(tm + T_O, umma_desc_k_sw128(sb + G_VNT) + 2 * k, umma_desc_k_sw128(sb + G_LOC) + 2 * k, idesc64, 1u);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16_ss(tm + T_S, umma_desc_k_sw128(sb + G_VNT) + 2 * k, umma_desc_mn_sw128(sb + G_KD + k * 2048, 8192),
                     idesc128mn, 1u);
      umma_commit(&S.bar);
    }
    alive = !__syncthreads_or(!gdn_wait(S, p.status, phase));
    phase ^= 1u;
    if (!alive) break;
    tc_fence_after();
    lap(8);
    // ---- outputs: stage out [token][dv] in fp32 (the X1 tile is free), refresh the bf16 copy of S^T -------------------
    float* stage = reinterpret_cast<float*>(sm + G_X1);
#pragma unroll
    for (int c0 = 0; c0 < GC; c0 += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(tm + T_O + lane_off + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 16; ++u) stage[(c0 + u) * GD + tid] = __uint_as_float(r[u]);
    }
    if (ch + 1 < n_chunks) {
#pragma unroll 1
      for (int c0 = 0; c0 < GD; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(tm + T_S + lane_off + c0, r);
        tmem_ld_wait();
        float f[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) f[u] = __uint_as_float(r[u]);
        store8(sm + G_SB, 128, tid, c0, f, 1.f);
        store8(sm + G_SB, 128, tid, c0 + 8, f + 8, 1.f);
      }
    }
    tc_fence_before();
    __syncthreads();
    // gated RMSNorm per token: warp w takes tokens w, w + 4, ...; lane l holds dv elements 4l .. 4l + 3.  The gate
    // rows z are fetched for all of the warp's tokens first, so that their latencies overlap.
    {
      float4 z[GC / 4];
#pragma unroll
      for (int u = 0; u < GC / 4; ++u) {
        const int i = warp + 4 * u;
        z[u] = i < n ? *reinterpret_cast<const float4*>(p.proj + (tc0 + i) * p.ldp + p.conv_dim + vh * GD + lane * 4)
                     : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < GC / 4; ++u) {
        const int i = warp + 4 * u;
        if (i >= n) break;
        const float4 o = *reinterpret_cast<const float4*>(stage + i * GD + lane * 4);
        const float ss = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
        const float rs = rsqrtf(ss / (float)GD + p.eps);
        auto fin = [&](float ov, float w, float zv) {
          const float y = __bfloat162float(__float2bfloat16(ov * rs));
          return y * w * (zv / (1.f + __expf(-zv)));
        };
        const uint2 pk = make_uint2(pack_bf16(fin(o.x, wj[0], z[u].x), fin(o.y, wj[1], z[u].y)),
                                    pack_bf16(fin(o.z, wj[2], z[u].z), fin(o.w, wj[3], z[u].w)));
        *reinterpret_cast<uint2*>(p.out + (tc0 + i) * value_dim + vh * GD + lane * 4) = pk;
      }
    }
    __syncthreads();                                  // the staging tile is X1 of the next chunk
    lap(9);
  }

  // ---- state out ------------------------------------------------------------------------------------------------------
  if (alive && !S.abort) {
    tc_fence_after();
#pragma unroll 1
    for (int c0 = 0; c0 < GD; c0 += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(tm + T_S + lane_off + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) Sg[(size_t)(c0 + i) * GD + tid] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
}

}  // namespace smc

// Delta rule + gated RMSNorm of prompt rows, chunk-parallel (the conv + SiLU pass must have filled conv_out).
// Rows as in smc_gdn_varlen; dk = dv = 128 only.
SMC_API int smc_gdn_chunked(const float* conv_out, const float* proj, int ldp, float* temporal, const int* state_rows,
                            const float* dt_bias, const float* A_log, const void* gnorm_w, void* out, int bs, int E,
                            const int* tok_off, const int* tok_len, int Hk, int Hv, int dk, int dv, float eps,
                            int* status, long long* trace, int pdl, cudaStream_t st) {
  using namespace smc;
  if ((tok_off == nullptr) != (tok_len == nullptr)) return -103;
  if (bs <= 0) return 0;
  if (dk != GD || dv != GD || Hv % Hk) return -104;
  GdnChunkParams p;
  p.conv_out = conv_out; p.proj = proj; p.temporal = temporal; p.state_rows = state_rows; p.tok_off = tok_off;
  p.tok_len = tok_len; p.dt_bias = dt_bias; p.A_log = A_log; p.gnorm_w = (const __nv_bfloat16*)gnorm_w;
  p.out = (__nv_bfloat16*)out; p.conv_dim = 2 * Hk * dk + Hv * dv; p.ldp = ldp; p.E = E; p.Hk = Hk; p.Hv = Hv;
  p.eps = eps; p.status = status; p.pdl = pdl; p.trace = trace;
  if ((p.conv_dim % 4) != 0 || (ldp % 4) != 0) return -105;       // float4 row loads
  const size_t smem = G_SMEM + 1024;
  CUDA_CHECK_RET(cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cfg.gridDim = dim3(bs, Hv);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = smem;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, gdn_chunk_kernel, p));
  return 0;
}
