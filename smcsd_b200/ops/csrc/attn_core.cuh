// Device-side building blocks shared by the attention kernels: asynchronous 16-byte gathers, the
// m16n8k16 tensor-core step and one flash-attention tile update (scores, running max / sum, P x V).
#pragma once
#include "common.cuh"

namespace smc {

constexpr int TK = 32;          // keys per streamed tile

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// wait until at most `pending` of this thread's copy groups are still in flight (pending in 0..4)
__device__ __forceinline__ void cp_async_wait_dyn(int pending) {
  switch (pending) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    case 3: cp_async_wait<3>(); break;
    default: cp_async_wait<4>(); break;
  }
}
__device__ __forceinline__ void group_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Running flash state of one warp: rows g and g+8 of its m-tile.
template <int D>
struct WarpState {
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[D / 8][4];
};

// One tile of NT*8 keys.  Kt / Vt: [keys][D + 8] bf16.  Key `col` of the tile is visible to this thread's
// query rows g / g+8 iff col < nvalid and col <= lim0 / lim1 (the causal limits, precomputed by the caller).
template <int D, int NT, bool Q_REGS>
__device__ __forceinline__ void process_tile(const __nv_bfloat16* Kt, const __nv_bfloat16* Vt,
                                             const uint32_t (&qa)[Q_REGS ? D / 16 : 1][4],
                                             const __nv_bfloat16* Qs_mt, float scale, WarpState<D>& st, int nvalid,
                                             int lim0, int lim1) {
  constexpr int LD = D + 8;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  float s[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    if constexpr (Q_REGS) {
      a[0] = qa[kk][0]; a[1] = qa[kk][1]; a[2] = qa[kk][2]; a[3] = qa[kk][3];
    } else {
      a[0] = *reinterpret_cast<const uint32_t*>(Qs_mt + g * LD + kk * 16 + 2 * t);
      a[1] = *reinterpret_cast<const uint32_t*>(Qs_mt + (g + 8) * LD + kk * 16 + 2 * t);
      a[2] = *reinterpret_cast<const uint32_t*>(Qs_mt + g * LD + kk * 16 + 2 * t + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(Qs_mt + (g + 8) * LD + kk * 16 + 2 * t + 8);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const __nv_bfloat16* kr = Kt + (nt * 8 + g) * LD + kk * 16 + 2 * t;
      mma16816(s[nt], a, *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 8));
    }
  }
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = nt * 8 + 2 * t + (c & 1);
      const bool vis = col < nvalid && col <= (c < 2 ? lim0 : lim1);
      const float v = vis ? s[nt][c] * scale : -INFINITY;
      s[nt][c] = v;
      if (c < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
    }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);
  const float c0 = mn0 == -INFINITY ? 1.f : __expf(st.m0 - mn0);
  const float c1 = mn1 == -INFINITY ? 1.f : __expf(st.m1 - mn1);
  st.m0 = mn0; st.m1 = mn1;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    s[nt][0] = mn0 == -INFINITY ? 0.f : __expf(s[nt][0] - mn0);
    s[nt][1] = mn0 == -INFINITY ? 0.f : __expf(s[nt][1] - mn0);
    s[nt][2] = mn1 == -INFINITY ? 0.f : __expf(s[nt][2] - mn1);
    s[nt][3] = mn1 == -INFINITY ? 0.f : __expf(s[nt][3] - mn1);
    sum0 += s[nt][0] + s[nt][1];
    sum1 += s[nt][2] + s[nt][3];
  }
  st.l0 = st.l0 * c0 + sum0;
  st.l1 = st.l1 * c1 + sum1;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    st.o[nt][0] *= c0; st.o[nt][1] *= c0; st.o[nt][2] *= c1; st.o[nt][3] *= c1;
  }
  // P (bf16) x V
  const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
  for (int k2 = 0; k2 < NT / 2; ++k2) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * k2][0], s[2 * k2][1]);
    a[1] = pack_bf16(s[2 * k2][2], s[2 * k2][3]);
    a[2] = pack_bf16(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
    a[3] = pack_bf16(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
#pragma unroll
    for (int nt = 0; nt < D / 8; nt += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, Vt + (k2 * 16 + (mat & 1) * 8 + rr) * LD + (nt + (mat >> 1)) * 8);
      mma16816(st.o[nt], a, b[0], b[1]);
      mma16816(st.o[nt + 1], a, b[2], b[3]);
    }
  }
}

}  // namespace smc
