// Fused attention step for uniform extend length E (1 = draft decode, 2 = draft head,
// gamma+1 = target verify) over the token-granular paged KV cache.  One launch per layer does
//   q/k/v of the new tokens from the fp32 QKV GEMM output: optional per-head RMSNorm, rotary
//   embedding, bf16 rounding; new K/V rows written to their pages
//   attention of the E*G query rows of one KV head (GQA packed) over [cached prefix | new tokens]
//   merge of the CTA's key-ways, optional sigmoid output gate, bf16 output rows
// so the separate rope / KV-write / split-merge kernels disappear from the hot loop.
//
// CTA = (sequence, kv head[, key split]); warps = m-tiles (16 query rows each) x key-ways.  Each
// key-way streams 32-key tiles: page ids are read once per range, K/V rows are gathered into
// padded shared-memory tiles with cp.async (all rows of a tile in flight together, double
// buffered), scores and P*V run on tensor cores (mma.sync m16n8k16, bf16 in / fp32 out) with
// flash-style running max / sum in registers.  The new tokens form a last, causally masked tile
// served from shared memory.
#include <stdlib.h>

#include <cuda_fp8.h>

#include "attn_core.cuh"
#include "common.cuh"

namespace smc {

struct FusedAttnParams {
  const float* qkv;          // [T, ld_qkv] fp32
  const __nv_bfloat16* q_in; // optional: rotated bf16 queries [T, Hq*D]; then K/V of the new tokens are already in
                             // their pages and every key is read through the block table (prefill passes)
  int ld_qkv, q_off, gate_off, k_off, v_off;
  const int* positions;      // [T]
  const int* cache_locs;     // [T]
  const float* rope;         // [max_pos, rd] cos | sin
  int rd, max_pos;
  const __nv_bfloat16* qn_w; // [D] or null: per-head RMSNorm weights for q and k
  const __nv_bfloat16* kn_w;
  float norm_eps;
  int norm_plus_one;
  __nv_bfloat16* k_pool;     // [pages + 1, Hkv * D]
  __nv_bfloat16* v_pool;
  int n_pages;
  const int* block_table;
  int bt_stride;
  const int* rows;           // [bs]
  const int* prefix_lens;    // [bs]
  __nv_bfloat16* out;        // [T, Hq * D]
  int gsub;                  // query heads of one kv head are dealt to gsub CTAs (grid z)
  int E, Hq, Hkv, KS, n_mt, n_kw, stg;    // stg: stages of each key-way's K/V tile ring (2..6)
  float scale;
  int* status;
  int pdl;
  // Shared-prefix ("cascade") passes.  A group pass serves the query rows of several sequences that share a prompt
  // from one stream of its keys (rotated queries in q_in, keys [0, prefix), no causal limit) and parks the
  // unnormalised state per (token, head) in part_out; the per-sequence pass then starts at key_begin[b] and folds
  // that state in (part_in) before it normalises.  State row: D values, running max, running sum.
  const int* key_begin;      // [bs] or null: first key of this sequence served by this launch
  float* part_out;           // [T, Hq, D + 2] or null
  const float* part_in;      // [part_in_n, T, Hq, D + 2] or null: states of the key splits of the group pass
  int part_in_n;             // number of states to fold in (>= 1 when part_in is given)
  long long part_in_stride;  // floats between consecutive states
  int causal;                // 0: every key of the range is visible to every query row
  // FP8 KV cache: a page row holds Hkv * D e4m3 bytes, then one fp32 scale per kv head, padded to 16 bytes
  // (kv_row_bytes); value = byte * scale.  k_pool / v_pool then point at bytes.
  int kv_row_bytes;
};

constexpr int RANGE = 2048;     // page ids staged per pass

// PFX = false compiles the shared-prefix options out (no key_begin, no parked states, causal): the plain decode and
// verify steps keep the lean kernel.
// KV8 = true reads and writes the e4m3 cache layout: tiles arrive as bytes in the upper half of their bf16 rows and are
// expanded in place (scaled) before the tensor-core loop; new K/V rows are quantised per (token, kv head) on their way
// to the pages.
template <int D, bool PFX, bool KV8>
__global__ void __launch_bounds__(256) attn_fused_kernel(const FusedAttnParams p) {
  const int* const pfx_key_begin = PFX ? p.key_begin : nullptr;
  float* const pfx_part_out = PFX ? p.part_out : nullptr;
  const float* const pfx_part_in = PFX ? p.part_in : nullptr;
  const int pfx_part_in_n = PFX ? p.part_in_n : 0;
  const long long pfx_part_in_stride = PFX ? p.part_in_stride : 0;
  const int pfx_causal = PFX ? p.causal : 1;
  constexpr int LD = D + 8;
  constexpr bool Q_REGS = D <= 128;
  extern __shared__ __align__(16) uint8_t smem_fa[];
  const int n_mt = p.n_mt, n_kw = p.n_kw;
  // G: query heads per kv head handled by this CTA; hbase: its first query head
  const int G = p.Hq / p.Hkv / p.gsub, R = p.E * G, Rpad = n_mt * 16;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_fa);             // [Rpad][LD]
  __nv_bfloat16* Kn = Qs + (size_t)Rpad * LD;                                 // [16][LD]
  __nv_bfloat16* Vn = Kn + 16 * LD;                                           // [16][LD]
  int* pg = reinterpret_cast<int*>(Vn + 16 * LD);                             // [RANGE]
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(pg + RANGE);        // [n_kw][stg stages][K|V][TK][LD]
  constexpr int TILE = TK * LD;

  const int b = blockIdx.x / p.Hkv, kvh = blockIdx.x % p.Hkv, ks = blockIdx.y;
  const int hbase = kvh * (p.Hq / p.Hkv) + (int)blockIdx.z * (p.Hq / p.Hkv / p.gsub);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = warp % n_mt, kw = warp / n_mt;
  const int nwarps = blockDim.x >> 5;
  if (p.pdl) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
  }
  const int prefix = p.prefix_lens[b];
  const size_t kv_row = (size_t)p.Hkv * D;
  const bool pool_only = p.q_in != nullptr;
  // A group pass without rotated queries (q_in == null, causal == 0) rotates its tokens' queries itself, but writes no
  // K/V rows and skips the new-token tile: the per-sequence pass that follows does both.
  const bool group_self = PFX && !pool_only && !pfx_causal;
  const int g = lane >> 2, t = lane & 3;

  // ---- key range of this CTA and the first K/V fetch (runs under the new-token work below) -----------
  const int n_keys = (pool_only && pfx_causal) ? prefix + p.E : prefix;     // keys served from the paged cache
  const int kbeg = pfx_key_begin != nullptr ? max(0, min(pfx_key_begin[b], n_keys)) : 0;
  int per = (n_keys - kbeg + p.KS - 1) / p.KS;
  per = (per + TK - 1) / TK * TK;
  const int kb = kbeg + ks * per, ke = min(n_keys, kb + per);
  const int* bt = p.block_table + (size_t)p.rows[b] * p.bt_stride;
  const int gsize = 32 * n_mt, gt = mt * 32 + lane;   // thread index inside this key-way's group
  const int stg = p.stg;
  __nv_bfloat16* my_tiles = tiles + (size_t)kw * stg * 2 * TILE;
  constexpr int CPR = D / 8;
  __shared__ int s_pos[16];
  auto load_pages = [&](int r0, int r1) {
    for (int i = threadIdx.x; i < r1 - r0; i += blockDim.x) {
      int page = bt[r0 + i];
      if (page < 0 || page > p.n_pages) { atomicOr(p.status, SMC_ERR_BOUNDS); page = 0; }
      pg[i] = page;
    }
  };
  auto issue = [&](int r0, int r1, int tile, int stage) {
    __nv_bfloat16* Kt = my_tiles + (size_t)stage * 2 * TILE;
    __nv_bfloat16* Vt = Kt + TILE;
    const int k0 = tile * TK;
    if constexpr (KV8) {
      // e4m3 rows: D bytes land in bytes [D, 2D) of the key's bf16 row, the scale in the row's padding at byte 2D
      constexpr int CPR8 = D / 16;
      const uint8_t* kp = reinterpret_cast<const uint8_t*>(p.k_pool);
      const uint8_t* vp = reinterpret_cast<const uint8_t*>(p.v_pool);
      for (int c = gt; c < TK * (CPR8 + 1); c += gsize) {
        const int key = c / (CPR8 + 1), col = c % (CPR8 + 1);
        const int page = (r0 + k0 + key < r1) ? pg[k0 + key] : 0;
        const size_t rowoff = (size_t)page * p.kv_row_bytes;
        uint8_t* kd = reinterpret_cast<uint8_t*>(Kt + key * LD);
        uint8_t* vd = reinterpret_cast<uint8_t*>(Vt + key * LD);
        if (col < CPR8) {
          cp_async16(kd + D + col * 16, kp + rowoff + (size_t)kvh * D + col * 16);
          cp_async16(vd + D + col * 16, vp + rowoff + (size_t)kvh * D + col * 16);
        } else {
          cp_async4(kd + 2 * D, kp + rowoff + (size_t)p.Hkv * D + kvh * 4);
          cp_async4(vd + 2 * D, vp + rowoff + (size_t)p.Hkv * D + kvh * 4);
        }
      }
    } else {
      for (int c = gt; c < TK * CPR; c += gsize) {
        const int key = c / CPR, col = c % CPR;
        const int page = (r0 + k0 + key < r1) ? pg[k0 + key] : 0;
        const size_t off = (size_t)page * kv_row + (size_t)kvh * D + col * 8;
        cp_async16(Kt + key * LD + col * 8, p.k_pool + off);
        cp_async16(Vt + key * LD + col * 8, p.v_pool + off);
      }
    }
  };
  // e4m3 tile -> bf16 in place: one thread per key row walks its 16-byte chunks in order (chunk c is read before the
  // 32 bytes it expands to are written; those never reach a chunk that is still unread)
  auto expand = [&](__nv_bfloat16* Kt) {
    for (int rr = gt; rr < 2 * TK; rr += gsize) {                // rows of the K tile, then of the V tile
      uint8_t* row = reinterpret_cast<uint8_t*>(Kt + (size_t)rr * LD);
      const float sc = *reinterpret_cast<const float*>(row + 2 * D);
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + D + c * 16);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xffffu), __NV_E4M3);
          const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
          const float2 b2 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
          o[2 * i] = pack_bf16(a.x * sc, a.y * sc);
          o[2 * i + 1] = pack_bf16(b2.x * sc, b2.y * sc);
        }
        *reinterpret_cast<uint4*>(row + c * 32) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(row + c * 32 + 16) = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  };
  // Ring of `stg` tiles per key-way: the prologue requests the first stg-1 tiles of a range, then every
  // iteration waits for its tile, refills the stage consumed one iteration earlier and computes.  One copy group
  // is committed per slot whether or not it holds a tile, so the group arithmetic stays uniform.
  auto prologue = [&](int r0, int r1) {
    const int nt_r = (r1 - r0 + TK - 1) / TK;
    for (int j = 0; j < stg - 1; ++j) {
      if (kw + j * n_kw < nt_r) issue(r0, r1, kw + j * n_kw, j);
      cp_async_commit();
    }
  };
  if (threadIdx.x < 16) {
    int pos = 0;
    if ((int)threadIdx.x < p.E) {
      pos = p.positions[b * p.E + threadIdx.x];
      if (pos < 0 || pos >= p.max_pos) {
        atomicOr(p.status, SMC_ERR_BOUNDS);
        pos = pos < 0 ? 0 : p.max_pos - 1;
      }
    }
    s_pos[threadIdx.x] = pos;
  }
  if (kb < ke) load_pages(kb, min(ke, kb + RANGE));
  __syncthreads();
  if (kb < ke) prologue(kb, min(ke, kb + RANGE));

  if (pool_only) {
    // queries were rotated by an earlier kernel; stage them (zero padded) and skip the new-token K/V work
    for (int idx = threadIdx.x; idx < Rpad * (D / 8); idx += blockDim.x) {
      const int r = idx / (D / 8), c = idx % (D / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < R) {
        const int e = r / G, gq = r % G;
        v = *reinterpret_cast<const uint4*>(p.q_in + ((size_t)(b * p.E + e) * p.Hq + hbase + gq) * D + c * 8);
      }
      *reinterpret_cast<uint4*>(Qs + (size_t)r * LD + c * 8) = v;
    }
    __syncthreads();
  } else {
  // ---- phase 0: q / k / v of the new tokens (norm, rope, bf16) ------------------------------------
    const int half = p.rd >> 1;
    // real rows: [0, R) queries, [R, R+E) keys, [R+E, R+2E) values
    auto real_row = [&](int j, __nv_bfloat16*& dst, const float*& src, int& pos) {
      if (j < R) {
        const int e = j / G, gq = j % G;
        dst = Qs + (size_t)j * LD;
        src = p.qkv + (size_t)(b * p.E + e) * p.ld_qkv + p.q_off + (size_t)(hbase + gq) * D;
        pos = s_pos[e];
      } else {
        const bool is_k = j < R + p.E;
        const int e = is_k ? j - R : j - R - p.E;
        dst = (is_k ? Kn : Vn) + (size_t)e * LD;
        src = p.qkv + (size_t)(b * p.E + e) * p.ld_qkv + (is_k ? p.k_off : p.v_off) + (size_t)kvh * D;
        pos = s_pos[e];
      }
    };
    auto store4 = [](__nv_bfloat16* dst, float4 v) {
      uint2 o;
      o.x = pack_bf16(v.x, v.y);
      o.y = pack_bf16(v.z, v.w);
      *reinterpret_cast<uint2*>(dst) = o;
    };
    // zero the padding rows
    for (int idx = threadIdx.x; idx < (Rpad - R) * (D / 8); idx += blockDim.x)
      *reinterpret_cast<uint4*>(Qs + (size_t)(R + idx / (D / 8)) * LD + (idx % (D / 8)) * 8) = make_uint4(0u, 0u, 0u, 0u);
    for (int idx = threadIdx.x; idx < 2 * (16 - p.E) * (D / 8); idx += blockDim.x) {
      const int rr = idx / (D / 8), c = idx % (D / 8);
      __nv_bfloat16* base = rr < 16 - p.E ? Kn + (size_t)(p.E + rr) * LD : Vn + (size_t)(p.E + rr - (16 - p.E)) * LD;
      *reinterpret_cast<uint4*>(base + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (p.qn_w == nullptr && p.kn_w == nullptr && (half & 3) == 0) {
      // no per-head norm: float4-wide, fully independent work items (few loop trips, all loads in flight)
      const int hq = half >> 2;
      for (int idx = threadIdx.x; idx < (R + p.E) * hq; idx += blockDim.x) {       // rotated part of q and k rows
        const int j = idx / hq, i4 = (idx % hq) * 4;
        __nv_bfloat16* dst; const float* src; int pos;
        real_row(j, dst, src, pos);
        const float* cs = p.rope + (size_t)pos * p.rd;
        const float4 a = *reinterpret_cast<const float4*>(src + i4);
        const float4 bb = *reinterpret_cast<const float4*>(src + half + i4);
        const float4 c = *reinterpret_cast<const float4*>(cs + i4);
        const float4 sn = *reinterpret_cast<const float4*>(cs + half + i4);
        store4(dst + i4, make_float4(a.x * c.x - bb.x * sn.x, a.y * c.y - bb.y * sn.y, a.z * c.z - bb.z * sn.z,
                                     a.w * c.w - bb.w * sn.w));
        store4(dst + half + i4, make_float4(bb.x * c.x + a.x * sn.x, bb.y * c.y + a.y * sn.y, bb.z * c.z + a.z * sn.z,
                                            bb.w * c.w + a.w * sn.w));
      }
      const int pq = (D - p.rd) >> 2;                                               // pass-through dims of q and k rows
      for (int idx = threadIdx.x; idx < (R + p.E) * pq; idx += blockDim.x) {
        const int j = idx / pq, i4 = p.rd + (idx % pq) * 4;
        __nv_bfloat16* dst; const float* src; int pos;
        real_row(j, dst, src, pos);
        store4(dst + i4, *reinterpret_cast<const float4*>(src + i4));
      }
      for (int idx = threadIdx.x; idx < p.E * (D / 4); idx += blockDim.x) {         // value rows
        const int j = R + p.E + idx / (D / 4), i4 = (idx % (D / 4)) * 4;
        __nv_bfloat16* dst; const float* src; int pos;
        real_row(j, dst, src, pos);
        store4(dst + i4, *reinterpret_cast<const float4*>(src + i4));
      }
    } else {
      // per-head RMSNorm (hybrid attention layers): one warp per row
      for (int j = warp; j < R + 2 * p.E; j += nwarps) {
        __nv_bfloat16* dst; const float* src; int pos;
        real_row(j, dst, src, pos);
        const bool is_v = j >= R + p.E;
        const __nv_bfloat16* nw = is_v ? nullptr : (j < R ? p.qn_w : p.kn_w);
        float rstd = 1.f;
        if (nw != nullptr) {
          float ss = 0.f;
          for (int i = lane; i < D; i += 32) ss += src[i] * src[i];
          rstd = rsqrtf(warp_sum(ss) / (float)D + p.norm_eps);
        }
        const float* cs = p.rope + (size_t)pos * p.rd;
        const float add = p.norm_plus_one ? 1.f : 0.f;
        for (int i = lane; i < D / 2; i += 32) {
          int i1, i2;
          bool rot;
          if (i < half) { i1 = i; i2 = i + half; rot = !is_v; }
          else { const int jj = i - half; i1 = p.rd + 2 * jj; i2 = i1 + 1; rot = false; }
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
    __syncthreads();
  }
  // new K/V rows go to their pages (one CTA per (sequence, kv head) writes them)
  if constexpr (KV8) {
    if (ks == p.KS - 1 && !pool_only && !group_self && blockIdx.z == 0) {
      // one warp per new K / V row: scale = max|x| / 448, e4m3 bytes and the scale go to the row's page
      uint8_t* kp = reinterpret_cast<uint8_t*>(p.k_pool);
      uint8_t* vp = reinterpret_cast<uint8_t*>(p.v_pool);
      for (int j = warp; j < 2 * p.E; j += nwarps) {
        const bool is_v = j >= p.E;
        const int e = is_v ? j - p.E : j;
        const __nv_bfloat16* src = (is_v ? Vn : Kn) + (size_t)e * LD;
        int loc = p.cache_locs[b * p.E + e];
        if (loc < 0 || loc > p.n_pages) { if (lane == 0) atomicOr(p.status, SMC_ERR_BOUNDS); loc = 0; }
        float amax = 0.f;
        for (int i = lane; i < D; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[i])));
        amax = warp_max(amax);
        const float sc = fmaxf(amax, 1e-12f) * (1.f / 448.f), inv = 1.f / sc;
        uint8_t* dst = (is_v ? vp : kp) + (size_t)loc * p.kv_row_bytes;
        for (int i = lane * 2; i < D; i += 64) {
          const __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(
              make_float2(__bfloat162float(src[i]) * inv, __bfloat162float(src[i + 1]) * inv), __NV_SATFINITE, __NV_E4M3);
          *reinterpret_cast<uint16_t*>(dst + (size_t)kvh * D + i) = (uint16_t)q;
        }
        if (lane == 0) *reinterpret_cast<float*>(dst + (size_t)p.Hkv * D + kvh * 4) = sc;
      }
    }
  } else
  if (ks == p.KS - 1 && !pool_only && !group_self && blockIdx.z == 0) {
    constexpr int CPR = D / 8;
    for (int c = threadIdx.x; c < p.E * CPR * 2; c += blockDim.x) {
      const bool is_v = c >= p.E * CPR;
      const int cc = is_v ? c - p.E * CPR : c;
      const int e = cc / CPR, col = cc % CPR;
      int loc = p.cache_locs[b * p.E + e];
      if (loc < 0 || loc > p.n_pages) { atomicOr(p.status, SMC_ERR_BOUNDS); loc = 0; }
      const uint4 v = *reinterpret_cast<const uint4*>((is_v ? Vn : Kn) + (size_t)e * LD + col * 8);
      *reinterpret_cast<uint4*>((is_v ? p.v_pool : p.k_pool) + (size_t)loc * kv_row + (size_t)kvh * D + col * 8) = v;
    }
  }

  // ---- phase 1: query fragments -----------------------------------------------------------------
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
  // new-token index of this thread's two query rows (rows past R are padding and masked out at the end)
  const int e_row0 = (mt * 16 + g) / G, e_row1 = (mt * 16 + g + 8) / G;
  WarpState<D> st;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) st.o[nt][0] = st.o[nt][1] = st.o[nt][2] = st.o[nt][3] = 0.f;

  // ---- phase 2: cached prefix, streamed in 32-key tiles -------------------------------------------
  for (int r0 = kb; r0 < ke; r0 += RANGE) {
    const int r1 = min(ke, r0 + RANGE);
    const int ntiles = (r1 - r0 + TK - 1) / TK;
    if (r0 != kb) {                       // the first range was staged (and its first tiles requested) above
      cp_async_wait<0>();
      __syncthreads();
      load_pages(r0, r1);
      __syncthreads();
      prologue(r0, r1);
    }
    int j = 0;
    for (int tile = kw; tile < ntiles; tile += n_kw, ++j) {
      cp_async_wait_dyn(stg - 2);         // tile j of this key-way has landed
      group_barrier(1 + kw, gsize);       // ... for every thread of the group, and tile j-1 is fully consumed
      const int jn = j + stg - 1;
      if (kw + jn * n_kw < ntiles) issue(r0, r1, kw + jn * n_kw, jn % stg);
      cp_async_commit();
      const int nvalid = min(TK, r1 - r0 - tile * TK);
      if constexpr (KV8) {
        expand(my_tiles + (size_t)(j % stg) * 2 * TILE);
        group_barrier(1 + kw, gsize);
      }
      const __nv_bfloat16* Kt = my_tiles + (size_t)(j % stg) * 2 * TILE;
      const int key0 = r0 + tile * TK;
      process_tile<D, TK / 8, Q_REGS>(Kt, Kt + TILE, qa, Qs_mt, p.scale, st, nvalid,
                                      pfx_causal ? prefix + e_row0 - key0 : 0x3fffffff,
                                      pfx_causal ? prefix + e_row1 - key0 : 0x3fffffff);
    }
  }
  cp_async_wait<0>();
  // ---- phase 3: the new tokens, causally masked (key-way 0 of the last split) ----------------------
  if (ks == p.KS - 1 && kw == 0 && !pool_only && !group_self) {
    process_tile<D, 2, Q_REGS>(Kn, Vn, qa, Qs_mt, p.scale, st, p.E, e_row0, e_row1);
  }
  st.l0 += __shfl_xor_sync(0xffffffffu, st.l0, 1);
  st.l0 += __shfl_xor_sync(0xffffffffu, st.l0, 2);
  st.l1 += __shfl_xor_sync(0xffffffffu, st.l1, 1);
  st.l1 += __shfl_xor_sync(0xffffffffu, st.l1, 2);

  // ---- phase 4: merge the key-ways in a fixed order, then write ------------------------------------
  __syncthreads();
  float* marea = reinterpret_cast<float*>(tiles);
  const int slot_floats = 16 * D + 64;
  if (kw > 0) {
    float* slot = marea + (size_t)((kw - 1) * n_mt + mt) * slot_floats;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      *reinterpret_cast<float2*>(slot + g * D + nt * 8 + 2 * t) = make_float2(st.o[nt][0], st.o[nt][1]);
      *reinterpret_cast<float2*>(slot + (g + 8) * D + nt * 8 + 2 * t) = make_float2(st.o[nt][2], st.o[nt][3]);
    }
    if (t == 0) {
      slot[16 * D + g] = st.m0; slot[16 * D + 8 + g] = st.m1;
      slot[16 * D + 16 + g] = st.l0; slot[16 * D + 24 + g] = st.l1;
    }
  }
  __syncthreads();
  if (kw == 0) {
    for (int k2 = 1; k2 < n_kw; ++k2) {
      const float* slot = marea + (size_t)((k2 - 1) * n_mt + mt) * slot_floats;
      const float m0b = slot[16 * D + g], m1b = slot[16 * D + 8 + g];
      const float l0b = slot[16 * D + 16 + g], l1b = slot[16 * D + 24 + g];
      const float M0 = fmaxf(st.m0, m0b), M1 = fmaxf(st.m1, m1b);
      const float a0 = M0 == -INFINITY ? 1.f : __expf(st.m0 - M0), b0 = M0 == -INFINITY ? 0.f : __expf(m0b - M0);
      const float a1 = M1 == -INFINITY ? 1.f : __expf(st.m1 - M1), b1 = M1 == -INFINITY ? 0.f : __expf(m1b - M1);
      st.l0 = st.l0 * a0 + l0b * b0; st.l1 = st.l1 * a1 + l1b * b1;
      st.m0 = M0; st.m1 = M1;
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        const float2 x0 = *reinterpret_cast<const float2*>(slot + g * D + nt * 8 + 2 * t);
        const float2 x1 = *reinterpret_cast<const float2*>(slot + (g + 8) * D + nt * 8 + 2 * t);
        st.o[nt][0] = st.o[nt][0] * a0 + x0.x * b0; st.o[nt][1] = st.o[nt][1] * a0 + x0.y * b0;
        st.o[nt][2] = st.o[nt][2] * a1 + x1.x * b1; st.o[nt][3] = st.o[nt][3] * a1 + x1.y * b1;
      }
    }
  }
  // ---- phase 5: merge the key splits across the cluster (CTA rank == split index), rank 0 writes ------
  if (p.KS > 1) {
    __syncthreads();                       // the key-way slots above have been consumed
    if (kw == 0 && ks > 0) {
      float* slot = marea + (size_t)mt * slot_floats;
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        *reinterpret_cast<float2*>(slot + g * D + nt * 8 + 2 * t) = make_float2(st.o[nt][0], st.o[nt][1]);
        *reinterpret_cast<float2*>(slot + (g + 8) * D + nt * 8 + 2 * t) = make_float2(st.o[nt][2], st.o[nt][3]);
      }
      if (t == 0) {
        slot[16 * D + g] = st.m0; slot[16 * D + 8 + g] = st.m1;
        slot[16 * D + 16 + g] = st.l0; slot[16 * D + 24 + g] = st.l1;
      }
    }
    cluster_sync();
    if (kw == 0 && ks == 0) {
      const uint32_t local = smem_u32(marea + (size_t)mt * slot_floats);
      for (int r2 = 1; r2 < p.KS; ++r2) {
        const uint32_t rem = dsmem_map(local, (uint32_t)r2);
        const float m0b = ld_dsmem_f32_at(rem + (16 * D + g) * 4), m1b = ld_dsmem_f32_at(rem + (16 * D + 8 + g) * 4);
        const float l0b = ld_dsmem_f32_at(rem + (16 * D + 16 + g) * 4), l1b = ld_dsmem_f32_at(rem + (16 * D + 24 + g) * 4);
        const float M0 = fmaxf(st.m0, m0b), M1 = fmaxf(st.m1, m1b);
        const float a0 = M0 == -INFINITY ? 1.f : __expf(st.m0 - M0), b0 = M0 == -INFINITY ? 0.f : __expf(m0b - M0);
        const float a1 = M1 == -INFINITY ? 1.f : __expf(st.m1 - M1), b1 = M1 == -INFINITY ? 0.f : __expf(m1b - M1);
        st.l0 = st.l0 * a0 + l0b * b0; st.l1 = st.l1 * a1 + l1b * b1;
        st.m0 = M0; st.m1 = M1;
#pragma unroll
        for (int n0 = 0; n0 < D / 8; n0 += 8) {      // batches of remote loads first, then the arithmetic
          float2 x0[8], x1[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            x0[i] = ld_dsmem_f32x2_at(rem + (g * D + (n0 + i) * 8 + 2 * t) * 4);
            x1[i] = ld_dsmem_f32x2_at(rem + ((g + 8) * D + (n0 + i) * 8 + 2 * t) * 4);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int nt = n0 + i;
            st.o[nt][0] = st.o[nt][0] * a0 + x0[i].x * b0; st.o[nt][1] = st.o[nt][1] * a0 + x0[i].y * b0;
            st.o[nt][2] = st.o[nt][2] * a1 + x1[i].x * b1; st.o[nt][3] = st.o[nt][3] * a1 + x1[i].y * b1;
          }
        }
      }
    }
  }
  if (kw == 0 && ks == 0) {
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      const int r = mt * 16 + g + 8 * hrow;
      if (r >= R) continue;
      const int e = r / G, gq = r % G, tkn = b * p.E + e, head = hbase + gq;
      float m = hrow ? st.m1 : st.m0, l = hrow ? st.l1 : st.l0;
      float a_self = 1.f;
      float a_in[8];
      const float* sin_row = nullptr;
      if (pfx_part_in != nullptr) {
        // fold in the states a group pass left for this (token, head): flash-decoding merge of partial softmaxes
        sin_row = pfx_part_in + ((size_t)tkn * p.Hq + head) * (D + 2);
        float M = m;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (q < pfx_part_in_n) M = fmaxf(M, sin_row[(size_t)q * pfx_part_in_stride + D]);
        a_self = M == -INFINITY ? 1.f : __expf(m - M);
        l *= a_self;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          a_in[q] = 0.f;
          if (q < pfx_part_in_n) {
            const float m_in = sin_row[(size_t)q * pfx_part_in_stride + D], l_in = sin_row[(size_t)q * pfx_part_in_stride + D + 1];
            a_in[q] = (M == -INFINITY || m_in == -INFINITY) ? 0.f : __expf(m_in - M);
            l += l_in * a_in[q];
          }
        }
        m = M;
      }
      if (pfx_part_out != nullptr) {
        float* so = pfx_part_out + ((size_t)tkn * p.Hq + head) * (D + 2);
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt)
          *reinterpret_cast<float2*>(so + nt * 8 + 2 * t) = make_float2(st.o[nt][2 * hrow], st.o[nt][2 * hrow + 1]);
        if (t == 0) { so[D] = m; so[D + 1] = l; }
        continue;
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)tkn * p.Hq + head) * D;
      const float* grow = p.gate_off >= 0 ? p.qkv + (size_t)tkn * p.ld_qkv + p.gate_off + (size_t)head * D : nullptr;
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        float v0 = st.o[nt][2 * hrow] * a_self, v1 = st.o[nt][2 * hrow + 1] * a_self;
        if (sin_row != nullptr) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (q < pfx_part_in_n) {
              const float2 x = *reinterpret_cast<const float2*>(sin_row + (size_t)q * pfx_part_in_stride + nt * 8 + 2 * t);
              v0 += x.x * a_in[q];
              v1 += x.y * a_in[q];
            }
        }
        v0 *= inv;
        v1 *= inv;
        if (grow != nullptr) {
          const float2 gg = *reinterpret_cast<const float2*>(grow + nt * 8 + 2 * t);
          v0 *= 1.f / (1.f + __expf(-gg.x));
          v1 *= 1.f / (1.f + __expf(-gg.y));
        }
        *reinterpret_cast<uint32_t*>(orow + nt * 8 + 2 * t) = pack_bf16(v0, v1);
      }
    }
  }
  // the other splits keep their shared memory alive until rank 0 has read it
  if (p.KS > 1) cluster_sync();
}

// Shared memory one CTA of a single-wave grid may take (SMC_ATTN_SMEM_KB overrides): large rings keep more K/V bytes
// in flight, small CTAs can share an SM with the CTAs of the neighbouring GEMM launches.
static int attn_smem_cap() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("SMC_ATTN_SMEM_KB"); v = (e != nullptr ? atoi(e) : 200) * 1024; }
  return v;
}

static size_t fused_smem_bytes(int D, int n_mt, int n_kw, int stg) {
  const size_t LD = D + 8;
  size_t b = ((size_t)n_mt * 16 + 32) * LD * 2 + RANGE * 4;
  size_t tiles = (size_t)n_kw * stg * 2 * TK * LD * 2;
  // key-way slots of the in-CTA merge; one slot per m-tile is also what the cross-split merge parks
  size_t merge = (size_t)(n_kw > 1 ? (n_kw - 1) * n_mt : n_mt) * (16 * D + 64) * 4;
  return b + (tiles > merge ? tiles : merge);
}

// Query heads of one kv head are dealt to 1, 2 or 4 CTAs when a single CTA would hold more than 64 query rows
// (more than 4 m-tiles leave no warps for key-ways) and the grid still fits one wave.
static int pick_head_groups(int E, int G, long long ctas) {
  int gsub = 1;
  while (gsub < 4 && E * (G / gsub) > 64 && (G / gsub) % 2 == 0 && ctas * gsub * 2 <= 148) gsub *= 2;
  return gsub;
}

// Key-ways per CTA: as many as fit in 8 warps and ~200 KB of shared memory.  Grids of several waves trade
// key-ways for residency (smaller CTAs, more of them per SM), so one CTA's serial phases overlap another's tiles.
static int pick_key_ways(int D, int n_mt, long long ctas) {
  int n_kw = 8 / n_mt;
  if (n_kw < 1) n_kw = 1;
  while (n_kw > 1 && fused_smem_bytes(D, n_mt, n_kw, 2) > (size_t)attn_smem_cap()) --n_kw;
  if (ctas > 2 * 148 && n_kw > 4) n_kw = 4;     // measured at 1024 CTAs: 4 key-ways 45 us, 8: 67 us, 2: 57 us
  return n_kw;
}

}  // namespace smc

// Key-range splits (1, 2, 4 or 8) for `bs` sequences of about `ctx` cached tokens.  A split is taken while the grid
// still fits one wave of one CTA per SM and every key-way keeps at least two 32-key tiles; kernels small enough
// for two CTAs per SM may go to two waves' worth of CTAs once every key-way would still stream eight tiles.
SMC_API int smc_attention_kv_splits(int bs, int E, int Hq, int Hkv, int D, int ctx) {
  using namespace smc;
  if (bs <= 0 || Hkv <= 0 || Hq % Hkv || E < 1) return 1;
  const int gsub = pick_head_groups(E, Hq / Hkv, (long long)bs * Hkv);
  const int R = E * (Hq / Hkv / gsub), n_mt = (R + 15) / 16;
  const int n_kw = pick_key_ways(D, n_mt, 0);
  const bool two_per_sm = fused_smem_bytes(D, n_mt, n_kw, 2) <= 110 * 1024;
  const long long base = (long long)bs * Hkv * gsub;
  int ks = 1;
  while (ks < 8) {
    const int nk = ks * 2;
    const int tiles_per_way = ctx / (nk * TK * n_kw);
    if (base * nk <= 148 && tiles_per_way >= 2) ks = nk;
    else if (two_per_sm && base * nk <= 296 && tiles_per_way >= 8) ks = nk;
    else break;
  }
  return ks;
}

// qkv: fp32 [T, ld_qkv] with query heads at q_off, optional gate heads at gate_off (< 0: none), key heads
// at k_off, value heads at v_off.  out: bf16 [T, Hq*D].  KS in {1, 2, 4, 8} key-range splits per
// (sequence, kv head) run as one thread-block cluster and are merged through distributed shared memory;
// part_acc / part_ml are ignored (kept so existing callers need not change).
SMC_API int smc_attention_fused_ex(const float* qkv, const void* q_in, int ld_qkv, int q_off, int gate_off, int k_off,
                                   int v_off, const int* positions, const int* cache_locs, const float* rope, int rd,
                                   int max_pos, const void* qn_w, const void* kn_w, float norm_eps, int norm_plus_one,
                                   void* k_pool, void* v_pool, int n_pages, const int* block_table, int bt_stride,
                                   const int* rows, const int* prefix_lens, void* out, int bs, int E, int Hq, int Hkv,
                                   int D, int KS, float scale, int* status, int pdl, const int* key_begin,
                                   float* part_out, const float* part_in, int part_in_n, long long part_in_stride,
                                   int causal, int kv_fp8, cudaStream_t st);

SMC_API int smc_attention_fused(const float* qkv, const void* q_in, int ld_qkv, int q_off, int gate_off, int k_off, int v_off,
                                const int* positions, const int* cache_locs, const float* rope, int rd, int max_pos,
                                const void* qn_w, const void* kn_w, float norm_eps, int norm_plus_one, void* k_pool,
                                void* v_pool, int n_pages, const int* block_table, int bt_stride, const int* rows,
                                const int* prefix_lens, void* out, float* part_acc, float* part_ml, int bs, int E,
                                int Hq, int Hkv, int D, int KS, float scale, int* status, int pdl, cudaStream_t st) {
  (void)part_acc;
  (void)part_ml;
  return smc_attention_fused_ex(qkv, q_in, ld_qkv, q_off, gate_off, k_off, v_off, positions, cache_locs, rope, rd, max_pos,
                                qn_w, kn_w, norm_eps, norm_plus_one, k_pool, v_pool, n_pages, block_table, bt_stride, rows,
                                prefix_lens, out, bs, E, Hq, Hkv, D, KS, scale, status, pdl, nullptr, nullptr, nullptr, 0, 0,
                                1, 0, st);
}

// Same, with the shared-prefix options: key_begin [bs] (first key served), part_out / part_in [T, Hq, D + 2] fp32
// (unnormalised attention state parked by a group pass / folded in by the per-sequence pass; part_in may hold up to
// eight states, part_in_stride floats apart, one per key split of the group pass), causal (0: no limit).
// A group pass takes rotated queries (q_in), may span more than 16 tokens per "sequence" (E * Hq / Hkv <= 128 query
// rows) and keeps all query heads of a kv head in one CTA so that its keys are streamed once.
SMC_API int smc_attention_fused_ex(const float* qkv, const void* q_in, int ld_qkv, int q_off, int gate_off, int k_off,
                                   int v_off, const int* positions, const int* cache_locs, const float* rope, int rd,
                                   int max_pos, const void* qn_w, const void* kn_w, float norm_eps, int norm_plus_one,
                                   void* k_pool, void* v_pool, int n_pages, const int* block_table, int bt_stride,
                                   const int* rows, const int* prefix_lens, void* out, int bs, int E, int Hq, int Hkv,
                                   int D, int KS, float scale, int* status, int pdl, const int* key_begin,
                                   float* part_out, const float* part_in, int part_in_n, long long part_in_stride,
                                   int causal, int kv_fp8, cudaStream_t st) {
  using namespace smc;
  if (part_in != nullptr && (part_in_n < 1 || part_in_n > 8)) return -75;
  if (bs <= 0) return 0;
  if (Hq % Hkv || E < 1 || (rd & 1) || rd > D) return -70;
  if (E > 16 && (q_in == nullptr || E * (Hq / Hkv) > 128)) return -70;
  if (!causal && q_in == nullptr && (E > 16 || part_out == nullptr)) return -74;   // self-rotating group pass: <= 16 tokens
  if (!(KS == 1 || KS == 2 || KS == 4 || KS == 8)) return -73;
  const int gsub = part_out != nullptr ? 1 : pick_head_groups(E, Hq / Hkv, (long long)bs * Hkv);
  const int G = Hq / Hkv / gsub, R = E * G;
  const int n_mt = (R + 15) / 16;
  if (n_mt > 8) return -71;
  int n_kw = pick_key_ways(D, n_mt, (long long)bs * Hkv * KS * gsub);
  // Ring depth: a grid that fits the GPU in one wave with one CTA per SM spends the whole shared memory on tiles
  // in flight; larger grids stay under half of it so two CTAs share an SM.
  const size_t budget = (size_t)bs * Hkv * KS * gsub <= 148 ? (size_t)attn_smem_cap() : 100 * 1024;
  int stg = 2;
  while (stg < 6 && fused_smem_bytes(D, n_mt, n_kw, stg + 1) <= budget) ++stg;
  FusedAttnParams p;
  p.qkv = qkv; p.q_in = (const __nv_bfloat16*)q_in; p.ld_qkv = ld_qkv; p.q_off = q_off; p.gate_off = gate_off; p.k_off = k_off; p.v_off = v_off;
  p.positions = positions; p.cache_locs = cache_locs; p.rope = rope; p.rd = rd; p.max_pos = max_pos;
  p.qn_w = (const __nv_bfloat16*)qn_w; p.kn_w = (const __nv_bfloat16*)kn_w; p.norm_eps = norm_eps;
  p.norm_plus_one = norm_plus_one;
  p.k_pool = (__nv_bfloat16*)k_pool; p.v_pool = (__nv_bfloat16*)v_pool; p.n_pages = n_pages;
  p.block_table = block_table; p.bt_stride = bt_stride; p.rows = rows; p.prefix_lens = prefix_lens;
  p.out = (__nv_bfloat16*)out;
  p.E = E; p.Hq = Hq; p.Hkv = Hkv; p.KS = KS; p.gsub = gsub; p.n_mt = n_mt; p.n_kw = n_kw; p.stg = stg; p.scale = scale; p.status = status;
  p.pdl = pdl;
  p.key_begin = key_begin; p.part_out = part_out; p.part_in = part_in; p.causal = causal ? 1 : 0;
  p.part_in_n = part_in_n; p.part_in_stride = part_in_stride;
  p.kv_row_bytes = kv_fp8 ? (Hkv * D + Hkv * 4 + 15) / 16 * 16 : 0;
  const size_t smem = fused_smem_bytes(D, n_mt, n_kw, stg);
  void (*kern)(const FusedAttnParams) = nullptr;
  const bool pfx = key_begin != nullptr || part_out != nullptr || part_in != nullptr || !causal;
  if (kv_fp8) {                                  // the e4m3 cache is served by the full-option build
    if (D == 64) kern = attn_fused_kernel<64, true, true>;
    else if (D == 128) kern = attn_fused_kernel<128, true, true>;
    else if (D == 256) kern = attn_fused_kernel<256, true, true>;
  } else if (D == 64) kern = pfx ? attn_fused_kernel<64, true, false> : attn_fused_kernel<64, false, false>;
  else if (D == 128) kern = pfx ? attn_fused_kernel<128, true, false> : attn_fused_kernel<128, false, false>;
  else if (D == 256) kern = pfx ? attn_fused_kernel<256, true, false> : attn_fused_kernel<256, false, false>;
  else return -72;
  CUDA_CHECK_RET(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (KS > 1) {                            // the splits of one (sequence, kv head) form a cluster along y
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = (unsigned)KS;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(bs * Hkv, KS, gsub);
  cfg.blockDim = dim3(32 * n_mt * n_kw);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, kern, p));
  return 0;
}
