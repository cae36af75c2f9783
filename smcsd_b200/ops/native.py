"""ctypes bindings of the sm_100a kernel library.

Every wrapper launches on PyTorch's current CUDA stream, takes torch tensors, allocates
nothing on its own (scratch buffers are passed in) and is therefore safe to capture in a CUDA
graph.  The library must be present on a GPU machine: ``lib()`` raises instead of falling
back to PyTorch.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsmcsd_b200.so")
_lib = None

EPI_PARTIAL_F32, EPI_BF16, EPI_SWIGLU_BF16, EPI_STORE_F32, EPI_RESID_F32 = 0, 1, 2, 3, 4
ERR_BARRIER_TIMEOUT, ERR_PEER_TIMEOUT, ERR_ALLOC_EXHAUSTED, ERR_BOUNDS = 1, 2, 4, 8


class NativeError(RuntimeError):
    pass


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            from . import build as _build
            _build.build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(L) -> None:
    vp, i, ll, f, d, ull = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_double, C.c_ulonglong
    L.smc_gemm_skinny.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp, i, vp]
    L.smc_gemm_bn_for.argtypes = [i]
    L.smc_gemm_default_splits.argtypes = [i, i, i]
    L.smc_gemm_cluster_splits.argtypes = [i, i, i]
    L.smc_gemm_cluster_splits.restype = C.c_int
    L.smc_add_rmsnorm.argtypes = [vp, vp, i, ll, vp, vp, vp, vp, i, i, i, f, i, vp, vp, i, vp]
    L.smc_gemm_skinny_norm.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp, i, vp, i, i, i, f, vp, vp, i, i, vp]
    L.smc_gemm_skinny_norm.restype = C.c_int
    L.smc_rope_kv_write.argtypes = [vp, i, ll, vp, vp, vp, i, i, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    L.smc_swiglu_partials.argtypes = [vp, i, ll, vp, i, i, i, i, i, vp]
    L.smc_attention_fused_ex.argtypes = [vp, vp, i, i, i, i, i, vp, vp, vp, i, i, vp, vp, f, i, vp, vp, i, vp, i, vp, vp,
                                         vp, i, i, i, i, i, i, f, vp, i, vp, vp, vp, i, ll, i, i, vp]
    L.smc_attention_fused_ex.restype = C.c_int
    L.smc_kv_store_e4m3.argtypes = [vp, vp, i, vp, vp, vp, i, i, i, i, vp, i, vp]
    L.smc_kv_store_e4m3.restype = C.c_int
    L.smc_sample_scratch_bytes.argtypes = [i, i]
    L.smc_sample_or_score.argtypes = [vp, i, ll, ll, i, i, f, f, f, vp, ull, vp, i, vp, i, vp, vp, vp, i, vp]
    L.smc_slot_arrays_size.argtypes = []
    L.smc_prepare_cycle.argtypes = [vp, vp, i, i, vp, vp, vp]
    L.smc_assemble_verify.argtypes = [vp, vp, i, i, vp]
    L.smc_cycle_io_size.argtypes = []
    L.smc_write_back.argtypes = [vp, vp, i, i, vp, vp, vp, vp, vp, f, i, vp, vp, vp]
    L.smc_collect_resample.argtypes = [vp, vp, i, vp, i, d, ull, vp, vp, vp, vp, vp]
    L.smc_state_copy.argtypes = [vp, ll, ll, i, i, vp, vp, vp, i, vp]
    for name in ("smc_gemm_skinny", "smc_add_rmsnorm", "smc_rope_kv_write", "smc_swiglu_partials",
                 "smc_sample_or_score", "smc_prepare_cycle", "smc_write_back",
                 "smc_collect_resample", "smc_state_copy", "smc_gemm_bn_for", "smc_gemm_default_splits",
                 "smc_sample_scratch_bytes", "smc_slot_arrays_size", "smc_assemble_verify", "smc_cycle_io_size"):
        getattr(L, name).restype = C.c_int


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


# kernels launched through this module (a captured graph replays the launches counted at capture)
launch_count = 0
_KERNELS_PER_CALL = {"smc_sample_or_score": 2, "smc_collect_resample": 2}


def _check(rc: int, what: str) -> None:
    global launch_count
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")
    launch_count += _KERNELS_PER_CALL.get(what, 1)


# ----------------------------------------------------------------------------- GEMM
def gemm_default_splits(N: int, K: int, M: int) -> int:
    return lib().smc_gemm_default_splits(N, K, M)


def gemm_cluster_splits(N: int, K: int, M: int) -> int:
    return lib().smc_gemm_cluster_splits(N, K, M)


def gemm_swiglu_splits(N: int, K: int, M: int) -> int:
    """Split-K factor of a gate/up GEMM with the SwiGLU epilogue.  Only grids that leave SMs idle are cut along K
    (cluster reduction before the activation): a tensor-parallel shard with 56 slabs runs as 112 CTAs, while 128
    slabs stay unsplit (measured on B200: 13.2 us unsplit, 14.0 us with two splits).  ``SMC_GU_SPLITS`` overrides."""
    env = os.environ.get("SMC_GU_SPLITS")
    if env:
        return max(1, int(env))
    bn = lib().smc_gemm_bn_for(M)
    tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
    kblocks = (K + 63) // 64
    s = 1
    while s < 4 and tiles * s * 2 <= 148 and kblocks // (s * 2) >= 4:
        s *= 2
    return s


def gemm_skinny(W: torch.Tensor, X: torch.Tensor, out: torch.Tensor, *, M: int, splits: int = 1,
                epi: int = EPI_PARTIAL_F32, ldx: Optional[int] = None, ldo: Optional[int] = None,
                status: torch.Tensor, pdl: bool = False) -> None:
    """out = X[:M] @ W.T on the tcgen05 tensor cores.  W [N, K] bf16; X rows of pitch ``ldx``."""
    N, K = W.shape
    ldx = ldx if ldx is not None else X.stride(0)
    ldo = ldo if ldo is not None else (out.stride(0) if out.dim() == 2 else N)
    _check(lib().smc_gemm_skinny(_p(W), _p(X), _p(out), N, K, M, ldx, ldo, splits, epi, _p(status), int(pdl),
                                 _stream()), "smc_gemm_skinny")


def gemm_skinny_fp8(W8: torch.Tensor, w_scale: torch.Tensor, X8: torch.Tensor, x_scale: Optional[torch.Tensor],
                    out: torch.Tensor, *, M: int, splits: int = 1, epi: int = EPI_PARTIAL_F32,
                    ldx: Optional[int] = None, ldo: Optional[int] = None, status: torch.Tensor, pdl: bool = False) -> None:
    """W8A8 GEMM on tcgen05 (kind::f8f6f4): out = (X8[:M] * x_scale[:, None]) @ (W8 * w_scale[:, None]).T with e4m3
    operands (uint8 / float8_e4m3fn storage), fp32 accumulation, scales applied in the epilogue."""
    N, K = W8.shape
    ldx = ldx if ldx is not None else X8.stride(0)
    ldo = ldo if ldo is not None else (out.stride(0) if out.dim() == 2 else N)
    L = lib()
    if not getattr(L, "_fp8_declared", False):
        vp, i = C.c_void_p, C.c_int
        L.smc_gemm_skinny_fp8.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp, vp, vp, i, vp]
        L.smc_gemm_skinny_fp8.restype = C.c_int
        L.smc_quant_rows_e4m3.argtypes = [vp, i, vp, i, vp, i, i, i, vp]
        L.smc_quant_rows_e4m3.restype = C.c_int
        L._fp8_declared = True
    _check(L.smc_gemm_skinny_fp8(_p(W8), _p(X8), _p(out), N, K, M, ldx, ldo, splits, epi, _p(w_scale), _p(x_scale),
                                 _p(status), int(pdl), _stream()), "smc_gemm_skinny_fp8")


def quant_rows_e4m3(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor, *, M: int, K: int, pdl: bool = False) -> None:
    """Per-row dynamic quantisation of bf16 rows to e4m3 bytes: ``scale[m] = max|x[m]| / 448``, ``q = x / scale``."""
    L = lib()
    if not getattr(L, "_fp8_declared", False):
        vp, i = C.c_void_p, C.c_int
        L.smc_gemm_skinny_fp8.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp, vp, vp, i, vp]
        L.smc_gemm_skinny_fp8.restype = C.c_int
        L.smc_quant_rows_e4m3.argtypes = [vp, i, vp, i, vp, i, i, i, vp]
        L.smc_quant_rows_e4m3.restype = C.c_int
        L._fp8_declared = True
    _check(L.smc_quant_rows_e4m3(_p(x), x.stride(0), _p(q), q.stride(0), _p(scale), M, K, int(pdl), _stream()),
           "smc_quant_rows_e4m3")


def quantize_weight_e4m3(w: torch.Tensor):
    """Per-output-row e4m3 quantisation of a weight matrix [N, K] (host-side helper, PyTorch): returns (bytes, scale)."""
    wf = w.float()
    scale = wf.abs().amax(dim=1).clamp_(min=1e-12) / 448.0
    q = (wf / scale[:, None]).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).contiguous(), scale.contiguous()


def gemm_skinny_norm(W: torch.Tensor, X: torch.Tensor, out: torch.Tensor, *, M: int, splits: int, epi: int, ldo: int,
                     status: torch.Tensor, ssq_in: Optional[torch.Tensor] = None, ssq_parts: int = 0, norm_d: int = 0,
                     norm_eps: float = 0.0, ssq_out: Optional[torch.Tensor] = None, hb_out: Optional[torch.Tensor] = None,
                     ldx: Optional[int] = None, pdl: bool = False, ssq_ld: int = 0, ssq_mstride: int = 1) -> None:
    """GEMM with the RMSNorm folded in: outputs scaled per token by rsqrt(sum_p ssq_in[p, m] / norm_d + eps); the
    residual epilogue can emit the bf16 copy of the new rows (``hb_out``) and their sums of squares (``ssq_out``
    [n_tiles, ld]) for the next consumer."""
    N, K = W.shape
    ldx = ldx if ldx is not None else X.stride(0)
    if not ssq_ld:
        ref = ssq_in if ssq_in is not None else ssq_out
        ssq_ld = ref.stride(0) if ref is not None and ref.dim() == 2 else 0
    _check(lib().smc_gemm_skinny_norm(_p(W), _p(X), _p(out), N, K, M, ldx, ldo, splits, epi, _p(status), int(pdl),
                                      _p(ssq_in), ssq_parts, ssq_ld, norm_d, norm_eps, _p(ssq_out), _p(hb_out),
                                      hb_out.stride(0) if hb_out is not None else 0, ssq_mstride, _stream()),
           "smc_gemm_skinny")


# ----------------------------------------------------------------------------- fused elementwise
def add_rmsnorm(h: torch.Tensor, w: Optional[torch.Tensor], xn: Optional[torch.Tensor], *, M: int, d: int, eps: float,
                partials: Optional[torch.Tensor] = None, splits: int = 0, split_stride: int = 0,
                ids: Optional[torch.Tensor] = None, embed: Optional[torch.Tensor] = None, ldx: Optional[int] = None,
                plus_one: bool = False, pdl: bool = False, hb: Optional[torch.Tensor] = None,
                ssq: Optional[torch.Tensor] = None) -> None:
    """h (+= partials | = embedding rows); optional outputs: normalised bf16 ``xn``, raw bf16 copy ``hb`` and the
    per-row sum of squares ``ssq`` (for GEMMs that apply the norm in their epilogue)."""
    ldx = ldx if ldx is not None else (xn.stride(0) if xn is not None else d)
    _check(lib().smc_add_rmsnorm(_p(h), _p(partials), splits, split_stride, _p(ids), _p(embed), _p(w), _p(xn), ldx, M,
                                 d, eps, int(plus_one), _p(hb), _p(ssq), int(pdl), _stream()), "smc_add_rmsnorm")


def add_rmsnorm_q8(h: torch.Tensor, w: torch.Tensor, xn: torch.Tensor, q8: torch.Tensor, qscale: torch.Tensor, *, M: int,
                   d: int, eps: float, ids: Optional[torch.Tensor] = None, embed: Optional[torch.Tensor] = None,
                   plus_one: bool = False, pdl: bool = False) -> None:
    """RMSNorm of the residual rows (or of embedding rows) that also emits the e4m3 copy of the normalised rows with
    per-row scales, for the W8A8 GEMMs."""
    L = lib()
    if not getattr(L, "_q8norm_declared", False):
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        L.smc_add_rmsnorm_q8.argtypes = [vp, vp, vp, vp, vp, i, i, i, f, i, vp, i, vp, i, vp]
        L.smc_add_rmsnorm_q8.restype = C.c_int
        L._q8norm_declared = True
    _check(L.smc_add_rmsnorm_q8(_p(h), _p(ids), _p(embed), _p(w), _p(xn), xn.stride(0), M, d, eps, int(plus_one),
                                _p(q8), q8.stride(0), _p(qscale), int(pdl), _stream()), "smc_add_rmsnorm_q8")


def kv_row_bytes_e4m3(Hkv: int, D: int) -> int:
    """Bytes of one page row of the e4m3 KV cache: Hkv * D value bytes, one fp32 scale per kv head, padded to 16."""
    return (Hkv * D + Hkv * 4 + 15) // 16 * 16


_KV8_TMP = {}


def rope_kv_write(partials: torch.Tensor, splits: int, split_stride: int, positions: torch.Tensor,
                  cache_locs: torch.Tensor, rope: torch.Tensor, q_out: torch.Tensor, k_pool: torch.Tensor,
                  v_pool: torch.Tensor, *, M: int, Hq: int, Hkv: int, D: int, status: torch.Tensor,
                  pdl: bool = False) -> None:
    """Rotary + bf16 rounding of the new tokens; q rows to ``q_out``, K/V rows to their cache pages.  With an e4m3
    cache (uint8 pools) the rotated K/V rows pass through a bf16 staging buffer and a quantising store kernel."""
    if k_pool.dtype == torch.uint8:
        key = (k_pool.device, Hkv * D)
        tmp = _KV8_TMP.get(key)
        if tmp is None or tmp[0].shape[0] < M + 1:
            n = max(M + 1, 4096)
            tmp = (torch.zeros(n, Hkv * D, dtype=torch.bfloat16, device=k_pool.device),
                   torch.zeros(n, Hkv * D, dtype=torch.bfloat16, device=k_pool.device),
                   torch.arange(n, dtype=torch.int32, device=k_pool.device))
            _KV8_TMP[key] = tmp
        tk, tv, iota = tmp
        _check(lib().smc_rope_kv_write(_p(partials), splits, split_stride, _p(positions), _p(iota), _p(rope),
                                       rope.shape[1], rope.shape[0], _p(q_out), _p(tk), _p(tv), tk.shape[0] - 1, M, Hq,
                                       Hkv, D, _p(status), int(pdl), _stream()), "smc_rope_kv_write")
        _check(lib().smc_kv_store_e4m3(_p(tk), _p(tv), M, _p(cache_locs), _p(k_pool), _p(v_pool), k_pool.shape[0] - 1,
                                       Hkv, D, kv_row_bytes_e4m3(Hkv, D), _p(status), int(pdl), _stream()),
               "smc_kv_store_e4m3")
        return
    _check(lib().smc_rope_kv_write(_p(partials), splits, split_stride, _p(positions), _p(cache_locs), _p(rope),
                                   rope.shape[1], rope.shape[0], _p(q_out), _p(k_pool), _p(v_pool),
                                   k_pool.shape[0] - 1, M, Hq, Hkv, D, _p(status), int(pdl), _stream()),
           "smc_rope_kv_write")


def rope_kv_write_heads(qkv: torch.Tensor, positions: torch.Tensor, cache_locs: torch.Tensor, rope: torch.Tensor,
                        q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *, M: int, Hq: int, Hkv: int,
                        D: int, status: torch.Tensor, q_off: int = 0, k_off: Optional[int] = None,
                        v_off: Optional[int] = None, qn_w: Optional[torch.Tensor] = None,
                        kn_w: Optional[torch.Tensor] = None, norm_eps: float = 1e-6, norm_plus_one: bool = False,
                        pdl: bool = False) -> None:
    """New-token stage on its own (prompt passes): per-head RMSNorm, rotary, bf16; q rows to ``q_out``, k/v rows to
    their cache pages.  Column offsets select q / k / v inside the fp32 projection rows."""
    L = lib()
    if not getattr(L, "_rkh_declared", False):
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        L.smc_rope_kv_write_heads.argtypes = [vp, i, i, i, i, vp, vp, vp, i, i, vp, vp, f, i, vp, vp, vp, i, i, i, i, i,
                                              vp, i, vp]
        L.smc_rope_kv_write_heads.restype = C.c_int
        L._rkh_declared = True
    k_off = Hq * D if k_off is None else k_off
    v_off = k_off + Hkv * D if v_off is None else v_off
    _check(L.smc_rope_kv_write_heads(_p(qkv), qkv.stride(0), q_off, k_off, v_off, _p(positions), _p(cache_locs),
                                     _p(rope), rope.shape[1], rope.shape[0], _p(qn_w), _p(kn_w), norm_eps,
                                     int(norm_plus_one), _p(q_out), _p(k_pool), _p(v_pool), k_pool.shape[0] - 1, M, Hq,
                                     Hkv, D, _p(status), int(pdl), _stream()), "smc_rope_kv_write_heads")


def swiglu_partials(partials: torch.Tensor, splits: int, split_stride: int, act: torch.Tensor, *, M: int, ffn: int,
                    blk: int, pdl: bool = False) -> None:
    _check(lib().smc_swiglu_partials(_p(partials), splits, split_stride, _p(act), M, ffn, blk, act.stride(0), int(pdl),
                                     _stream()), "smc_swiglu_partials")


def attention_fused(qkv: torch.Tensor, positions: torch.Tensor, cache_locs: torch.Tensor, rope: torch.Tensor,
                    k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, rows: torch.Tensor,
                    prefix_lens: torch.Tensor, out: Optional[torch.Tensor], part_acc: Optional[torch.Tensor] = None,
                    part_ml: Optional[torch.Tensor] = None, *,
                    bs: int, E: int, Hq: int, Hkv: int, D: int, KS: int, scale: float, status: torch.Tensor,
                    q_off: int = 0, gate_off: int = -1, k_off: Optional[int] = None, v_off: Optional[int] = None,
                    qn_w: Optional[torch.Tensor] = None, kn_w: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
                    norm_plus_one: bool = False, pdl: bool = False, q_in: Optional[torch.Tensor] = None,
                    key_begin: Optional[torch.Tensor] = None, part_out: Optional[torch.Tensor] = None,
                    part_in: Optional[torch.Tensor] = None, causal: bool = True, part_in_n: int = 1,
                    part_in_stride: int = 0) -> None:
    """Norm/rope/KV-write of the new tokens + paged causal attention + split merge, one launch per layer.
    K/V pools of dtype uint8 hold the e4m3 cache layout (``kv_row_bytes_e4m3``): tiles are dequantised after they
    land, new rows are quantised on their way to the pages.
    Shared-prefix passes: ``causal=False`` with ``q_in`` and ``part_out`` serves the rows of several sequences from
    one stream of their common keys and parks the unnormalised state; ``key_begin`` / ``part_in`` make the
    per-sequence launch start after those keys and fold the state in.  (``part_acc`` / ``part_ml`` are ignored.)"""
    k_off = Hq * D if k_off is None else k_off
    v_off = k_off + Hkv * D if v_off is None else v_off
    _check(lib().smc_attention_fused_ex(_p(qkv), _p(q_in), qkv.stride(0), q_off, gate_off, k_off, v_off, _p(positions),
                                        _p(cache_locs), _p(rope), rope.shape[1], rope.shape[0], _p(qn_w), _p(kn_w),
                                        norm_eps, int(norm_plus_one), _p(k_pool), _p(v_pool), k_pool.shape[0] - 1,
                                        _p(block_table), block_table.stride(0), _p(rows), _p(prefix_lens), _p(out),
                                        bs, E, Hq, Hkv, D, KS, scale, _p(status), int(pdl), _p(key_begin),
                                        _p(part_out), _p(part_in), part_in_n if part_in is not None else 0,
                                        part_in_stride, int(causal), int(k_pool.dtype == torch.uint8), _stream()),
           "smc_attention_fused")


def attention_tc_splits(n_seq: int, Hkv: int, keys: int, rows: int = 128) -> int:
    L = lib()
    L.smc_attention_tc_splits.argtypes = [C.c_int] * 4
    L.smc_attention_tc_splits.restype = C.c_int
    return L.smc_attention_tc_splits(n_seq, Hkv, keys, rows)


def attention_prefix_tc(q: Optional[torch.Tensor], k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                        rows: torch.Tensor, key_count: torch.Tensor, part_out: torch.Tensor, *, n_seq: int, E: int,
                        T: int, Hq: int, Hkv: int, D: int, KS: int, scale: float, status: torch.Tensor,
                        trace: Optional[torch.Tensor] = None, use_tma: bool = True, qkv: Optional[torch.Tensor] = None,
                        q_off: int = 0, positions: Optional[torch.Tensor] = None,
                        rope: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """Shared-prefix attention pass on tcgen05: the E tokens (all query heads) of every (super-)sequence against keys
    [0, key_count) of its block-table row, no causal limit; parks the unnormalised state of every key split in
    ``part_out`` [KS, T, Hq, D + 2].  ``trace`` (int64 [CTAs, 12], optional) receives the cycles every CTA spent in
    its waits: softmax {scores ready, score load, P buffer free, exp + store, total}, MMA {K/V, score buffer, P}, first
    loader warp {stage free, copy issue, landing, total}.  Tiles of 64 consecutive pages are fetched by TMA unless
    ``use_tma`` is off; scattered tiles are gathered row by row.  With ``q`` None the kernel rotates the fp32 query
    projections ``qkv`` (heads at ``q_off``) itself, given ``positions`` and the ``rope`` table."""
    L = lib()
    if not getattr(L, "_atc_declared", False):
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        L.smc_attention_prefix_tc.argtypes = [vp, vp, vp, i, vp, i, vp, vp, vp, i, i, i, i, i, i, i, f, vp, vp, i, vp, i, i, vp, vp, i,
                                              i, vp]
        L.smc_attention_prefix_tc.restype = C.c_int
        L._atc_declared = True
    _check(L.smc_attention_prefix_tc(_p(q), _p(k_pool), _p(v_pool), k_pool.shape[0] - 1, _p(block_table),
                                     block_table.stride(0), _p(rows), _p(key_count), _p(part_out), n_seq, E, T, Hq, Hkv,
                                     D, KS, scale, _p(status), _p(trace), int(use_tma), _p(qkv),
                                     qkv.stride(0) if qkv is not None else 0, q_off, _p(positions), _p(rope),
                                     rope.shape[1] if rope is not None else 0, int(pdl), _stream()), "smc_attention_prefix_tc")


def attn_kv_splits(ctx: int, bs: int, Hkv: int, E: int = 1, G: int = 4, D: int = 128) -> int:
    """Key-range splits (1, 2, 4 or 8) the fused attention step should use for ``bs`` sequences of about ``ctx``
    cached tokens with ``E`` new tokens, ``G`` query heads per kv head and head size ``D``.  The splits of one
    (sequence, kv head) run as a thread-block cluster and are merged on chip."""
    L = lib()
    if not getattr(L, "_aks_declared", False):
        L.smc_attention_kv_splits.argtypes = [C.c_int] * 6
        L.smc_attention_kv_splits.restype = C.c_int
        L._aks_declared = True
    return L.smc_attention_kv_splits(bs, E, Hkv * G, Hkv, D, int(ctx))


def sample_scratch_bytes(rows: int, nchunks: int) -> int:
    return lib().smc_sample_scratch_bytes(rows, nchunks)


def sample_or_score(logits: torch.Tensor, *, rows: int, V: int, splits: int, split_stride: int, row_stride: int,
                    temperature: float, alpha: float, softcap: float, tokens_in: Optional[torch.Tensor], seed: int,
                    cycle_counter: torch.Tensor, call_id: int, scratch: torch.Tensor, nchunks: int,
                    tok_out: torch.Tensor, logp_out: torch.Tensor, logz_out: Optional[torch.Tensor],
                    pdl: bool = False) -> None:
    _check(lib().smc_sample_or_score(_p(logits), splits, split_stride, row_stride, rows, V, temperature, alpha,
                                     softcap, _p(tokens_in), seed & 0xFFFFFFFFFFFFFFFF, _p(cycle_counter), call_id,
                                     _p(scratch), nchunks, _p(tok_out), _p(logp_out), _p(logz_out), int(pdl),
                                     _stream()), "smc_sample_or_score")


def lm_parts_bytes(rows: int, V: int) -> int:
    L = lib()
    L.smc_lm_parts_bytes.argtypes = [C.c_int, C.c_int]
    L.smc_lm_parts_bytes.restype = C.c_int
    return L.smc_lm_parts_bytes(rows, V)


def lm_head_sample(W: torch.Tensor, X: torch.Tensor, *, M: int, V: int, ldx: int, status: torch.Tensor,
                   temperature: float, alpha: float, softcap: float, tokens_in: Optional[torch.Tensor], seed: int,
                   cycle_counter: torch.Tensor, call_id: int, parts: torch.Tensor, tok_out: torch.Tensor,
                   logp_out: torch.Tensor, logz_out: Optional[torch.Tensor], ssq_in: Optional[torch.Tensor] = None,
                   ssq_parts: int = 0, ssq_ld: int = 0, norm_d: int = 0, norm_eps: float = 0.0, ssq_mstride: int = 1,
                   pdl: bool = False) -> None:
    """lm_head GEMM whose epilogue samples / scores every row straight out of tensor memory (the logits are never
    stored) followed by the per-row merge of the vocabulary slabs.  W [rows >= V, K] bf16; X rows of pitch ``ldx``."""
    L = lib()
    if not getattr(L, "_lmhs_declared", False):
        vp, i, f, ull = C.c_void_p, C.c_int, C.c_float, C.c_ulonglong
        L.smc_lm_head_sample.argtypes = [vp, vp, i, i, i, i, vp, i, vp, i, i, i, f, i, f, f, f, vp, ull, vp, i, vp, vp,
                                         vp, vp, vp]
        L.smc_lm_head_sample.restype = C.c_int
        L._lmhs_declared = True
    assert parts.numel() * parts.element_size() >= lm_parts_bytes(M, V)
    _check(L.smc_lm_head_sample(_p(W), _p(X), V, W.shape[1], M, ldx, _p(status), int(pdl), _p(ssq_in), ssq_parts,
                                ssq_ld, norm_d, norm_eps, ssq_mstride, temperature, alpha, softcap, _p(tokens_in),
                                seed & 0xFFFFFFFFFFFFFFFF, _p(cycle_counter), call_id, _p(parts), _p(tok_out),
                                _p(logp_out), _p(logz_out), _stream()), "smc_lm_head_sample")


_KERNELS_PER_CALL["smc_lm_head_sample"] = 2


# ----------------------------------------------------------------------------- SMC state
class SlotArrays(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished",
                                         "finished_len", "finish_code", "matched_eos", "ignore_eos",
                                         "max_new_tokens", "eos_ids", "log_weights", "interval_weights",
                                         "all_token_ids")] + \
               [("max_out", C.c_int), ("block_table", C.c_void_p), ("bt_stride", C.c_int), ("refcount", C.c_void_p),
                ("free_stack", C.c_void_p), ("free_count", C.c_void_p), ("alloc_error", C.c_void_p),
                ("n_pages", C.c_int)]


def make_slot_arrays(state) -> SlotArrays:
    a = SlotArrays()
    for n in ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished", "finished_len", "finish_code",
              "matched_eos", "ignore_eos", "max_new_tokens", "eos_ids", "log_weights", "interval_weights",
              "all_token_ids"):
        setattr(a, n, getattr(state, n).data_ptr())
    a.max_out = state.max_output_len
    a.block_table = state.bt.table.data_ptr()
    a.bt_stride = state.bt.table.stride(0)
    a.refcount = state.alloc.refcount.data_ptr()
    a.free_stack = state.alloc.free_stack.data_ptr()
    a.free_count = state.alloc.free_count.data_ptr()
    a.alloc_error = state.alloc.error_flag.data_ptr()
    a.n_pages = state.alloc.size
    assert C.sizeof(a) == lib().smc_slot_arrays_size(), "SlotArrays layout mismatch"
    return a


class CycleIO(C.Structure):
    NAMES = ("orig_seq", "x0", "prev", "cache_locs", "positions_verify", "step_pos", "step_locs", "head_ids",
             "head_pos", "head_locs", "head_prefix", "verify_ids", "verify_given")
    _fields_ = [(n, C.c_void_p) for n in NAMES]


def make_cycle_io(bufs: dict) -> CycleIO:
    io = CycleIO()
    for n in CycleIO.NAMES:
        setattr(io, n, bufs[n].data_ptr())
    assert C.sizeof(io) == lib().smc_cycle_io_size()
    return io


def prepare_cycle(arrays: SlotArrays, active, bs, G, counters, io: CycleIO):
    _check(lib().smc_prepare_cycle(C.byref(arrays), _p(active), bs, G, _p(counters), C.byref(io), _stream()),
           "smc_prepare_cycle")


def assemble_verify(io: CycleIO, drafts, bs, gamma):
    _check(lib().smc_assemble_verify(C.byref(io), _p(drafts), bs, gamma, _stream()), "smc_assemble_verify")


def write_back(arrays: SlotArrays, active, bs, gamma, drafts, logq, verify_tok, verify_logp, verify_logz, alpha,
               use_logz, tokens_out, diff_out):
    _check(lib().smc_write_back(C.byref(arrays), _p(active), bs, gamma, _p(drafts), _p(logq), _p(verify_tok),
                                _p(verify_logp), _p(verify_logz), alpha, int(use_logz), _p(tokens_out), _p(diff_out),
                                _stream()), "smc_write_back")


def collect_resample(arrays: SlotArrays, active_rows, n_groups, group_to_slots, N, threshold, seed, counters,
                     group_log_z, job_dst, job_src):
    _check(lib().smc_collect_resample(C.byref(arrays), _p(active_rows), n_groups, _p(group_to_slots), N, threshold,
                                      seed & 0xFFFFFFFFFFFFFFFF, _p(counters), _p(group_log_z), _p(job_dst),
                                      _p(job_src), _stream()), "smc_collect_resample")


def state_copy(state_tensor: torch.Tensor, n_layers: int, n_rows: int, counters, job_dst, job_src, max_jobs: int):
    row_bytes = state_tensor[0, 0].numel() * state_tensor.element_size()
    _check(lib().smc_state_copy(_p(state_tensor), state_tensor.stride(0) * state_tensor.element_size(), row_bytes,
                                n_layers, n_rows, _p(counters), _p(job_dst), _p(job_src), max_jobs, _stream()),
           "smc_state_copy")


# ----------------------------------------------------------------------------- tensor-parallel links
EPI_RS_F32 = 5


class TpLink(C.Structure):
    _fields_ = [("ag_flag", C.c_void_p), ("epoch", C.c_void_p), ("ag_uses", C.c_longlong), ("ag_idx", C.c_longlong),
                ("ag_inc", C.c_longlong), ("peer_base", C.c_ulonglong * 8), ("rs_off", C.c_longlong),
                ("rs_flag_off", C.c_longlong), ("tp", C.c_int), ("rank", C.c_int), ("rows_per_rank", C.c_int),
                ("pad", C.c_int), ("arrive", C.c_void_p)]


class TpPeers(C.Structure):
    _fields_ = [("base", C.c_ulonglong * 8), ("tp", C.c_int), ("rank", C.c_int)]


def _declare_tp(L) -> None:
    if getattr(L, "_tp_declared", False):
        return
    vp, i, ll, f, ull = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong
    L.smc_gemm_skinny_tp.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp, i, vp, vp]
    L.smc_tp_norm_allgather.argtypes = [vp, vp, vp, vp, ll, ll, ll, vp, vp, vp, vp, ll, ll, i, i, i, f, i, vp, vp, i, vp]
    L.smc_tp_sample_or_score.argtypes = [vp, vp, ll, i, i, i, i, f, f, f, vp, ull, vp, i, ll, vp, ll, vp, ll, ll, vp, i,
                                         vp, vp, vp, vp, vp, i, i, vp]
    L.smc_tp_bump_counter.argtypes = [vp, ull, vp]
    L.smc_tp_wait_counter.argtypes = [vp, ull, vp, vp, vp]
    for n in ("smc_gemm_skinny_tp", "smc_tp_norm_allgather", "smc_tp_sample_or_score", "smc_tp_bump_counter",
              "smc_tp_wait_counter", "smc_tp_link_size", "smc_tp_peers_size", "smc_tp_partial_bytes"):
        getattr(L, n).restype = C.c_int
    assert C.sizeof(TpLink) == L.smc_tp_link_size(), "TpLink layout mismatch"
    assert C.sizeof(TpPeers) == L.smc_tp_peers_size(), "TpPeers layout mismatch"
    L._tp_declared = True


def tp_lib():
    L = lib()
    _declare_tp(L)
    return L


def gemm_skinny_tp(W: torch.Tensor, X: torch.Tensor, out: Optional[torch.Tensor], *, M: int, splits: int, epi: int,
                   link: TpLink, ldx: Optional[int] = None, ldo: int, status: torch.Tensor, pdl: bool = False) -> None:
    N, K = W.shape
    ldx = ldx if ldx is not None else X.stride(0)
    _check(tp_lib().smc_gemm_skinny_tp(_p(W), _p(X), _p(out), N, K, M, ldx, ldo, splits, epi, _p(status), int(pdl),
                                       C.byref(link), _stream()), "smc_gemm_skinny_tp")


def tp_norm_allgather(peers: TpPeers, h_local, rs_buf, rs_flag_ptr: int, rs_uses: int, rs_idx: int, rs_inc: int,
                      epoch, ids, embed, w, xn_off: int, ag_flag_off: int, rows_per_rank: int, my_rows: int, d: int,
                      eps: float, plus_one: bool, arrive, status, pdl: bool = False) -> None:
    _check(tp_lib().smc_tp_norm_allgather(C.byref(peers), _p(h_local), _p(rs_buf), C.c_void_p(rs_flag_ptr), rs_uses,
                                          rs_idx, rs_inc, _p(epoch), _p(ids), _p(embed), _p(w), xn_off, ag_flag_off,
                                          rows_per_rank, my_rows, d, eps, int(plus_one), _p(arrive), _p(status), int(pdl),
                                          _stream()), "smc_tp_norm_allgather")


def tp_sample_or_score(peers: TpPeers, logits, *, rows: int, Vshard: int, v0: int, Vtotal: int, temperature: float,
                       alpha: float, softcap: float, tokens_in, seed: int, cycle_counter, call_id: int,
                       gather_off: int, gather_local_ptr: int, flag_off: int, flag_local_ptr: int, uses: int, idx: int,
                       epoch, nchunks: int, tok_out, logp_out, logz_out, arrive, status, pdl: bool = False,
                       phase: int = 0) -> None:
    _check(tp_lib().smc_tp_sample_or_score(C.byref(peers), _p(logits), logits.stride(0), rows, Vshard, v0, Vtotal,
                                           temperature, alpha, softcap, _p(tokens_in), seed & 0xFFFFFFFFFFFFFFFF,
                                           _p(cycle_counter), call_id, gather_off, C.c_void_p(gather_local_ptr),
                                           flag_off, C.c_void_p(flag_local_ptr), uses, idx, _p(epoch), nchunks,
                                           _p(tok_out), _p(logp_out), _p(logz_out), _p(arrive), _p(status), int(pdl), phase,
                                           _stream()), "smc_sample_or_score" if phase == 0 else "smc_tp_sample_phase")


def tp_bump_counter(flag_ptr: int, by: int) -> None:
    _check(tp_lib().smc_tp_bump_counter(C.c_void_p(flag_ptr), by, _stream()), "smc_tp_bump_counter")


def tp_wait_counter(flag_ptr: int, want: int, outcome: torch.Tensor, status: torch.Tensor) -> None:
    _check(tp_lib().smc_tp_wait_counter(C.c_void_p(flag_ptr), want, _p(outcome), _p(status), _stream()),
           "smc_tp_wait_counter")


# ----------------------------------------------------------------------------- gated delta net
GDN_CHUNK_MIN_TOKENS = 64      # rows at least this long (on average) take the chunk-parallel tensor-core kernel


def gdn_step(proj: torch.Tensor, conv_state: torch.Tensor, temporal: torch.Tensor, state_rows: torch.Tensor,
             conv_w: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, gnorm_w: torch.Tensor,
             conv_out: torch.Tensor, out: torch.Tensor, *, bs: int, E: int, Hk: int, Hv: int, dk: int, dv: int, W: int,
             eps: float, pdl: bool = False, tok_off: Optional[torch.Tensor] = None,
             tok_len: Optional[torch.Tensor] = None, chunked: bool = False, status: Optional[torch.Tensor] = None,
             max_len: int = 0, trace: Optional[torch.Tensor] = None) -> None:
    """Conv + gated delta rule + gated RMSNorm for E new tokens per row; advances the state of one layer in place.
    conv_state [rows, conv_dim, W-1] fp32 and temporal [rows, Hv, dk, dv] fp32 are that layer's slices.
    ``tok_off`` / ``tok_len`` (int32 per row) give rows of different lengths at arbitrary token offsets.
    ``chunked`` (prompt passes, dk = dv = 128): the delta rule runs chunk-parallel on tcgen05 (64 tokens per step)
    instead of token by token; ``status`` receives its error bits; ``max_len`` (host-side bound of ``tok_len``) lets
    the conv pass run token-parallel as well; ``trace`` (int64 [10]) accumulates the cycles the first CTA of the
    chunk-parallel kernel spends per phase."""
    L = lib()
    if not getattr(L, "_gdn_declared", False):
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        L.smc_gdn_varlen.argtypes = [vp, i, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, vp, vp, i, i, i, i, i, f, i, vp]
        L.smc_gdn_varlen.restype = C.c_int
        L.smc_gdn_conv.argtypes = [vp, i, vp, vp, vp, vp, i, i, vp, vp, i, i, i, i, vp]
        L.smc_gdn_conv.restype = C.c_int
        L.smc_gdn_chunked.argtypes = [vp, vp, i, vp, vp, vp, vp, vp, vp, i, i, vp, vp, i, i, i, i, f, vp, vp, i, vp]
        L.smc_gdn_chunked.restype = C.c_int
        L._gdn_declared = True
    if chunked and gdn_chunked_supported(dk, dv):
        if status is None:
            raise ValueError("the chunk-parallel kernel needs a status word")
        conv_dim = 2 * Hk * dk + Hv * dv
        _check(L.smc_gdn_conv(_p(proj), proj.stride(0), _p(conv_state), _p(state_rows), _p(conv_w), _p(conv_out), bs, E,
                              _p(tok_off), _p(tok_len), conv_dim, W, int(max_len), int(pdl), _stream()), "smc_gdn_conv")
        _check(L.smc_gdn_chunked(_p(conv_out), _p(proj), proj.stride(0), _p(temporal), _p(state_rows), _p(dt_bias),
                                 _p(A_log), _p(gnorm_w), _p(out), bs, E, _p(tok_off), _p(tok_len), Hk, Hv, dk, dv, eps,
                                 _p(status), _p(trace), int(pdl), _stream()), "smc_gdn_chunked")
        return
    _check(L.smc_gdn_varlen(_p(proj), proj.stride(0), _p(conv_state), _p(temporal), _p(state_rows), _p(conv_w),
                            _p(dt_bias), _p(A_log), _p(gnorm_w), _p(conv_out), _p(out), bs, E, _p(tok_off),
                            _p(tok_len), Hk, Hv, dk, dv, W, eps, int(pdl), _stream()), "smc_gdn_varlen")


def gdn_chunked_supported(dk: int, dv: int) -> bool:
    return dk == 128 and dv == 128


_KERNELS_PER_CALL["smc_gdn_step"] = 2
