"""The allocation-free sampler entry point, called through its exported C symbol.

Some callers of this library may not allocate device memory (a serving loop with a fixed memory
budget, a host framework that owns the device heap, a plug-in that only receives buffers).  For
them ``smc_sample_or_score_static`` keeps its scratch in a fixed array inside the library.  This
test checks that it returns what the regular entry point returns, on two calls in a row (the
second call reuses whatever the first left in the shared scratch), and that it refuses requests
beyond its stated maximum.  The file name makes pytest collect it last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from smcsd_b200.ops import native
    L = native.lib()
    vp, i, ll, f, ull = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong
    L.smc_sample_or_score_static.argtypes = [vp, i, ll, ll, i, i, f, f, f, vp, ull, vp, i, vp, vp, vp, vp]
    L.smc_sample_or_score_static.restype = C.c_int
    L.smc_no_alloc_last_error.restype = C.c_char_p
    return native, L


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def test_static_sampler_matches_regular_entry_point_twice():
    native, L = _lib()
    torch.manual_seed(0)
    dev = "cuda"
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (rows, V, alpha, T) in enumerate([(72, 128256, 1.0, 0.7), (9, 32000, 1.7, 0.9)]):
        logits = torch.randn(rows, V, device=dev) * 2.5
        given = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        given[::2] = torch.randint(0, V, (len(given[::2]),), device=dev, dtype=torch.int32)
        ctr = torch.tensor([call + 3], dtype=torch.int64, device=dev)
        # regular entry point (scratch supplied by the caller)
        scratch = torch.empty(native.sample_scratch_bytes(rows, 32), dtype=torch.uint8, device=dev)
        tok_a = torch.zeros(rows, dtype=torch.int32, device=dev)
        lp_a, lz_a = torch.zeros(rows, device=dev), torch.zeros(rows, device=dev)
        native.sample_or_score(logits, rows=rows, V=V, splits=1, split_stride=0, row_stride=logits.stride(0),
                               temperature=T, alpha=alpha, softcap=0.0, tokens_in=given, seed=99, cycle_counter=ctr,
                               call_id=call, scratch=scratch, nchunks=32, tok_out=tok_a, logp_out=lp_a, logz_out=lz_a)
        # allocation-free entry point, straight through the C symbol
        tok_b = torch.zeros(rows, dtype=torch.int32, device=dev)
        lp_b, lz_b = torch.zeros(rows, device=dev), torch.zeros(rows, device=dev)
        rc = L.smc_sample_or_score_static(_ptr(logits), 1, 0, logits.stride(0), rows, V, T, alpha, 0.0, _ptr(given), 99,
                                          _ptr(ctr), call, _ptr(tok_b), _ptr(lp_b), _ptr(lz_b), stream)
        assert rc == 0, L.smc_no_alloc_last_error()
        torch.cuda.synchronize()
        assert torch.equal(tok_a, tok_b)
        assert (lp_a - lp_b).abs().max().item() < 2e-3
        assert (lz_a - lz_b).abs().max().item() < 2e-3
        # and both agree with the plain PyTorch definition on the scored rows
        ref = (logits[::2] / T).gather(1, given[::2].long().unsqueeze(1)).squeeze(1) - torch.logsumexp(logits[::2] / T, -1)
        assert (lp_b[::2] - ref).abs().max().item() < 2e-3


def test_static_sampler_rejects_oversized_requests():
    _, L = _lib()
    x = torch.zeros(4, 8, device="cuda")
    out_i = torch.zeros(4, dtype=torch.int32, device="cuda")
    out_f = torch.zeros(4, device="cuda")
    ctr = torch.zeros(1, dtype=torch.int64, device="cuda")
    rc = L.smc_sample_or_score_static(_ptr(x), 1, 0, 8, 100000, 8, 1.0, 1.0, 0.0, None, 0, _ptr(ctr), 0, _ptr(out_i),
                                      _ptr(out_f), None, None)
    assert rc == -90
    assert b"at most" in L.smc_no_alloc_last_error()
