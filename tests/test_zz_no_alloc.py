"""The entry point that allocates nothing: rfx_attention_decode_noalloc.

It is for callers that cannot allocate device memory when they call the
library: a host that gave the whole GPU to its own arena at start-up, a loop
that cannot afford the device synchronisation an allocation may cause, or a
plain C program with no allocator to lend.  The split-KV decode attention needs
scratch for its partial results; this variant keeps that scratch in a 4 MiB
array inside the library.

The test goes through the exported C symbol, the way such a caller would, and
holds the output against the ordinary entry point's (whose scratch the caller
allocates) on two calls in a row: the array keeps the first call's contents,
which the second call must not mistake for its own.  It also checks that a call
too large for the array is refused with the library's error code.  The file
sorts last so that a run that stops at the first failure has already run every
other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

ARGTYPES = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 3 + \
    [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_void_p]


def _library():
    from reflex_b200.csrc import build

    lib = ctypes.CDLL(build.ensure_built())
    lib.rfx_attention_decode_noalloc.argtypes = ARGTYPES
    lib.rfx_attention_decode_noalloc.restype = ctypes.c_int
    lib.rfx_attention_decode_noalloc_capacity.restype = ctypes.c_longlong
    return lib


def _case(seed, R, nq, nkv, d, ctxs):
    g = torch.Generator().manual_seed(seed)
    pages_per = [(c + 63) // 64 for c in ctxs]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, generator=g)
    table = torch.zeros((R, max(pages_per)), dtype=torch.int32)
    o = 0
    for i, n in enumerate(pages_per):
        table[i, :n] = perm[o:o + n].int()
        o += n
    k = torch.randn(total, nkv, 64, d, generator=g).bfloat16().to(DEV)
    v = torch.randn(total, nkv, 64, d, generator=g).bfloat16().to(DEV)
    q = (torch.randn(R, nq * d, generator=g) * 1.5).bfloat16().to(DEV)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=DEV)
    slot = torch.arange(R, dtype=torch.int32, device=DEV)
    return q, k, v, table.to(DEV), pos, slot


def _call(lib, q, k, v, table, pos, slot, nq, nkv, d, n_splits, window=0):
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    st = lib.rfx_attention_decode_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], 64,
        pos.data_ptr(), slot.data_ptr(), out.data_ptr(), q.shape[0], nq, nkv, d, n_splits, window,
        float(d) ** -0.5, stream)
    return st, out


def test_noalloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from reflex_b200 import ops

    lib = _library()
    assert lib.rfx_attention_decode_noalloc_capacity() == 1 << 20
    # first call: 8 rows, 5 splits; second: other sizes, fewer floats of scratch,
    # so stale partials of the first call lie beyond and inside what it uses
    for seed, (R, nq, nkv, d, ctxs, splits) in enumerate([
            (8, 32, 8, 128, [640, 1, 64, 65, 300, 999, 128, 77], 5),
            (3, 6, 1, 32, [129, 500, 31], 3)]):
        q, k, v, table, pos, slot = _case(seed, R, nq, nkv, d, ctxs)
        st, got = _call(lib, q, k, v, table, pos, slot, nq, nkv, d, splits)
        assert st == 0
        want = ops.attention_decode(q, k, v, table, 64, pos, slot, nq, nkv, d, None, d ** -0.5,
                                    n_splits=splits)
        torch.cuda.synchronize()
        assert not bool(torch.isnan(got.float()).any())
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < 8e-3, err  # the bound the kernel tests use; the two are in fact bit-equal
        assert torch.equal(got, want)


def test_noalloc_entry_point_refuses_more_than_its_array_holds():
    lib = _library()
    R, nq, nkv, d = 64, 32, 8, 128
    q, k, v, table, pos, slot = _case(3, R, nq, nkv, d, [70] * R)
    before = torch.full_like(q, 3.0)
    out = before.clone()
    # 64 * 32 * 16 * 130 floats = 4.26 M > 1 M
    st = lib.rfx_attention_decode_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], 64,
        pos.data_ptr(), slot.data_ptr(), out.data_ptr(), R, nq, nkv, d, 16, 0, float(d) ** -0.5,
        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == -4
    assert torch.equal(out, before)  # nothing was launched
    lib.rfx_error_string.restype = ctypes.c_char_p
    lib.rfx_error_string.argtypes = [ctypes.c_int]
    assert b"scratch" in lib.rfx_error_string(st)
    # one split needs no scratch at all, whatever the size
    st, got = _call(lib, q, k, v, table, pos, slot, nq, nkv, d, 1)
    torch.cuda.synchronize()
    assert st == 0 and not bool(torch.isnan(got.float()).any())
