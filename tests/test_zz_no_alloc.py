"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some users of the kernels cannot allocate device memory when they need attention: a
plug-in whose host program owns the device heap, a server that gave all free memory to
its cache pool at start-up, a latency-critical loop that cannot afford an allocation's
synchronisation.  ``b200_decode_attention_static`` keeps the split-KV scratch in an array
inside the library instead of taking it from the caller.  This test calls it twice in a
row through ctypes, with raw pointers, and compares each result with the ordinary entry
point's (which is given scratch by the caller); both run the same kernels, so they agree
within the tolerance of the kernel tests.  It also checks that a problem larger than the
array is refused with the documented code and that nothing is launched then.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOO_LARGE = -4


def _case(n_rows, nh, nkv, d, page, ctx, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    pages_per_row = -(-ctx // page)
    total = n_rows * pages_per_row
    perm = torch.randperm(total, generator=g) + 1
    table = perm.view(n_rows, pages_per_row).to(torch.int32)
    kc = torch.randn(total + 1, nkv, page, d, generator=g).to(dtype)
    vc = torch.randn(total + 1, nkv, page, d, generator=g).to(dtype)
    q = torch.randn(n_rows, nh * d, generator=g).to(dtype)
    kv_len = torch.tensor([ctx - 3 * r for r in range(n_rows)], dtype=torch.int32)
    cu = torch.arange(n_rows + 1, dtype=torch.int32)
    rows = torch.arange(n_rows, dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, table, cu, kv_len, rows)]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_entry_point_matches_the_ordinary_one_twice(dtype):
    from llm_infer_rust_b200.kernels import ops
    from llm_infer_rust_b200.kernels.build import load_cuda_library
    nh, nkv, d, page, splits = 8, 2, 64, 16, 4
    lib = load_cuda_library("decode_attention_static.cu", {"HEAD_DIM": d})
    lib.b200_decode_attention_static_max_floats.restype = ctypes.c_longlong
    limit = lib.b200_decode_attention_static_max_floats()
    assert limit == 1 << 20
    scale = 1.0 / math.sqrt(d)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = 1 if dtype == torch.bfloat16 else 0
    for call, (n_rows, ctx, seed) in enumerate(((5, 700, 1), (3, 333, 2))):   # the second call reuses the array
        q, kc, vc, table, cu, kv_len, rows = _case(n_rows, nh, nkv, d, page, ctx, dtype, seed)
        assert n_rows * nh * splits * (d + 2) <= limit
        got = torch.full_like(q, 9.0)
        rc = lib.b200_decode_attention_static(
            _ptr(q), _ptr(kc), _ptr(vc), _ptr(got), _ptr(table), table.shape[1], _ptr(cu), _ptr(kv_len), _ptr(rows),
            n_rows, nh, nkv, page, 0, ctypes.c_float(scale), splits, code, stream)
        assert rc == 0, rc
        want = torch.full_like(q, 9.0)
        scratch = torch.empty(ops.decode_scratch_floats(n_rows, nh, d, splits), device=DEV)
        ops.decode_attention(q, kc, vc, want, scratch, table, cu, kv_len, rows, n_rows, nh, nkv, d, page, None,
                             scale, splits)
        torch.cuda.synchronize()
        if dtype == torch.bfloat16:
            torch.testing.assert_close(got.float(), want.float(), atol=2e-3, rtol=2.0 ** -7)
        else:
            torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
        assert not (got == 9.0).any(), call


def test_a_problem_beyond_the_array_is_refused_and_nothing_runs():
    from llm_infer_rust_b200.kernels.build import load_cuda_library
    nh, nkv, d, page = 8, 2, 64, 16
    lib = load_cuda_library("decode_attention_static.cu", {"HEAD_DIM": d})
    lib.b200_decode_attention_static_max_floats.restype = ctypes.c_longlong
    limit = lib.b200_decode_attention_static_max_floats()
    q, kc, vc, table, cu, kv_len, rows = _case(4, nh, nkv, d, page, 64, torch.bfloat16, 3)
    out = torch.full_like(q, 9.0)
    n_rows = limit // (nh * 2 * (d + 2)) + 1                  # one row too many for two splits
    rc = lib.b200_decode_attention_static(
        _ptr(q), _ptr(kc), _ptr(vc), _ptr(out), _ptr(table), table.shape[1], _ptr(cu), _ptr(kv_len), _ptr(rows),
        int(n_rows), nh, nkv, page, 0, ctypes.c_float(0.125), 2, 1,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == TOO_LARGE and (out == 9.0).all()
