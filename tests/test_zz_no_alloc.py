"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some users of the kernels cannot allocate device memory when they need attention: a
plug-in whose host program owns the device heap, a server that gave all free memory to
its cache pool at start-up, a latency-critical loop that cannot afford an allocation's
synchronisation.  ``b200_decode_attention_static`` keeps the split-KV scratch in an array
inside the library instead of taking it from the caller.  This test calls it twice in a
row through ctypes, with raw pointers (the second call finds the first call's partials in
the array), once over all keys and once with a window, and compares each result with a
plain float32 reference of paged attention (tests/kernel_refs.py) within the bounds that
the kernel tests state, and with the ordinary entry point (which is given scratch by the
caller).  The static entry point always runs the all-sizes CUDA-core kernels of
attention.cu; the ordinary one takes the same kernels for float32 and the tensor-core
kernel for this bfloat16 case, so in bfloat16 the two agree within twice that bound, not
bit for bit.  It also checks that a problem larger than the array is refused with the
documented code and that nothing is launched then.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes
import math

import pytest
import torch

import kernel_refs as R

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
    for call, (n_rows, ctx, seed, window) in enumerate(((5, 700, 1, None), (3, 333, 2, 90))):   # the second call reuses the array
        q, kc, vc, table, cu, kv_len, rows = _case(n_rows, nh, nkv, d, page, ctx, dtype, seed)
        assert n_rows * nh * splits * (d + 2) <= limit
        got = torch.full_like(q, 9.0)
        rc = lib.b200_decode_attention_static(
            _ptr(q), _ptr(kc), _ptr(vc), _ptr(got), _ptr(table), table.shape[1], _ptr(cu), _ptr(kv_len), _ptr(rows),
            n_rows, nh, nkv, page, int(window or 0), ctypes.c_float(scale), splits, code, stream)
        assert rc == 0, rc
        ordinary = torch.full_like(q, 9.0)
        scratch = torch.empty(ops.decode_scratch_floats(n_rows, nh, d, splits), device=DEV)
        ops.decode_attention(q, kc, vc, ordinary, scratch, table, cu, kv_len, rows, n_rows, nh, nkv, d, page, window,
                             scale, splits)
        torch.cuda.synchronize()
        want = R.ref_paged_attention(q, kc, vc, table, cu, kv_len, kv_len - 1, nh, nkv, d, page, window, scale)
        if dtype == torch.bfloat16:
            # the bound of the kernel tests: a probability rounded to bfloat16 as the operand of P.V and the result's
            # own rounding, 2^-8 * max |v| in all (the CUDA-core kernel only pays the second half of it)
            bound = 2.0 ** -8 * float(vc.float().abs().max())
            assert (got.float() - want.float()).abs().max() <= bound
            assert (got.float() - ordinary.float()).abs().max() <= 2 * bound
        else:
            torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
            torch.testing.assert_close(got, ordinary, atol=2e-5, rtol=1e-4)
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
