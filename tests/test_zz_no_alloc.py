"""GPU test of qgemm_w4a16_noalloc, the entry point for callers that cannot allocate device memory
(for instance a runtime plugin that is only handed its tensors, or a bare FFI caller).

It is called here straight through the C ABI with nothing but input and output pointers, twice in a row
on different inputs, and each result is compared with what the ordinary entry point (caller-provided
workspace) returns for the same inputs.  The second call finds the built-in scratch array full of the
first call's data, which is exactly the situation the entry point has to cope with.  The file name keeps
this test last in collection order.
"""
import pytest
import torch

from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, A, P, S, zero, group, out_dtype):
    from tilelang_ascend_b200 import _lib
    M, K = A.shape
    N = P.shape[0]
    C = torch.empty((M, N), dtype=out_dtype, device=A.device)
    abi = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}
    rc = lib.qgemm_w4a16_noalloc(A.data_ptr(), P.data_ptr(), None if S is None else S.data_ptr(), zero, group,
                                 C.data_ptr(), M, N, K, abi[A.dtype], abi[out_dtype], None,
                                 torch.cuda.current_stream().cuda_stream)
    return rc, C


def test_noalloc_matches_regular_entry_point_twice():
    import tilelang_ascend_b200 as q
    from tilelang_ascend_b200 import _lib
    lib = _lib.load()
    cases = [(16, 4096, 4096, "float16", 128, 11), (5, 2048, 640, "bfloat16", 64, 12)]
    for M, K, N, dt, group, seed in cases:  # two calls in a row, the second on a dirty scratch array
        A, P, S = [t.cuda() for t in oc.make_w4a16_inputs(M, K, N, dt, group, seed=seed)]
        want = q.w4a16_gemm(A, P, S, 8, group)
        rc, got = _call_noalloc(lib, A, P, S, 8, group, A.dtype)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-2)
        assert torch.equal(got, want)  # same kernels, same fixed summation order
        ref = oc.dequant_gemm_fp16_ref(A.cpu(), P.cpu(), dt, S.cpu(), 8, group)
        torch.testing.assert_close(got.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from tilelang_ascend_b200 import _lib
    lib = _lib.load()
    A, P, S = [t.cuda() for t in oc.make_w4a16_inputs(33, 256, 128, "float16", 128, seed=1)]
    rc, _ = _call_noalloc(lib, A, P, S, 8, 128, torch.float16)
    assert rc != 0 and "M <= 32" in _lib.last_error()
    # K beyond the built-in array's activation area
    A, P, S = [t.cuda() for t in oc.make_w4a16_inputs(1, 16384 + 128, 8, "float16", 128, seed=3)]
    rc, _ = _call_noalloc(lib, A, P, S, 8, 128, torch.float16)
    assert rc != 0 and "K <= 16384" in _lib.last_error()
    # arguments the ordinary entry point rejects are rejected here too, before anything is put on the stream
    A, P, S = [t.cuda() for t in oc.make_w4a16_inputs(4, 256, 128, "float16", 128, seed=4)]
    rc, _ = _call_noalloc(lib, A, P, S, 8, 48, torch.float16)
    assert rc != 0 and "group" in _lib.last_error()
    # still usable afterwards
    A, P, S = [t.cuda() for t in oc.make_w4a16_inputs(8, 256, 128, "float16", 128, seed=2)]
    rc, got = _call_noalloc(lib, A, P, S, 8, 128, torch.float16)
    assert rc == 0
    ref = oc.dequant_gemm_fp16_ref(A.cpu(), P.cpu(), "float16", S.cpu(), 8, 128)
    torch.testing.assert_close(got.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)
