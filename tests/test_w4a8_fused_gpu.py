"""GPU parity of the fused W4A8 kernel (int4 weights unpacked on the way to the tensor core, up to 128 tokens)
through the C ABI entry qgemm_w4a8, exact int32 against the CPU oracle."""
import pytest
import torch

import tilelang_ascend_b200 as q
from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu

# (M, N, K): every token-tile height (16 / 32 / 64 / 128), ragged N and K (K not a multiple of the 256-wide slab),
# sizes large enough for the kernel's scratch to fit into the caller's [N, K] workspace
CASES = [(1, 1024, 4096), (16, 1040, 4128), (17, 2048, 4096), (32, 2064, 4064), (40, 4096, 4096),
         (64, 4112, 4096), (100, 4096, 8192), (128, 4096, 8224)]


@pytest.mark.parametrize("M,N,K", CASES)
def test_signed_nibbles_exact_and_no_int8_copy(M, N, K):
    g = torch.Generator().manual_seed(M * 7 + N)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=g)
    Bi = torch.randint(-8, 8, (N, K), dtype=torch.int8, generator=g)
    qB = oc.pack_int4_signed(Bi)
    ws = torch.full((N, K), 0x55, dtype=torch.int8, device="cuda")
    C = torch.zeros(M, N, dtype=torch.int32, device="cuda")
    out = q.w4a8_gemm_cv(M, N, K)(A.cuda(), qB.cuda(), ws, C)
    assert torch.equal(out.cpu(), oc.w4a8_gemm_ref(A, qB))
    # the fused kernel uses only the head of the workspace as scratch: the int8 copy of the weights is never written
    assert torch.all(ws[-1] == 0x55) and not torch.equal(ws[-1].cpu(), Bi[-1])
    # a second call on the same (dirty) workspace gives the same result
    out2 = q.w4a8_gemm_cv(M, N, K)(A.cuda(), qB.cuda(), ws, torch.zeros_like(C))
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M,N,K", [(8, 1024, 4096), (48, 4096, 4096)])
def test_unsigned_nibbles_int8_mode_exact(M, N, K):
    g = torch.Generator().manual_seed(K + M)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=g)
    P = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    C = q.dequant_gemm_int8_wrapper(M, N, K, 128, 128, 64, "int32")(A.cuda(), P.cuda())
    assert torch.equal(C.cpu(), oc.dequant_gemm_int8_ref(A, P, "int32"))


def test_extreme_values():
    M, N, K = 16, 1024, 4096
    A = torch.full((M, K), -128, dtype=torch.int8)
    Bi = torch.full((N, K), -8, dtype=torch.int8)
    Bi[::2] = 7
    qB = oc.pack_int4_signed(Bi)
    ws = torch.zeros(N, K, dtype=torch.int8, device="cuda")
    C = torch.zeros(M, N, dtype=torch.int32, device="cuda")
    out = q.w4a8_gemm_cv(M, N, K)(A.cuda(), qB.cuda(), ws, C)
    assert torch.equal(out.cpu(), oc.w4a8_gemm_ref(A, qB))
