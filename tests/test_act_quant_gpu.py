"""GPU parity of the per-token activation quantiser (examples/deepseek_v4/act_quant.py) through the C ABI."""
import pytest
import torch

import tilelang_ascend_b200 as q
from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,round_scale,bf16", [("act_quant_2d", False, ("x",)),
                                                   ("act_quant_3d_round", True, ("x",)),
                                                   ("act_quant_f16", False, ())])
def test_reference_vectors(golden, name, round_scale, bf16):
    c = golden.case(name, bf16=bf16)
    y, s = q.act_quant(c["x"].cuda(), round_scale=round_scale)
    assert y.shape == c["y"].shape and s.shape == c["s"].shape
    assert torch.equal(y.cpu(), c["y"])
    assert torch.equal(s.cpu(), c["s"])


# rows of 8 .. 16392 elements: one warp per row up to a whole block per row, and the re-read path beyond
SHAPES = [(1, 8), (7, 264), (64, 1024), (33, 2056), (130, 4096), (48, 7168), (5, 16384), (3, 16392), (2, 40000)]


@pytest.mark.parametrize("M,N", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_matches_oracle_bit_for_bit(M, N, dtype):
    g = torch.Generator().manual_seed(M * 100003 + N)
    x = (torch.randn(M, N, generator=g) * torch.rand(M, 1, generator=g) * 8).to(dtype)
    y_ref, s_ref = oc.act_quant_torch_ref(x)
    y, s = q.act_quant(x.cuda())
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(y.cpu(), y_ref)


def test_round_scale_is_a_power_of_two_not_below_amax_over_127():
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(200, 512, generator=g) * 5).to(torch.bfloat16)
    x[0] = 0
    x[1, :] = 127.0  # amax / 127 == 1 exactly: the power of two is 1, not 2
    y, s = q.act_quant(x.cuda(), round_scale=True)
    y_ref, s_ref = oc.act_quant_torch_ref(x, round_scale=True)
    assert torch.equal(s.cpu(), s_ref) and torch.equal(y.cpu(), y_ref)
    m, e = torch.frexp(s.cpu())
    assert torch.all(m == 0.5)
    assert float(s[1]) == 1.0 and torch.all(y[1] == 127)


def test_zero_rows_and_empty_input():
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    y, s = q.act_quant(x)
    assert torch.all(y == 0)
    assert torch.equal(s.cpu(), torch.full((4, 1), 1e-4, dtype=torch.float32) / 127.0)
    y, s = q.act_quant(torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (0, 64) and s.shape == (0, 1)


def test_feeds_the_w8a8_gemm():
    """act_quant -> quant_matmul(A, B, scale_b, scale_a) equals the oracle chain on the same inputs."""
    g = torch.Generator().manual_seed(11)
    M, K, N = 96, 512, 272
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    B = torch.randint(-128, 128, (K, N), dtype=torch.int8, generator=g)
    sb = torch.rand(N, generator=g) * 0.02 + 0.001
    a8, sa = q.act_quant(x.cuda())
    C = q.quant_matmul(a8, B.cuda(), sb.cuda(), scale_a=sa.view(-1), out_dtype="bfloat16")
    a8_ref, sa_ref = oc.act_quant_torch_ref(x)
    C_ref = oc.quant_matmul_ref(a8_ref, B, sb, "bfloat16", scale_a=sa_ref.view(-1))
    assert torch.equal(C.cpu(), C_ref)


def test_factory_signature_and_errors():
    kernel = q.act_quant_kernel_int8_optimized(256, block_M=16, block_N=256, round_scale=False)
    x = torch.randn(20, 256).to(torch.bfloat16)
    y, s = kernel(x.cuda())
    y_ref, s_ref = oc.act_quant_torch_ref(x)
    assert s.shape == (20,) and torch.equal(y.cpu(), y_ref) and torch.equal(s.cpu(), s_ref.view(-1))
    with pytest.raises(ValueError):
        kernel(torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        q.act_quant_kernel_int8_optimized(100)
    with pytest.raises(ValueError):
        q.act_quant(torch.zeros(4, 64, dtype=torch.float32, device="cuda"))
    with pytest.raises(q.QGemmError):
        q.act_quant(torch.zeros(4, 12, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("M,K,N,dtype,round_scale", [(1, 1024, 4096, torch.bfloat16, False), (16, 8192, 1024, torch.bfloat16, False),
                                                     (37, 4096, 2560, torch.float16, True), (128, 2048, 10240, torch.bfloat16, False),
                                                     (5, 16384 + 256, 272, torch.float16, False)])
def test_quantiser_fused_into_the_w4a8_operator(M, K, N, dtype, round_scale):
    """bf16 / f16 activations straight into the W4A8 operator: scales and int32 results are those of the oracle's
    act_quant followed by its W4A8 GEMM, bit for bit, and of the two separate device calls."""
    g = torch.Generator().manual_seed(M + K + N)
    x = (torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 4).to(dtype)
    qB = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    a8_ref, sa_ref = oc.act_quant_torch_ref(x, round_scale=round_scale)
    C_ref = oc.w4a8_gemm_ref(a8_ref, qB)
    ws = torch.empty((N, K), dtype=torch.int8, device="cuda")
    C = torch.empty((M, N), dtype=torch.int32, device="cuda")
    kernel = q.w4a8_gemm_act_quant(M, N, K, round_scale=round_scale)
    C, sa = kernel(x.cuda(), qB.cuda(), ws, C)
    assert torch.equal(sa.cpu(), sa_ref.view(-1))
    assert torch.equal(C.cpu(), C_ref)
    a8, sa2 = q.act_quant(x.cuda(), round_scale=round_scale)
    C2 = q.w4a8_gemm_cv(M, N, K)(a8, qB.cuda(), ws, torch.empty_like(C))
    assert torch.equal(C, C2) and torch.equal(sa, sa2.view(-1))


def test_fused_quantiser_needs_room_for_its_scratch_in_the_workspace():
    """The [N, K] int8 workspace is the only scratch the operator gets; a weight matrix smaller than the kernel's own
    scratch (a few MB) is rejected with a message instead of being overrun."""
    M, K, N = 4, 256, 128
    kernel = q.w4a8_gemm_act_quant(M, N, K)
    with pytest.raises(q.QGemmError, match="workspace is too small"):
        kernel(torch.zeros((M, K), dtype=torch.bfloat16, device="cuda"), torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda"),
               torch.empty((N, K), dtype=torch.int8, device="cuda"), torch.empty((M, N), dtype=torch.int32, device="cuda"))


def test_fused_quantiser_rejects_more_than_128_tokens():
    M, K, N = 129, 256, 128
    kernel = q.w4a8_gemm_act_quant(M, N, K)
    with pytest.raises(q.QGemmError, match="M <= 128"):
        kernel(torch.zeros((M, K), dtype=torch.bfloat16, device="cuda"), torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda"),
               torch.empty((N, K), dtype=torch.int8, device="cuda"), torch.empty((M, N), dtype=torch.int32, device="cuda"))
