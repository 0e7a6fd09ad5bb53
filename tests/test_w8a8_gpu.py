"""GPU parity tests for the W8A8 path: CUDA kernels (through libqgemm.so) against the CPU oracle.

Bars (from the reference's own checks): int32 accumulators bit-exact
(examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:373-374), fp16/bf16 outputs within
rtol = atol = 1e-2 (examples/quant_batch_matmul/example_quant_batch_matmul.py:116).  Because the
epilogue is one fp32 multiply per scale after an exact integer sum, outputs are also compared bit for bit.
"""
import pytest
import torch

from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu


def _q():
    import tilelang_ascend_b200 as q
    return q


def _cmp(C, ref, exact=True):
    torch.testing.assert_close(C.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)
    if exact:
        assert torch.equal(C.cpu(), ref), f"not bit-exact: {(C.cpu() != ref).sum().item()} of {ref.numel()} differ"


@pytest.mark.parametrize("name,odt", [("w8a8_b_s1_f16", "float16"), ("w8a8_b_sN_bf16", "bfloat16"),
                                      ("w8a8_u_s1_bf16", "bfloat16"), ("w8a8_u_sN_f16", "float16")])
def test_golden_vectors(golden, name, odt):
    """Reference-produced vectors (its check_case recipe: randint(-128, 127), scale = randn)."""
    q = _q()
    c = golden.case(name, bf16=("C",) if odt == "bfloat16" else ())
    A, B, s = c["A"].cuda(), c["B"].cuda(), c["scale"].cuda()
    if A.dim() == 3:
        k = q.simple_quant_batch_matmul(A.shape[0], A.shape[1], B.shape[2], A.shape[2], "N" if s.numel() > 1 else "1",
                                        128, 256, 64, out_dtype=odt)
    else:
        k = q.simple_quant_matmul(A.shape[0], B.shape[1], A.shape[1], "N" if s.numel() > 1 else 1, 128, 256, 64,
                                  out_dtype=odt)
    _cmp(k(A, B, s), c["C"])


def test_two_scale_golden_nk_layout(golden):
    """examples/deepseek_v4/int8_gemm.py golden: B stored [N, K], per-token and per-channel scales."""
    q = _q()
    c = golden.case("w8a8_two_scale_bf16", bf16=("C",))
    C = q.quant_matmul(c["A"].cuda(), c["B_nk"].cuda(), c["scale_b"].squeeze(1).contiguous().cuda(),
                       scale_a=c["scale_a"].squeeze(1).contiguous().cuda(), out_dtype=torch.bfloat16, b_layout="NK")
    torch.testing.assert_close(C.cpu().float(), c["C"].float(), rtol=1e-2, atol=1e-2)
    ref = oc.quant_matmul_ref(c["A"], c["B_nk"].t().contiguous(), c["scale_b"].squeeze(1), "bfloat16",
                              scale_a=c["scale_a"].squeeze(1))
    assert torch.equal(C.cpu(), ref)


SHAPES = [
    # batch (0 = unbatched), M, K, N
    (0, 128, 128, 128),
    (0, 128, 128, 256),
    (0, 1, 16, 16),
    (0, 7, 48, 80),
    (0, 129, 272, 400),
    (0, 300, 1040, 528),
    (3, 65, 144, 272),
    (2, 256, 2048, 1024),
    (0, 1024, 1024, 1024),
    (8, 1024, 1024, 1024),  # the reference example's default case (example_quant_batch_matmul.py:120-133)
    (20, 300, 272, 528),    # enough 256 x 256 tiles for the two-CTA kernel, ragged in M, N and K
    (0, 2304, 528, 2320),
]


@pytest.mark.parametrize("batch,M,K,N", SHAPES)
@pytest.mark.parametrize("odt", ["float16", "bfloat16"])
def test_accumulators_and_output_exact(batch, M, K, N, odt):
    q = _q()
    A, B, sa, sb = oc.make_w8a8_inputs(batch, M, K, N, seed=batch * 7 + M)
    ref, acc_ref = oc.quant_matmul_ref(A, B, sb, odt, scale_a=sa, return_acc=True)
    C, acc = q.quant_matmul(A.cuda(), B.cuda(), sb.cuda(), scale_a=sa.cuda(), out_dtype=odt, return_accumulators=True)
    assert torch.equal(acc.cpu(), acc_ref), "int32 accumulators differ"
    _cmp(C, ref)


@pytest.mark.parametrize("batch,M,K,N", [(0, 96, 160, 144), (2, 130, 512, 272), (0, 512, 4096, 256), (24, 260, 144, 528)])
def test_nk_layout_and_int32_output(batch, M, K, N):
    q = _q()
    A, B, sa, sb = oc.make_w8a8_inputs(batch, M, K, N, seed=5)
    acc_ref = oc.int_matmul_exact(A, B)
    B_nk = B.transpose(-1, -2).contiguous()
    acc = q.quant_matmul(A.cuda(), B_nk.cuda(), None, out_dtype=torch.int32, b_layout="NK")
    assert torch.equal(acc.cpu(), acc_ref)
    acc2 = q.quant_matmul(A.cuda(), B.cuda(), None, out_dtype=torch.int32)
    assert torch.equal(acc2.cpu(), acc_ref)


def test_single_scale_and_shared_scales():
    q = _q()
    A, B, sa, sb = oc.make_w8a8_inputs(4, 100, 256, 208, seed=11)
    one = sb[0, :1].contiguous()
    ref = oc.quant_matmul_ref(A, B, one, "float16")
    _cmp(q.quant_matmul(A.cuda(), B.cuda(), one.cuda()), ref)
    shared = sb[0].contiguous()
    ref = oc.quant_matmul_ref(A, B, shared, "bfloat16", scale_a=sa[0].contiguous())
    _cmp(q.quant_matmul(A.cuda(), B.cuda(), shared.cuda(), scale_a=sa[0].contiguous().cuda(), out_dtype="bfloat16"), ref)


def test_extreme_values_large_k():
    """All operands at -128 with K = 4096: accumulators reach 2**26 and the int32 -> fp32 conversion rounds."""
    q = _q()
    M, K, N = 130, 4096, 144
    A = torch.full((M, K), -128, dtype=torch.int8)
    B = torch.full((K, N), -128, dtype=torch.int8)
    B[::3] = 127
    s = torch.full((N,), 1e-4)
    ref, acc_ref = oc.quant_matmul_ref(A, B, s, "float16", return_acc=True)
    C, acc = q.quant_matmul(A.cuda(), B.cuda(), s.cuda(), return_accumulators=True)
    assert torch.equal(acc.cpu(), acc_ref)
    _cmp(C, ref)


def test_config1_and_reference_recipe():
    """BASELINE config 1 (1 x 256 x 1024 x 1024 -> fp16) and the reference's own input recipe on it."""
    q = _q()
    A, B, sa, sb = oc.make_config_inputs("cfg1")
    ref = oc.quant_matmul_ref(A, B, sb, "float16", scale_a=sa)
    k = q.simple_quant_batch_matmul(1, 256, 1024, 1024, "N", 128, 256, 64)
    _cmp(k(A.cuda(), B.cuda(), sb.cuda(), sa.cuda()), ref)
    torch.manual_seed(0)
    A = torch.randint(-128, 127, [1, 256, 1024], dtype=torch.int8)
    B = torch.randint(-128, 127, [1, 1024, 1024], dtype=torch.int8)
    scale = torch.randn([1024])
    _cmp(k(A.cuda(), B.cuda(), scale.cuda()), oc.quant_matmul_ref(A, B, scale, "float16"))


def test_config4_batched_full_size():
    """BASELINE config 4 (16 x 512 x 7168 x 2048 -> bf16), full size, accumulators bit-exact."""
    q = _q()
    A, B, sa, sb = oc.make_config_inputs("cfg4")
    ref, acc_ref = oc.quant_matmul_ref(A, B, sb, "bfloat16", scale_a=sa, return_acc=True)
    C, acc = q.quant_matmul(A.cuda(), B.cuda(), sb.cuda(), scale_a=sa.cuda(), out_dtype="bfloat16",
                            return_accumulators=True)
    assert torch.equal(acc.cpu(), acc_ref)
    _cmp(C, ref)


def test_config3_full_size_properties():
    """BASELINE config 3 (4096 x 4096 x 14336 -> bf16) at full size: exact on a band of rows and columns
    against the oracle, plus size-independent properties over the whole output (linearity in A:
    acc(A1) + acc(A2) == acc(A1 + A2) for operands that do not overflow int8; a checksum of columns)."""
    q = _q()
    A, B, sa, sb = oc.make_config_inputs("cfg3")
    Ad, Bd = A.cuda(), B.cuda()
    C, acc = q.quant_matmul(Ad, Bd, sb.cuda(), scale_a=sa.cuda(), out_dtype="bfloat16", return_accumulators=True)
    rows = torch.cat([torch.arange(0, 160), torch.arange(2000, 2100), torch.arange(4000, 4096)])
    ref, acc_ref = oc.quant_matmul_ref(A[rows], B, sb, "bfloat16", scale_a=sa[rows], return_acc=True)
    assert torch.equal(acc[rows.cuda()].cpu(), acc_ref)
    assert torch.equal(C[rows.cuda()].cpu(), ref)
    # column checksum: sum_n acc[m, n] == A[m, :] . (sum_n B[:, n])   (int64, exact)
    colsum = B.to(torch.int64).sum(dim=1)
    want = (A.to(torch.int64) * colsum[None, :]).sum(dim=1)
    assert torch.equal(acc.to(torch.int64).sum(dim=1).cpu(), want)
    # linearity: halves of A (arithmetic shift keeps them in range) recombine exactly
    A1 = (A >> 1)
    A2 = A - A1
    acc1 = q.quant_matmul(A1.cuda(), Bd, None, out_dtype=torch.int32)
    acc2 = q.quant_matmul(A2.cuda(), Bd, None, out_dtype=torch.int32)
    assert torch.equal(acc1 + acc2, acc)


SPLITK_SHAPES = [(0, 256, 4096, 1024), (2, 200, 4224, 528), (0, 130, 7168, 272), (3, 256, 4608, 1024)]


@pytest.mark.parametrize("batch,M,K,N", SPLITK_SHAPES)
def test_k_split_over_cta_pairs_is_exact(batch, M, K, N):
    """Few tiles and a long K: the kernel runs in clusters of two CTAs that each accumulate half of K and exchange
    halves of the tile through distributed shared memory.  Ragged M, N and K, both layouts: accumulators and outputs
    bit-exact against the oracle."""
    q = _q()
    A, B, sa, sb = oc.make_w8a8_inputs(batch, M, K, N, seed=M + K)
    ref, acc_ref = oc.quant_matmul_ref(A, B, sb, "bfloat16", scale_a=sa, return_acc=True)
    C, acc = q.quant_matmul(A.cuda(), B.cuda(), sb.cuda(), scale_a=sa.cuda(), out_dtype="bfloat16", return_accumulators=True)
    assert torch.equal(acc.cpu(), acc_ref) and torch.equal(C.cpu(), ref)
    acc2 = q.quant_matmul(A.cuda(), B.transpose(-1, -2).contiguous().cuda(), None, out_dtype=torch.int32, b_layout="NK")
    assert torch.equal(acc2.cpu(), acc_ref)


def test_k_split_and_unsplit_kernels_give_the_same_bits():
    """The same shapes with the K split switched off (QGEMM_W8_SPLITK=0 is read once per process, hence a child
    process): identical outputs, which also shows that the shapes above really take the split path's place."""
    import os
    import subprocess
    import sys
    code = r"""
import torch
from oracle import qgemm_oracle as oc
import tilelang_ascend_b200 as q
for batch, M, K, N in %r:
    A, B, sa, sb = oc.make_w8a8_inputs(batch, M, K, N, seed=M + K)
    ref = oc.quant_matmul_ref(A, B, sb, "bfloat16", scale_a=sa)
    C = q.quant_matmul(A.cuda(), B.cuda(), sb.cuda(), scale_a=sa.cuda(), out_dtype="bfloat16")
    assert torch.equal(C.cpu(), ref), (batch, M, K, N)
print("unsplit ok")
""" % (SPLITK_SHAPES,)
    env = dict(os.environ, QGEMM_W8_SPLITK="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "unsplit ok" in r.stdout, r.stdout + r.stderr


def test_rejects_bad_arguments():
    q = _q()
    k = q.simple_quant_matmul(64, 64, 64, "N", 128, 256, 64)
    A = torch.zeros(64, 64, dtype=torch.int8, device="cuda")
    s = torch.ones(64, device="cuda")
    with pytest.raises(ValueError, match="contiguous"):
        k(A.t(), A, s)
    with pytest.raises(ValueError, match="dtype mismatch"):
        k(A.float(), A, s)
    with pytest.raises(ValueError, match="device mismatch"):
        k(A, A.cpu(), s)
    with pytest.raises(ValueError, match="shape mismatch"):
        k(A[:32].contiguous(), A, s)
    with pytest.raises(q.QGemmError, match="multiples of 16"):
        q.quant_matmul(torch.zeros(8, 24, dtype=torch.int8, device="cuda"),
                       torch.zeros(24, 40, dtype=torch.int8, device="cuda"), torch.ones(40, device="cuda"))
    # the context is still usable after rejected calls
    assert torch.equal(k(A, A, s).cpu(), torch.zeros(64, 64, dtype=torch.float16))


def test_empty_inputs_give_empty_outputs():
    """No rows / no tokens: an empty result, no launch (the reference wrapper allocates the output with torch.empty)."""
    q = _q()
    B = torch.zeros(128, 64, dtype=torch.int8, device="cuda")
    sb = torch.ones(64, device="cuda")
    C = q.quant_matmul(torch.zeros(0, 128, dtype=torch.int8, device="cuda"), B, sb)
    assert C.shape == (0, 64) and C.dtype == torch.float16
    Cb = q.quant_matmul(torch.zeros(0, 5, 128, dtype=torch.int8, device="cuda"), torch.zeros(0, 128, 64, dtype=torch.int8, device="cuda"), sb)
    assert Cb.shape == (0, 5, 64)
    P = torch.zeros(64, 64, dtype=torch.uint8, device="cuda")
    C4 = q.w4a16_gemm(torch.zeros(0, 128, dtype=torch.float16, device="cuda"), P, None)
    assert C4.shape == (0, 64)
