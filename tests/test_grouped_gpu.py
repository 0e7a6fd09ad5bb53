"""GPU parity of the grouped (ragged) W8A8 matmul through the C ABI, against the CPU oracle and the
reference-produced vectors (examples/grouped_gemm/example_grouped_gemm_fwd.py)."""
import pytest
import torch

import tilelang_ascend_b200 as q
from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu


def test_reference_vectors(golden):
    c = golden.case("grouped_gemm")
    acc = q.grouped_quant_matmul(c["A"].cuda(), c["B"].cuda(), c["meta"].cuda(), None, out_dtype=torch.int32)
    assert torch.equal(acc.cpu(), c["acc"])


def _inputs(sizes, K, N, seed, per_group_scale=True):
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-128, 128, (sum(sizes), K), dtype=torch.int8, generator=g)
    B = torch.randint(-128, 128, (len(sizes), K, N), dtype=torch.int8, generator=g)
    sb = torch.rand((len(sizes), N) if per_group_scale else (N,), generator=g) * 0.019 + 0.001
    sa = torch.rand(sum(sizes), generator=g) * 0.019 + 0.001
    return A, B, sb, sa


# the reference's own size lists (example_grouped_gemm_fwd.py:199-203) with smaller K, N, and ragged extras
CASES = [([64], 256, 272, 64), ([64, 128, 256], 512, 528, 64), ([63], 256, 64, 64), ([100, 200, 300, 400], 144, 256, 128),
         ([63, 77, 111, 280], 272, 528, 64), ([1, 0, 129, 5, 260], 128, 2320, 128), ([300] * 12, 512, 512, 128)]


@pytest.mark.parametrize("sizes,K,N,bm", CASES)
@pytest.mark.parametrize("odt", ["float16", "bfloat16"])
def test_matches_oracle_bit_for_bit(sizes, K, N, bm, odt):
    A, B, sb, sa = _inputs(sizes, K, N, seed=len(sizes) * 1000 + K)
    meta = oc.build_block_metadata_ref(sizes, bm)
    ref, acc_ref = oc.grouped_quant_matmul_ref(A, B, meta, sb, odt, scale_a=sa, return_acc=True)
    kernel = q.grouped_quant_gemm(tuple(sizes), K, N, bm, 256, 128, out_dtype=odt)
    assert torch.equal(kernel.block_metadata("cpu"), meta)
    C, acc = kernel(A.cuda(), B.cuda(), meta.cuda(), sb.cuda(), sa.cuda(), return_accumulators=True)
    assert torch.equal(acc.cpu(), acc_ref)
    assert torch.equal(C.cpu(), ref)


def test_transposed_weights_and_shared_scale():
    sizes, K, N = [70, 200, 33], 256, 144
    A, B, sb, sa = _inputs(sizes, K, N, seed=5, per_group_scale=False)
    meta = oc.build_block_metadata_ref(sizes, 128)
    ref = oc.grouped_quant_matmul_ref(A, B, meta, sb, "bfloat16")
    Bt = B.transpose(1, 2).contiguous()
    C = q.grouped_quant_matmul(A.cuda(), Bt.cuda(), meta.cuda(), sb.cuda(), out_dtype="bfloat16", b_layout="NK")
    assert torch.equal(C.cpu(), ref)


def test_equal_groups_equal_the_batched_operator():
    """Config-4-like special case: equal group sizes give the same result as the batched kernel."""
    G, M, K, N = 4, 256, 512, 256
    A, B, sb, sa = _inputs([M] * G, K, N, seed=9)
    meta = q.build_block_metadata([M] * G, 128, "cuda")
    C = q.grouped_quant_matmul(A.cuda(), B.cuda(), meta, sb.cuda(), sa.cuda(), out_dtype="bfloat16")
    Cb = q.quant_matmul(A.view(G, M, K).cuda(), B.cuda(), sb.cuda(), scale_a=sa.view(G, M).cuda(), out_dtype="bfloat16")
    assert torch.equal(C.view(G, M, N), Cb)


def test_uncovered_rows_and_bad_entries_are_left_alone():
    sizes, K, N = [40, 50], 128, 64
    A, B, sb, sa = _inputs(sizes, K, N, seed=2)
    meta = torch.tensor([[0, 0, 40], [7, 40, 50], [1, 4000, 10], [1, 60, 30]], dtype=torch.int32)  # entries 1, 2 invalid
    out = torch.full((90, N), 7.0, dtype=torch.float16, device="cuda")
    C = q.grouped_quant_matmul(A.cuda(), B.cuda(), meta.cuda(), sb.cuda(), out_dtype="float16", out=out)
    good = torch.tensor([[0, 0, 40], [1, 60, 30]], dtype=torch.int32)
    ref = oc.grouped_quant_matmul_ref(A, B, good, sb, "float16")
    assert torch.equal(C[:40].cpu(), ref[:40]) and torch.equal(C[60:].cpu(), ref[60:])
    assert torch.all(C[40:60] == 7.0)


def test_empty_and_rejects():
    A = torch.zeros(0, 128, dtype=torch.int8, device="cuda")
    B = torch.zeros(2, 128, 64, dtype=torch.int8, device="cuda")
    sb = torch.ones(64, device="cuda")
    C = q.grouped_quant_matmul(A, B, q.build_block_metadata([0, 0], 128, "cuda"), sb)
    assert C.shape == (0, 64)
    with pytest.raises(ValueError):
        q.grouped_quant_gemm((64, 64), 128, 64, block_M=256)
    with pytest.raises(ValueError):
        q.grouped_quant_matmul(torch.zeros(8, 128, dtype=torch.int8, device="cuda"), B,
                               torch.zeros(1, 2, dtype=torch.int32, device="cuda"), sb)
    with pytest.raises(q.QGemmError):
        q.grouped_quant_matmul(torch.zeros(8, 40, dtype=torch.int8, device="cuda"),
                               torch.zeros(2, 40, 64, dtype=torch.int8, device="cuda"),
                               q.build_block_metadata([8], 128, "cuda"), sb)
