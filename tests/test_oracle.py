"""CPU tests: the oracle restatement against the reference's golden vectors and, when the
reference tree is mounted, against the reference's own functions."""
import pytest
import torch

from oracle import lift_reference as lr
from oracle import qgemm_oracle as oc

needs_ref = pytest.mark.skipif(not lr.reference_available(), reason="reference tree not mounted")


def test_int_matmul_exact_equals_int32_matmul():
    g = torch.Generator().manual_seed(1)
    A = torch.randint(-128, 128, (2, 37, 1100), dtype=torch.int8, generator=g)
    B = torch.randint(-128, 128, (2, 1100, 29), dtype=torch.int8, generator=g)
    assert torch.equal(oc.int_matmul_exact(A, B), A.to(torch.int32) @ B.to(torch.int32))
    # worst case magnitudes stay exact
    A = torch.full((4, 2048), -128, dtype=torch.int8)
    B = torch.full((2048, 4), -128, dtype=torch.int8)
    assert torch.equal(oc.int_matmul_exact(A, B), A.to(torch.int32) @ B.to(torch.int32))


@pytest.mark.parametrize("name,odt", [("w8a8_b_s1_f16", "float16"), ("w8a8_b_sN_bf16", "bfloat16"),
                                      ("w8a8_u_s1_bf16", "bfloat16"), ("w8a8_u_sN_f16", "float16")])
def test_w8a8_golden(golden, name, odt):
    c = golden.case(name, bf16=("C",) if odt == "bfloat16" else ())
    out = oc.quant_matmul_ref(c["A"], c["B"], c["scale"], odt)
    assert out.dtype == c["C"].dtype
    assert torch.equal(out, c["C"])  # integer accumulate + one fp32 multiply: bit-exact
    out2 = oc.quant_matmul_ref(c["A"], c["B"], c["scale"], odt, exact_fast=False)
    assert torch.equal(out2, c["C"])


def test_w8a8_two_scale_golden(golden):
    c = golden.case("w8a8_two_scale_bf16", bf16=("C",))
    out = oc.quant_matmul_ref(c["A"], c["B_nk"].t().contiguous(), c["scale_b"].squeeze(1), "bfloat16",
                              scale_a=c["scale_a"].squeeze(1))
    # The reference kernel multiplies scale_a then scale_b; its golden multiplies by outer(sa, sb):
    # the two orders differ by fp32 rounding only; the reference gate is rtol = atol = 1e-2.
    torch.testing.assert_close(out.float(), c["C"].float(), rtol=1e-2, atol=1e-2)
    assert (out != c["C"]).float().mean() < 0.02


def test_unpack_known_answer(golden):
    c = golden.case("unpack_kat")
    got = oc.unpack_uint4(c["packed"])
    assert got.tolist() == [[2, 1, 4, 3]]
    assert torch.equal(got.to(torch.float16), c["f16"])
    assert torch.equal(got.to(torch.int8), c["i8"])


def test_unpack_random_golden(golden):
    c = golden.case("unpack_rand")
    got = oc.unpack_uint4(c["packed"])
    assert torch.equal(got.to(torch.float16), c["f16"])
    assert torch.equal(got.to(torch.int8), c["i8"])
    assert torch.equal(oc.pack_uint4(got), c["packed"])


@pytest.mark.parametrize("name,odt", [("dq_f16", "float16"), ("dq_bf16", "bfloat16")])
def test_dequant_fp16_golden(golden, name, odt):
    bf = ("A", "C") if odt == "bfloat16" else ()
    c = golden.case(name, bf16=bf)
    out = oc.dequant_gemm_fp16_ref(c["A"], c["packed"], odt)
    torch.testing.assert_close(out, c["C"], rtol=1e-2, atol=1e-2)
    assert torch.equal(out, c["C"])  # same fp32 matmul on the same machine family: expected identical


@pytest.mark.parametrize("name,odt", [("dq_i8_i32", "int32"), ("dq_i8_f16", "float16")])
def test_dequant_int8_golden(golden, name, odt):
    c = golden.case(name)
    out = oc.dequant_gemm_int8_ref(c["A"], c["packed"], odt)
    assert torch.equal(out, c["C"])


def test_w4a8_golden(golden):
    c = golden.case("w4a8")
    assert torch.equal(oc.unpack_int4_signed(c["qB"]), c["conv"])
    assert torch.equal(c["conv"], c["B_int8"])
    assert torch.equal(oc.pack_int4_signed(c["B_int8"]), c["qB"])
    assert torch.equal(oc.w4a8_gemm_ref(c["A"], c["qB"]), c["C_nm"].t())


def test_general_compress_golden(golden):
    c = golden.case("general_compress")
    assert torch.equal(oc.pack_uint4(c["vals"]), c["packed"])
    assert torch.equal(oc.unpack_uint4(c["packed"]).to(torch.int8), c["vals"])


def test_gen_quant4_pins_scaled_dequant(golden):
    """gen_quant4's own dequantised weights pin W = (q - 8).half() * s[k // g, n] and the [K/g, N] layout."""
    c = golden.case("gen_quant4")
    q = (c["q_minus8"].to(torch.int16) + 8)  # [K, N], values 0..16 (the reference clamps to 16, not 15)
    keep = (q <= 15).all(dim=0)  # columns that fit a nibble
    assert keep.any()
    qn = q[:, keep].t().contiguous().clamp(0, 15)  # [N', K]
    packed = oc.pack_uint4(qn)
    s = c["s"][:, keep].contiguous()
    W = oc.dequant_weight_ref(packed, s, zero=8, group_size=128)
    assert torch.equal(W, c["ref_weight_nk"][keep])


def test_config_generators_shapes():
    A, B, sa, sb = oc.make_w8a8_inputs(1, 256, 1024, 1024)
    assert A.shape == (1, 256, 1024) and B.shape == (1, 1024, 1024) and sa.shape == (1, 256) and sb.shape == (1, 1024)
    assert A.min() == -128 and A.max() == 127
    assert 0.001 <= float(sa.min()) and float(sb.max()) <= 0.02
    A, P, S = oc.make_w4a16_inputs(16, 512, 256)
    assert P.shape == (256, 256) and S.shape == (4, 256) and S.dtype == torch.float16
    assert float(S.min()) >= 0.005 - 1e-4 and float(S.max()) <= 0.02 + 1e-4


@needs_ref
def test_restatement_matches_live_reference():
    fg = lr.dequant_fine_grained()
    fg["ref_program_fp16"].__globals__.update(fg)
    g = torch.Generator().manual_seed(3)
    Bp = torch.randint(0, 256, (6, 16), dtype=torch.uint8, generator=g)
    A = torch.randn(5, 32, generator=g).half()
    assert torch.equal(oc.unpack_uint4(Bp).half(), fg["torch_unpack_uint4_to_fp16"](Bp))
    assert torch.equal(oc.dequant_gemm_fp16_ref(A, Bp, "float16"), fg["ref_program_fp16"](A, Bp, "float16"))
    ref = lr.w8a8_ref_program()
    A8 = torch.randint(-128, 128, (2, 9, 48), dtype=torch.int8, generator=g)
    B8 = torch.randint(-128, 128, (2, 48, 24), dtype=torch.int8, generator=g)
    sc = torch.randn(24, generator=g)
    assert torch.equal(oc.quant_matmul_ref(A8, B8, sc, torch.float16), ref(A8, B8, sc, torch.float16, torch.int32))
    qu = lr.load_quantize_utils()
    v = torch.randint(0, 16, (4, 16), dtype=torch.int8, generator=g)
    assert torch.equal(oc.pack_uint4(v), qu.general_compress(v, 4, torch.uint8))


ACT_QUANT_CASES = [("act_quant_2d", False, ("x",)), ("act_quant_3d_round", True, ("x",)), ("act_quant_f16", False, ())]


@pytest.mark.parametrize("name,round_scale,bf16", ACT_QUANT_CASES)
def test_act_quant_restatement_matches_reference_vectors(golden, name, round_scale, bf16):
    """examples/deepseek_v4/act_quant.py:112-142 (golden act_quant_torch): int8 values and scales, bit for bit."""
    c = golden.case(name, bf16=bf16)
    y, s = oc.act_quant_torch_ref(c["x"], round_scale=round_scale)
    assert torch.equal(y, c["y"])
    assert torch.equal(s, c["s"])
    assert y.shape == c["x"].shape and s.shape == tuple(c["x"].shape[:-1]) + (1,)


@needs_ref
def test_lifted_act_quant_equals_restatement():
    ref = lr.act_quant_golden()
    torch.manual_seed(7)
    for shape, rs in (((33, 264), False), ((3, 4, 128), True), ((5, 72), True)):
        x = (torch.randn(*shape) * 2).to(torch.bfloat16)
        y0, s0 = ref(x, round_scale=rs)
        y1, s1 = oc.act_quant_torch_ref(x, round_scale=rs)
        assert torch.equal(y0, y1) and torch.equal(s0, s1)


def test_grouped_gemm_restatement_matches_reference_vectors(golden):
    """examples/grouped_gemm/example_grouped_gemm_fwd.py: the table of construct_inputs (:147-166) and the block
    loop of torch_gmm (:7-41) on integer operands = the exact accumulators of the grouped W8A8 form."""
    c = golden.case("grouped_gemm")
    sizes, bm = c["sizes"].tolist(), int(c["block_M"][0])
    assert torch.equal(oc.build_block_metadata_ref(sizes, bm), c["meta"])
    one = torch.ones(1)
    _, acc = oc.grouped_quant_matmul_ref(c["A"], c["B"], c["meta"], one, "float16", return_acc=True)
    assert torch.equal(acc, c["acc"])
    _, acc_t = oc.grouped_quant_matmul_ref(c["A"], c["B"].transpose(1, 2).contiguous(), c["meta"], one, "float16",
                                           b_layout="NK", return_acc=True)
    assert torch.equal(acc_t, c["acc"])


def test_block_metadata_builder_matches_oracle():
    import tilelang_ascend_b200.ops as ops
    for sizes, bm in (([64], 64), ([63, 77, 111, 280], 64), ([100, 0, 300, 5], 128), ([], 128)):
        assert torch.equal(ops.build_block_metadata(sizes, bm), oc.build_block_metadata_ref(sizes, bm))
