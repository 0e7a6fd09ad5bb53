"""CPU tests of the host layer: the C-ABI library loads and exports every declared symbol, the Python
factories keep the reference's signatures and error behaviour, packing helpers match the oracle."""
import inspect
import os
import re

import pytest
import torch

from oracle import qgemm_oracle as oc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from tilelang_ascend_b200 import _lib
    header = open(os.path.join(ROOT, "include", "qgemm.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(qgemm_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.qgemm_version() >= 1000


def test_factory_signatures_match_reference():
    import tilelang_ascend_b200 as q
    sig = inspect.signature(q.simple_quant_batch_matmul.__wrapped__)
    assert list(sig.parameters) == ["Batch", "M", "N", "K", "scale_size", "block_M", "block_N", "block_K",
                                    "in_dtype", "out_dtype", "accum_dtype", "scale_dtype"]
    assert sig.parameters["out_dtype"].default == "float16"
    sig = inspect.signature(q.simple_quant_matmul.__wrapped__)
    assert list(sig.parameters)[:7] == ["M", "N", "K", "scale_size", "block_M", "block_N", "block_K"]
    sig = inspect.signature(q.dequant_gemm_fp16_wrapper.__wrapped__)
    assert list(sig.parameters) == ["M", "N", "K", "block_M", "block_N", "block_K", "input_dtype", "output_dtype"]
    sig = inspect.signature(q.dequant_gemm_int8_wrapper.__wrapped__)
    assert list(sig.parameters) == ["M", "N", "K", "block_M", "block_N", "block_K", "output_dtype"]
    assert list(inspect.signature(q.w4a8_gemm_cv.__wrapped__).parameters) == ["M", "N", "K"]
    # factories are memoised per argument tuple, like the reference's jit wrapper
    assert q.simple_quant_matmul(64, 64, 64, "N", 128, 256, 64) is q.simple_quant_matmul(64, 64, 64, "N", 128, 256, 64)


def test_no_cpu_path_and_argument_errors():
    import tilelang_ascend_b200 as q
    k = q.simple_quant_matmul(16, 16, 16, "N", 128, 256, 64)
    z = torch.zeros(16, 16, dtype=torch.int8)
    with pytest.raises(ValueError, match="CUDA tensor"):
        k(z, z, torch.ones(16))
    with pytest.raises(ValueError):
        q.simple_quant_matmul(16, 16, 16, "N", 128, 256, 64, out_dtype="float32")
    with pytest.raises(ValueError):
        q.simple_quant_batch_matmul(1, 16, 16, 16, "M", 128, 256, 64)
    with pytest.raises(ValueError):
        q.dequant_gemm_fp16_wrapper(16, 16, 32, 0, 256, 64)


def test_packing_helpers_match_oracle(golden):
    import tilelang_ascend_b200 as q
    c = golden.case("general_compress")
    assert torch.equal(q.general_compress(c["vals"], 4, torch.uint8), c["packed"])
    assert q.general_compress(c["vals"]).dtype == torch.int8
    assert torch.equal(q.general_compress(c["vals"]).view(torch.uint8), c["packed"])
    w = golden.case("w4a8")
    assert torch.equal(q.pack_int4(w["B_int8"]), w["qB"])
    g = torch.Generator().manual_seed(0)
    v = torch.randint(0, 4, (5, 16), dtype=torch.int8, generator=g)
    two_bit = q.general_compress(v, 2, torch.uint8)
    assert two_bit.shape == (5, 4)
    assert int(two_bit[0, 0]) == int(v[0, 0] | (v[0, 1] << 2) | (v[0, 2] << 4) | (v[0, 3] << 6))
    assert torch.equal(oc.unpack_uint4(q.pack_int4(torch.arange(16).view(1, 16))).view(-1), torch.arange(16, dtype=torch.uint8))


def test_interleave_weight_matches_reference_vectors(golden):
    """tilelang/quantize/utils.py:73-126, the (nbits, target) combinations that run in the reference."""
    from tilelang_ascend_b200 import quantize as qz
    from oracle import qgemm_oracle as oc
    c = golden.case("interleave_weight")
    qw = c["qweight"]
    assert torch.equal(qz.interleave_weight(qw, 4, "float16"), c["i4_f16"])
    assert torch.equal(qz.interleave_weight(qw, 4, "int8"), c["i4_i8"])
    assert torch.equal(qz.interleave_weight(qw, 2, "int8"), c["i2_i8"])
    assert torch.equal(oc.interleave_int4_f16_ref(qw.view(torch.uint8)), c["i4_f16"].view(torch.uint8))
    assert torch.equal(qz.deinterleave_weight_int4_f16(c["i4_f16"]), qw.view(torch.uint8))
    for nbits, tgt in ((1, "int8"), (1, "float16"), (2, "float16")):  # run here; they raise in the reference
        out = qz.interleave_weight(qw, nbits, tgt)
        assert out.shape == qw.shape and out.dtype == torch.int8
    with pytest.raises(ValueError):
        qz.interleave_weight(qw, 3, "float16")


def test_group_quantiser_matches_reference_vector(golden):
    """gen_quant4 (tilelang/quantize/utils.py:5-50): scales, integers and dequantised weights."""
    from tilelang_ascend_b200 import quantize as qz
    c = golden.case("gen_quant4")
    torch.manual_seed(0)
    original_w, linear, s, centred = qz.gen_quant4(256, 16, 128)
    assert torch.equal(s, c["s"]) and torch.equal(centred.to(torch.int8), c["q_minus8"])
    assert torch.equal(linear.weight.data, c["ref_weight_nk"])
    q, s2 = qz.quantize_int4_groupwise(original_w, 128)
    assert torch.equal(s2, s) and int(q.max()) <= 15 and int(q.min()) >= 0
    assert torch.equal(q.to(torch.int32), torch.clamp(centred + 8, 0, 15))
    z = qz.unpack_qzeros(qz.pack_int4(torch.tensor([[1, 15, 8, 0]])), 4)
    assert torch.equal(z, torch.tensor([[1, 15, 8, 0]], dtype=torch.float16))
