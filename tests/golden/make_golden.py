"""Generate the committed golden vectors from the reference's own torch functions.

Run where the reference tree is mounted (it is not needed afterwards):

    python tests/golden/make_golden.py

Each vector set holds seeded inputs and the output that the reference's
function produced for them.  The functions are executed from the reference
tree (see oracle/lift_reference.py); nothing of the reference is stored here
but these small input/output arrays.  bf16 tensors are stored as their uint16
bit patterns so that the files stay plain numpy.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import lift_reference as lr  # noqa: E402


def to_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main():
    assert lr.reference_available(), "reference tree not found"
    out = {}

    # --- W8A8: the reference's check_case recipe (randint(-128, 127), scale = randn), seed 0 ----
    ref_b = lr.w8a8_ref_program()
    ref_u = lr.w8a8_unbatched_ref_program()
    torch.manual_seed(0)
    for tag, (batch, M, N, K, ssz, odt) in {
        "w8a8_b_s1_f16": (3, 70, 48, 160, "1", torch.float16),
        "w8a8_b_sN_bf16": (2, 130, 272, 96, "N", torch.bfloat16),
    }.items():
        A = torch.randint(-128, 127, [batch, M, K], dtype=torch.int8)
        B = torch.randint(-128, 127, [batch, K, N], dtype=torch.int8)
        scale = torch.randn([N if ssz == "N" else 1], dtype=torch.float32)
        C = ref_b(A, B, scale, odt, torch.int32)
        out[tag] = dict(A=to_np(A), B=to_np(B), scale=to_np(scale), C=to_np(C))
    for tag, (M, N, K, ssz, odt) in {
        "w8a8_u_s1_bf16": (129, 64, 1024, "1", torch.bfloat16),
        "w8a8_u_sN_f16": (33, 144, 4096, "N", torch.float16),
    }.items():
        A = torch.randint(-128, 127, [M, K], dtype=torch.int8)
        B = torch.randint(-128, 127, [K, N], dtype=torch.int8)
        scale = torch.randn([N if ssz == "N" else 1], dtype=torch.float32)
        C = ref_u(A, B, scale, odt, torch.int32)
        out[tag] = dict(A=to_np(A), B=to_np(B), scale=to_np(scale), C=to_np(C))

    # --- two-scale golden (examples/deepseek_v4/int8_gemm.py), B stored [N, K], seed 42 --------
    two = lr.two_scale_golden()
    torch.manual_seed(42)
    M, N, K = 48, 80, 256
    a = torch.randn(M, K, dtype=torch.bfloat16).float()
    sa = torch.clamp(a.abs().amax(dim=1, keepdim=True), min=1e-4) / 127.0
    a8 = torch.clamp(a / sa, -128, 127).round().to(torch.int8)
    b = torch.randn(N, K, dtype=torch.bfloat16).float()
    sb = torch.clamp(b.abs().amax(dim=1, keepdim=True), min=1e-4) / 127.0
    b8 = torch.clamp(b / sb, -128, 127).round().to(torch.int8)
    C = two(a8, sa, b8, sb, out_dtype=torch.bfloat16)
    out["w8a8_two_scale_bf16"] = dict(A=to_np(a8), B_nk=to_np(b8), scale_a=to_np(sa), scale_b=to_np(sb), C=to_np(C))

    # --- unsigned int4 unpack: the reference's known-answer vector and a random case -----------
    fg = lr.dequant_fine_grained()
    fg["check_unpack_functions"].__globals__.update(fg)
    fg["check_unpack_functions"]()  # asserts [[0x12, 0x34]] -> [2, 1, 4, 3] inside the reference
    kat = torch.tensor([[0x12, 0x34]], dtype=torch.uint8)
    out["unpack_kat"] = dict(packed=to_np(kat), f16=to_np(fg["torch_unpack_uint4_to_fp16"](kat)),
                             i8=to_np(fg["torch_unpack_uint4_to_int8"](kat)))
    torch.manual_seed(0)
    Bp = torch.randint(0, 255, [12, 24], dtype=torch.uint8)
    out["unpack_rand"] = dict(packed=to_np(Bp), f16=to_np(fg["torch_unpack_uint4_to_fp16"](Bp)),
                              i8=to_np(fg["torch_unpack_uint4_to_int8"](Bp)))

    # --- unscaled dequant GEMM, fp16 / bf16 / int8 modes (reference check_case recipes) ---------
    fg["ref_program_fp16"].__globals__.update(fg)
    for tag, (M, N, K, idt, odt) in {
        "dq_f16": (20, 40, 64, torch.float16, "float16"),
        "dq_bf16": (9, 24, 128, torch.bfloat16, "bfloat16"),
    }.items():
        A = torch.randn(M, K, dtype=idt)
        Bp = torch.randint(0, 255, [N, K // 2], dtype=torch.uint8)
        C = fg["ref_program_fp16"](A, Bp, odt)
        out[tag] = dict(A=to_np(A), packed=to_np(Bp), C=to_np(C))
    for tag, (M, N, K, odt) in {"dq_i8_i32": (17, 24, 96, "int32"), "dq_i8_f16": (8, 16, 64, "float16")}.items():
        A = torch.randint(-128, 127, [M, K], dtype=torch.int8)
        Bp = torch.randint(0, 255, [N, K // 2], dtype=torch.uint8)
        C = fg["ref_program_int8"](A, Bp, odt)
        out[tag] = dict(A=to_np(A), packed=to_np(Bp), C=to_np(C))

    # --- W4A8 signed nibbles (seed 42 as in the reference) -----------------------------------
    w = lr.w4a8()
    w["ref_program"].__globals__.update(w)
    torch.manual_seed(42)
    M, N, K = 24, 32, 64
    A = torch.randint(-8, 8, (M, K), dtype=torch.int8)
    qB, B_int8 = w["generate_quantized_weight"](N, K)
    C_nm = w["ref_program"](A, qB)  # [N, M]
    out["w4a8"] = dict(A=to_np(A), qB=to_np(qB), B_int8=to_np(B_int8), conv=to_np(w["torch_convert"](qB)),
                       C_nm=to_np(C_nm.contiguous()))

    # --- tilelang/quantize: general_compress and gen_quant4 (scale layout, zero 8, formula) ----
    qu = lr.load_quantize_utils()
    torch.manual_seed(0)
    vals = torch.randint(0, 16, (10, 32), dtype=torch.int8)
    out["general_compress"] = dict(vals=to_np(vals), packed=to_np(qu.general_compress(vals, 4, torch.uint8)))
    torch.manual_seed(0)
    k, n, g = 256, 16, 128
    _, linear, s, w_minus8 = qu.gen_quant4(k, n, g)
    out["gen_quant4"] = dict(s=to_np(s), q_minus8=to_np(w_minus8.to(torch.int8)),
                             ref_weight_nk=to_np(linear.weight.data.contiguous()))

    # --- per-token activation quantiser golden (examples/deepseek_v4/act_quant.py, seed 42) -------
    aq = lr.act_quant_golden()
    torch.manual_seed(42)
    x = torch.randn(40, 1024, dtype=torch.bfloat16)
    x[3] = 0  # an all-zero row exercises the 1e-4 floor
    x[5] *= 1000.0
    x[7, :512] = 0.5  # exact ties after scaling
    x[7, 512:] = 127.0
    y, s = aq(x, round_scale=False)
    out["act_quant_2d"] = dict(x=to_np(x), y=to_np(y), s=to_np(s))
    x3 = (torch.randn(2, 5, 256) * 3).to(torch.bfloat16)
    y, s = aq(x3, round_scale=True)
    out["act_quant_3d_round"] = dict(x=to_np(x3), y=to_np(y), s=to_np(s))
    xh = torch.randn(6, 4104, dtype=torch.float16)
    y, s = aq(xh, round_scale=False)
    out["act_quant_f16"] = dict(x=to_np(xh), y=to_np(y), s=to_np(s))

    # --- grouped GEMM block loop and table (examples/grouped_gemm/example_grouped_gemm_fwd.py), seed 0 ----
    # torch_gmm on integer-valued int32 operands gives the exact accumulators of the quantized form; the
    # table comes from construct_inputs with the reference's own block_M (ragged sizes, one empty tail block).
    gg = lr.grouped_gemm_reference()
    torch.manual_seed(0)
    sizes, K, N, bm = [63, 77, 111, 280], 96, 48, 64
    _, _, meta = gg["construct_inputs"](sizes, K, N, False, bm, "cpu", torch.float32)
    A = torch.randint(-128, 127, [sum(sizes), K], dtype=torch.int8)
    B = torch.randint(-128, 127, [len(sizes), K, N], dtype=torch.int8)
    acc = gg["torch_gmm"](A.to(torch.int32), B.to(torch.int32), meta)
    acc_t = gg["torch_gmm"](A.to(torch.int32), B.transpose(1, 2).contiguous().to(torch.int32), meta, trans_b=True)
    assert torch.equal(acc, acc_t)
    out["grouped_gemm"] = dict(sizes=np.array(sizes, dtype=np.int64), block_M=np.array([bm], dtype=np.int64),
                               A=to_np(A), B=to_np(B), meta=to_np(meta), acc=to_np(acc))

    # --- interleave_weight (tilelang/quantize/utils.py:73-126): the combinations that run in the reference ----
    torch.manual_seed(3)
    qw = torch.randint(-128, 128, (6, 32), dtype=torch.int8)
    out["interleave_weight"] = dict(qweight=to_np(qw),
                                    i4_f16=to_np(qu.interleave_weight(qw.clone(), 4, "float16")),
                                    i4_i8=to_np(qu.interleave_weight(qw.clone(), 4, "int8")),
                                    i2_i8=to_np(qu.interleave_weight(qw.clone(), 2, "int8")))

    flat = {f"{case}/{key}": v for case, d in out.items() for key, v in d.items()}
    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **flat)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "cases")


if __name__ == "__main__":
    main()
