"""CPU oracle for the quantized-GEMM hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch-on-CPU, the torch reference programs that
tile-ai/tilelang-ascend ships beside its quantized-GEMM examples.  It is the
checker for the CUDA kernels: only the test-suite, the smoke entry and the CPU
baseline leg of the benchmark may import it.  Nothing in the product package
imports or falls back to it.

Parity status
-------------
* W8A8 (``quant_matmul_ref``), unsigned/signed int4 unpack, int8-mode and
  fp16-mode unscaled dequant GEMM, W4A8: pinned.  The restatement is checked
  against the reference's own functions (lifted from the reference tree by
  ``oracle/lift_reference.py``) and against the committed golden vectors under
  ``tests/golden`` which those lifted functions produced, including the
  reference's known-answer vector ``[[0x12, 0x34]] -> [2, 1, 4, 3]``.
* Scaled W4A16 (``scales`` given, zero point 8): the formula
  ``W[k, n] = (q[n, k] - zero).half() * s[k // g, n]`` is taken from
  ``tilelang/quantize/utils.py:33,46`` (``gen_quant4``).  No test of the
  reference exercises that formula together with a GEMM, so for this
  extension the golden vectors pin only the dequantised weights (against
  ``gen_quant4``'s own ``ref`` output); the GEMM on top of it is
  "parity unpinned" by the reference and pinned only by this restatement.

Every function cites the reference file:line it follows (paths are relative to
the reference project root).
"""
from __future__ import annotations

import torch

__all__ = [
    "int_matmul_exact",
    "quant_matmul_ref",
    "unpack_uint4",
    "unpack_int4_signed",
    "pack_uint4",
    "pack_int4_signed",
    "dequant_weight_ref",
    "dequant_gemm_fp16_ref",
    "dequant_gemm_int8_ref",
    "w4a8_gemm_ref",
    "act_quant_ref",
    "make_config_inputs",
    "CONFIG_SHAPES",
]

_DTYPES = {
    "float16": torch.float16,
    "bfloat16": torch.bfloat16,
    "float32": torch.float32,
    "int32": torch.int32,
    "int8": torch.int8,
}


def _dt(x):
    return _DTYPES[x] if isinstance(x, str) else x


# ----------------------------------------------------------------------------
# W8A8
# ----------------------------------------------------------------------------
def int_matmul_exact(A: torch.Tensor, B: torch.Tensor, chunk: int = 512) -> torch.Tensor:
    """Exact ``A.to(int32) @ B.to(int32)`` for int8 operands, evaluated with fp32 BLAS.

    Definition followed: ``C = A.to(accum_dtype) @ B.to(accum_dtype)``
    (examples/quant_batch_matmul/example_quant_batch_matmul.py:94).  Every
    partial sum over at most ``chunk`` <= 512 products of int8 values is
    bounded by 512 * 128 * 128 = 2**23 < 2**24 and therefore exact in fp32;
    the partials are added as int32.  Bit-identical to the int32 matmul and
    about 15x faster on CPU.  ``A`` is [..., M, K], ``B`` is [..., K, N].
    """
    assert chunk <= 512
    K = A.shape[-1]
    assert B.shape[-2] == K
    out = None
    for k0 in range(0, K, chunk):
        a = A[..., :, k0:k0 + chunk].to(torch.float32)
        b = B[..., k0:k0 + chunk, :].to(torch.float32)
        part = torch.matmul(a, b).to(torch.int32)
        out = part if out is None else out + part
    return out


def quant_matmul_ref(A, B, scale, out_dtype, accum_dtype=torch.int32, scale_a=None,
                     exact_fast=True, return_acc=False):
    """W8A8 reference: ``(int32(A @ B).to(fp32) * scale).to(out_dtype)``.

    Follows ``ref_program`` of
    examples/quant_batch_matmul/example_quant_batch_matmul.py:93-95 and
    examples/quant_batch_matmul/example_quant_matmul.py:92-94.  ``A`` is
    [M, K] or [Batch, M, K] int8, ``B`` is [K, N] or [Batch, K, N] int8,
    ``scale`` is fp32 of shape [1], [N] or (per-batch extension) [Batch, N].

    ``scale_a`` (optional, [M] or [Batch, M]) is the per-token activation
    scale of the two-scale form; the multiplication order is the one of the
    reference kernel in examples/deepseek_v4/int8_gemm.py:95-101 — accumulator
    to fp32, times scale_a[m], times scale_b[n], then the cast.
    """
    out_dtype = _dt(out_dtype)
    accum_dtype = _dt(accum_dtype)
    assert accum_dtype == torch.int32
    if exact_fast:
        C = int_matmul_exact(A, B)
    else:
        C = A.to(accum_dtype) @ B.to(accum_dtype)
    Cf = C.to(scale.dtype)
    if scale_a is not None:
        Cf = Cf * scale_a.unsqueeze(-1)
    sb = scale
    if sb.dim() == 2:  # [Batch, N] -> broadcast over M
        sb = sb.unsqueeze(-2)
    out = (Cf * sb).to(out_dtype)
    if return_acc:
        return out, C
    return out


# ----------------------------------------------------------------------------
# int4 packing
# ----------------------------------------------------------------------------
def unpack_uint4(packed: torch.Tensor) -> torch.Tensor:
    """[N, K/2] uint8 -> [N, K] uint8 with values 0..15, low nibble = even k.

    Vectorised restatement of the element loop
    ``u4 = (tensor[i, j // 2] >> ((j % 2) * 4)) & 0xF`` in
    examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:10-32
    (fp16 result) and :35-57 (int8 result); the same decode expression is
    ``_tir_packed_to_unsigned_convert`` in tilelang/quantize/quantization.py:198-206.
    """
    assert packed.dtype == torch.uint8
    lo = packed & 0xF
    hi = packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def unpack_int4_signed(packed: torch.Tensor) -> torch.Tensor:
    """[N, K/2] uint8 -> [N, K] int8 in -8..7 (two's-complement nibbles).

    Follows ``torch_convert`` in
    examples/dequantize_gemm/example_dequant_gemm_w4a8.py:124-145
    (``i4 = ((val >> 4*pos) & 0xF) << 4 >> 4`` on int8) and
    ``_tir_packed_int_to_int_convert`` in tilelang/quantize/quantization.py:221-231.
    """
    u = unpack_uint4(packed).to(torch.int16)
    return torch.where(u >= 8, u - 16, u).to(torch.int8)


def pack_uint4(q: torch.Tensor) -> torch.Tensor:
    """[..., K] integer values 0..15 -> [..., K/2] uint8, element j in byte j//2 at bits 4*(j%2).

    Follows ``general_compress(w, source_bits=4)`` in
    tilelang/quantize/utils.py:53-69 and ``generate_quantized_weight`` in
    examples/dequantize_gemm/example_dequant_gemm_w4a8.py:156-165.
    """
    assert q.shape[-1] % 2 == 0
    q = q.to(torch.int16) & 0xF
    return (q[..., 0::2] | (q[..., 1::2] << 4)).to(torch.uint8)


def pack_int4_signed(w: torch.Tensor) -> torch.Tensor:
    """[..., K] int8 in -8..7 -> [..., K/2] uint8 (``(high << 4) | low`` on the masked nibbles).

    Follows examples/dequantize_gemm/example_dequant_gemm_w4a8.py:156-165.
    """
    return pack_uint4(w.to(torch.int16) & 0xF)


# ----------------------------------------------------------------------------
# W4A16 / W4 -> int8
# ----------------------------------------------------------------------------
def dequant_weight_ref(packed, scales=None, zero=8, group_size=128):
    """Dequantised weight matrix W[N, K] in fp16.

    ``scales is None``: the reference example's semantics — unsigned values
    0..15 as fp16, no zero point, no scale
    (examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:10-32).

    Otherwise ``W[n, k] = (q[n, k] - zero).half() * s[k // g, n]`` with ``s`` of
    shape [K/g, N] fp16: ``ref = (w - 8).half() * s`` and
    ``s = s.reshape((-1, n))`` in tilelang/quantize/utils.py:33,46; zero mode
    "original" ``(q - z) * s`` of tilelang/quantize/lop3.py:165-166.  The
    subtraction is exact and the product rounds once to fp16 (RN-even), as a
    torch fp16 multiply does.
    """
    q = unpack_uint4(packed)
    if scales is None:
        return q.to(torch.float16)
    N, K = q.shape
    assert scales.dtype == torch.float16 and scales.shape == (K // group_size, N), scales.shape
    s_full = scales.t().repeat_interleave(group_size, dim=1)  # [N, K]
    return (q.to(torch.int16) - int(zero)).to(torch.float16) * s_full


def dequant_weight_zeros_ref(packed, scales, zeros, group_size=128, zeros_mode="original"):
    """Dequantised W[N, K] fp16 with one zero point per (group, output feature): ``zeros`` fp16 [K/g, N].

    The three zero modes of tilelang/quantize/lop3.py (selected at :1097,1172-1180), each with the roundings of
    the f16x2 instructions its decode routine issues:
      "original"   (:135-168)  h = q - z (sub.f16x2), then h * s (fma with +0): two roundings
      "rescale"    (:232-262)  fma(q, s, -|z|): one rounding (the routine ORs the sign bit into z, :247)
      "quantized"  (:325-358)  (q - qz) * s with integer qz: the subtraction is exact, one rounding
    ``q`` is the raw nibble value 0..15 (exact in f16)."""
    q = unpack_uint4(packed).to(torch.float16)
    N, K = q.shape
    assert scales.shape == (K // group_size, N) and zeros.shape == (K // group_size, N)
    s_full = scales.t().repeat_interleave(group_size, dim=1)
    z_full = zeros.to(torch.float16).t().repeat_interleave(group_size, dim=1)
    if zeros_mode in ("original", "quantized"):
        return (q - z_full) * s_full
    if zeros_mode == "rescale":
        # q * s is exact in fp64 (4 x 11 significant bits) and so is the difference: one rounding to f16
        return (q.double() * s_full.double() - z_full.double().abs()).to(torch.float16)
    raise ValueError(zeros_mode)


def interleave_int4_f16_ref(packed):
    """interleave_weight(qweight, 4, "float16") of tilelang/quantize/utils.py:73-99, restated per 32-bit word:
    element o (bits 4o) moves to bits (o % 2) * 16 + (o // 2) * 4."""
    w = packed.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(w)
    for o in range(8):
        out |= ((w >> (4 * o)) & 0xF) << ((o % 2) * 16 + (o // 2) * 4)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)
    return out.view(torch.uint8).reshape(packed.shape)


def dequant_gemm_fp16_ref(A, packed, output_dtype, scales=None, zero=8, group_size=128):
    """``C = fp32(A) @ fp32(W).T`` cast to ``output_dtype``.

    Follows ``ref_program_fp16`` in
    examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:269-289: A is
    taken to fp32 directly from its own dtype (fp16 or bf16, :283), the weights
    go through fp16 (:281,284), fp32 matmul (:285), cast (:288).
    """
    W = dequant_weight_ref(packed, scales, zero, group_size)
    C = torch.matmul(A.to(torch.float32), W.to(torch.float32).t())
    return C.to(_dt(output_dtype))


def dequant_gemm_int8_ref(A, packed, output_dtype="int32"):
    """``C = int32(A) @ int32(unpack_u4(B)).T`` (exact), optionally cast.

    Follows ``ref_program_int8`` in
    examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:292-312.
    """
    W = unpack_uint4(packed).to(torch.int8)
    C = int_matmul_exact(A, W.t())
    return C.to(_dt(output_dtype))


def w4a8_gemm_ref(A, qB):
    """Signed-int4 weights times int8 activations, exact int32, returned as [M, N].

    Follows ``ref_program`` in
    examples/dequantize_gemm/example_dequant_gemm_w4a8.py:148-153
    (``matmul(A.float(), B.T.float()).to(int32)``; the reference returns the
    transpose [N, M] and its test transposes the kernel result to match, :182).
    """
    W = unpack_int4_signed(qB)
    return int_matmul_exact(A, W.t())


# ----------------------------------------------------------------------------
# Per-token activation quantisation (the step before the W8A8 GEMM)
# ----------------------------------------------------------------------------
def act_quant_ref(x: torch.Tensor):
    """bf16/fp16 [M, K] -> (int8 [M, K], fp32 scale [M]) by abs-max / 127 per row.

    Follows the test-data recipe in examples/deepseek_v4/int8_gemm.py:143-151:
    ``scale = clamp(absmax, min=1e-4) / 127``; ``q = clamp(x / scale, -128, 127).round()``.
    """
    xf = x.to(torch.float32)
    amax = torch.clamp(xf.abs().amax(dim=1, keepdim=True), min=1e-4)
    scale = amax / 127.0
    q = torch.clamp(xf / scale, -128, 127).round().to(torch.int8)
    return q, scale.squeeze(1)


def build_block_metadata_ref(batch_sizes_list, block_M):
    """(group, first row, valid rows) per row block, as construct_inputs builds it in
    examples/grouped_gemm/example_grouped_gemm_fwd.py:147-166."""
    rows, off = [], 0
    for g, size in enumerate(batch_sizes_list):
        for i in range((size + block_M - 1) // block_M):
            rows.append([g, off + i * block_M, min(block_M, size - i * block_M)])
        off += size
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 3)


def grouped_quant_matmul_ref(A, B, block_metadata, scale, out_dtype, scale_a=None, b_layout="KN", return_acc=False):
    """Ragged grouped W8A8 reference: the block loop of torch_gmm
    (examples/grouped_gemm/example_grouped_gemm_fwd.py:7-41) with the W8A8 arithmetic of ``quant_matmul_ref``
    per block: ``out[m0:m0+rows] = cast(int32(A[m0:m0+rows] @ B[g]) [* scale_a] * scale[g or 0])``.

    A [total_M, K] int8; B [G, K, N] (or [G, N, K] with ``b_layout="NK"``, torch_gmm's ``trans_b``, :33-34);
    scale fp32 [1], [N] or [G, N]; scale_a fp32 [total_M] or None.  Rows no block covers stay zero."""
    out_dtype = _dt(out_dtype)
    G = B.shape[0]
    N = B.shape[2] if b_layout == "KN" else B.shape[1]
    out = torch.zeros((A.shape[0], N), dtype=out_dtype)
    acc = torch.zeros((A.shape[0], N), dtype=torch.int32)
    for g, m0, rows in block_metadata.cpu().tolist():
        part_b = B[g] if b_layout == "KN" else B[g].transpose(0, 1)
        sc = scale[g] if scale.dim() == 2 and scale.shape[0] == G else scale
        sa = None if scale_a is None else scale_a[m0:m0 + rows]
        c, a32 = quant_matmul_ref(A[m0:m0 + rows], part_b.contiguous(), sc.reshape(-1), out_dtype, scale_a=sa, return_acc=True)
        out[m0:m0 + rows] = c
        acc[m0:m0 + rows] = a32
    return (out, acc) if return_acc else out


def act_quant_torch_ref(x: torch.Tensor, round_scale: bool = False):
    """Per-token int8 quantiser: x [M, N] or [batch, seq, N] -> (int8 like x, fp32 scales [..., 1]).

    Follows the golden act_quant_torch of examples/deepseek_v4/act_quant.py:112-142 step by step:
    ``amax = clamp(max|x|, min=1e-4)`` per row in fp32 (:126-128); ``scales = amax / 127`` or, with
    ``round_scale``, ``2 ** ceil(log2(amax / 127))`` (:130-133); ``q = round(clamp(x / scales, -127, 127))``
    cast through float16 to int8 (:135-137); 3-D inputs keep their shape and get scales [batch, seq, 1]
    (:139-141).  (The recipe in examples/deepseek_v4/int8_gemm.py:143-151, restated in ``act_quant_ref``,
    differs only in clamping to -128.)"""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).to(torch.float32)
    amax = torch.clamp(x2.abs().amax(dim=1, keepdim=True), min=1e-4)
    if round_scale:
        scales = 2 ** torch.ceil(torch.log2(amax / 127.0))
    else:
        scales = amax / 127.0
    q = torch.round(torch.clamp(x2 / scales, -127, 127)).to(torch.float16).to(torch.int8)
    return q.reshape(shape), scales.reshape(tuple(shape[:-1]) + (1,))


# ----------------------------------------------------------------------------
# Seeded synthetic inputs for the five benchmark configurations
# ----------------------------------------------------------------------------
CONFIG_SHAPES = {
    "cfg1": dict(kind="w8a8", batch=1, M=256, K=1024, N=1024, out="float16"),
    "cfg2": dict(kind="w4a16", M=16, K=4096, N=4096, a="float16", out="float16", group=128),
    "cfg3": dict(kind="w8a8", batch=0, M=4096, K=4096, N=14336, out="bfloat16"),
    "cfg4": dict(kind="w8a8", batch=16, M=512, K=7168, N=2048, out="bfloat16"),
    "cfg5": dict(kind="w4a16", M=None, K=8192, N=28672, a="bfloat16", out="bfloat16", group=128),
}


def make_w8a8_inputs(batch, M, K, N, seed=0):
    """int8 operands uniform in [-128, 127]; fp32 scales uniform in [0.001, 0.02].

    ``batch == 0`` means unbatched ([M, K] x [K, N]); scales are per batch when
    batched ([Batch, M] and [Batch, N]).  Tensors are created on the CPU from
    one seeded generator in the order A, B, scale_a, scale_b.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    bs = () if batch == 0 else (batch,)
    A = torch.randint(-128, 128, bs + (M, K), dtype=torch.int8, generator=g)
    B = torch.randint(-128, 128, bs + (K, N), dtype=torch.int8, generator=g)
    sa = torch.rand(bs + (M,), dtype=torch.float32, generator=g) * 0.019 + 0.001
    sb = torch.rand(bs + (N,), dtype=torch.float32, generator=g) * 0.019 + 0.001
    return A, B, sa, sb


def make_w4a16_inputs(M, K, N, a_dtype="float16", group=128, seed=0):
    """A ~ N(0,1); int4 weights uniform 0..15 packed low-nibble-first; fp16 scales in [0.005, 0.02]."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    A = torch.randn((M, K), dtype=torch.float32, generator=g).to(_dt(a_dtype))
    packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    scales = (torch.rand((K // group, N), dtype=torch.float32, generator=g) * 0.015 + 0.005).to(torch.float16)
    return A, packed, scales


def make_config_inputs(name, M=None, seed=0):
    c = CONFIG_SHAPES[name]
    if c["kind"] == "w8a8":
        return make_w8a8_inputs(c["batch"], c["M"], c["K"], c["N"], seed)
    return make_w4a16_inputs(M if M is not None else c["M"], c["K"], c["N"], c["a"], c["group"], seed)
