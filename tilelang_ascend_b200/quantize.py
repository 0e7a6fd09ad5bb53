"""Host-side int4 packing helpers with the layout of the reference's ``tilelang/quantize``.

One layout everywhere: element ``j`` of a row lives in byte ``j // 2`` at bits ``4 * (j % 2)``
(low nibble = even index), packed tensor shape ``[..., K/2]``
(tilelang/quantize/utils.py:53-69; examples/dequantize_gemm/example_dequant_gemm_w4a8.py:156-165).
These are vectorised torch ops and run on whatever device the input tensor lives on.
"""
from __future__ import annotations

import torch


def pack_int4(values: torch.Tensor) -> torch.Tensor:
    """Pack integer values (unsigned 0..15, or signed -8..7 as two's-complement nibbles) two per byte
    along the last axis; returns uint8 of shape [..., K/2]."""
    if values.shape[-1] % 2 != 0:
        raise ValueError("last dimension must be even to pack two int4 values per byte")
    v = values.to(torch.int16) & 0xF
    return (v[..., 0::2] | (v[..., 1::2] << 4)).to(torch.uint8)


def general_compress(lowprecision_weight: torch.Tensor, source_bits: int = 4, storage_dtype=None) -> torch.Tensor:
    """Same name, arguments and result as tilelang/quantize/utils.py:53-69 (``8 // source_bits`` values per
    byte, lowest bits first, default int8 storage); vectorised instead of the reference's column loop."""
    if storage_dtype is None:
        storage_dtype = torch.int8
    if source_bits not in (1, 2, 4, 8):
        raise ValueError("source_bits must be 1, 2, 4 or 8")
    epb = 8 // source_bits
    w = lowprecision_weight
    if w.dtype == torch.float16:
        w = w.to(torch.int8)
    if w.shape[-1] % epb != 0:
        raise ValueError("last dimension must be a multiple of 8 // source_bits")
    w = w.to(torch.int16).reshape(*w.shape[:-1], w.shape[-1] // epb, epb)
    out = torch.zeros(w.shape[:-1], dtype=torch.int16, device=w.device)
    for k in range(epb):
        # the reference shifts the value and truncates to int8 before OR-ing: keep the low 8 bits
        out |= (w[..., k] << (source_bits * k)) & 0xFF
    out = out.to(torch.uint8)
    if storage_dtype == torch.uint8:
        return out
    return out.view(torch.int8).to(storage_dtype)


# --------------------------------------------------------------------------- group-wise int4 quantiser
def quantize_int4_groupwise(w: torch.Tensor, groupsize: int = -1, clamp_max: int = 15):
    """Symmetric group-wise int4 quantisation of a ``[K, N]`` weight, the arithmetic of ``gen_quant4``
    (tilelang/quantize/utils.py:14-33): per (group of ``groupsize`` rows, column) ``s = max|w| * 2 / 16`` and
    ``q = clamp(round(w / s) + 8, 0, clamp_max)``.

    Returns ``(q, s)``: ``q`` uint8 ``[K, N]`` and ``s`` ``[K / groupsize, N]`` in ``w``'s dtype, the layout
    ``scales[k // g, n]`` the W4A16 operator takes (:46).  The reference clamps to 16, which does not fit a
    nibble (the largest element of every group reaches it); ``clamp_max=15`` (default) is what a packer needs,
    ``clamp_max=16`` reproduces the reference's integers."""
    if w.dim() != 2:
        raise ValueError("w must be [K, N]")
    K, N = w.shape
    g = K if groupsize == -1 else int(groupsize)
    if g <= 0 or K % g != 0:
        raise ValueError(f"groupsize {groupsize} must divide K={K}")
    wg = w.reshape(K // g, g, N)
    s = wg.abs().amax(dim=1, keepdim=True)
    s = s * (2 / 16)
    q = torch.round(wg / s).to(torch.int32) + 8
    q = torch.clamp(q, 0, clamp_max)
    return q.reshape(K, N).to(torch.uint8), s.reshape(K // g, N).contiguous()


def gen_quant4(k: int, n: int, groupsize: int = -1):
    """Same name, arguments and results as tilelang/quantize/utils.py:5-50: random fp16 weights ``[k, n]``
    quantised group-wise to int4.  Returns ``(original_w, linear, s, q - 8)`` with ``linear`` an
    ``nn.Linear(k, n)`` holding the dequantised weights ``((q - 8).half() * s).T`` and ``s`` of shape
    ``[k / groupsize, n]``.  As in the reference the integers are clamped to 16, so ``q - 8`` reaches +8: clamp to
    7 (or use ``quantize_int4_groupwise``) before packing."""
    w = torch.randn((k, n), dtype=torch.half, device="cpu")
    original_w = w.clone()
    g = k if groupsize == -1 else groupsize
    q, s = quantize_int4_groupwise(w, g, clamp_max=16)
    centred = q.to(torch.int32) - 8
    ref = (centred.reshape(k // g, g, n).half() * s.reshape(k // g, 1, n)).reshape(k, n)
    linear = torch.nn.Linear(k, n, bias=False)
    linear.weight.data = ref.t()
    return original_w, linear, s, centred


# --------------------------------------------------------------------------- interleaved ("fast decode") layout
def _interleave_positions(nbits: int, target_dtype: str):
    """dest bit position of source element ``o`` (at bits ``nbits * o``) inside each 32-bit word."""
    stride = 8 if target_dtype == "int8" else 16
    lanes = 32 // stride
    return [(o % lanes) * stride + (o // lanes) * nbits for o in range(32 // nbits)]


def _move_fields(word: torch.Tensor, moves):
    """OR together ``((word >> src) & mask) << dst`` for ``(src, dst, mask)`` in ``moves`` (int64 arithmetic)."""
    out = torch.zeros_like(word)
    for src, dst, mask in moves:
        out |= ((word >> src) & mask) << dst
    return out


def interleave_weight(qweight: torch.Tensor, nbits: int = 4, target_dtype: str = "float16") -> torch.Tensor:
    """Same name, arguments and result as tilelang/quantize/utils.py:73-126: permute the ``32 / nbits`` packed
    elements of every 32-bit word so that the lop3 decode emits consecutive elements.  For 4 bits and a float16
    target, element ``o`` moves to bits ``(o % 2) * 16 + (o // 2) * 4``: the low half-word holds elements
    0, 2, 4, 6 and the high half-word 1, 3, 5, 7.  ``qweight`` is int8 / uint8 with a last dimension that is a
    multiple of 4 bytes; the result has the same shape and dtype int8.

    The W4A16 operator takes this layout with ``weight_layout="interleaved"``.  (In the reference the 1-bit
    formats and 2-bit / float16 raise a TypeError in their extra shuffle, :102-124; they are restated here from
    the masks and shifts written there and are not pinned by reference vectors.)"""
    if target_dtype not in ("float16", "int8"):
        raise ValueError("target_dtype must be 'float16' or 'int8'")
    if nbits not in (1, 2, 4):
        raise ValueError("nbits must be 1, 2 or 4")
    if qweight.dtype not in (torch.int8, torch.uint8) or qweight.shape[-1] % 4 != 0:
        raise ValueError("qweight must be int8/uint8 with a last dimension that is a multiple of 4")
    word = qweight.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    mask = (1 << nbits) - 1
    pos = _interleave_positions(nbits, target_dtype)
    word = _move_fields(word, [(nbits * o, pos[o], mask) for o in range(32 // nbits)])
    # the extra field shuffles of the 1-bit and 2-bit formats (utils.py:101-124)
    if nbits == 1 and target_dtype == "int8":
        word = (word & 0xF0F00F0F) | _move_fields(word, [(4, 16, 0xF), (12, 24, 0xF), (16, 4, 0xF), (24, 12, 0xF)])
    elif nbits == 2 and target_dtype == "float16":
        word = (word & 0xFF0000FF) | _move_fields(word, [(8, 16, 0xFF), (16, 8, 0xFF)])
    elif nbits == 1 and target_dtype == "float16":
        word = (word & 0xF000000F) | _move_fields(word, [(4, 8, 0xF), (8, 16, 0xF), (12, 24, 0xF), (16, 4, 0xF),
                                                         (20, 12, 0xF), (24, 20, 0xF)])
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    return word.view(torch.int8).reshape(qweight.shape)


def deinterleave_weight_int4_f16(qweight: torch.Tensor) -> torch.Tensor:
    """Inverse of ``interleave_weight(qweight, 4, "float16")``: back to sequential nibbles (uint8)."""
    word = qweight.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    pos = _interleave_positions(4, "float16")
    word = _move_fields(word, [(pos[o], 4 * o, 0xF) for o in range(8)])
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    return word.view(torch.uint8).reshape(qweight.shape)


def unpack_qzeros(qzeros: torch.Tensor, n: int) -> torch.Tensor:
    """Packed integer zero points ``[K / g, n / 2]`` (two per byte along the output features, low nibble first, the
    layout ``general_compress`` produces) -> fp16 ``[K / g, n]``, the form the operator's ``zeros=`` takes for
    zero mode "quantized" (``(q - qz) * s``, tilelang/quantize/lop3.py:325-358)."""
    b = qzeros.to(torch.int16) & 0xFF
    z = torch.stack([b & 0xF, (b >> 4) & 0xF], dim=-1).reshape(*qzeros.shape[:-1], -1)
    if z.shape[-1] != n:
        raise ValueError(f"qzeros holds {z.shape[-1]} zero points per group, expected {n}")
    return z.to(torch.float16)
