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
