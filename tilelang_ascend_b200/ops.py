"""Operator factories with the names, argument order and call signatures of the reference examples.

Reference                                                              here
---------------------------------------------------------------------  -------------------------------
examples/quant_batch_matmul/example_quant_batch_matmul.py:17-91        simple_quant_batch_matmul
examples/quant_batch_matmul/example_quant_matmul.py:17-90              simple_quant_matmul
examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:176-223  dequant_gemm_fp16_wrapper
examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:226-266  dequant_gemm_int8_wrapper
examples/dequantize_gemm/example_dequant_gemm_w4a8.py:25-121           w4a8_gemm_cv

As in the reference, a factory is called with the static shape and returns a callable that takes
torch tensors and returns a torch tensor; outputs and workspaces are allocated by the wrapper on the
device of the first input (tilelang/jit/adapter/cython/cython_wrapper.pyx:102-141), inputs must be
contiguous, of the declared dtype and on one device, else ``ValueError`` (:148-180).  The ``block_*``
arguments are kept for signature parity; the tile sizes of the B200 kernels are fixed by the library.
Every call goes through the C ABI of libqgemm.so; there is no fallback path.
"""
from __future__ import annotations

import functools
import os
from typing import Optional

import torch

from . import _lib

_TORCH_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32,
             "int8": torch.int8, "int32": torch.int32}
_ABI_DT = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16, torch.int32: _lib.DT_I32}


def _dt(x):
    if isinstance(x, torch.dtype):
        return x
    try:
        return _TORCH_DT[x]
    except KeyError:
        raise ValueError(f"unsupported dtype {x!r}") from None


def _stream_handle(stream, device) -> int:
    if stream is None or stream == -1:
        return torch.cuda.current_stream(device).cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


def _check_tensor(t, idx, name, dtype, shape, device):
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"Unsupported tensor type: {type(t)}")
    if not t.is_contiguous():
        raise ValueError(f"Input tensor at index {idx} must be contiguous")
    if t.device != device:
        raise ValueError(f"Buffer device mismatch for parameter {name}: expected {device}, got {t.device}")
    if t.dtype != dtype:
        raise ValueError(f"Buffer dtype mismatch for parameter {name}: expected {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"Static shape mismatch for parameter {name}: expected {tuple(shape)}, got {tuple(t.shape)}")


def _require_cuda(t, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise ValueError(f"parameter {name} must be a CUDA tensor (this operator has no CPU path)")


def _check_blocks(*blocks):
    for b in blocks:
        if not isinstance(b, int) or b <= 0:
            raise ValueError(f"block sizes must be positive integers, got {b!r}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------------------------------- W8A8
def quant_matmul(A, B, scale, scale_a=None, out_dtype=torch.float16, b_layout="KN", stream=None,
                 return_accumulators=False, status=None):
    """``C = cast((int32(A @ B)).float() [* scale_a[..., None]] * scale)`` on CUDA int8 tensors.

    A: [M, K] or [Batch, M, K]; B: [K, N] / [Batch, K, N] (``b_layout="KN"``) or [N, K] / [Batch, N, K]
    (``"NK"``).  scale: fp32 [1], [N] or [Batch, N].  scale_a: optional fp32 [M] or [Batch, M].
    ``out_dtype`` float16 / bfloat16, or int32 for the raw accumulators.
    """
    lib = _lib.load()
    _require_cuda(A, "A")
    dev = A.device
    out_dtype = _dt(out_dtype)
    if A.dim() not in (2, 3) or B.dim() != A.dim():
        raise ValueError("A and B must both be 2-D or both be 3-D")
    batched = A.dim() == 3
    batch = A.shape[0] if batched else 1
    M, K = A.shape[-2], A.shape[-1]
    if b_layout == "KN":
        N = B.shape[-1]
        b_shape = ((batch,) if batched else ()) + (K, N)
    elif b_layout == "NK":
        N = B.shape[-2]
        b_shape = ((batch,) if batched else ()) + (N, K)
    else:
        raise ValueError("b_layout must be 'KN' or 'NK'")
    _check_tensor(A, 0, "A", torch.int8, None, dev)
    _check_tensor(B, 1, "B", torch.int8, b_shape, dev)
    sb_len = sa_len = 0
    if out_dtype != torch.int32:
        _check_tensor(scale, 2, "scale", torch.float32, None, dev)
        sb_len = scale.numel()
        if sb_len not in (1, N, batch * N):
            raise ValueError(f"Static shape mismatch for parameter scale: expected [1], [{N}] or [{batch}, {N}], got {tuple(scale.shape)}")
        if scale_a is not None:
            _check_tensor(scale_a, 3, "scale_a", torch.float32, None, dev)
            sa_len = scale_a.numel()
            if sa_len not in (M, batch * M):
                raise ValueError(f"Static shape mismatch for parameter scale_a: expected [{M}] or [{batch}, {M}], got {tuple(scale_a.shape)}")
    elif out_dtype not in _ABI_DT:
        raise ValueError(f"unsupported out_dtype {out_dtype}")
    out_shape = ((batch,) if batched else ()) + (M, N)
    C = torch.empty(out_shape, dtype=out_dtype, device=dev)
    acc = torch.empty(out_shape, dtype=torch.int32, device=dev) if (return_accumulators and out_dtype != torch.int32) else None
    if C.numel() == 0:  # no rows (or an empty batch): nothing to launch
        return (C, acc) if acc is not None else C
    with torch.cuda.device(dev):
        rc = lib.qgemm_w8a8(A.data_ptr(), B.data_ptr(), _ptr(scale) if out_dtype != torch.int32 else None,
                            _ptr(scale_a) if out_dtype != torch.int32 else None, C.data_ptr(), _ptr(acc),
                            batch, M, N, K, sb_len, sa_len, _ABI_DT[out_dtype],
                            _lib.B_KN if b_layout == "KN" else _lib.B_NK, _ptr(status), _stream_handle(stream, dev))
    _lib.check(rc, "qgemm_w8a8")
    if acc is not None:
        return C, acc
    return C


class _QuantMatmulKernel:
    """Callable returned by the W8A8 factories: ``kernel(A, B, scale[, scale_a]) -> C``."""

    def __init__(self, batch, M, N, K, scale_size, out_dtype):
        self.batch, self.M, self.N, self.K = batch, M, N, K
        self.scale_size = scale_size
        self.out_dtype = out_dtype

    def __call__(self, A, B, scale, scale_a=None, stream=None, return_accumulators=False):
        lead = () if self.batch is None else (self.batch,)
        _require_cuda(A, "A")
        _check_tensor(A, 0, "A", torch.int8, lead + (self.M, self.K), A.device)
        _check_tensor(B, 1, "B", torch.int8, lead + (self.K, self.N), A.device)
        if isinstance(scale, torch.Tensor) and scale_a is None:
            n_scale = self.N if str(self.scale_size) == "N" else 1
            allowed = {n_scale} | ({self.batch * self.N} if (self.batch and n_scale != 1) else set())
            if scale.numel() not in allowed:
                raise ValueError(f"Static shape mismatch for parameter scale: expected [{n_scale}], got {tuple(scale.shape)}")
        return quant_matmul(A, B, scale, scale_a=scale_a, out_dtype=self.out_dtype, stream=stream,
                            return_accumulators=return_accumulators)


def _check_w8a8_dtypes(in_dtype, out_dtype, accum_dtype, scale_dtype):
    if _dt(in_dtype) != torch.int8:
        raise ValueError("in_dtype must be int8")
    if _dt(out_dtype) not in (torch.float16, torch.bfloat16):
        raise ValueError("out_dtype must be float16 or bfloat16")
    if _dt(accum_dtype) != torch.int32:
        raise ValueError("accum_dtype must be int32")
    if _dt(scale_dtype) != torch.float32:
        raise ValueError("scale_dtype must be float32")


@functools.lru_cache(maxsize=None)
def simple_quant_batch_matmul(Batch: int, M: int, N: int, K: int, scale_size, block_M: int, block_N: int,
                              block_K: int, in_dtype="int8", out_dtype="float16", accum_dtype="int32",
                              scale_dtype="float32"):
    """Factory with the signature of examples/quant_batch_matmul/example_quant_batch_matmul.py:17-22.

    Returns ``kernel(A[Batch,M,K], B[Batch,K,N], scale[N or 1]) -> C[Batch,M,N]``.  Extension: an optional
    fourth argument ``scale_a`` ([M] or [Batch, M], per-token activation scale, applied before ``scale``)
    and per-batch ``scale`` of shape [Batch, N].
    """
    _check_blocks(block_M, block_N, block_K)
    _check_w8a8_dtypes(in_dtype, out_dtype, accum_dtype, scale_dtype)
    if str(scale_size) not in ("1", "N"):
        raise ValueError('scale_size must be "1" or "N"')
    return _QuantMatmulKernel(int(Batch), int(M), int(N), int(K), scale_size, _dt(out_dtype))


@functools.lru_cache(maxsize=None)
def simple_quant_matmul(M: int, N: int, K: int, scale_size, block_M: int, block_N: int, block_K: int,
                        in_dtype="int8", out_dtype="float16", accum_dtype="int32", scale_dtype="float32"):
    """Factory with the signature of examples/quant_batch_matmul/example_quant_matmul.py:17-22.

    Returns ``kernel(A[M,K], B[K,N], scale[N or 1]) -> C[M,N]`` (optional ``scale_a[M]`` as above).
    """
    _check_blocks(block_M, block_N, block_K)
    _check_w8a8_dtypes(in_dtype, out_dtype, accum_dtype, scale_dtype)
    if str(scale_size) not in ("1", "N"):
        raise ValueError('scale_size must be 1 or "N"')
    return _QuantMatmulKernel(None, int(M), int(N), int(K), scale_size, _dt(out_dtype))


# ------------------------------------------------------------------------------------------ W4A16
_ZERO_MODES = {"original": 0, "rescale": 1, "quantized": 2}
_WEIGHT_LAYOUTS = {"sequential": 0, "interleaved": 1}


def release_workspaces():
    """Kept for callers of earlier versions: scratch buffers are allocated per call now (as the reference wrapper
    allocates its workspaces, tilelang/jit/adapter/cython/cython_wrapper.pyx:102-141), so there is nothing to drop."""


def _w4a16_workspace(lib, batch, M, N, K, device, stream_handle, zeros_tensor=False):
    """Scratch buffer of one call (split-K partial sums + arrival counters + prepared activations, and from 1024
    tokens on, or with a zeros tensor, the f16 copy of the weights).

    It needs no initialisation: the call zeroes its arrival counters itself, on its stream.  It is allocated per
    call from torch's caching allocator, so no launch ever sees a buffer that another call may still be using or
    that a captured CUDA graph still points to; when the launch stream is not torch's current stream the buffer
    is tied to that stream so that the allocator does not hand it out again too early."""
    need = lib.qgemm_w4a16_ex_workspace_bytes(batch, M, N, K, 1 if zeros_tensor else 0)
    if need < 0:
        raise _lib.QGemmError("qgemm_w4a16_ex_workspace_bytes: " + _lib.last_error())
    ws = torch.empty(need, dtype=torch.uint8, device=device)
    if stream_handle != torch.cuda.current_stream(device).cuda_stream:
        ws.record_stream(torch.cuda.ExternalStream(stream_handle, device=device))
    return ws, need


def w4a16_gemm(A, B_packed, scales=None, zeros=8, group_size=128, out_dtype=None, stream=None, status=None,
               zeros_mode="original", weight_layout="sequential", check_status=False):
    """``C[M,N] = A[M,K] @ W[N,K].T`` with ``W = (unpack_u4(B_packed) - zeros).half() * scales[k // g, n]``
    (or the raw nibble values when ``scales is None``).  CUDA tensors in, CUDA tensor out.

    ``zeros`` is an integer zero point or an fp16 tensor ``[K/g, N]`` of per-(group, feature) zero points;
    ``zeros_mode`` is one of the reference's three (tilelang/quantize/lop3.py:1097): "original" ``(q - z) * s``,
    "rescale" ``q * s - |z|``, "quantized" ``(q - qz) * s`` with integer ``qz`` (see ``quantize.unpack_qzeros``).
    ``weight_layout="interleaved"`` takes weights permuted by ``interleave_weight(qweight, 4, "float16")``.

    Batched form: ``A[Batch,M,K]``, ``B_packed[Batch,N,K/2]``, ``scales[Batch,K/g,N]`` -> ``C[Batch,M,N]``,
    independent problems of one shape in a single launch (the batch dimension of ``simple_quant_batch_matmul``
    carried over to the W4A16 operator).

    ``status``: optional int32 CUDA tensor of one element that receives a non-zero code if a bounded wait inside
    the kernel ran out (the result is then unspecified).  ``check_status=True`` allocates that word, waits for the
    launch to finish and raises ``QGemmError`` if it is non-zero - a synchronising debug aid, off by default."""
    lib = _lib.load()
    _require_cuda(A, "A")
    dev = A.device
    if A.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"Buffer dtype mismatch for parameter A: expected float16 or bfloat16, got {A.dtype}")
    out_dtype = A.dtype if out_dtype is None else _dt(out_dtype)
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("output dtype must be float16 or bfloat16")
    if A.dim() not in (2, 3) or B_packed.dim() != A.dim():
        raise ValueError("A must be [M, K] and B_packed [N, K/2] (or both with a leading batch dimension)")
    batched = A.dim() == 3
    batch = A.shape[0] if batched else 1
    lead = (batch,) if batched else ()
    M, K = A.shape[-2], A.shape[-1]
    N = B_packed.shape[-2]
    _check_tensor(A, 0, "A", A.dtype, lead + (M, K), dev)
    _check_tensor(B_packed, 1, "B_packed", torch.uint8, lead + (N, K // 2), dev)
    if K % 2 != 0:
        raise ValueError("K must be divisible by 2 (INT4 packed format)")
    if zeros_mode not in _ZERO_MODES:
        raise ValueError(f"zeros_mode must be one of {sorted(_ZERO_MODES)}, got {zeros_mode!r}")
    if weight_layout not in _WEIGHT_LAYOUTS:
        raise ValueError(f"weight_layout must be one of {sorted(_WEIGHT_LAYOUTS)}, got {weight_layout!r}")
    zeros_t = None
    if scales is not None:
        if group_size in (-1, None):
            group_size = K
        if K % group_size != 0:
            raise ValueError("group_size must divide K")
        _check_tensor(scales, 2, "scales", torch.float16, lead + (K // group_size, N), dev)
        if isinstance(zeros, torch.Tensor):
            _check_tensor(zeros, 3, "zeros", torch.float16, lead + (K // group_size, N), dev)
            zeros_t, zeros = zeros, 0
        elif not isinstance(zeros, int):
            raise ValueError("zeros must be an integer zero point or an fp16 tensor [K/g, N]")
        elif zeros_mode == "rescale":
            raise ValueError("zeros_mode 'rescale' needs a zeros tensor")
    else:
        if isinstance(zeros, torch.Tensor):
            raise ValueError("a zeros tensor needs scales")
        zeros, group_size = 0, K
    sh = _stream_handle(stream, dev)
    C = torch.empty(lead + (M, N), dtype=out_dtype, device=dev)
    if C.numel() == 0:  # no tokens: nothing to launch
        return C
    if check_status and status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        # integer zero points at decode sizes are taken in flight: no room for dequantised weights is needed
        inflight = (zeros_t is not None and zeros_mode == "quantized" and M <= 64
                    and (group_size == 128 or group_size % 256 == 0 or group_size >= K)
                    and os.environ.get("QGEMM_W4_ZEROS_INFLIGHT", "1") != "0" and os.environ.get("QGEMM_W4_GS", "1") != "0"
                    and "QGEMM_W4_GS_MIN_M" not in os.environ)
        ws, need = _w4a16_workspace(lib, batch, M, N, K, dev, sh, zeros_t is not None and not inflight)
        rc = lib.qgemm_w4a16_ex(A.data_ptr(), B_packed.data_ptr(), _ptr(scales), _ptr(zeros_t), int(zeros),
                                _ZERO_MODES[zeros_mode], _WEIGHT_LAYOUTS[weight_layout], int(group_size),
                                C.data_ptr(), ws.data_ptr(), need, batch, M, N, K, _ABI_DT[A.dtype],
                                _ABI_DT[out_dtype], _ptr(status), sh)
    _lib.check(rc, "qgemm_w4a16")
    if check_status:
        torch.cuda.synchronize(dev)  # the launch may be on any stream
        code = int(status.item())
        if code != 0:
            raise _lib.QGemmError(f"qgemm_w4a16: a bounded wait ran out on the device ({_lib.STATUS_NAMES.get(code, code)}); "
                                  "the result is unspecified")
    return C


def w4a16_gemm_gather(A, B_packed, scales, zeros, group_size, dst_ptrs, ldc, col0, out_dtype=None, stream=None,
                      status=None):
    """This rank's ``[M, N]`` block of a column-sharded W4A16 layer, written by the kernel into columns
    ``[col0, col0 + N)`` of every buffer of ``dst_ptrs``: device addresses of row-major ``[M, ldc]`` buffers, this
    rank's own and its peers' (mapped with ``ipc_open``).  Returns nothing; the buffers are complete once every
    rank's call has finished (see ``dist.ColumnShardedW4A16``).  Arguments otherwise as ``w4a16_gemm`` (2-D only)."""
    import ctypes
    lib = _lib.load()
    _require_cuda(A, "A")
    dev = A.device
    if A.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"Buffer dtype mismatch for parameter A: expected float16 or bfloat16, got {A.dtype}")
    out_dtype = A.dtype if out_dtype is None else _dt(out_dtype)
    if A.dim() != 2 or B_packed.dim() != 2:
        raise ValueError("A must be [M, K] and B_packed [N, K/2]")
    M, K = A.shape
    N = B_packed.shape[0]
    _check_tensor(A, 0, "A", A.dtype, (M, K), dev)
    _check_tensor(B_packed, 1, "B_packed", torch.uint8, (N, K // 2), dev)
    if scales is not None:
        if group_size in (-1, None):
            group_size = K
        _check_tensor(scales, 2, "scales", torch.float16, (K // group_size, N), dev)
    else:
        zeros, group_size = 0, K
    if not 1 <= len(dst_ptrs) <= 8:
        raise ValueError(f"1 to 8 destination buffers required, got {len(dst_ptrs)}")
    if M == 0:
        return
    sh = _stream_handle(stream, dev)
    ptr_array = (ctypes.c_void_p * len(dst_ptrs))(*[int(x) for x in dst_ptrs])
    with torch.cuda.device(dev):
        ws, need = _w4a16_workspace(lib, 1, M, N, K, dev, sh)
        rc = lib.qgemm_w4a16_gather(A.data_ptr(), B_packed.data_ptr(), _ptr(scales), int(zeros), int(group_size),
                                    ctypes.cast(ptr_array, ctypes.c_void_p), len(dst_ptrs), int(ldc), int(col0),
                                    ws.data_ptr(), need, M, N, K, _ABI_DT[A.dtype], _ABI_DT[out_dtype], _ptr(status), sh)
    _lib.check(rc, "qgemm_w4a16_gather")


def ipc_export(t: torch.Tensor):
    """(handle bytes, byte offset) under which another process of this node can map the device buffer of ``t``."""
    import ctypes
    lib = _lib.load()
    handle = (ctypes.c_ubyte * 64)()
    off = ctypes.c_int64(0)
    with torch.cuda.device(t.device):
        rc = lib.qgemm_ipc_export(t.data_ptr(), ctypes.cast(handle, ctypes.c_void_p), ctypes.cast(ctypes.byref(off), ctypes.c_void_p))
    _lib.check(rc, "qgemm_ipc_export")
    return bytes(handle), int(off.value)


def peer_signal_wait(flag_slots, local_flags: torch.Tensor, epoch: int = 0, epoch_counter: Optional[torch.Tensor] = None,
                     stream=None, status=None):
    """Store an epoch into this rank's slot of every rank's flag array (``flag_slots``: one device address per rank)
    and wait, on the stream, until every slot of ``local_flags`` (int32 ``[ranks]``) has reached it: the stream-ordered
    "all peers' blocks have landed" of the gathered W4A16 form without a collective.  The epoch is ``epoch`` or, with
    ``epoch_counter`` (an int32 CUDA tensor of one element that the kernel increments), counted on the device, which
    keeps counting when a captured graph is replayed.  The wait is bounded (``qgemm_set_wait_limit_ms``); ``status``
    receives QGEMM_ST_TIMEOUT_PEER if it runs out."""
    import ctypes
    lib = _lib.load()
    n = len(flag_slots)
    arr = (ctypes.c_void_p * n)(*[int(p) for p in flag_slots])
    dev = local_flags.device
    if local_flags.dtype != torch.int32 or local_flags.numel() < n or not local_flags.is_cuda:
        raise ValueError("local_flags must be a CUDA int32 tensor with one element per rank")
    with torch.cuda.device(dev):
        rc = lib.qgemm_peer_signal_wait(ctypes.cast(arr, ctypes.c_void_p), n, local_flags.data_ptr(), int(epoch) & 0xFFFFFFFF,
                                        _ptr(epoch_counter), _ptr(status), _stream_handle(stream, dev))
    _lib.check(rc, "qgemm_peer_signal_wait")


_ipc_mappings = {}  # (device index, handle) -> [base address, users]: an allocation is mapped once per process


def ipc_open(handle: bytes, device) -> int:
    """Map a buffer exported by ``ipc_export`` in another process; returns the base address of its allocation.

    Several exported buffers can lie in one allocation (torch's allocator carves small tensors out of larger
    segments) and an allocation can be mapped only once, so mappings are shared and counted."""
    import ctypes
    lib = _lib.load()
    key = (torch.device(device).index, bytes(handle))
    hit = _ipc_mappings.get(key)
    if hit is not None:
        hit[1] += 1
        return hit[0]
    buf = (ctypes.c_ubyte * 64).from_buffer_copy(handle)
    base = ctypes.c_void_p(0)
    with torch.cuda.device(device):
        rc = lib.qgemm_ipc_open(ctypes.cast(buf, ctypes.c_void_p), ctypes.cast(ctypes.byref(base), ctypes.c_void_p))
    _lib.check(rc, "qgemm_ipc_open")
    _ipc_mappings[key] = [int(base.value), 1]
    return int(base.value)


def ipc_close(base: int, device):
    """Drop one use of a mapping made by ``ipc_open``; the last one unmaps the allocation."""
    lib = _lib.load()
    idx = torch.device(device).index
    for key, ent in list(_ipc_mappings.items()):
        if key[0] == idx and ent[0] == base:
            ent[1] -= 1
            if ent[1] > 0:
                return
            del _ipc_mappings[key]
            break
    with torch.cuda.device(device):
        _lib.check(lib.qgemm_ipc_close(base), "qgemm_ipc_close")


@functools.lru_cache(maxsize=None)
def dequant_gemm_fp16_wrapper(M: int, N: int, K: int, block_M: int, block_N: int, block_K: int,
                              input_dtype: str = "float16", output_dtype: str = "float16"):
    """Factory with the signature of examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:176-185.

    Returns ``wrapper(A[M,K], B_packed[N,K/2]) -> C[M,N]``.  Like the reference wrapper (:208-221) it takes
    CPU tensors and returns a CPU tensor; CUDA tensors are accepted too and then the result stays on the
    GPU.  Extension: ``wrapper(A, B_packed, scales, zeros=8, group_size=128)`` applies group-wise fp16
    scales of shape [K/group_size, N] and an integer zero point, ``W = (q - zeros) * scales``.
    """
    _check_blocks(block_M, block_N, block_K)
    in_dt, out_dt = _dt(input_dtype), _dt(output_dtype)
    if in_dt not in (torch.float16, torch.bfloat16) or out_dt not in (torch.float16, torch.bfloat16):
        raise ValueError("input_dtype / output_dtype must be float16 or bfloat16")

    def wrapper(A: torch.Tensor, B_packed: torch.Tensor, scales=None, zeros: int = 8, group_size: int = 128):
        if tuple(A.shape) != (M, K) or tuple(B_packed.shape) != (N, K // 2):
            raise ValueError(f"Static shape mismatch: expected A {(M, K)}, B_packed {(N, K // 2)}; "
                             f"got {tuple(A.shape)}, {tuple(B_packed.shape)}")
        if A.dtype != in_dt:
            raise ValueError(f"Buffer dtype mismatch for parameter A: expected {in_dt}, got {A.dtype}")
        on_cpu = not A.is_cuda
        if on_cpu:
            # copies queue on the current stream without a host round trip each (pinned sources); the final
            # .cpu() below waits for everything, so the sources may be reused as soon as the call returns
            dev = torch.device("cuda", torch.cuda.current_device())
            A_, B_ = A.to(dev, non_blocking=True), B_packed.to(dev, non_blocking=True)
            s_ = None if scales is None else scales.to(dev, non_blocking=True)
        else:
            A_, B_, s_ = A, B_packed, scales
        C = w4a16_gemm(A_, B_, s_, zeros, group_size, out_dtype=out_dt)
        return C.cpu() if on_cpu else C

    return wrapper


# --------------------------------------------------------------------------- W4 -> int8 (exact int32)
def unpack_int4(B_packed, signed=False, out=None, stream=None):
    """[N, K/2] uint8 -> [N, K] int8 on the GPU (unsigned 0..15, or two's-complement -8..7 when ``signed``)."""
    lib = _lib.load()
    _require_cuda(B_packed, "B_packed")
    dev = B_packed.device
    _check_tensor(B_packed, 0, "B_packed", torch.uint8, None, dev)
    N, K = B_packed.shape[0], B_packed.shape[1] * 2
    if out is None:
        out = torch.empty((N, K), dtype=torch.int8, device=dev)
    else:
        _check_tensor(out, 1, "out", torch.int8, (N, K), dev)
    with torch.cuda.device(dev):
        rc = lib.qgemm_unpack_int4(B_packed.data_ptr(), out.data_ptr(), N, K, 1 if signed else 0,
                                   _stream_handle(stream, dev))
    _lib.check(rc, "qgemm_unpack_int4")
    return out


def _w4a8(A, qB, workspace, C, signed, stream=None, status=None):
    lib = _lib.load()
    dev = A.device
    M, K = A.shape
    N = qB.shape[0]
    with torch.cuda.device(dev):
        rc = lib.qgemm_w4a8(A.data_ptr(), qB.data_ptr(), workspace.data_ptr(), C.data_ptr(), M, N, K,
                            1 if signed else 0, _lib.DT_I32, _ptr(status), _stream_handle(stream, dev))
    _lib.check(rc, "qgemm_w4a8")
    return C


@functools.lru_cache(maxsize=None)
def w4a8_gemm_cv(M: int, N: int, K: int):
    """Factory with the signature of examples/dequantize_gemm/example_dequant_gemm_w4a8.py:26.

    Returns ``kernel(A[M,K] int8, qB[N,K/2] uint8, workspace[N,K] int8, C[M,N] int32) -> C`` with signed
    (two's-complement) nibbles; like the reference, the caller provides ``workspace`` and ``C`` (:174-177)."""

    def kernel(A, qB, workspace, C, stream=None):
        _require_cuda(A, "A")
        dev = A.device
        _check_tensor(A, 0, "A", torch.int8, (M, K), dev)
        _check_tensor(qB, 1, "qB", torch.uint8, (N, K // 2), dev)
        _check_tensor(workspace, 2, "workspace", torch.int8, (N, K), dev)
        _check_tensor(C, 3, "C", torch.int32, (M, N), dev)
        return _w4a8(A, qB, workspace, C, signed=True, stream=stream)

    return kernel


@functools.lru_cache(maxsize=None)
def w4a8_gemm_act_quant(M: int, N: int, K: int, round_scale: bool = False):
    """The per-token activation quantiser (examples/deepseek_v4/act_quant.py:33-92) fused into the W4A8 operator
    (examples/dequantize_gemm/example_dequant_gemm_w4a8.py:26) for up to 128 tokens.

    Returns ``kernel(X[M,K] bf16/f16, qB[N,K/2] uint8, workspace[N,K] int8, C[M,N] int32) -> (C, scale_a[M] fp32)``
    with ``C`` and ``scale_a`` bit-identical to ``act_quant`` followed by ``w4a8_gemm_cv``; the dequantised product is
    ``C * scale_a[:, None] * weight_scale``."""

    def kernel(X, qB, workspace, C, stream=None, status=None):
        lib = _lib.load()
        _require_cuda(X, "X")
        dev = X.device
        if X.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"Buffer dtype mismatch for parameter X: expected float16 or bfloat16, got {X.dtype}")
        _check_tensor(X, 0, "X", X.dtype, (M, K), dev)
        _check_tensor(qB, 1, "qB", torch.uint8, (N, K // 2), dev)
        _check_tensor(workspace, 2, "workspace", torch.int8, (N, K), dev)
        _check_tensor(C, 3, "C", torch.int32, (M, N), dev)
        scale_a = torch.empty((M,), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = lib.qgemm_w4a8_act_quant(X.data_ptr(), _ABI_DT[X.dtype], qB.data_ptr(), workspace.data_ptr(), C.data_ptr(),
                                          scale_a.data_ptr(), 1 if round_scale else 0, M, N, K, 1, _ptr(status),
                                          _stream_handle(stream, dev))
        _lib.check(rc, "qgemm_w4a8_act_quant")
        return C, scale_a

    return kernel


@functools.lru_cache(maxsize=None)
def dequant_gemm_int8_wrapper(M: int, N: int, K: int, block_M: int, block_N: int, block_K: int,
                              output_dtype: str = "int32"):
    """Factory with the signature of examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:226-234.

    Returns ``wrapper(A[M,K] int8, B_packed[N,K/2] uint8) -> C[M,N]``: unsigned nibbles, exact int32
    accumulation, then the cast to ``output_dtype`` (int32 / float16 / bfloat16) as the reference does
    (:263).  CPU tensors in give a CPU tensor out, as in the reference; CUDA tensors stay on the GPU."""
    _check_blocks(block_M, block_N, block_K)
    out_dt = _dt(output_dtype)
    if out_dt not in (torch.int32, torch.float16, torch.bfloat16):
        raise ValueError("output_dtype must be int32, float16 or bfloat16")

    def wrapper(A: torch.Tensor, B_packed: torch.Tensor):
        if tuple(A.shape) != (M, K) or tuple(B_packed.shape) != (N, K // 2):
            raise ValueError(f"Static shape mismatch: expected A {(M, K)}, B_packed {(N, K // 2)}; "
                             f"got {tuple(A.shape)}, {tuple(B_packed.shape)}")
        on_cpu = not A.is_cuda
        dev = torch.device("cuda", torch.cuda.current_device()) if on_cpu else A.device
        A_, B_ = (A.to(dev), B_packed.to(dev)) if on_cpu else (A, B_packed)
        _check_tensor(A_, 0, "A", torch.int8, (M, K), dev)
        _check_tensor(B_, 1, "B_packed", torch.uint8, (N, K // 2), dev)
        ws = torch.empty((N, K), dtype=torch.int8, device=dev)
        C = torch.empty((M, N), dtype=torch.int32, device=dev)
        _w4a8(A_, B_, ws, C, signed=False)
        C = C.to(out_dt)
        return C.cpu() if on_cpu else C

    return wrapper


# --------------------------------------------------------------------------- per-token activation quantiser
def act_quant(x, round_scale: bool = False, stream=None):
    """bf16/f16 ``x`` [M, N] or [batch, seq, N] -> (int8 of the same shape, fp32 scales [M, 1] or [batch, seq, 1]).

    Same arguments and results as the reference golden ``act_quant_torch(x, round_scale)``
    (examples/deepseek_v4/act_quant.py:112-142), computed on the GPU: per row ``scale = max(amax, 1e-4) / 127``
    (a power of two not below it when ``round_scale``), ``y = round(clamp(x / scale, -127, 127))``.  The
    outputs are what ``quant_matmul`` takes as ``A`` and ``scale_a``."""
    lib = _lib.load()
    _require_cuda(x, "x")
    dev = x.device
    if x.dim() not in (2, 3):
        raise ValueError(f"x must be 2-D or 3-D, got {x.dim()}-D")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"x must be bfloat16 or float16, got {x.dtype}")
    if not x.is_contiguous():
        raise ValueError("Input tensor at index 0 (x) must be contiguous")
    N = x.shape[-1]
    M = x.numel() // N if N else 0
    y = torch.empty(x.shape, dtype=torch.int8, device=dev)
    s = torch.empty(tuple(x.shape[:-1]) + (1,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.qgemm_act_quant(x.data_ptr(), y.data_ptr(), s.data_ptr(), M, N,
                                 _lib.DT_BF16 if x.dtype == torch.bfloat16 else _lib.DT_F16,
                                 1 if round_scale else 0, _stream_handle(stream, dev))
    _lib.check(rc, "qgemm_act_quant")
    return y, s


@functools.lru_cache(maxsize=None)
def act_quant_kernel_int8_optimized(N: int, block_M: int = 32, block_N: int = 32, round_scale: bool = False):
    """Factory with the signature of examples/deepseek_v4/act_quant.py:33.

    Returns ``kernel(X[M, N] bf16) -> (Y[M, N] int8, S[M] fp32)`` with M free, as in the reference (:34,
    outputs at ``out_idx=[-2, -1]``, :25); ``block_M`` / ``block_N`` are accepted as hints only."""
    if N <= 0 or N % 8:
        raise ValueError(f"N must be a positive multiple of 8, got {N}")
    if block_M <= 0 or block_N <= 0:
        raise ValueError("block_M and block_N must be positive")

    def kernel(X, stream=None):
        if X.dim() != 2 or X.shape[1] != N:
            raise ValueError(f"X must have shape [M, {N}], got {tuple(X.shape)}")
        y, s = act_quant(X, round_scale=round_scale, stream=stream)
        return y, s.view(-1)

    return kernel


# --------------------------------------------------------------------------- grouped (ragged) W8A8
def build_block_metadata(batch_sizes_list, block_M: int = 128, device=None):
    """Row-block table [total_blocks, 3] int32 = (group, first row, valid rows) for stacked row groups.

    The same table as ``construct_inputs`` builds on the host in
    examples/grouped_gemm/example_grouped_gemm_fwd.py:147-166: blocks never cross a group boundary, the last
    block of a group may be partial.  Empty groups contribute no block."""
    if not isinstance(block_M, int) or block_M <= 0:
        raise ValueError(f"block_M must be a positive integer, got {block_M!r}")
    rows, off = [], 0
    for g, size in enumerate(batch_sizes_list):
        size = int(size)
        if size < 0:
            raise ValueError(f"group sizes must not be negative, got {size}")
        for start in range(0, size, block_M):
            rows.append((g, off + start, min(block_M, size - start)))
        off += size
    meta = torch.tensor(rows, dtype=torch.int32).reshape(-1, 3)
    return meta if device is None else meta.to(device)


def grouped_quant_matmul(A, B, block_metadata, scale, scale_a=None, out_dtype=torch.float16, b_layout="KN",
                         stream=None, return_accumulators=False, status=None, out=None):
    """Ragged grouped W8A8: for every table row (g, m0, rows): ``C[m0:m0+rows] = cast(int32(A[m0:m0+rows] @ B[g])
    [* scale_a[m0:m0+rows, None]] * scale[g or 0])``.

    A: [total_M, K] int8; B: [G, K, N] (``"KN"``) or [G, N, K] (``"NK"``) int8; block_metadata: CUDA int32
    [blocks, 3] with at most 128 rows per block; scale: fp32 [1], [N] or [G, N]; scale_a: optional fp32 [total_M].
    Rows of the result that no block covers keep the contents of ``out`` (zeros when ``out`` is not given)."""
    lib = _lib.load()
    _require_cuda(A, "A")
    dev = A.device
    out_dtype = _dt(out_dtype)
    if A.dim() != 2 or B.dim() != 3:
        raise ValueError("A must be 2-D [total_M, K] and B 3-D [G, K, N] or [G, N, K]")
    total_M, K = A.shape
    G = B.shape[0]
    if b_layout == "KN":
        N, b_shape = B.shape[2], (G, K, B.shape[2])
    elif b_layout == "NK":
        N, b_shape = B.shape[1], (G, B.shape[1], K)
    else:
        raise ValueError("b_layout must be 'KN' or 'NK'")
    _check_tensor(A, 0, "A", torch.int8, None, dev)
    _check_tensor(B, 1, "B", torch.int8, b_shape, dev)
    _check_tensor(block_metadata, 2, "block_metadata", torch.int32, None, dev)
    if block_metadata.dim() != 2 or block_metadata.shape[1] != 3:
        raise ValueError(f"Static shape mismatch for parameter block_metadata: expected [blocks, 3], got {tuple(block_metadata.shape)}")
    sb_len = sa_len = 0
    if out_dtype != torch.int32:
        _check_tensor(scale, 3, "scale", torch.float32, None, dev)
        sb_len = scale.numel()
        if sb_len not in (1, N, G * N):
            raise ValueError(f"Static shape mismatch for parameter scale: expected [1], [{N}] or [{G}, {N}], got {tuple(scale.shape)}")
        if scale_a is not None:
            _check_tensor(scale_a, 4, "scale_a", torch.float32, None, dev)
            sa_len = scale_a.numel()
            if sa_len != total_M:
                raise ValueError(f"Static shape mismatch for parameter scale_a: expected [{total_M}], got {tuple(scale_a.shape)}")
    elif out_dtype not in _ABI_DT:
        raise ValueError(f"unsupported out_dtype {out_dtype}")
    if out is None:
        C = torch.zeros((total_M, N), dtype=out_dtype, device=dev)
    else:
        _check_tensor(out, 5, "out", out_dtype, (total_M, N), dev)
        C = out
    acc = torch.zeros((total_M, N), dtype=torch.int32, device=dev) if (return_accumulators and out_dtype != torch.int32) else None
    with torch.cuda.device(dev):
        rc = lib.qgemm_w8a8_grouped(A.data_ptr(), B.data_ptr(), _ptr(scale) if out_dtype != torch.int32 else None,
                                    _ptr(scale_a) if out_dtype != torch.int32 else None, C.data_ptr(), _ptr(acc),
                                    block_metadata.data_ptr(), block_metadata.shape[0], G, total_M, N, K, sb_len,
                                    sa_len, _ABI_DT[out_dtype], _lib.B_KN if b_layout == "KN" else _lib.B_NK,
                                    _ptr(status), _stream_handle(stream, dev))
    _lib.check(rc, "qgemm_w8a8_grouped")
    if acc is not None:
        return C, acc
    return C


@functools.lru_cache(maxsize=None)
def grouped_quant_gemm(batch_sizes_list, K: int, N: int, block_M: int = 128, block_N: int = 256, block_K: int = 128,
                       out_dtype="float16", b_layout: str = "KN"):
    """Factory with the signature of ``grouped_gemm`` in examples/grouped_gemm/example_grouped_gemm_fwd.py:44,
    for int8 operands: returns ``kernel(A, B, block_metadata, scale[, scale_a]) -> C``.

    ``batch_sizes_list`` (a tuple, as the reference passes it, :174) fixes total_M and the group count;
    ``block_M`` is the row-block height the caller's table was built with and must not exceed 128 (one tile);
    ``block_N`` / ``block_K`` are hints.  ``kernel.block_metadata(device)`` returns the table for these sizes."""
    sizes = tuple(int(x) for x in batch_sizes_list)
    _check_blocks(block_M, block_N, block_K)
    if block_M > 128:
        raise ValueError(f"block_M must not exceed 128 rows (one output tile), got {block_M}")
    total_M, G = sum(sizes), len(sizes)
    blocks = sum((x + block_M - 1) // block_M for x in sizes)

    def kernel(A, B, block_metadata, scale, scale_a=None, stream=None, return_accumulators=False):
        if A.dim() != 2 or tuple(A.shape) != (total_M, K):
            raise ValueError(f"Static shape mismatch for parameter A: expected ({total_M}, {K}), got {tuple(A.shape)}")
        if B.dim() != 3 or B.shape[0] != G:
            raise ValueError(f"Static shape mismatch for parameter B: expected {G} groups, got {tuple(B.shape)}")
        if block_metadata.dim() != 2 or block_metadata.shape[0] != blocks:
            raise ValueError(f"Static shape mismatch for parameter block_metadata: expected ({blocks}, 3), got {tuple(block_metadata.shape)}")
        return grouped_quant_matmul(A, B, block_metadata, scale, scale_a, out_dtype=out_dtype, b_layout=b_layout,
                                    stream=stream, return_accumulators=return_accumulators)

    kernel.block_metadata = lambda device="cuda": build_block_metadata(sizes, block_M, device)
    return kernel
