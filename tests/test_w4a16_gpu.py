"""GPU parity tests for the W4A16 / W4A8 paths: CUDA kernels (through libqgemm.so) against the CPU oracle.

Bars: fp16/bf16 outputs within rtol = atol = 1e-2
(examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:341-344); int32 outputs exact (:373-374,
examples/dequantize_gemm/example_dequant_gemm_w4a8.py:182).  The kernel accumulates exact f16 x f16
products in fp32 in a different order than the CPU matmul, so float results are close, not identical.
"""
import pytest
import torch

from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu


def _q():
    import tilelang_ascend_b200 as q
    return q


def _close(C, ref):
    assert C.dtype == ref.dtype
    torch.testing.assert_close(C.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("name,dt", [("dq_f16", "float16"), ("dq_bf16", "bfloat16")])
def test_golden_unscaled(golden, name, dt):
    """Reference-produced vectors of ref_program_fp16 (unsigned nibbles, no scale, no zero point)."""
    q = _q()
    bf = ("A", "C") if dt == "bfloat16" else ()
    c = golden.case(name, bf16=bf)
    M, K = c["A"].shape
    N = c["packed"].shape[0]
    if K % 32 != 0 or N % 8 != 0:
        pytest.skip("shape below the kernel's granularity")
    w = q.dequant_gemm_fp16_wrapper(M, N, K, 128, 256, 64, dt, dt)
    C = w(c["A"], c["packed"])  # CPU in -> CPU out, like the reference wrapper
    assert not C.is_cuda
    _close(C, c["C"])


def test_reference_known_answer_through_kernel():
    """The reference's nibble-order vector [[0x12, 0x34]] -> [2, 1, 4, 3], observed through the GEMM:
    with A = identity rows the output row m is column m of the unpacked weights."""
    q = _q()
    K, N = 32, 8
    packed = torch.zeros(N, K // 2, dtype=torch.uint8)
    packed[0, 0], packed[0, 1] = 0x12, 0x34
    A = torch.eye(K, dtype=torch.float16)[:4]
    C = q.w4a16_gemm(A.cuda(), packed.cuda()).cpu()
    assert C[:, 0].tolist() == [2.0, 1.0, 4.0, 3.0]
    assert torch.equal(C.float(), oc.unpack_uint4(packed).float().t()[:4])


W4_SHAPES = [
    # M, K, N, group
    (16, 256, 128, 128),
    (1, 32, 8, 32),
    (5, 96, 40, 32),
    (16, 1024, 256, 128),
    (8, 4096, 512, 128),
    (33, 640, 264, 64),
    (64, 2048, 384, 128),
    (100, 512, 136, 256),
    (256, 1024, 256, 128),
    (300, 768, 520, -1),
    # two blocks of 128 tokens per tile (above 128 tokens): ragged second block, odd and even block counts, split K
    (130, 512, 272, 128),
    (200, 2048, 136, 32),
    (513, 1024, 264, 64),
    (640, 4096, 384, 128),
]


@pytest.mark.parametrize("M,K,N,group", W4_SHAPES)
@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_scaled_against_oracle(M, K, N, group, dt):
    q = _q()
    g = K if group == -1 else group
    A, packed, scales = oc.make_w4a16_inputs(M, K, N, dt, g, seed=M + N)
    ref = oc.dequant_gemm_fp16_ref(A, packed, dt, scales, 8, g)
    C = q.w4a16_gemm(A.cuda(), packed.cuda(), scales.cuda(), 8, group)
    _close(C, ref)
    # a second, tighter bar than the reference's: error relative to the output scale
    err = (C.cpu().float() - ref.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref.float().abs().max().item()) * (1 if dt == "float16" else 4)


@pytest.mark.parametrize("M,K,N", [(16, 512, 128), (256, 256, 256), (512, 512, 512)])
def test_unscaled_reference_semantics(M, K, N):
    """scales=None: raw unsigned nibble values, exactly the reference example (its 256^3 / 512^3 ladder)."""
    q = _q()
    g = torch.Generator().manual_seed(0)
    A = torch.randn(M, K, generator=g).half()
    packed = torch.randint(0, 255, (N, K // 2), dtype=torch.uint8, generator=g)
    w = q.dequant_gemm_fp16_wrapper(M, N, K, 128, 256, 64)
    C = w(A.cuda(), packed.cuda())
    assert C.is_cuda
    _close(C, oc.dequant_gemm_fp16_ref(A, packed, "float16"))


def test_dequant_is_exact_via_identity_activations():
    """With A = I (K x K) the GEMM returns W^T: every dequantised weight must equal the oracle's fp16 value
    bit for bit ((q - 8) is exact, the product with the scale rounds once)."""
    q = _q()
    K, N = 256, 136
    _, packed, scales = oc.make_w4a16_inputs(1, K, N, "float16", 128, seed=3)
    A = torch.eye(K, dtype=torch.float16)
    C = q.w4a16_gemm(A.cuda(), packed.cuda(), scales.cuda(), 8, 128).cpu()
    W = oc.dequant_weight_ref(packed, scales, 8, 128)  # [N, K]
    assert torch.equal(C, W.t())
    for zero in (0, 3, 15):
        C = q.w4a16_gemm(A.cuda(), packed.cuda(), scales.cuda(), zero, 128).cpu()
        assert torch.equal(C, oc.dequant_weight_ref(packed, scales, zero, 128).t())


def test_split_k_is_deterministic_and_counters_stay_clean():
    q = _q()
    A, packed, scales = oc.make_config_inputs("cfg2")
    Ad, Pd, Sd = A.cuda(), packed.cuda(), scales.cuda()
    ref = oc.dequant_gemm_fp16_ref(A, packed, "float16", scales, 8, 128)
    outs = [q.w4a16_gemm(Ad, Pd, Sd, 8, 128) for _ in range(5)]
    _close(outs[0], ref)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("batch,M,K,N,dt", [(3, 5, 512, 264, "float16"), (4, 16, 1024, 256, "bfloat16"),
                                             (2, 70, 256, 384, "float16"), (6, 1, 2048, 128, "bfloat16")])
def test_batched_matches_oracle_and_single_calls(batch, M, K, N, dt):
    """Independent problems of one shape in one launch: every batch entry must match the oracle and the
    same problem launched on its own (identical arithmetic per element, possibly another fp32 split order)."""
    q = _q()
    ins = [oc.make_w4a16_inputs(M, K, N, dt, 128, seed=100 + b) for b in range(batch)]
    A = torch.stack([i[0] for i in ins]).cuda()
    P = torch.stack([i[1] for i in ins]).cuda()
    S = torch.stack([i[2] for i in ins]).cuda()
    C = q.w4a16_gemm(A, P, S, 8, 128)
    assert C.shape == (batch, M, N)
    for b in range(batch):
        ref = oc.dequant_gemm_fp16_ref(ins[b][0], ins[b][1], dt, ins[b][2], 8, 128)
        _close(C[b], ref)
        single = q.w4a16_gemm(A[b].contiguous(), P[b].contiguous(), S[b].contiguous(), 8, 128)
        torch.testing.assert_close(C[b].float(), single.float(), rtol=2e-3, atol=2e-3)
    C2 = q.w4a16_gemm(A, P, None)  # unscaled, batched
    for b in range(batch):
        _close(C2[b], oc.dequant_gemm_fp16_ref(ins[b][0], ins[b][1], dt))


@pytest.mark.parametrize("M", [1, 8, 64])
def test_config5_decode_full_size(M):
    """BASELINE config 5 decode shapes at full size (K = 8192, N = 28672, bf16): a band of output columns
    against the oracle plus linearity in A over the whole output (f(A) + f(2A) == f(3A) up to rounding)."""
    q = _q()
    A, packed, scales = oc.make_config_inputs("cfg5", M=M)
    Ad, Pd, Sd = A.cuda(), packed.cuda(), scales.cuda()
    C = q.w4a16_gemm(Ad, Pd, Sd, 8, 128)
    cols = torch.cat([torch.arange(0, 256), torch.arange(14000, 14200), torch.arange(28672 - 200, 28672)])
    ref = oc.dequant_gemm_fp16_ref(A, packed[cols], "bfloat16", scales[:, cols].contiguous(), 8, 128)
    _close(C[:, cols.cuda()], ref)
    C2 = q.w4a16_gemm((Ad * 2), Pd, Sd, 8, 128)
    torch.testing.assert_close(C2.float(), C.float() * 2, rtol=1e-2, atol=1e-2)  # exact power-of-two scaling in fp32
    assert torch.isfinite(C.float()).all()


def test_config5_prefill_m512_band():
    q = _q()
    A, packed, scales = oc.make_config_inputs("cfg5", M=512)
    C = q.w4a16_gemm(A.cuda(), packed.cuda(), scales.cuda(), 8, 128)
    cols = torch.cat([torch.arange(0, 128), torch.arange(20000, 20128)])
    ref = oc.dequant_gemm_fp16_ref(A, packed[cols], "bfloat16", scales[:, cols].contiguous(), 8, 128)
    _close(C[:, cols.cuda()], ref)


@pytest.mark.parametrize("M,N,K", [(64, 64, 256), (128, 128, 512), (256, 256, 1024)])
def test_w4a8_signed_exact(M, N, K):
    """The reference's three W4A8 levels (example_dequant_gemm_w4a8.py:202-208), exact int32."""
    q = _q()
    g = torch.Generator().manual_seed(42)
    A = torch.randint(-8, 8, (M, K), dtype=torch.int8, generator=g)
    Bi = torch.randint(-8, 8, (N, K), dtype=torch.int8, generator=g)
    qB = oc.pack_int4_signed(Bi)
    kernel = q.w4a8_gemm_cv(M, N, K)
    ws = torch.zeros(N, K, dtype=torch.int8, device="cuda")
    C = torch.zeros(M, N, dtype=torch.int32, device="cuda")
    out = kernel(A.cuda(), qB.cuda(), ws, C)
    assert torch.equal(ws.cpu(), Bi)
    assert torch.equal(out.cpu(), oc.w4a8_gemm_ref(A, qB))


def test_w4a8_golden(golden):
    q = _q()
    c = golden.case("w4a8")
    M, K = c["A"].shape
    N = c["qB"].shape[0]
    ws = torch.zeros(N, K, dtype=torch.int8, device="cuda")
    C = torch.zeros(M, N, dtype=torch.int32, device="cuda")
    q.w4a8_gemm_cv(M, N, K)(c["A"].cuda(), c["qB"].cuda(), ws, C)
    assert torch.equal(ws.cpu(), c["conv"])
    assert torch.equal(C.cpu(), c["C_nm"].t())


@pytest.mark.parametrize("M,N,K,odt", [(256, 256, 256, "int32"), (512, 512, 512, "int32"), (512, 512, 512, "float16")])
def test_int8_mode_unsigned_exact(M, N, K, odt):
    """dequant_gemm_int8_wrapper ladder (example_dequant_gemm_fine_grained.py:459-469)."""
    q = _q()
    g = torch.Generator().manual_seed(0)
    A = torch.randint(-128, 127, (M, K), dtype=torch.int8, generator=g)
    packed = torch.randint(0, 255, (N, K // 2), dtype=torch.uint8, generator=g)
    C = q.dequant_gemm_int8_wrapper(M, N, K, 128, 128, 64, odt)(A, packed)
    ref = oc.dequant_gemm_int8_ref(A, packed, odt)
    if odt == "int32":
        assert torch.equal(C, ref)
    else:
        torch.testing.assert_close(C, ref, rtol=1e-2, atol=1e-2)


def test_unpack_kernel_matches_oracle_on_ragged_sizes():
    q = _q()
    g = torch.Generator().manual_seed(1)
    for N, K in [(1, 2), (3, 34), (17, 96), (64, 1000)]:
        packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
        assert torch.equal(q.unpack_int4(packed.cuda()).cpu(), oc.unpack_uint4(packed).to(torch.int8))
        assert torch.equal(q.unpack_int4(packed.cuda(), signed=True).cpu(), oc.unpack_int4_signed(packed))


def test_rejects_bad_arguments():
    q = _q()
    A = torch.zeros(4, 64, dtype=torch.float16, device="cuda")
    P = torch.zeros(16, 32, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="dtype mismatch"):
        q.w4a16_gemm(A.float(), P)
    with pytest.raises(ValueError, match="shape mismatch"):
        q.w4a16_gemm(A, P[:, :16].contiguous())
    with pytest.raises(q.QGemmError, match="multiple of 32"):
        q.w4a16_gemm(A[:, :48].contiguous(), P[:, :24].contiguous())
    with pytest.raises(q.QGemmError, match="group"):
        q.w4a16_gemm(A, P, torch.ones(4, 16, dtype=torch.float16, device="cuda"), 8, 16)
    assert torch.equal(q.w4a16_gemm(A, P).cpu(), torch.zeros(4, 16, dtype=torch.float16))


def test_dequantise_once_path_small_shapes():
    """Above QGEMM_W4_GEMM_MIN_M tokens (default 1792) the weights are dequantised to f16 once and multiplied by
    the f16 tensor-core GEMM.  The threshold is read once per process, so a child process with a low threshold
    runs that path on small ragged shapes: scaled / unscaled, every group size, f16 / bf16, batched."""
    import os
    import subprocess
    import sys
    code = r"""
import torch
from oracle import qgemm_oracle as oc
import tilelang_ascend_b200 as q
def close(C, ref): torch.testing.assert_close(C.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)
for M, K, N, dt, group in [(17, 256, 128, "float16", 128), (40, 512, 272, "bfloat16", 64), (200, 1024, 528, "float16", 32),
                           (130, 768, 2320, "bfloat16", 256), (300, 512, 144, "float16", 512), (129, 2048, 1024, "bfloat16", 128)]:
    A, P, S = oc.make_w4a16_inputs(M, K, N, dt, group, seed=M + K)
    C = q.w4a16_gemm(A.cuda(), P.cuda(), S.cuda(), 8, group)
    close(C, oc.dequant_gemm_fp16_ref(A, P, dt, S, 8, group))
    C0 = q.w4a16_gemm(A.cuda(), P.cuda(), None)
    close(C0, oc.dequant_gemm_fp16_ref(A, P, dt))
# exact dequantisation: unit activations read back half(q - zero) * s bit for bit
K, N, group = 256, 144, 64
_, P, S = oc.make_w4a16_inputs(1, K, N, "float16", group, seed=3)
eye = torch.eye(K, dtype=torch.float16)
W = q.w4a16_gemm(eye.cuda(), P.cuda(), S.cuda(), 8, group)   # [K, N] = dequantised weights, transposed
assert torch.equal(W.cpu().t().contiguous(), oc.dequant_weight_ref(P, S, 8, group).half())
# batched
ins = [oc.make_w4a16_inputs(48, 512, 272, "float16", 128, seed=s) for s in range(3)]
A, P, S = [torch.stack([x[i] for x in ins]).cuda() for i in range(3)]
C = q.w4a16_gemm(A, P, S, 8, 128)
for b in range(3): close(C[b], oc.dequant_gemm_fp16_ref(ins[b][0], ins[b][1], "float16", ins[b][2], 8, 128))
print("dequantise-once ok")
"""
    env = dict(os.environ, QGEMM_W4_GEMM_MIN_M="17")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "dequantise-once ok" in r.stdout, r.stdout + r.stderr


def test_config5_prefill_m4096_band_and_linearity():
    """Config 5 at 4096 tokens goes through the dequantise-once path at full size: bands of output columns
    against the oracle, and f(2A) == 2 f(A) over the whole output."""
    q = _q()
    A, packed, scales = oc.make_config_inputs("cfg5", M=4096)
    Ad, Pd, Sd = A.cuda(), packed.cuda(), scales.cuda()
    C = q.w4a16_gemm(Ad, Pd, Sd, 8, 128)
    cols = torch.cat([torch.arange(0, 64), torch.arange(20000, 20064), torch.arange(28672 - 64, 28672)])
    ref = oc.dequant_gemm_fp16_ref(A, packed[cols], "bfloat16", scales[:, cols].contiguous(), 8, 128)
    _close(C[:, cols.cuda()], ref)
    C2 = q.w4a16_gemm(Ad * 2, Pd, Sd, 8, 128)
    torch.testing.assert_close(C2.float(), C.float() * 2, rtol=1e-2, atol=1e-2)


def _cfg5_column_sum_of_weights(packed, scales, zero=8, group=128):
    """sum over n of the dequantised weights W[n, k] = half(q - zero) * s[k / g, n], in float64, group by group."""
    N, K = packed.shape[0], packed.shape[1] * 2
    q = oc.unpack_uint4(packed).to(torch.float32)  # [N, K]
    wsum = torch.empty(K, dtype=torch.float64)
    for g in range(K // group):
        w = ((q[:, g * group:(g + 1) * group] - zero).half() * scales[g, :, None]).double()  # one f16 rounding, as the operator's contract says
        wsum[g * group:(g + 1) * group] = w.sum(dim=0)
    return wsum


@pytest.fixture(scope="module")
def cfg5_weights():
    _, packed, scales = oc.make_config_inputs("cfg5", M=1)
    return packed, scales, _cfg5_column_sum_of_weights(packed, scales), packed.cuda(), scales.cuda()


@pytest.mark.parametrize("M", [1, 8, 16, 64, 512, 4096])
def test_config5_whole_output_identity(cfg5_weights, M):
    """An identity every output tile takes part in, at full size: sum_n C[m, n] == A[m, :] . sum_n W[n, :].
    A tile written to the wrong place, left out or added twice (a lost or duplicated split-K hand-over) moves a
    row sum by about sqrt(128) * |C|, far outside the bar, which is the rounding of 28672 bf16 outputs."""
    q = _q()
    packed, scales, wsum, Pd, Sd = cfg5_weights
    A, _, _ = oc.make_config_inputs("cfg5", M=M)
    C = q.w4a16_gemm(A.cuda(), Pd, Sd, 8, 128)
    got = C.double().sum(dim=1).cpu()
    want = A.half().double() @ wsum  # the operator converts bf16 activations to f16 first, as the reference wrapper does
    N = packed.shape[0]
    cmax = C.float().abs().max().item()
    bar = 6.0 * (N ** 0.5) * cmax * 2.0 ** -9 + 1e-3 * want.abs().max().item()
    assert (got - want).abs().max().item() <= bar, ((got - want).abs().max().item(), bar)
    assert torch.isfinite(C.float()).all()


def test_kernels_on_either_side_of_a_switch_agree():
    """Up to 64 tokens the group scale multiplies the group's fp32 sum, above that every weight is scaled in f16
    first: the same token row through both kernels differs by at most that f16 product's rounding, 2^-11
    relative per term - far inside the operator's tolerance, and the bar here."""
    q = _q()
    M, K, N = 65, 2048, 512
    A, packed, scales = oc.make_w4a16_inputs(M, K, N, "float16", 128, seed=11)
    Ad, Pd, Sd = A.cuda(), packed.cuda(), scales.cuda()
    C65 = q.w4a16_gemm(Ad, Pd, Sd, 8, 128)                      # per-weight scale (tcgen05 kernel, 128-token tile)
    C64 = q.w4a16_gemm(Ad[:64].contiguous(), Pd, Sd, 8, 128)    # group-sum kernel, 64-token tile
    C32 = q.w4a16_gemm(Ad[:32].contiguous(), Pd, Sd, 8, 128)    # group-sum kernel, 32-token tile
    C8 = q.w4a16_gemm(Ad[:8].contiguous(), Pd, Sd, 8, 128)      # group-sum kernel, 16-token tile
    ref = oc.dequant_gemm_fp16_ref(A, packed, "float16", scales, 8, 128)
    _close(C65, ref)
    _close(C64, ref[:64])
    # the group-sum kernel does the same arithmetic per row whatever the token count and tile height ...
    assert torch.equal(C32, C64[:32])
    # ... up to the order in which the K ranges of a split tile are added in fp32 (the single-launch form of small
    # problems cuts K over a cluster, the two-launch form over the persistent grid)
    torch.testing.assert_close(C8.float(), C64[:8].float(), rtol=2e-3, atol=2e-3)
    # |sum_k a w (1 + e_k)| with |e_k| <= 2^-11: bounded by 2^-11 * sum |a w|, plus the output's own rounding
    W = oc.dequant_weight_ref(packed, scales, 8, 128).float()
    bound = (A.float().abs() @ W.abs().t()) * 2.0 ** -11 + ref.float().abs() * 2.0 ** -9 + 1e-3
    assert ((C65[:64].float() - C64.float()).abs().cpu() <= bound[:64]).all()


def test_bounded_wait_expires_cleanly_and_the_next_call_is_exact():
    """The time-out path end to end, without faulting or hanging anything: with the test hook on, one
    accumulator hand-over of the launch is never signalled, so one wait of the epilogue runs into its limit
    (20 ms here).  The kernel must return by itself with QGEMM_ST_TIMEOUT_EPILOGUE in the status word, and the
    next ordinary call on the same device must be correct."""
    q = _q()
    from tilelang_ascend_b200 import _lib
    lib = _lib.load()
    A, packed, scales = oc.make_w4a16_inputs(16, 1024, 256, "float16", 128, seed=5)
    Ad, Pd, Sd = A.cuda(), packed.cuda(), scales.cuda()
    ref = oc.dequant_gemm_fp16_ref(A, packed, "float16", scales, 8, 128)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    try:
        lib.qgemm_set_wait_limit_ms(20)
        lib.qgemm_debug_withhold_commit(1)
        q.w4a16_gemm(Ad, Pd, Sd, 8, 128, status=status)
        torch.cuda.synchronize()  # returns: the kernel gave up by itself
        assert int(status.item()) == 3  # QGEMM_ST_TIMEOUT_EPILOGUE
        with pytest.raises(q.QGemmError, match="bounded wait ran out"):
            q.w4a16_gemm(Ad, Pd, Sd, 8, 128, check_status=True)
    finally:
        lib.qgemm_debug_withhold_commit(0)
        lib.qgemm_set_wait_limit_ms(2000)
    status.zero_()
    C = q.w4a16_gemm(Ad, Pd, Sd, 8, 128, status=status)
    _close(C, ref)
    assert int(status.item()) == 0
    C2 = q.w4a16_gemm(Ad, Pd, Sd, 8, 128, check_status=True)
    assert torch.equal(C, C2)


def test_back_to_back_calls_that_feed_each_other():
    """Calls issued back to back overlap: a call's pre-pass is resident and its GEMM kernel is already streaming
    weights while the call in front still runs.  Here every call reads the previous call's output as its
    activations and all calls share one scratch area (the built-in one), so any step taken too early shows: the
    chain must be bit-identical to the same chain with the device drained between calls, and match the oracle."""
    from tilelang_ascend_b200 import _lib
    lib = _lib.load()
    M, K, layers = 16, 2048, 6
    g = torch.Generator().manual_seed(77)
    A0, _, _ = oc.make_w4a16_inputs(M, K, K, "float16", 128, seed=70)
    Ws = []
    for l in range(layers):
        _, P, S = oc.make_w4a16_inputs(M, K, K, "float16", 128, seed=71 + l)
        # keep the chain's magnitude steady: rescale so that one layer maps unit-variance rows to about unit variance
        W = oc.dequant_weight_ref(P, S, 8, 128).float()
        gain = (torch.randn(64, K, generator=g) @ W.t()).std().item()
        Ws.append((P, (S.float() / gain).to(torch.float16)))
    dev = [(P.cuda(), S.cuda()) for P, S in Ws]
    stream = torch.cuda.current_stream().cuda_stream

    def chain(drain):
        x = A0.cuda()
        outs = []
        for P, S in dev:
            C = torch.empty((M, K), dtype=torch.float16, device="cuda")
            rc = lib.qgemm_w4a16_noalloc(x.data_ptr(), P.data_ptr(), S.data_ptr(), 8, 128, C.data_ptr(), M, K, K,
                                         _lib.DT_F16, _lib.DT_F16, None, stream)
            assert rc == 0, _lib.last_error()
            if drain:
                torch.cuda.synchronize()
            outs.append(C)
            x = C
        torch.cuda.synchronize()
        return outs

    want = chain(drain=True)
    for _ in range(3):
        got = chain(drain=False)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    x = A0
    for (P, S), c in zip(Ws, want):
        ref = oc.dequant_gemm_fp16_ref(x, P, "float16", S, 8, 128)
        _close(c, ref)
        x = c.cpu()


SMALL_SHAPES = [
    # M, K, N, group, dtype, batch: clusters of 1 (K <= 1024), 2 and 4 CTAs, K beyond the form's range, ragged N, batches
    (16, 1024, 256, 128, "float16", None), (5, 512, 136, 128, "bfloat16", None), (16, 2048, 512, 128, "float16", None),
    (9, 4096, 1024, 128, "bfloat16", None), (16, 4096, 4096, 128, "float16", None), (1, 8192, 2048, 128, "float16", None),
    (16, 8192, 2304, 256, "bfloat16", None), (12, 4096, 264, 4096, "float16", None), (16, 2048, 384, 128, "float16", 3),
]


@pytest.mark.parametrize("M,K,N,group,dt,batch", SMALL_SHAPES)
def test_single_launch_form_of_small_problems(M, K, N, group, dt, batch):
    """Problems of at most four slabs per CTA run as one launch (activations prepared inside the kernel, K cut over a
    thread-block cluster whose CTAs add their sums through distributed shared memory): results against the oracle,
    one-hot rows bit for bit, the interleaved layout identical, and two runs identical."""
    q = _q()
    if batch is None:
        A, P, S = oc.make_w4a16_inputs(M, K, N, dt, group, seed=M + N)
        ref = oc.dequant_gemm_fp16_ref(A, P, dt, S, 8, group)
    else:
        parts = [oc.make_w4a16_inputs(M, K, N, dt, group, seed=40 + i) for i in range(batch)]
        A, P, S = [torch.stack([p[i] for p in parts]) for i in range(3)]
        ref = torch.stack([oc.dequant_gemm_fp16_ref(*p[:2], dt, p[2], 8, group) for p in parts])
    C = q.w4a16_gemm(A.cuda(), P.cuda(), S.cuda(), 8, group)
    _close(C, ref)
    assert torch.equal(C, q.w4a16_gemm(A.cuda(), P.cuda(), S.cuda(), 8, group))
    if batch is None:
        Pi = q.interleave_weight(P, 4, "float16").view(torch.uint8)
        assert torch.equal(C, q.w4a16_gemm(A.cuda(), Pi.cuda(), S.cuda(), 8, group, weight_layout="interleaved"))
        W = oc.dequant_weight_ref(P, S, 8, group)
        for k0 in (0, K // 2 - 3, K - M):
            hot = torch.zeros((M, K), dtype=A.dtype)
            hot[torch.arange(M), k0 + torch.arange(M)] = 1
            Wt = q.w4a16_gemm(hot.cuda(), P.cuda(), S.cuda(), 8, group, out_dtype=torch.float16)
            assert torch.equal(Wt.cpu(), W[:, k0:k0 + M].t().contiguous())


def test_single_launch_form_gives_up_cleanly_when_a_cluster_signal_is_missing():
    """The bounded wait of the single-launch form, made to expire in the safe way: with the test hook at 2, CTA 1 of
    the last cluster writes its sums but keeps its signal back, so the first CTA's wait runs into the limit (20 ms).
    The kernel must return by itself with QGEMM_ST_TIMEOUT_EPILOGUE, and the next ordinary call must be exact."""
    q = _q()
    from tilelang_ascend_b200 import _lib
    lib = _lib.load()
    A, packed, scales = oc.make_w4a16_inputs(16, 4096, 512, "float16", 128, seed=9)  # four clusters of four CTAs
    Ad, Pd, Sd = A.cuda(), packed.cuda(), scales.cuda()
    ref = oc.dequant_gemm_fp16_ref(A, packed, "float16", scales, 8, 128)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    try:
        lib.qgemm_set_wait_limit_ms(20)
        lib.qgemm_debug_withhold_commit(2)
        C_bad = q.w4a16_gemm(Ad, Pd, Sd, 8, 128, status=status)
        torch.cuda.synchronize()  # returns: the kernel gave up by itself
        assert int(status.item()) == 3  # QGEMM_ST_TIMEOUT_EPILOGUE
        # the clusters whose signals all arrived wrote their tiles
        _close(C_bad[:, :384], ref[:, :384])
    finally:
        lib.qgemm_debug_withhold_commit(0)
        lib.qgemm_set_wait_limit_ms(2000)
    status.zero_()
    C = q.w4a16_gemm(Ad, Pd, Sd, 8, 128, status=status)
    _close(C, ref)
    assert int(status.item()) == 0
