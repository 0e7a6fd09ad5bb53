"""GPU parity of the other weight formats of tilelang/quantize through the C ABI (qgemm_w4a16_ex):
interleaved nibble layout, per-(group, feature) zero points and the three zero modes."""
import pytest
import torch

import tilelang_ascend_b200 as q
from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu


def _close(C, ref):
    torch.testing.assert_close(C.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,K,N,dt,group", [(1, 256, 128, "float16", 128), (8, 512, 272, "bfloat16", 64),
                                            (16, 1024, 528, "float16", 128), (40, 512, 144, "bfloat16", 32),
                                            (200, 768, 256, "float16", 256)])
def test_interleaved_layout_gives_identical_results(M, K, N, dt, group):
    """The same weights in the interleaved layout: bit-identical output on every kernel (decode, tcgen05)."""
    A, P, S = oc.make_w4a16_inputs(M, K, N, dt, group, seed=M)
    Pi = q.interleave_weight(P, 4, "float16").view(torch.uint8)
    assert torch.equal(Pi, oc.interleave_int4_f16_ref(P))
    C = q.w4a16_gemm(A.cuda(), P.cuda(), S.cuda(), 8, group)
    Ci = q.w4a16_gemm(A.cuda(), Pi.cuda(), S.cuda(), 8, group, weight_layout="interleaved")
    assert torch.equal(C, Ci)
    _close(Ci, oc.dequant_gemm_fp16_ref(A, P, dt, S, 8, group))


@pytest.mark.parametrize("mode", ["original", "rescale", "quantized"])
@pytest.mark.parametrize("M,K,N,group", [(1, 256, 144, 128), (24, 512, 272, 64), (130, 768, 528, 256)])
def test_zero_modes_exact_dequantisation_and_gemm(mode, M, K, N, group):
    g = torch.Generator().manual_seed(K + N)
    A, P, S = oc.make_w4a16_inputs(M, K, N, "float16", group, seed=K)
    if mode == "quantized":
        zeros = torch.randint(0, 16, (K // group, N), generator=g).to(torch.float16)
    else:
        zeros = (torch.rand((K // group, N), generator=g) * 6 + 5).to(torch.float16)
        if mode == "rescale":
            zeros = zeros * S  # rescale-mode zeros live in scaled units
    W = oc.dequant_weight_zeros_ref(P, S, zeros, group, mode)
    # unit activations read the dequantised weights back bit for bit
    eye = torch.eye(K, dtype=torch.float16)
    Wt = q.w4a16_gemm(eye.cuda(), P.cuda(), S.cuda(), zeros.cuda(), group, zeros_mode=mode)
    assert torch.equal(Wt.cpu().t().contiguous(), W)
    C = q.w4a16_gemm(A.cuda(), P.cuda(), S.cuda(), zeros.cuda(), group, zeros_mode=mode)
    ref = (A.float() @ W.float().t()).to(torch.float16)
    _close(C, ref)
    # interleaved layout with a zeros tensor
    Pi = q.interleave_weight(P, 4, "float16").view(torch.uint8)
    Ci = q.w4a16_gemm(A.cuda(), Pi.cuda(), S.cuda(), zeros.cuda(), group, zeros_mode=mode, weight_layout="interleaved")
    _close(Ci, ref)


@pytest.mark.parametrize("M,K,N,group,dt", [(1, 256, 144, 128, "float16"), (16, 1024, 528, 128, "bfloat16"),
                                            (24, 1024, 272, 256, "float16"), (40, 2048, 1040, 128, "float16"),
                                            (64, 1024, 264 + 8, 1024, "bfloat16"), (16, 8192, 4096, 128, "float16")])
def test_integer_zeros_in_flight_up_to_64_tokens(M, K, N, group, dt):
    """Zero mode "quantized" with up to 64 tokens and groups of 128, a multiple of 256 or the whole K stays on the
    streaming kernel (no dequantised copy of the weights): one-hot rows read (q - qz) * s back bit for bit, results
    match the oracle, the interleaved layout gives the same bits, and the whole-matrix path agrees within the
    operator's tolerance."""
    g = torch.Generator().manual_seed(M + K + N)
    A, P, S = oc.make_w4a16_inputs(M, K, N, dt, group, seed=K + M)
    zeros = torch.randint(0, 16, (K // group, N), generator=g).to(torch.float16)
    W = oc.dequant_weight_zeros_ref(P, S, zeros, group, "quantized")
    Pd, Sd, Zd = P.cuda(), S.cuda(), zeros.cuda()
    for k0 in (0, K // 2 - 8, K - M):
        hot = torch.zeros((M, K), dtype=A.dtype)
        hot[torch.arange(M), k0 + torch.arange(M)] = 1
        Wt = q.w4a16_gemm(hot.cuda(), Pd, Sd, Zd, group, zeros_mode="quantized", out_dtype=torch.float16)
        assert torch.equal(Wt.cpu(), W[:, k0:k0 + M].t().contiguous())
    C = q.w4a16_gemm(A.cuda(), Pd, Sd, Zd, group, zeros_mode="quantized")
    ref = (A.float() @ W.float().t()).to(A.dtype)
    _close(C, ref)
    Pi = q.interleave_weight(P, 4, "float16").view(torch.uint8)
    Ci = q.w4a16_gemm(A.cuda(), Pi.cuda(), Sd, Zd, group, zeros_mode="quantized", weight_layout="interleaved")
    assert torch.equal(C, Ci)
    C65 = q.w4a16_gemm(torch.cat([A, A[:1].expand(65 - M, K)]).cuda(), Pd, Sd, Zd, group, zeros_mode="quantized")
    _close(C65[:M], ref)


def test_integer_zero_tensor_equals_scalar_zero():
    A, P, S = oc.make_w4a16_inputs(32, 512, 256, "bfloat16", 128, seed=4)
    zeros = torch.full((4, 256), 8.0, dtype=torch.float16)
    C0 = q.w4a16_gemm(A.cuda(), P.cuda(), S.cuda(), 8, 128)
    C1 = q.w4a16_gemm(A.cuda(), P.cuda(), S.cuda(), zeros.cuda(), 128, zeros_mode="quantized")
    assert torch.equal(C1, C0)  # both on the streaming kernel: the same arithmetic


def test_quantiser_round_trip_through_the_operator():
    """quantize_int4_groupwise -> pack -> operator equals the dequantised-weight GEMM."""
    g = torch.Generator().manual_seed(0)
    K, N, group = 512, 256, 128
    w = torch.randn((K, N), generator=g).half()
    qv, s = q.quantize_int4_groupwise(w, group)
    P = q.pack_int4(qv.t().contiguous())          # [N, K/2]
    A = torch.randn((16, K), generator=g).half()
    C = q.w4a16_gemm(A.cuda(), P.cuda(), s.cuda(), 8, group)
    Wd = oc.dequant_weight_ref(P, s, 8, group)
    _close(C, (A.float() @ Wd.float().t()).half())
    # half a step everywhere, one step for each group's largest element (16 does not fit a nibble: clamped to 15)
    assert (Wd.float().t() - w.float()).abs().max() <= s.float().max() + 1e-3


def test_rejects():
    A, P, S = [t.cuda() for t in oc.make_w4a16_inputs(8, 256, 128, "float16", 128, seed=1)]
    with pytest.raises(ValueError):
        q.w4a16_gemm(A, P, S, 8, 128, zeros_mode="rescale")          # needs a zeros tensor
    with pytest.raises(ValueError):
        q.w4a16_gemm(A, P, S, 8, 128, weight_layout="ladder")
    with pytest.raises(ValueError):
        q.w4a16_gemm(A, P, None, torch.zeros(2, 128, dtype=torch.float16, device="cuda"))
    A2, P2, S2 = [t.cuda() for t in oc.make_w4a16_inputs(8, 256, 136, "float16", 128, seed=1)]
    with pytest.raises(q.QGemmError):
        q.w4a16_gemm(A2, P2, S2, torch.zeros(2, 136, dtype=torch.float16, device="cuda"), 128)  # N % 16 != 0
