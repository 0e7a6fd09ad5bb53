"""Seeded random shapes through every operator against the CPU oracle: ragged M, N and K at the kernels' granularity,
every scale-group width, both activation types, both weight layouts, scalar and per-group zero points - shapes nobody
picked by hand, so that tile edges, split-K segment boundaries and kernel-selection thresholds are hit where they fall.
The case lists are fixed by the seeds below (same cases on every run)."""
import random

import pytest
import torch

import tilelang_ascend_b200 as q
from oracle import qgemm_oracle as oc

pytestmark = pytest.mark.gpu


def _w4a16_cases(n, seed):
    rnd = random.Random(seed)
    cases = []
    for i in range(n):
        M = rnd.choice([1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 48, 63, 64, 65, 100, 128, 129, 200, 257, 300])
        group = rnd.choice([32, 64, 128, 128, 128, 256, -1])
        gk = 256 if group == -1 else max(group, 32)
        K = gk * rnd.randint(1, 24 if M <= 64 else 8)
        if group == 256 and K % 256:
            K += 256 - K % 256
        N = 8 * rnd.randint(1, 160)
        dt = rnd.choice(["float16", "bfloat16"])
        layout = rnd.choice(["sequential", "sequential", "interleaved"])
        zeros = rnd.choice(["scalar", "scalar", "tensor"])
        if zeros == "tensor":
            N = max(16, N - N % 16)
        cases.append((i, M, K, N, group, dt, layout, zeros))
    return cases


@pytest.mark.parametrize("i,M,K,N,group,dt,layout,zeros", _w4a16_cases(60, 20240))
def test_w4a16_random_shape(i, M, K, N, group, dt, layout, zeros):
    g = K if group == -1 else group
    A, P, S = oc.make_w4a16_inputs(M, K, N, dt, g, seed=1000 + i)
    Pd = P
    if layout == "interleaved":
        Pd = q.interleave_weight(P, 4, "float16").view(torch.uint8)
    if zeros == "tensor":
        Z = torch.randint(0, 16, (K // g, N), generator=torch.Generator().manual_seed(i)).to(torch.float16)
        W = oc.dequant_weight_zeros_ref(P, S, Z, g, "quantized")
        ref = (A.float() @ W.float().t()).to(A.dtype)
        C = q.w4a16_gemm(A.cuda(), Pd.cuda(), S.cuda(), Z.cuda(), group, zeros_mode="quantized", weight_layout=layout)
    else:
        zero = (i % 16)
        ref = oc.dequant_gemm_fp16_ref(A, P, dt, S, zero, g)
        C = q.w4a16_gemm(A.cuda(), Pd.cuda(), S.cuda(), zero, group, weight_layout=layout)
    assert C.shape == (M, N) and C.dtype == A.dtype
    torch.testing.assert_close(C.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)


def _w8a8_cases(n, seed):
    rnd = random.Random(seed)
    cases = []
    for i in range(n):
        batch = rnd.choice([1, 1, 2, 3, 5])
        M = rnd.choice([1, 17, 100, 128, 129, 255, 256, 300, 513, 1000])
        K = 16 * rnd.randint(1, 96)
        N = 16 * rnd.randint(1, 80)
        layout = rnd.choice(["KN", "KN", "NK"])
        odt = rnd.choice(["float16", "bfloat16"])
        cases.append((i, batch, M, K, N, layout, odt))
    return cases


@pytest.mark.parametrize("i,batch,M,K,N,layout,odt", _w8a8_cases(30, 777))
def test_w8a8_random_shape_bit_exact(i, batch, M, K, N, layout, odt):
    A, B, sa, sb = oc.make_w8a8_inputs(batch, M, K, N, seed=2000 + i)
    ref, acc_ref = oc.quant_matmul_ref(A, B, sb, odt, scale_a=sa, return_acc=True)
    Bd = B.transpose(1, 2).contiguous() if layout == "NK" else B
    C, acc = q.quant_matmul(A.cuda(), Bd.cuda(), sb.cuda(), scale_a=sa.cuda(), out_dtype=odt, b_layout=layout,
                            return_accumulators=True)
    assert torch.equal(acc.cpu(), acc_ref)
    assert torch.equal(C.cpu(), ref)


def _w4a8_cases(n, seed):
    rnd = random.Random(seed)
    return [(i, rnd.choice([1, 5, 16, 33, 64, 100, 128, 130, 260]), 32 * rnd.randint(8, 64), 16 * rnd.randint(8, 80))
            for i in range(n)]


@pytest.mark.parametrize("i,M,K,N", _w4a8_cases(16, 99))
def test_w4a8_random_shape_exact(i, M, K, N):
    g = torch.Generator().manual_seed(3000 + i)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=g)
    qB = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    ref = oc.w4a8_gemm_ref(A, qB)
    ws = torch.empty((N, K), dtype=torch.int8, device="cuda")
    C = torch.empty((M, N), dtype=torch.int32, device="cuda")
    q.w4a8_gemm_cv(M, N, K)(A.cuda(), qB.cuda(), ws, C)
    assert torch.equal(C.cpu(), ref)
