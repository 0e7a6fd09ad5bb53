"""CPU tests (gloo, world_size 2) of the multi-GPU host logic: batch sharding of the batched W8A8 operator
and column sharding + all-gather of the W4A16 operator.  The GEMM itself is replaced by the CPU oracle
here; on GPUs the same code path calls the CUDA kernels and NCCL."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import qgemm_oracle as oc
from tilelang_ascend_b200.dist import ColumnShardedW4A16, GroupShardedW8A8, shard_batches, shard_groups, shard_range


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_gemm(A, P, S, zero, group):
    return oc.dequant_gemm_fp16_ref(A, P, A.dtype, S, zero, group)


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _worker_column_shard(rank, world, port, q):
    try:
        _init(rank, world, port)
        M, K, N = 5, 256, 512
        A, P, S = oc.make_w4a16_inputs(M, K, N, "float16", 128, seed=3)  # same seed on every rank
        layer = ColumnShardedW4A16(P, S, 8, 128, gemm=_cpu_gemm)
        assert layer.B_local.shape == (N // world, K // 2) and layer.s_local.shape == (K // 128, N // world)
        out = layer(A)
        ref = oc.dequant_gemm_fp16_ref(A, P, "float16", S, 8, 128)
        local = layer.forward(A, gather=False)
        ok = torch.equal(out, ref) and torch.equal(local, ref[:, layer.n0:layer.n1])
        q.put((rank, bool(ok), ""))
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        q.put((rank, False, repr(exc)))


def _worker_batch_shard(rank, world, port, q):
    try:
        _init(rank, world, port)
        A, B, sa, sb = oc.make_w8a8_inputs(6, 40, 64, 48, seed=1)
        Al, Bl, sal, sbl = shard_batches([A, B, sa, sb], world, rank)
        out_local = oc.quant_matmul_ref(Al, Bl, sbl, "bfloat16", scale_a=sal)
        parts = [torch.empty_like(out_local) for _ in range(world)]
        dist.all_gather(parts, out_local)  # only for the check: the data path itself has no collective
        ref = oc.quant_matmul_ref(A, B, sb, "bfloat16", scale_a=sa)
        q.put((rank, bool(torch.equal(torch.cat(parts, 0), ref)), ""))
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        q.put((rank, False, repr(exc)))


def _worker_peer_leaves(rank, world, port, q):
    """Rank 1 leaves between steps; rank 0's next collective must end with an error, not hang."""
    try:
        _init(rank, world, port, timeout_s=8)
        t = torch.ones(4)
        dist.all_reduce(t)  # step 1: everybody present
        if rank == 1:
            q.put((rank, True, "left"))
            q.close()
            q.join_thread()  # make sure the message is out before the process disappears
            os._exit(0)
        try:
            dist.all_reduce(t)  # step 2: the peer is gone
            dist.all_reduce(t)
            q.put((rank, False, "collective succeeded without its peer"))
        except Exception as exc:
            q.put((rank, True, type(exc).__name__))
    except Exception as exc:  # pragma: no cover
        q.put((rank, False, repr(exc)))


def _cpu_grouped(A, B, meta, scale, scale_a=None, out_dtype=torch.bfloat16):
    return oc.grouped_quant_matmul_ref(A, B, meta, scale, out_dtype, scale_a=scale_a)


def _cpu_meta(sizes, block_M, device=None):
    return oc.build_block_metadata_ref(sizes, block_M)


def _worker_group_shard(rank, world, port, q):
    try:
        _init(rank, world, port)
        sizes, K, N = [63, 0, 140, 77, 5], 64, 48
        g = torch.Generator().manual_seed(8)  # same seed on every rank
        A = torch.randint(-128, 128, (sum(sizes), K), dtype=torch.int8, generator=g)
        B = torch.randint(-128, 128, (len(sizes), K, N), dtype=torch.int8, generator=g)
        sb = torch.rand((len(sizes), N), generator=g) * 0.02 + 0.001
        sa = torch.rand(sum(sizes), generator=g) * 0.02 + 0.001
        layer = GroupShardedW8A8(sizes, B, sb, out_dtype=torch.bfloat16, gemm=_cpu_grouped, metadata=_cpu_meta)
        r0, r1 = layer.row0, layer.row1
        full = layer(A[r0:r1], sa[r0:r1], gather=True)
        ref = oc.grouped_quant_matmul_ref(A, B, oc.build_block_metadata_ref(sizes, 128), sb, torch.bfloat16, scale_a=sa)
        local = layer(A[r0:r1], sa[r0:r1])
        ok = torch.equal(full, ref) and torch.equal(local, ref[r0:r1]) and layer.B_local.shape[0] == layer.g1 - layer.g0
        q.put((rank, bool(ok), ""))
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        q.put((rank, False, repr(exc)))


def _run(worker, world=2, timeout=120):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=timeout) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    return sorted(results)


def test_shard_range_properties():
    for total, world, mult in [(16, 8, 1), (16, 3, 1), (28672, 8, 128), (28672, 5, 128), (7, 8, 1)]:
        spans = [shard_range(total, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a0 <= a1
        assert all((b - a) % mult == 0 for a, b in spans)
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= mult
    with pytest.raises(ValueError):
        shard_range(100, 4, 0, 128)


def test_single_process_layer_equals_oracle():
    A, P, S = oc.make_w4a16_inputs(3, 128, 256, "bfloat16", 128, seed=0)
    layer = ColumnShardedW4A16(P, S, 8, 128, gemm=_cpu_gemm)
    assert torch.equal(layer(A), oc.dequant_gemm_fp16_ref(A, P, "bfloat16", S, 8, 128))


def test_column_sharded_w4a16_two_ranks():
    res = _run(_worker_column_shard)
    assert all(ok for _, ok, _ in res), res


def test_batch_sharded_w8a8_two_ranks():
    res = _run(_worker_batch_shard)
    assert all(ok for _, ok, _ in res), res


def test_peer_leaving_between_steps_gives_an_error():
    res = _run(_worker_peer_leaves)
    assert all(ok for _, ok, _ in res), res


def test_shard_groups_covers_all_rows():
    sizes = [63, 0, 140, 77, 5, 300, 12]
    for world in (1, 2, 3, 8):
        spans = [shard_groups(sizes, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[0][2] == 0 and spans[-1][1] == len(sizes) and spans[-1][3] == sum(sizes)
        for a, b in zip(spans, spans[1:]):
            assert a[1] == b[0] and a[3] == b[2]
        for g0, g1, r0, r1 in spans:
            assert r1 - r0 == sum(sizes[g0:g1])


def test_group_sharded_w8a8_two_ranks():
    res = _run(_worker_group_shard)
    assert all(ok for _, ok, _ in res), res


def test_column_sharded_layer_argument_checks():
    """Host-side validation: the form of the "landed" signal must be one of the two known ones, layers that share
    output buffers must have the same output width, and on CPU tensors the layer falls back to the collective form."""
    _, P, S = oc.make_w4a16_inputs(1, 256, 256, "float16", 128, seed=3)
    with pytest.raises(ValueError, match="landed"):
        ColumnShardedW4A16(P, S, 8, 128, gemm=_cpu_gemm, landed="carrier pigeon")
    a = ColumnShardedW4A16(P, S, 8, 128, gemm=_cpu_gemm)
    _, P2, S2 = oc.make_w4a16_inputs(1, 256, 384, "float16", 128, seed=4)
    with pytest.raises(ValueError, match="same N"):
        ColumnShardedW4A16(P2, S2, 8, 128, gemm=_cpu_gemm, share_buffers_with=a)
    A, _, _ = oc.make_w4a16_inputs(4, 256, 256, "float16", 128, seed=5)
    assert not a._use_peers(A)  # CPU tensors, custom GEMM: never the peer-store form
    assert a.forward(A).shape == (4, 256)
