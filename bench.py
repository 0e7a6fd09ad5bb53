#!/usr/bin/env python
"""Benchmark of the quantized-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-suite]
    python bench.py --case cfg5 --m 8 --launches 3      # a few launches of one configuration, for ncu

Headline workload (N = 1): BASELINE config[1], the W4A16 decode GEMM M=16, K=4096, N=4096, group 128,
zero point 8, fp16.  One problem is only 8.9 MB, far below the L2 size, so a *step* is one pass over
LAYERS = 32 distinct weight sets of that shape (285 MB > L2), issued as one batched call (one small
activation pre-pass and one GEMM launch, replayed from a CUDA graph); the same work issued as 32 separate
calls is timed too and reported under `per_layer_launch`.  `value` is algorithmic bytes (each input read once, output written once) over device time, GB/s,
whole job over all ranks.  With N > 1 the headline config does not shard ("replicas only"): every rank
runs its own replica (weak scaling).  The sharded configurations (config 4 by batch, config 5 by weight
columns with an all-gather of outputs) and the other single-GPU configurations are measured in the same
run and reported under `suite`.

`--impl reference` times the reference's torch CPU program for this path (the restatement in oracle/,
all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

LAYERS = 32
KERNELS_PER_LAYER = 2  # activation pre-pass + GEMM
CFG2 = dict(M=16, K=4096, N=4096, group=128)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the committed ncu
# summary under profiles/.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 293437952  # profiles/w4a16_gs_cfg2_headline.md (284.0 MB read + 9.5 MB written)


def w4a16_bytes(M, K, N, group, out_bytes=2, a_bytes=2):
    return K * N // 2 + 2 * (K // group) * N + a_bytes * M * K + out_bytes * M * N


def w8a8_bytes(batch, M, K, N, out_bytes=2):
    return batch * (M * K + K * N + 4 * M + 4 * N + out_bytes * M * N)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {}
        for n in dir(nv):
            if n.startswith("nvmlClocksEventReason") or n.startswith("nvmlClocksThrottleReason"):
                v = getattr(nv, n)
                if isinstance(v, int) and v not in (0,):
                    names.setdefault(v, n.replace("nvmlClocksEventReason", "").replace("nvmlClocksThrottleReason", ""))
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                if get_reasons is not None:
                    r = get_reasons(self.h)
                    for bit, name in names.items():
                        if r & bit and bit & (bit - 1) == 0 and name not in ("GpuIdle", "All", "None"):
                            self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        # NCCL's own log lines (version banner, NCCL_DEBUG output) must not land on stdout, which carries the JSON line
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms, world):
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed(fn_step, steps, warmup, world, fn_k_steps=None, graph_events=None):
    """W untimed steps, then exactly K steps between barrier + synchronize, CUDA events, max over ranks.
    `fn_k_steps`, when given, issues all K steps at once (one CUDA graph holding K steps); `graph_events` are the two
    timing events recorded inside that graph, in front of the first step and behind the last one, so that the host's
    latency of launching the graph is not counted as device time of the steps."""
    for _ in range(warmup):
        fn_step()
    if fn_k_steps is not None:
        fn_k_steps()  # untimed: the first replay of a graph uploads it to the device
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if fn_k_steps is not None:
        fn_k_steps()
    else:
        for _ in range(steps):
            fn_step()
    e1.record()
    barrier(world)
    ms = e0.elapsed_time(e1)
    if fn_k_steps is not None and graph_events is not None:
        try:
            inner = graph_events[0].elapsed_time(graph_events[1])
            if 0.0 < inner <= ms:
                ms = inner
        except Exception as exc:  # pragma: no cover - depends on driver support for event nodes with timing
            sys.stderr.write(f"[bench] events inside the graph could not be read ({exc}); using the outer events\n")
    return max_over_ranks(ms, world)


def make_graph_step(launch_all, stream, repeat=1, events=None):
    """Capture `repeat` steps (all their launches) in a CUDA graph on `stream`; fall back to eager launches.
    `events`: two external timing events to record inside the graph, around the steps."""
    try:
        with torch.cuda.stream(stream):
            launch_all()  # warm: the library is loaded and set up before capture
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            if events is not None:
                events[0].record(stream)
            for _ in range(repeat):
                launch_all()
            if events is not None:
                events[1].record(stream)
        return (lambda: g.replay()), "cuda_graph"
    except Exception as exc:  # pragma: no cover - depends on driver behaviour
        sys.stderr.write(f"[bench] CUDA graph capture failed ({exc}); timing eager launches\n")

        def eager():
            for _ in range(repeat):
                launch_all()
        return eager, "eager"


# ----------------------------------------------------------------------------------------- our arm
def headline_inputs(seed0):
    from oracle import qgemm_oracle as oc  # input generator only (shared with the tests)
    layers = []
    for l in range(LAYERS):
        A, P, S = oc.make_w4a16_inputs(CFG2["M"], CFG2["K"], CFG2["N"], "float16", CFG2["group"], seed=seed0 + l)
        layers.append((A.pin_memory(), P.pin_memory(), S.pin_memory()))
    return layers


def run_ours(args):
    import tilelang_ascend_b200 as q

    world, rank, local = dist_setup(args.gpus)
    peaks, peaks_src = load_peaks()
    host_layers = headline_inputs(1000 * rank)
    dev_layers = [tuple(t.cuda(non_blocking=True) for t in lay) for lay in host_layers]
    torch.cuda.synchronize()
    outs = [None] * LAYERS
    # The step's 32 weight sets as one batched problem: [32, M, K], [32, N, K/2], [32, K/g, N].
    Ab = torch.stack([l[0] for l in dev_layers]).contiguous()
    Pb = torch.stack([l[1] for l in dev_layers]).contiguous()
    Sb = torch.stack([l[2] for l in dev_layers]).contiguous()
    batched_out = [None]

    def launch_batched():
        batched_out[0] = q.w4a16_gemm(Ab, Pb, Sb, 8, CFG2["group"])

    def launch_all():
        for i, (A, P, S) in enumerate(dev_layers):
            outs[i] = q.w4a16_gemm(A, P, S, 8, CFG2["group"])

    stream = torch.cuda.Stream()
    step, launch_mode = make_graph_step(launch_batched, stream)
    try:  # timing events that live inside the K-step graph (event-record nodes)
        inner_events = (torch.cuda.Event(enable_timing=True, external=True), torch.cuda.Event(enable_timing=True, external=True))
    except TypeError:  # pragma: no cover - older torch
        inner_events = None
    k_steps, k_mode = make_graph_step(launch_batched, stream, repeat=args.steps, events=inner_events)  # the timed region: K steps, one graph
    if k_mode != "cuda_graph":
        inner_events = None
    step_single, _ = make_graph_step(launch_all, stream)
    bytes_step = LAYERS * w4a16_bytes(**CFG2)
    with torch.cuda.stream(stream):
        with ClockSampler(local) as clk:
            ms = timed(step, args.steps, args.warmup, world, fn_k_steps=k_steps, graph_events=inner_events)
            # keep the sampler fed with the same work for a little longer: the timed region is short
            t_end = time.time() + 0.25
            while time.time() < t_end:
                step()
            torch.cuda.synchronize()
        ms_single = timed(step_single, args.steps, args.warmup, world)
    value = world * bytes_step * args.steps / (ms * 1e-3) / 1e9
    ms_per_step = ms / args.steps
    launch_us = ms_per_step * 1e3  # one batched GEMM launch (plus its activation pre-pass) per step
    achieved = bytes_step / (launch_us * 1e-6) / 1e9
    per_layer = {"what": "the same 32 weight sets as 32 separate calls (one launch each: the single-launch form of small problems)",
                 "ms_per_step": round(ms_single / args.steps, 5),
                 "value": round(world * bytes_step * args.steps / (ms_single * 1e-3) / 1e9, 2), "unit": "GB/s",
                 "us_per_call": round(ms_single / args.steps * 1e3 / LAYERS, 3)}

    # end to end through the reference-facing wrapper: host tensors in, host tensor out, every step
    wrapper = q.dequant_gemm_fp16_wrapper(CFG2["M"], CFG2["N"], CFG2["K"], 128, 256, 64, "float16", "float16")

    def e2e_step():
        for (A, P, S) in host_layers:
            wrapper(A, P, S, 8, CFG2["group"])

    e2e_steps = max(1, min(args.steps, 5))
    e2e_ms = timed(e2e_step, e2e_steps, 1, world)
    h2d = LAYERS * sum(t.numel() * t.element_size() for t in host_layers[0])
    d2h = LAYERS * CFG2["M"] * CFG2["N"] * 2
    e2e_value = world * bytes_step * e2e_steps / (e2e_ms * 1e-3) / 1e9

    suite = None
    if not args.no_suite:
        suite = run_suite(q, world, rank, peaks)

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base = cpu_baseline(sample_seconds=12.0)

    if rank == 0:
        line = {
            "metric": "w4a16_decode_gbs", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 (int4 weights, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": "BASELINE configs[1]: W4A16 dequantize_gemm decode M=16 K=4096 N=4096 group=128 zero=8 fp16; "
                                   f"one step = {LAYERS} distinct weight sets ({LAYERS * 8.9:.0f} MB > L2, so no L2 flush needed), "
                                   "issued as ONE batched call w4a16_gemm(A[32,M,K], B_packed[32,N,K/2], scales[32,K/g,N])",
                       "layers_per_step": LAYERS, "launch": launch_mode + " (the K timed steps are one graph" + (", timed by two events recorded inside it" if inner_events is not None else "") + ")",
                       "multi_gpu": "replicas only for this config; sharded configs are under suite"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                         "kernel": "w4a16_gs_kernel<16,f16>, batch 32 (time includes its w4a16_prepare_activations pre-pass)",
                         "us_per_launch": round(launch_us, 3),
                         "algorithmic_bytes_per_launch": bytes_step, "peak_source": peaks_src + " (copy)"},
            "per_layer_launch": per_layer,
            "e2e": {"value": round(e2e_value, 3), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "dequant_gemm_fp16_wrapper(CPU tensors) -> CPU tensor"},
            "gpu_launches": world * KERNELS_PER_LAYER * args.steps,
            "clocks": clk.summary(),
        }
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        if suite is not None:
            by_key = {e["key"]: e for e in suite if "key" in e}
            if "cfg3" in by_key:  # the metric's first half: W8A8 prefill TOPS against the int8 tensor roofline
                c3 = by_key["cfg3"]
                line["w8a8_prefill"] = {
                    "config": "BASELINE configs[2]: W8A8 M=4096 K=4096 N=14336, per-token and per-channel fp32 scales, bf16 out",
                    "tops": c3["tops"], "us_per_launch": round(c3["ms"] * 1e3, 2),
                    "kernel": "w8a8_gemm_kernel<256, [K,N] B, bf16> (tcgen05 kind::i8)",
                    "roofline": {"bound": "tensor", "achieved": c3["tops"], "peak": round(2 * peaks["bf16_tflops"], 1),
                                 "unit": "TOP/s", "frac": c3["frac_of_2x_measured_bf16"],
                                 "peak_source": "2 x measured bf16 burst (no measured int8 figure is provided)"},
                    "int8_yardstick": _int8_yardstick(),
                    "timing": "median of 5 CUDA-graph replays of 10 launches"}
            # the sharded configurations in one compact table: [ms] per configuration at this rank count
            line["sharded"] = {"n_gpus": world,
                               "cfg4_batch_sharded_ms": by_key["cfg4"]["ms"], "cfg4_tops": by_key["cfg4"]["tops"],
                               "cfg5_column_sharded_ms": {k[6:]: [by_key[k]["ms_compute"], by_key[k]["ms_gathered"]]
                                                          for k in by_key if k.startswith("cfg5_m")},
                               "cfg5_columns": "[compute only, with the output gathered on every rank]",
                               "cfg5_gather": next(by_key[k]["gather"] for k in by_key if k.startswith("cfg5_m")),
                               "checked_against_oracle": world > 1}
            line["suite"] = suite
        emit(line)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


L2_BYTES = 126 * 1024 * 1024


def _time_rotating(fn_of_idx, n_sets, iters, world, repeats=5):
    """Device time per launch: `iters` launches that cycle over `n_sets` input sets are captured in one CUDA graph
    (collectives included) on a side stream, the graph is replayed `repeats` times between barriers, each replay
    timed with CUDA events, max over ranks; the median of the repeats is returned.  Falls back to eager launches
    when capture is not possible."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(min(3, max(n_sets, 2))):  # warm-up: workspaces, peer buffers, NCCL channels exist before capture
            fn_of_idx(i % n_sets)
        stream.synchronize()
        barrier(world)
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(iters):
                    fn_of_idx(i % n_sets)
            run = g.replay
        except Exception as exc:  # pragma: no cover - depends on driver / NCCL behaviour
            sys.stderr.write(f"[bench] CUDA graph capture failed ({exc}); timing eager launches\n")
            torch.cuda.synchronize()

            def run():
                for i in range(iters):
                    fn_of_idx(i % n_sets)
        run()
        stream.synchronize()
        samples = []
        for _ in range(repeats):
            barrier(world)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            run()
            e1.record(stream)
            stream.synchronize()
            barrier(world)
            samples.append(max_over_ranks(e0.elapsed_time(e1), world) / iters)
    return statistics.median(samples)


def _int8_yardstick():
    """cuBLASLt's plain int8 GEMM (torch._int_mm, 8192^3) on this GPU, in the same run: a yardstick beside the
    2 x measured-bf16 denominator, not a target of its own.  Burst = best of 10, sustained = a loop of about 1 s."""
    try:
        n = 8192
        a = torch.randint(-128, 127, (n, n), dtype=torch.int8, device="cuda")
        b = torch.randint(-128, 127, (n, n), dtype=torch.int8, device="cuda")
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(1000.0 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        ops = 2.0 * n ** 3
        return {"what": "torch._int_mm 8192^3 (cuBLASLt int8), same run", "burst_tops": round(ops / best / 1e9, 1),
                "sustained_tops": round(ops * reps / e0.elapsed_time(e1) / 1e9, 1)}
    except Exception as exc:  # pragma: no cover
        return {"unavailable": repr(exc)[:120]}


def _fail(msg):
    sys.stderr.write("[bench] PARITY FAILURE: " + msg + "\n")
    raise SystemExit(3)


def run_suite(q, world, rank, peaks):
    """The other BASELINE configurations, sharded where they shard.  Device-resident inputs, CUDA events, max over
    ranks, launches replayed from CUDA graphs, median of 5 repeats; inputs either exceed L2 or rotate over enough
    copies to exceed it.  With more than one rank every sharded configuration is first checked against the CPU
    oracle on a band of its output (exit code 3 on a mismatch)."""
    from oracle import qgemm_oracle as oc  # input generators, and the checker of the sharded outputs
    from tilelang_ascend_b200.dist import ColumnShardedW4A16, shard_batches, shard_range
    int8_peak = 2 * peaks["bf16_tflops"]  # denominator: 2x the measured bf16 burst; the int8 yardstick is reported beside it
    res = []

    if world == 1:
        A, B, sa, sb = [t.cuda() for t in oc.make_config_inputs("cfg1")]
        ms = _time_rotating(lambda i: q.quant_matmul(A, B, sb, scale_a=sa, out_dtype="float16"), 1, 50, world)
        ops = 2 * 256 * 1024 * 1024
        res.append({"config": "cfg1 W8A8 1x256x1024x1024 fp16 (L2-warm, latency-bound)", "ms": round(ms, 5),
                    "tops": round(ops / ms / 1e9, 2)})
        del A, B
        A, B, sa, sb = [t.cuda() for t in oc.make_config_inputs("cfg3")]
        ms = _time_rotating(lambda i: q.quant_matmul(A, B, sb, scale_a=sa, out_dtype="bfloat16"), 1, 10, world)
        ops = 2 * 4096 * 4096 * 14336
        res.append({"config": "cfg3 W8A8 4096x4096x14336 bf16", "ms": round(ms, 5), "tops": round(ops / ms / 1e9, 1),
                    "frac_of_2x_measured_bf16": round(ops / ms / 1e9 / int8_peak, 4), "key": "cfg3"})
        del A, B

    if world == 1:
        # the step in front of the W8A8 GEMM: per-token activation quantiser, rows x 8192 bf16 (805 MB moved > L2)
        Mq, Nq = 32768, 8192
        X = torch.randn((Mq, Nq), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
        ms = _time_rotating(lambda i: q.act_quant(X), 1, 6, world)
        by = 3 * Mq * Nq + 4 * Mq
        res.append({"config": f"act_quant {Mq}x{Nq} bf16 -> int8 + fp32 row scales", "ms": round(ms, 5),
                    "gbs": round(by / ms / 1e6, 1), "frac_of_measured_hbm": round(by / ms / 1e6 / peaks["hbm_gbs"], 4)})
        del X

    if world == 1:
        # fused W4A8 at decode size on the config-5 weight shape: signed int4 weights, int8 activations, int32 out
        Kq, Nq, Mq = 8192, 28672, 16
        gen = torch.Generator().manual_seed(6)
        qBs = [torch.randint(0, 256, (Nq, Kq // 2), dtype=torch.uint8, generator=gen).cuda() for _ in range(3)]
        A8 = torch.randint(-128, 128, (Mq, Kq), dtype=torch.int8, generator=gen).cuda()
        wsq = torch.empty((Nq, Kq), dtype=torch.int8, device="cuda")
        Cq = torch.empty((Mq, Nq), dtype=torch.int32, device="cuda")
        kq = q.w4a8_gemm_cv(Mq, Nq, Kq)
        ms = _time_rotating(lambda i: kq(A8, qBs[i], wsq, Cq), 3, 12, world)
        by = Nq * Kq // 2 + Mq * Kq + 4 * Mq * Nq
        res.append({"config": f"W4A8 fused M={Mq} K={Kq} N={Nq} (signed int4 x int8 -> int32)", "ms": round(ms, 5),
                    "gbs": round(by / ms / 1e6, 1), "frac_of_measured_hbm": round(by / ms / 1e6 / peaks["hbm_gbs"], 4)})
        del qBs, wsq

    # config 4: batch sharded, no collective
    A, B, sa, sb = oc.make_config_inputs("cfg4")
    Ah, Bh, sah, sbh = shard_batches([A, B, sa, sb], world, rank)
    A, B, sa, sb = [t.cuda() for t in (Ah, Bh, sah, sbh)]
    if world > 1:  # this rank's first batch entry, a band of rows, bit for bit against the oracle
        got = q.quant_matmul(A, B, sb, scale_a=sa, out_dtype="bfloat16")[0, 100:164].cpu()
        want = oc.quant_matmul_ref(Ah[0:1, 100:164], Bh[0:1], sbh[0:1], "bfloat16", scale_a=sah[0:1, 100:164])[0]
        if not torch.equal(got, want):
            _fail(f"cfg4 batch shard of rank {rank} differs from the oracle")
    ms = _time_rotating(lambda i: q.quant_matmul(A, B, sb, scale_a=sa, out_dtype="bfloat16"), 1, 10, world)
    ops = 2 * 16 * 512 * 7168 * 2048
    res.append({"config": f"cfg4 W8A8 16x512x7168x2048 bf16, batch sharded over {world}", "ms": round(ms, 5),
                "tops": round(ops / ms / 1e9, 1), "frac_of_2x_measured_bf16": round(ops / ms / 1e9 / (world * int8_peak), 4),
                "key": "cfg4", "checked_against_oracle": world > 1})
    del A, B

    if world == 1:
        # ragged form of config 4: 16 experts, the same 8192 tokens split unevenly (seeded), same K and N
        Kg, Ng, G = 7168, 2048, 16
        gen = torch.Generator().manual_seed(4)
        w = torch.rand(G, generator=gen) + 0.2
        sizes = (w / w.sum() * 8192).floor().to(torch.int64)
        sizes[-1] += 8192 - int(sizes.sum())
        sizes = [int(x) for x in sizes]
        Ag = torch.randint(-128, 128, (8192, Kg), dtype=torch.int8, generator=gen).cuda()
        Bg = torch.randint(-128, 128, (G, Kg, Ng), dtype=torch.int8, generator=gen).cuda()
        sbg = (torch.rand((G, Ng), generator=gen) * 0.019 + 0.001).cuda()
        sag = (torch.rand(8192, generator=gen) * 0.019 + 0.001).cuda()
        meta = q.build_block_metadata(sizes, 128, "cuda")
        Cg = torch.empty((8192, Ng), dtype=torch.bfloat16, device="cuda")
        ms = _time_rotating(lambda i: q.grouped_quant_matmul(Ag, Bg, meta, sbg, sag, out_dtype="bfloat16", out=Cg), 1, 10, world)
        ops = 2 * 8192 * Kg * Ng
        res.append({"config": f"grouped W8A8, 16 ragged groups {min(sizes)}..{max(sizes)} rows (8192 total) x 7168 x 2048 bf16",
                    "ms": round(ms, 5), "tops": round(ops / ms / 1e9, 1), "row_blocks": int(meta.shape[0]),
                    "frac_of_2x_measured_bf16": round(ops / ms / 1e9 / int8_peak, 4)})
        del Ag, Bg

    # config 5: weight columns sharded; the gathered form leaves the whole [M, N] output on every rank.  The weight
    # copies rotate so that a rank's reads stay L2-cold: enough copies of its shard to exceed 2.5 x L2.
    K, N = 8192, 28672
    _, P, S = oc.make_config_inputs("cfg5", M=1)
    shard_bytes = (N // world) * K // 2
    n_sets = max(2, -(-int(2.5 * L2_BYTES) // shard_bytes))
    layers = [ColumnShardedW4A16(P, S, 8, 128).to("cuda")]
    for c in range(1, n_sets):  # further copies: the same weights with their rows rolled, one shared set of output buffers
        layers.append(ColumnShardedW4A16(P.roll(c * 128, 0).contiguous(), S.roll(c * 128, 1).contiguous(), 8, 128,
                                         share_buffers_with=layers[0]).to("cuda"))
    n0, n1 = shard_range(N, world, rank, 128)
    for M in (1, 8, 16, 64, 512, 4096):
        g = torch.Generator().manual_seed(M)
        Ah = torch.randn((M, K), generator=g).to(torch.bfloat16)
        A = Ah.cuda()
        if world > 1:
            # the gathered output of the first weight copy: a band of this rank's columns and a band of the next
            # rank's, against the oracle, on a few token rows
            out = layers[0].forward(A, gather=True)
            torch.cuda.synchronize()
            rows = torch.arange(0, M, max(1, M // 8))[:8]
            nn0 = shard_range(N, world, (rank + 1) % world, 128)[0]
            cols = torch.cat([torch.arange(n0, n0 + 64), torch.arange(nn0 + 32, nn0 + 96)])
            want = oc.dequant_gemm_fp16_ref(Ah[rows], P[cols], "bfloat16", S[:, cols].contiguous(), 8, 128)
            got = out[rows.cuda()][:, cols.cuda()].cpu()
            if not torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-2):
                _fail(f"cfg5 M={M}: gathered output on rank {rank} differs from the oracle "
                      f"(max abs diff {(got.float() - want.float()).abs().max().item():.4g})")
        sets = n_sets if M <= 64 else 2
        iters = 2 * sets if M <= 512 else 4
        ms_c = _time_rotating(lambda i: layers[i].forward(A, gather=False), sets, iters, world)
        ms_g = _time_rotating(lambda i: layers[i].forward(A, gather=True), sets, iters, world) if world > 1 else ms_c
        by = w4a16_bytes(M, K, N, 128)
        fl = 2 * M * K * N
        entry = {"config": f"cfg5 W4A16 M={M} K=8192 N=28672 bf16, columns sharded over {world}", "key": f"cfg5_m{M}",
                 "ms_compute": round(ms_c, 5), "ms_gathered": round(ms_g, 5),
                 "gather": "none (one rank)" if world == 1 else ("peer stores from the GEMM epilogue" if layers[0].peer_stores is not False else "NCCL all-gather + copy"),
                 "gbs": round(by / ms_c / 1e6, 1), "tflops": round(fl / ms_c / 1e9, 1), "weight_copies_rotated": sets,
                 "checked_against_oracle": world > 1}
        if M <= 64:
            entry["frac_of_measured_hbm"] = round(by / ms_c / 1e6 / (world * peaks["hbm_gbs"]), 4)
        else:
            entry["frac_of_measured_bf16"] = round(fl / ms_c / 1e9 / (world * peaks["bf16_tflops"]), 4)
        res.append(entry)
        if world == 1 and M == 16:
            # config 5 at 16 tokens with a zeros tensor [K/g, N] (zero mode "quantized"): taken in flight by the same kernel
            Z = torch.randint(0, 16, (K // 128, N), generator=torch.Generator().manual_seed(9)).to(torch.float16).cuda()
            Ps = [l.B_local for l in layers]
            Ss = [l.s_local for l in layers]
            ms = _time_rotating(lambda i: q.w4a16_gemm(A, Ps[i], Ss[i], Z, 128, zeros_mode="quantized"), n_sets, 2 * n_sets, world)
            by = w4a16_bytes(M, K, N, 128) + 2 * (K // 128) * N
            res.append({"config": f"cfg5 W4A16 M={M} with per-group zero points (zeros tensor, mode 'quantized'), in flight",
                        "ms": round(ms, 5), "gbs": round(by / ms / 1e6, 1),
                        "frac_of_measured_hbm": round(by / ms / 1e6 / peaks["hbm_gbs"], 4)})
        del A
    if world > 1:
        layers[0].close()
    return res


# ------------------------------------------------------------------------------- CPU reference arm
def cpu_baseline(sample_seconds=12.0):
    """The reference's torch CPU program for the headline config (restated in oracle/), all host threads.

    Sample: whole layers of the headline workload (unpack, (q - 8) * s dequant, fp32 matmul, cast) for
    about `sample_seconds` seconds."""
    from oracle import qgemm_oracle as oc
    torch.set_num_threads(os.cpu_count() or 1)
    A, P, S = oc.make_w4a16_inputs(CFG2["M"], CFG2["K"], CFG2["N"], "float16", CFG2["group"], seed=0)
    oc.dequant_gemm_fp16_ref(A, P, "float16", S, 8, CFG2["group"])
    t0, n = time.perf_counter(), 0
    while True:
        oc.dequant_gemm_fp16_ref(A, P, "float16", S, 8, CFG2["group"])
        n += 1
        dt = time.perf_counter() - t0
        if dt > sample_seconds or n >= 400:
            break
    gbs = n * w4a16_bytes(**CFG2) / dt / 1e9
    return {"value": round(gbs, 4), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n} layers of configs[1] (M=16 K=4096 N=4096) in {dt:.1f} s: vectorised unpack + (q-8)*s + fp32 matmul + cast",
            "ms_per_layer": round(dt / n * 1e3, 2)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import qgemm_oracle as oc
    torch.set_num_threads(os.cpu_count() or 1)
    A, P, S = oc.make_w4a16_inputs(CFG2["M"], CFG2["K"], CFG2["N"], "float16", CFG2["group"], seed=0)

    def step():  # one layer per step: a bounded sample of the 32-layer step
        oc.dequant_gemm_fp16_ref(A, P, "float16", S, 8, CFG2["group"])

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    gbs = args.steps * w4a16_bytes(**CFG2) / dt / 1e9
    cores = torch.get_num_threads()
    sample = f"one layer of configs[1] per step ({args.steps} steps, {dt:.2f} s): the reference's torch CPU program restated in oracle/"
    line = {
        "impl": "reference", "metric": "w4a16_decode_gbs", "value": round(gbs, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 (int4 weights, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": "BASELINE configs[1]: W4A16 dequantize_gemm decode M=16 K=4096 N=4096 group=128 zero=8 fp16; "
                               "CPU sample: one layer per step", "layers_per_step": 1},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def run_case(args):
    """A few eager launches of one configuration, for profilers: `--case cfg2|cfg3|cfg4|cfg5|act_quant|w4a8 [--m M] [--launches L]`.

    Weight sets rotate so that reads stay L2-cold (cfg2: 20 sets = 160 MB; cfg5: 2 sets = 235 MB)."""
    import tilelang_ascend_b200 as q
    from oracle import qgemm_oracle as oc  # input generators only
    torch.cuda.set_device(0)
    n = args.launches
    if args.case == "w4a8":  # fused W4A8 on the config-5 weight shape, --m tokens (default 16), two weight copies
        Kq, Nq, Mq = 8192, 28672, args.m or 16
        qBs = [torch.randint(0, 256, (Nq, Kq // 2), dtype=torch.uint8, device="cuda") for _ in range(2)]
        A8 = torch.randint(-128, 128, (Mq, Kq), dtype=torch.int8, device="cuda")
        wsq = torch.empty((Nq, Kq), dtype=torch.int8, device="cuda")
        C = torch.empty((Mq, Nq), dtype=torch.int32, device="cuda")
        kq = q.w4a8_gemm_cv(Mq, Nq, Kq)
        for i in range(n):
            kq(A8, qBs[i % 2], wsq, C)
    elif args.case == "act_quant":  # --m rows (default 8192) of 8192 bf16 values
        X = torch.randn((args.m or 8192, 8192), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
        for _ in range(n):
            C, _s = q.act_quant(X)
    elif args.case in ("cfg3", "cfg4", "cfg1"):
        A, B, sa, sb = [t.cuda() for t in oc.make_config_inputs(args.case)]
        odt = "float16" if args.case == "cfg1" else "bfloat16"
        for _ in range(n):
            C = q.quant_matmul(A, B, sb, scale_a=sa, out_dtype=odt)
    else:
        M = args.m if args.m is not None else (16 if args.case == "cfg2" else 8)
        A, P, S = [t.cuda() for t in oc.make_config_inputs(args.case, M=M)]
        sets = 20 if args.case == "cfg2" else 2
        Ps = [P] + [torch.randint(0, 256, P.shape, dtype=torch.uint8, device="cuda") for _ in range(sets - 1)]
        if args.batch > 1:  # the bench headline: `batch` weight sets of this shape in one launch
            Pb = torch.randint(0, 256, (args.batch,) + tuple(P.shape), dtype=torch.uint8, device="cuda")
            Ab = A.unsqueeze(0).repeat(args.batch, 1, 1).contiguous()
            Sb = S.unsqueeze(0).repeat(args.batch, 1, 1).contiguous()
            for i in range(n):
                C = q.w4a16_gemm(Ab, Pb, Sb, 8, 128)
        elif args.zeros:  # a zeros tensor [K/g, N] of integer zero points (zero mode "quantized")
            Z = torch.randint(0, 16, tuple(S.shape), generator=torch.Generator().manual_seed(9)).to(torch.float16).cuda()
            for i in range(n):
                C = q.w4a16_gemm(A, Ps[i % sets], S, Z, 128, zeros_mode="quantized")
        else:
            for i in range(n):
                C = q.w4a16_gemm(A, Ps[i % sets], S, 8, 128)
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "launches": n, "checksum": float(C.float().abs().mean())}))


_RESULT_FD = None  # the process's original stdout, kept for the one JSON line


def emit(line: dict):
    """Write the result line to the original stdout (everything else this process and its libraries print goes to
    stderr, see main())."""
    text = json.dumps(line) + "\n"
    if _RESULT_FD is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text.encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-suite", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "act_quant", "w4a8"], default=None,
                    help="profiling helper: launch one configuration a few times and exit")
    ap.add_argument("--m", type=int, default=None)
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--zeros", action="store_true", help="with --case cfg2|cfg5: per-group zero points from a zeros tensor")
    args = ap.parse_args()
    if args.case is not None:
        return run_case(args)
    # stdout carries exactly one JSON line: libraries that print there from native code (NCCL's version banner
    # under torchrun) are sent to stderr for the rest of the run
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
        run_ours(args)


if __name__ == "__main__":
    main()
