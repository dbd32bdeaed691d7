#!/usr/bin/env python
"""Benchmark of the transformer-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (single GPU and per rank): BERT-base fp16, 64 requests with lengths uniform in [8, 512] drawn
from seed 0, run unpadded ("smart batch": packed tokens + prefix-sum offsets). One step = one forward of
that batch through the reference-facing API (BertModelSmartBatch). With N > 1 every rank serves its own
64-request batch with replicated weights and no collective on the data path (weak scaling).

Prints ONE JSON line on rank 0. `value` is sequences/s with the ids already in HBM; `e2e` starts from
pinned host ids and ends with the pooled output back on the host. `roofline` is for the tensor-core GEMM
(the dominant kernel), timed alone with CUDA events on the four shapes of one encoder layer.
`--impl reference` times the reference's own CPU implementation (oracle/_ref) on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bert_base_fp16_varlen_b64_sequences_per_s"
UNIT = "sequences/s"
BATCH, LO, HI, SEED = 64, 8, 512, 0
LAYERS, HIDDEN, HEADS, FFN = 12, 768, 12, 3072


def workload_config(n_gpus):
    return {"workload": "bert-base fp16 smart-batch: 64 requests/GPU, lengths U[8,512] seed 0, packed tokens",
            "requests_per_gpu": BATCH, "parallelism": f"replicas x{n_gpus} (requests sharded, weights replicated, no collective)",
            "cache": "working set (170 MB of fp16 weights + ~0.4 GB of activations per step) exceeds the 126 MB L2",
            "result_returned": "pooled_output [64,768] fp16 (sequence_output stays on the device)"}


def flops_per_sequence(L):
    """Algorithmic FLOPs of one BERT-base sequence of length L: n*(24*H^2*L + 4*H*L^2)."""
    return LAYERS * (24 * HIDDEN * HIDDEN * L + 4 * HIDDEN * L * L)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML in a thread of this process
    (cheap reads every 25 ms), or, when the NVML binding is missing, through an `nvidia-smi -lms` child process."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.window = index, [], None, (0.0, float("inf"))
        self.nvml, self.handle, self.alive, self.thread = None, None, False, None

    def start(self):
        """Start early (before the warm-up): whatever comes up slowly must not do so inside the timed region."""
        try:
            import pynvml
            pynvml.nvmlInit()
            # NVML numbers devices by PCI order; CUDA_VISIBLE_DEVICES may remap, so go through the UUID of the CUDA device
            import torch
            uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except pynvml.NVMLError:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml, self.alive = pynvml, True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:  # no binding / no NVML: fall back to the command-line tool
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        bits = (("hw_slowdown", n.nvmlClocksThrottleReasonHwSlowdown), ("hw_thermal_slowdown", n.nvmlClocksThrottleReasonHwThermalSlowdown),
                ("sw_thermal_slowdown", n.nvmlClocksThrottleReasonSwThermalSlowdown), ("sw_power_cap", n.nvmlClocksThrottleReasonSwPowerCap))
        try:
            mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        except n.NVMLError:
            mx = 0
        while self.alive:
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                row = [str(self.index), str(sm), str(mx), "", ""] + ["Active" if mask & b else "Not Active" for _, b in bits]
                self.rows.append((time.time(), row))
            except n.NVMLError:
                pass
            time.sleep(0.025)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.nvml:
            self.alive = False
            if self.thread:
                self.thread.join(timeout=1)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        lo, hi = self.window
        inside = [r for t, r in self.rows if lo <= t <= hi + 0.05] or [r for _, r in self.rows[-3:]]
        for r in inside:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except (ValueError, IndexError):
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvml" if self.nvml else "nvidia-smi"}


def load_synthetic():
    """The seeded-input module loaded from its file, without importing the package around it: the reference arm must not
    load this repository's native libraries."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("ttb_synthetic", os.path.join(ROOT, "turbotransformers_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_batch(vocab, rank, synthetic=None):
    synthetic = synthetic or load_synthetic()
    lens = synthetic.varlen_lengths(BATCH, LO, HI, SEED + rank)
    ids = synthetic.varlen_ids(lens, vocab, SEED + rank)
    return lens, ids


# ----------------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU implementation on the host cores
# ----------------------------------------------------------------------------------------------------
def time_reference_cpu(steps, warmup, budget_s, rank0=True):
    import torch
    from oracle import ref_driver
    synthetic = load_synthetic()
    torch.set_grad_enabled(False)
    if not ref_driver.available():
        raise RuntimeError("oracle/_ref is not built")
    cores = os.cpu_count() or 1
    ref_driver.set_num_threads(cores)
    torch.set_num_threads(cores)
    hf = synthetic.make_hf_bert("bert-base", SEED)
    W = ref_driver.pack_bert_weights(hf)
    ref = ref_driver.RefBert(W, HEADS)
    lens, ids = make_batch(hf.config.vocab_size, 0, synthetic)
    # calibrate on one short request, then size the per-step sample to the time budget
    t = time.perf_counter()
    ref.forward_smart_batch(ids[:1])
    per_token = (time.perf_counter() - t) / max(1, lens[0])
    per_step_budget = budget_s / max(1, steps + warmup)
    n, tok = 0, 0
    while n < BATCH and (n == 0 or (tok + lens[n]) * per_token <= per_step_budget):
        tok += lens[n]
        n += 1
    sample = ids[:n]
    for _ in range(warmup):
        ref.forward_smart_batch(sample)
    t0 = time.perf_counter()
    for _ in range(steps):
        ref.forward_smart_batch(sample)
    dt = (time.perf_counter() - t0) / steps
    return {"value": n / dt, "ms_per_step": dt * 1e3, "cores": cores, "kind": "reference",
            "sample": f"first {n} of the 64 requests ({tok} tokens) per step through the compiled reference CPU code "
                      f"(MultiHeadedAttentionSmartBatch + BertIntermediate + BertOutput, OpenBLAS + OpenMP, {cores} threads)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    try:
        r = time_reference_cpu(args.steps, args.warmup, budget_s=150.0)
    except Exception as e:  # the oracle always exists on a prepared tree; say why if it does not
        print(json.dumps({"impl": "reference", "unavailable": str(e)[:200]}))
        return
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus),
            "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------------
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel (the CTA-pair GEMM on the QKV shape,
# M = 18424, N = 2304, K = 768), from an ncu capture of that launch.
# The algorithmic bytes of that launch are 116.7 MB (A 28.3 + W 3.5 + out 84.9); most of the output is still in L2 when
# the kernel ends, so the DRAM counter sees less than that.
QKV_LAUNCH_DRAM_BYTES = 61.5e6


def burst_us(torch, fns, rounds):
    """Mean device time of one launch in a back-to-back run over several buffer sets (CUDA events on the launching
    stream; the rotating sets keep each launch's activations out of L2)."""
    for _ in range(2):
        for f in fns:
            f()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(rounds):
        for f in fns:
            f()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (rounds * len(fns))


def graph_us(torch, ctx, fns, rounds):
    """Mean device time of one launch with the host out of the picture, for kernels shorter than the host's launch path:
    the launches of `fns` (different buffer sets) are recorded once into a CUDA graph on a side stream and the graph is
    replayed `rounds` times between two CUDA events."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        if ctx is not None:
            ctx.set_stream(side.cuda_stream)
        for f in fns:
            f()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for f in fns:
                f()
    torch.cuda.current_stream().wait_stream(side)
    if ctx is not None:
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(rounds):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (rounds * len(fns))


def gemm_roofline(torch, lens, peaks):
    """Times the kernels of one encoder layer at this batch's size the way they run inside a step: launches back to back,
    each on another of eight buffer sets so that no launch finds its activations in L2 (8 x >= 85 MB against 126 MB).
    Each run lasts a few milliseconds at full clocks, so the denominators are the burst figures. The roofline object
    is the QKV-shape launch of the dominant kernel; the other GEMM shapes, the attention kernel and the LayerNorm kernel
    are listed beside it with their own fractions."""
    import numpy as np
    from turbotransformers_b200 import _capi
    tokens = sum(lens)
    ctx = _capi.Context(torch.cuda.current_device())
    shapes = [("qkv", HIDDEN, 3 * HIDDEN, _capi.EPI_BIAS), ("attn_out", HIDDEN, HIDDEN, _capi.EPI_BIAS_RESIDUAL),
              ("ffn1", HIDDEN, FFN, _capi.EPI_BIAS_GELU), ("ffn2", FFN, HIDDEN, _capi.EPI_BIAS_RESIDUAL)]
    sets, rounds = 8, 6
    f16 = torch.float16
    per_shape, total_us, total_flops = {}, 0.0, 0.0
    for name, K, N, epi in shapes:
        w = torch.randn(N, K, device="cuda", dtype=f16) * 0.03
        b = torch.randn(N, device="cuda", dtype=f16)
        bufs = [(torch.randn(tokens, K, device="cuda", dtype=f16), torch.randn(tokens, N, device="cuda", dtype=f16),
                 torch.empty(tokens, N, device="cuda", dtype=f16)) for _ in range(sets)]
        us = burst_us(torch, [lambda a=a, r=r, o=o: ctx.call("linear", _capi.F16, a, K, w, b, r, N, tokens, N, K, epi, o, N)
                              for a, r, o in bufs], rounds)
        # the vendor library on the same operands for orientation (torch.addmm = cuBLAS GEMM + bias, no activation and
        # no residual), replayed from a CUDA graph to keep torch's host path out of the number
        wt = w.t()
        lib_us = graph_us(torch, None, [lambda a=a, o=o: torch.addmm(b, a, wt, out=o) for a, _, o in bufs], rounds)
        fl = 2.0 * tokens * N * K
        per_shape[name] = {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac": round(fl / us / 1e6 / peaks["tflops"], 4),
                           "cublas_bias_only_us": round(lib_us, 1)}
        total_us += us
        total_flops += fl
        del bufs, w, b
    # attention over the packed batch (tensor bound: 4*H*L^2 FLOPs per sequence, padding never counts)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    abufs = [(torch.randn(tokens, 3 * HIDDEN, device="cuda", dtype=f16), torch.empty(tokens, HIDDEN, device="cuda", dtype=f16))
             for _ in range(sets)]
    us = burst_us(torch, [lambda q=q, o=o: ctx.call("attention_fwd", _capi.F16, q, tokens, cu, len(lens), max(lens), HEADS, HIDDEN // HEADS,
                                                    None, 0, 0, 0, 0.125, o) for q, o in abufs], rounds)
    afl = sum(4.0 * HIDDEN * L * L for L in lens)
    attention = {"us": round(us, 1), "tflops": round(afl / us / 1e6, 1), "frac": round(afl / us / 1e6 / peaks["tflops"], 4), "bound": "tensor"}
    del abufs
    # LayerNorm over the residual sum the GEMM epilogue wrote (HBM bound: read + write of [tokens, H] fp16)
    g, z = torch.ones(HIDDEN, device="cuda", dtype=f16), torch.zeros(HIDDEN, device="cuda", dtype=f16)
    lbufs = [(torch.randn(tokens, HIDDEN, device="cuda", dtype=f16), torch.empty(tokens, HIDDEN, device="cuda", dtype=f16)) for _ in range(sets * 4)]
    lfns = [lambda x=x, o=o: ctx.call("layernorm", _capi.F16, x, o, g, z, tokens, HIDDEN, 1e-12) for x, o in lbufs]
    us_host = burst_us(torch, lfns, rounds)
    us = graph_us(torch, ctx, lfns, rounds)  # the kernel is shorter than the host's launch path: replayed from a graph
    lbytes = 2.0 * tokens * HIDDEN * 2
    layernorm = {"us": round(us, 1), "gbs": round(lbytes / us / 1e3, 1), "frac": round(lbytes / us / 1e3 / peaks["hbm_gbs"], 4), "bound": "hbm",
                 "timing": "CUDA-graph replay of 32 launches on 32 buffer sets", "us_launched_from_python": round(us_host, 1)}
    del lbufs
    ctx.close()
    qkv_flops = 2.0 * tokens * 3 * HIDDEN * HIDDEN
    achieved = per_shape["qkv"]["tflops"]
    return {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
            "frac": round(achieved / peaks["tflops"], 4), "traffic": QKV_LAUNCH_DRAM_BYTES,
            "peak_source": peaks["source"] + " (cuBLAS bf16, burst: the kernel is timed in a run of a few milliseconds at full clocks)",
            "frac_of_sustained_peak": round(achieved / peaks["tflops_sustained"], 4),
            "kernel": "gemm_tc_kernel<256, f16, pair> (tcgen05 cta_group::2 + TMEM + TMA) on the QKV shape "
                      f"[{tokens} x {3 * HIDDEN} x {HIDDEN}]; 36 of the 48 GEMM launches per step run this kernel",
            "avg_launch_us": per_shape["qkv"]["us"], "algorithmic_flops_per_launch": qkv_flops,
            "algorithmic_bytes_per_launch": 2.0 * (tokens * HIDDEN + 3 * HIDDEN * HIDDEN + tokens * 3 * HIDDEN),
            "per_shape": per_shape, "all_four_shapes_tflops": round(total_flops / total_us / 1e6, 1),
            "attention_kernel": attention, "layernorm_kernel": layernorm}


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.set_grad_enabled(False)
    import turbotransformers_b200 as tt
    from turbotransformers_b200 import sharding, synthetic
    cxx = tt._cxx_module
    peaks = load_peaks()

    hf = synthetic.make_hf_bert("bert-base", SEED)
    vocab = hf.config.vocab_size
    model = tt.BertModelSmartBatch.from_torch(hf.to(dev).half(), dev)
    lens, ids = make_batch(vocab, rank, synthetic)
    tokens = sum(lens)
    ids_host = torch.cat(ids).pin_memory()
    ids_dev = ids_host.to(dev)
    # End to end the way a serving loop runs it: every step copies its ids from pinned host memory and its pooled output back
    # to pinned host memory; the host waits for the result of step i-1 only after it has enqueued step i (two result buffers),
    # so the GPU never sits idle while the host enqueues. Every result has reached the host before the timed region ends.
    pooled_host = [torch.empty(BATCH, HIDDEN, dtype=torch.float16).pin_memory() for _ in range(2)]
    arrived = [torch.cuda.Event(), torch.cuda.Event()]
    e2e_state = {"i": 0}

    def step_device():
        return model(ids_dev, lens)

    def step_e2e():
        i = e2e_state["i"]
        d = ids_host.to(dev, non_blocking=True)
        seq, pooled = model(d, lens)[:2]
        pooled_host[i & 1].copy_(pooled, non_blocking=True)
        arrived[i & 1].record()
        if i > 0:
            arrived[(i - 1) & 1].synchronize()  # the caller has the previous step's result on the host
        e2e_state["i"] = i + 1
        return pooled_host[(i - 1) & 1]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = cxx.launch_count(local)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = cxx.launch_count(local) - l0
        ms = sharding.reduce_max_ms(ms, dev)  # the job is as slow as its slowest rank
        return ms, launches

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step_device()
    torch.cuda.synchronize()
    t_lo = time.time()
    ms, launches = timed(step_device, args.steps)
    sampler.window = (t_lo, time.time())
    clocks = sampler.stop() if rank == 0 else None
    if cxx.device_status(local) != 0:
        raise RuntimeError("the device status word reports a kernel error")
    for _ in range(3):
        step_e2e()
    ms_e2e, _ = timed(step_e2e, args.steps)

    if rank == 0:
        seq_per_s = BATCH * world * args.steps / (ms / 1e3)
        e2e_seq_per_s = BATCH * world * args.steps / (ms_e2e / 1e3)
        step_flops = sum(flops_per_sequence(L) for L in lens)
        line = {"metric": METRIC, "value": round(seq_per_s, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(world),
                "e2e": {"value": round(e2e_seq_per_s, 1), "unit": UNIT, "h2d_bytes_per_step": int(ids_host.numel() * 8),
                        "d2h_bytes_per_step": int(pooled_host[0].numel() * 2), "ms_per_step": round(ms_e2e / args.steps, 4),
                        "pipelining": "the host waits for step i-1's result after enqueueing step i; all results on the host before the region ends"},
                "gpu_launches": int(launches), "clocks": clocks,
                "tokens_per_step_per_gpu": tokens,
                "model_tflops": round(step_flops * world * args.steps / (ms / 1e3) / 1e12, 1),
                "model_tflops_frac_of_sustained_peak": round(step_flops * args.steps / (ms / 1e3) / 1e12 / peaks["tflops_sustained"], 4)}
        if args.no_extras:
            print(json.dumps(line))
            return
        line["roofline"] = gemm_roofline(torch, lens, peaks)
        # p50 latency of one 128-token request (the other half of the headline metric)
        fixed = tt.BertModel.from_torch(hf, dev)
        one = synthetic.random_ids(1, 128, vocab, SEED).to(dev)
        for _ in range(10):
            fixed(one)
        lat = []
        for _ in range(50):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fixed(one)
            e.record()
            e.synchronize()
            lat.append(s.elapsed_time(e))
        lat.sort()
        line["latency_b1_s128_ms"] = {"p50": round(lat[len(lat) // 2], 4), "p90": round(lat[int(len(lat) * 0.9)], 4)}
        # the same request through a CUDA-graph replay of the forward pass (one graph launch instead of ~90 kernel launches)
        try:
            from turbotransformers_b200.graphs import CapturedForward
            replay = CapturedForward(lambda ids: fixed(ids), one.clone())
            for _ in range(10):
                replay(one)
            glat = []
            for _ in range(50):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                replay(one)
                e.record()
                e.synchronize()
                glat.append(s.elapsed_time(e))
            glat.sort()
            line["latency_b1_s128_ms"].update({"graph_replay_p50": round(glat[len(glat) // 2], 4),
                                               "graph_replay_p90": round(glat[int(len(glat) * 0.9)], 4)})
        except Exception as ex:  # the eager numbers above stand on their own
            line["latency_b1_s128_ms"]["graph_replay_error"] = str(ex)[:160]
        if world == 1 and not args.no_cpu_baseline:
            try:
                r = time_reference_cpu(steps=1, warmup=0, budget_s=20.0)
                line["cpu_baseline"] = {"value": round(r["value"], 3), "unit": UNIT, "cores": r["cores"], "kind": r["kind"],
                                        "sample": r["sample"]}
            except Exception as e:
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                        "sample": f"unavailable: {str(e)[:120]}"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="timed regions only (for profiler launch lists)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
