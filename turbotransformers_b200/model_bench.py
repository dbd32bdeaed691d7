"""Whole-model timing of the benchmark configurations other than the headline one (which bench.py measures).

    python -m turbotransformers_b200.model_bench --config c1     # BERT-base fp32 b1 s128
    python -m turbotransformers_b200.model_bench --config sweep  # BERT-base fp16, batch {1,8,32} x seq {32,128,512}
    python -m turbotransformers_b200.model_bench --config c3     # BERT-base int8, batch {1,16,64}, seq 128
    python -m turbotransformers_b200.model_bench --config c4     # BERT-large fp16, 32 sequences of 512 (one GPU's shard of 256)
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m turbotransformers_b200.model_bench --config c4
                                                                 # the 256 sequences split over N GPUs, max over ranks
    python -m turbotransformers_b200.model_bench --config c5     # GPT-2 small fp16, b8 s1024, logits
    python -m turbotransformers_b200.model_bench --config c5gen  # GPT-2 small fp16 generation: 512-token prompt, then token by token
    python -m turbotransformers_b200.model_bench --config cpp [--devices N]   # the Python-free C++ host on the headline batch

One JSON line per point: sequences/s, ms per forward (mean and p50 over CUDA-event-timed iterations, inputs resident on
the device), and the algorithmic TFLOP/s (padding never counts; causal attention counts the lower triangle only).
Weights are seeded synthetic (synthetic.py); ids are uniform.
"""
import argparse
import json
import os

import torch

import turbotransformers_b200 as tt
from turbotransformers_b200 import synthetic


def enc_flops(layers, H, L, causal=False):
    att = 2.0 * H * L * (L + 1) if causal else 4.0 * H * L * L
    return layers * (24.0 * H * H * L + att)


def timeit(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        evs.append((s, e))
    torch.cuda.synchronize()
    t = sorted(s.elapsed_time(e) for s, e in evs)
    return sum(t) / len(t), t[len(t) // 2]


def report(name, batch, seq, flops_per_seq, mean_ms, p50_ms, **extra):
    print(json.dumps({"config": name, "batch": batch, "seq_len": seq, "ms_mean": round(mean_ms, 4), "ms_p50": round(p50_ms, 4),
                      "sequences_per_s": round(batch / (mean_ms / 1e3), 1),
                      "tflops": round(batch * flops_per_seq / (mean_ms / 1e3) / 1e12, 1), **extra}), flush=True)


def cpp_host(a):
    """BERT-base fp16 on the headline batch (64 requests U[8,512]) through `bert_model_example`: archive from disk, ids from
    a text file, one model and one host thread per device; every batch uploads its ids and downloads its pooled output."""
    import os
    import re
    import subprocess
    import tempfile

    from . import build
    from .tools.convert_huggingface_bert_pytorch_to_npz import save_bert_npz
    hf = synthetic.make_hf_bert("bert-base", 0)
    lens = synthetic.varlen_lengths(64, 8, 512, 0)
    ids = synthetic.varlen_ids(lens, hf.config.vocab_size, 0)
    with tempfile.TemporaryDirectory() as d:
        npz, txt = os.path.join(d, "bert_base.npz"), os.path.join(d, "ids.txt")
        save_bert_npz(hf, npz, compressed=False)
        with open(txt, "w") as f:
            f.write("\n".join(" ".join(str(int(v)) for v in r) for r in ids) + "\n")
        r = subprocess.run([build.build_example(), npz, "12", "12", "--dtype", "float16", "--ids", txt, "--devices", str(a.devices),
                            "--requests", str(max(a.iters, 20))], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(r.stderr)
    m = re.search(r"([0-9.]+) sequences/s \(([0-9.]+) ms per batch per device\)", r.stdout)
    print(json.dumps({"config": "bert-base fp16, 64 requests U[8,512], C++ host (npz archive, no Python), pooled output to the host",
                      "devices": a.devices, "sequences_per_s": float(m.group(1)), "ms_per_batch_per_device": float(m.group(2))}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["c1", "sweep", "c3", "c4", "c5", "c5gen", "cpp"])
    ap.add_argument("--devices", type=int, default=1, help="cpp: GPUs the serving loop drives (one host thread each)")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    torch.set_grad_enabled(False)
    dev = torch.device("cuda:0")
    if a.config == "cpp":
        return cpp_host(a)
    if a.config in ("c1", "sweep", "c3"):
        hf = synthetic.make_hf_bert("bert-base", 0)
        V = hf.config.vocab_size
        if a.config == "c1":
            model = tt.BertModel.from_torch(hf.to(dev), dev)
            points, name = [(1, 128)], "bert-base fp32"
        elif a.config == "sweep":
            model = tt.BertModel.from_torch(hf.to(dev).half(), dev)
            points, name = [(b, s) for b in (1, 8, 32) for s in (32, 128, 512)], "bert-base fp16"
        else:
            model = tt.QBertModel.from_torch(hf.to(dev).half(), dev)
            points, name = [(1, 128), (16, 128), (64, 128)], "bert-base int8 (all six Linears)"
        for b, s in points:
            ids = synthetic.random_ids(b, s, V, 0).to(dev)
            mean, p50 = timeit(lambda: model(ids), a.warmup, a.iters)
            report(name, b, s, enc_flops(12, 768, s), mean, p50)
    elif a.config == "c4":
        # BERT-large fp16, 256 sequences of 512: the batch is split into contiguous shards, one per GPU, weights replicated,
        # no collective on the data path. Under torch.distributed.run every rank runs its shard of 256 / world sequences and
        # the job's rate is all 256 sequences over the slowest rank's device time; a plain single-process run times one
        # GPU's shard of an 8-GPU job (32 sequences).
        import torch.distributed as dist
        from turbotransformers_b200 import sharding
        world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
        if world > 1:
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            torch.cuda.set_device(dev)
            dist.init_process_group("nccl", device_id=dev)
        shards = sharding.contiguous_shards(256, world if world > 1 else 8)
        mine = shards[rank if world > 1 else 0]
        hf = synthetic.make_hf_bert("bert-large", 0)
        model = tt.BertModel.from_torch(hf.to(dev).half(), dev)
        all_ids = synthetic.random_ids(256, 512, hf.config.vocab_size, 0)
        ids = all_ids[mine].to(dev)
        if world > 1:
            dist.barrier()
        mean, p50 = timeit(lambda: model(ids), a.warmup, a.iters)
        if world > 1:
            mean, p50 = sharding.reduce_max_ms(mean, dev), sharding.reduce_max_ms(p50, dev)
            if rank == 0:
                report(f"bert-large fp16, 256 sequences over {world} GPUs ({len(mine)} per GPU, max over ranks)", 256, 512,
                       enc_flops(24, 1024, 512), mean, p50, n_gpus=world)
            assert tt._cxx_module.device_status(dev.index) == 0
            dist.barrier()
            dist.destroy_process_group()
            return
        report("bert-large fp16 (32 of the 256 sequences: one GPU's shard at 8 GPUs)", len(mine), 512, enc_flops(24, 1024, 512), mean, p50)
    elif a.config == "c5gen":
        hf = synthetic.make_hf_gpt2("gpt2-small", 0)
        model = tt.GPT2Model.from_torch(hf.to(dev).half(), dev)
        for B in (8, 64):
            prompt = synthetic.random_ids(B, 512, hf.config.vocab_size, 0).to(dev)
            nxt = synthetic.random_ids(B, 1, hf.config.vocab_size, 1).to(dev)

            def prefill():
                past = model.new_cache()
                model(prompt, return_logits=False, past=past)
                return past
            mean, p50 = timeit(prefill, 2, 10)
            past = prefill()
            steps = 128

            def decode():
                model(nxt, return_logits=True, past=past)
            for _ in range(5):
                decode()
            torch.cuda.synchronize()
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(steps):
                decode()
            e0.record()
            torch.cuda.synchronize()
            ms_tok = s0.elapsed_time(e0) / steps
            print(json.dumps({"config": "gpt2-small fp16 generation with a key/value cache", "batch": B, "prompt": 512, "prefill_ms": round(mean, 3),
                              "decode_ms_per_step": round(ms_tok, 4), "decode_tokens_per_s": round(B / (ms_tok / 1e3), 1),
                              "cached_tokens_at_end": model.cached_length(past)}), flush=True)
    else:
        hf = synthetic.make_hf_gpt2("gpt2-small", 0)
        model = tt.GPT2Model.from_torch(hf.to(dev).half(), dev)
        ids = synthetic.random_ids(8, 1024, hf.config.vocab_size, 0).to(dev)
        mean, p50 = timeit(lambda: model(ids), a.warmup, a.iters)
        fl = enc_flops(12, 768, 1024, causal=True) + 2.0 * 1024 * 768 * hf.config.vocab_size
        report("gpt2-small fp16, full-sequence forward with tied-embedding logits", 8, 1024, fl, mean, p50)
        mean, p50 = timeit(lambda: model(ids, contiguous_logits=False), a.warmup, a.iters)
        report("gpt2-small fp16, logits left in rows padded to a multiple of 8 entries (a strided view)", 8, 1024, fl, mean, p50)
        mean, p50 = timeit(lambda: model(ids, return_logits=False), a.warmup, a.iters)
        report("gpt2-small fp16, hidden states only", 8, 1024, enc_flops(12, 768, 1024, causal=True), mean, p50)
    assert tt._cxx_module.device_status(0) == 0


if __name__ == "__main__":
    main()
