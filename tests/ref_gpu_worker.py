"""Worker process of test_reference_gpu_build.py (TEST INFRASTRUCTURE).

Holds the reference's own GPU build (oracle/_ref/cuda: its fp32 kernels + cuBLAS, compiled unmodified for sm_100a) and this
library in one process, runs both on the same seeded BERT-base weights and inputs on cuda:0, and prints one JSON line with
the largest differences and the device time of each.  It is a separate process because the reference's CPU and GPU builds
export the same C++ types and cannot be imported together.

    python tests/ref_gpu_worker.py [--layers 12] [--iters 10]
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from oracle import ref_driver  # noqa: E402


def timed(fn, iters, warmup=3):
    """Mean device milliseconds of fn() (events on the legacy default stream, which orders after the reference's stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    ref_driver.use_cuda_build()
    import turbotransformers_b200 as tt
    from turbotransformers_b200 import synthetic
    torch.set_grad_enabled(False)
    dev = torch.device("cuda:0")
    hf = synthetic.make_hf_bert("bert-base", 0, a.layers)
    vocab = hf.config.vocab_size
    ref = ref_driver.RefBert(ref_driver.pack_bert_weights(hf), hf.config.num_attention_heads)
    ours32 = tt.BertModel.from_torch(synthetic.make_hf_bert("bert-base", 0, a.layers).to(dev), dev)
    ours32_sb = tt.BertModelSmartBatch.from_torch(synthetic.make_hf_bert("bert-base", 0, a.layers).to(dev), dev)
    ours16_sb = tt.BertModelSmartBatch.from_torch(synthetic.make_hf_bert("bert-base", 0, a.layers).to(dev).half(), dev)
    out = {"layers": a.layers}

    # fixed-length batches: b1 s128 (the reference's CPU-runnable configuration) and b20 s128
    for name, b, s in (("b1_s128", 1, 128), ("b20_s128", 20, 128)):
        ids = synthetic.random_ids(b, s, vocab, 3).to(dev)
        want, want_pooled = ref.forward(ids)
        got, got_pooled = ours32(ids)[:2]
        out[name] = {"seq_maxdiff": (got.float() - want).abs().max().item(),
                     "pooled_maxdiff": (got_pooled.float() - want_pooled).abs().max().item(),
                     "reference_gpu_ms": timed(lambda: ref.forward(ids), a.iters),
                     "ours_fp32_ms": timed(lambda: ours32(ids), a.iters)}

    # the benchmark's batch: 64 requests, lengths U[8,512], packed (the reference's smart-batch layers)
    lens = synthetic.varlen_lengths(64, 8, 512, 0)
    id_list = [i.to(dev) for i in synthetic.varlen_ids(lens, vocab, 0)]
    want = ref.forward_smart_batch(id_list)
    got = ours32_sb(id_list, lens)[0]
    got16 = ours16_sb(id_list, lens)[0]
    out["varlen_b64"] = {"tokens": sum(lens),
                         "seq_maxdiff": (got.float().reshape(want.shape) - want).abs().max().item(),
                         "fp16_seq_maxdiff": (got16.float().reshape(want.shape) - want).abs().max().item(),
                         "reference_gpu_ms": timed(lambda: ref.forward_smart_batch(id_list), max(2, a.iters // 3), warmup=1),
                         "ours_fp32_ms": timed(lambda: ours32_sb(id_list, lens), a.iters),
                         "ours_fp16_ms": timed(lambda: ours16_sb(id_list, lens), a.iters)}
    assert tt._cxx_module.device_status(0) == 0
    print("REF_GPU_RESULT " + json.dumps(out))


if __name__ == "__main__":
    main()
