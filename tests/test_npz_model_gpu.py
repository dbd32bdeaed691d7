"""The Python-free model of the C++ API: `.npz` archive -> BertModel (csrc/host/bert_model.cpp), reached through its
pybind handle and through the `bert_model_example` executable, against the numpy restatement of the reference on the same
seeded weights and ids (what example/cpp/bert_model_test.cpp did with a pretrained checkpoint that is not available offline).

Tolerances as for the Python-loaded models: fp32 1e-3 max-abs; fp16 2e-2 max-abs and 2e-3 mean-abs.
"""
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import ref_driver, restate
from turbotransformers_b200 import build, synthetic
from turbotransformers_b200._cxx import cxx
from turbotransformers_b200.tools.convert_huggingface_bert_pytorch_to_npz import save_bert_npz

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
LENS = [50, 7, 33]


@pytest.fixture(scope="module")
def mini(tmp_path_factory):
    hf = synthetic.make_hf_bert("bert-mini", 3)
    path = str(tmp_path_factory.mktemp("npz") / "bert_mini.npz")
    save_bert_npz(hf, path, compressed=True)
    W = ref_driver.pack_bert_weights(hf)
    ids = [r.tolist() for r in synthetic.varlen_ids(LENS, hf.config.vocab_size, 5)]
    # oracle: every request alone (requests are independent), fp32
    want_seq = [restate.bert_model(np.asarray(i, np.int64)[None], W, hf.config.num_attention_heads)[0][0] for i in ids]
    want_pool = np.stack([restate.bert_model(np.asarray(i, np.int64)[None], W, hf.config.num_attention_heads)[1][0] for i in ids])
    return {"path": path, "layers": hf.config.num_hidden_layers, "heads": hf.config.num_attention_heads, "H": hf.config.hidden_size,
            "ids": ids, "seq": want_seq, "pool": want_pool}


@pytest.mark.parametrize("dtype,max_tol,mean_tol", [("float32", 1e-3, 1e-4), ("float16", 2e-2, 2e-3)])
def test_npz_bert_model_matches_oracle(mini, dtype, max_tol, mean_tol):
    m = cxx.NpzBertModel(mini["path"], mini["layers"], mini["heads"], dtype, 0)
    assert m.hidden_size == mini["H"]
    out = np.asarray(m(mini["ids"]), np.float32).reshape(len(LENS), max(LENS), mini["H"])
    for b, L in enumerate(LENS):
        d = np.abs(out[b, :L] - mini["seq"][b])
        assert d.max() < max_tol and d.mean() < mean_tol, (b, d.max(), d.mean())
    if dtype == "float16":  # the packed path leaves padding rows at zero
        assert not out[1, LENS[1]:].any()
    pooled = np.asarray(m(mini["ids"], pooling="First", use_pooler=True), np.float32).reshape(len(LENS), mini["H"])
    d = np.abs(pooled - mini["pool"])
    assert d.max() < max_tol and d.mean() < mean_tol


def test_npz_bert_model_position_and_segment_ids(mini):
    # explicit positions 0..L-1 and segment 0 are the defaults: same numbers through the padded path in every dtype
    m = cxx.NpzBertModel(mini["path"], mini["layers"], mini["heads"], "float16", 0)
    pos = [list(range(len(r))) for r in mini["ids"]]
    seg = [[0] * len(r) for r in mini["ids"]]
    a = np.asarray(m(mini["ids"]), np.float32).reshape(len(LENS), max(LENS), mini["H"])
    b = np.asarray(m(mini["ids"], pos, seg), np.float32).reshape(len(LENS), max(LENS), mini["H"])
    for i, L in enumerate(LENS):
        assert np.abs(a[i, :L] - b[i, :L]).max() < 2e-2
    with pytest.raises(RuntimeError):
        m(mini["ids"], pos[:1], [])
    with pytest.raises(RuntimeError):
        cxx.NpzBertModel(mini["path"], mini["layers"] + 1, mini["heads"], "float32", 0)  # a layer the archive does not have


def test_bert_model_example_executable(mini, tmp_path):
    exe = build.build_example()
    ids_file, out_file = tmp_path / "ids.txt", tmp_path / "out.bin"
    ids_file.write_text("\n".join(" ".join(str(v) for v in r) for r in mini["ids"]) + "\n")
    r = subprocess.run([exe, mini["path"], str(mini["layers"]), str(mini["heads"]), "--dtype", "float32", "--ids", str(ids_file),
                        "--out", str(out_file)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    out = np.fromfile(out_file, np.float32).reshape(len(LENS), max(LENS), mini["H"])
    for b, L in enumerate(LENS):
        assert np.abs(out[b, :L] - mini["seq"][b]).max() < 1e-3
    # the serving loop: one thread per device, pooled outputs, reports throughput
    r = subprocess.run([exe, mini["path"], str(mini["layers"]), str(mini["heads"]), "--dtype", "float16", "--ids", str(ids_file),
                        "--devices", "1", "--requests", "5"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert "sequences/s" in r.stdout
    r = subprocess.run([exe, str(tmp_path / "missing.npz"), "2", "2"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 1 and "cannot open" in r.stderr
