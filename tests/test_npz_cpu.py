"""The C++ `.npz` reader (csrc/host/npz.cpp) against numpy on archives numpy wrote: stored and deflated members, the zip64
fields numpy always emits, float32 / float16 / int64 members, scalars and empty arrays, prefix views. No GPU needed."""
import numpy as np
import pytest

from turbotransformers_b200 import synthetic
from turbotransformers_b200._cxx import cxx
from turbotransformers_b200.tools.convert_huggingface_bert_pytorch_to_npz import bert_state_to_arrays

DT = {"<f4": np.float32, "<f2": np.float16, "<i8": np.int64, "<i4": np.int32, "|u1": np.uint8}


def read_back(path):
    out = {}
    for name, (descr, shape, raw) in cxx.npz_load(str(path)).items():
        out[name] = np.frombuffer(raw, dtype=DT[descr]).reshape(shape)
    return out


@pytest.mark.parametrize("compressed", [False, True])
def test_reader_matches_numpy(tmp_path, compressed):
    r = np.random.default_rng(0)
    arrays = {"a.weight": r.standard_normal((37, 5)).astype(np.float32), "a.bias": r.standard_normal(5).astype(np.float32),
              "deep.er.half": r.standard_normal((3, 4, 2)).astype(np.float16), "ids": r.integers(0, 1 << 40, (7,), dtype=np.int64),
              "scalar": np.float32(3.5), "empty": np.zeros((0, 4), np.float32), "bytes": np.arange(10, dtype=np.uint8),
              "big": r.standard_normal((300, 1000)).astype(np.float32)}
    path = tmp_path / "t.npz"
    (np.savez_compressed if compressed else np.savez)(path, **arrays)
    got = read_back(path)
    assert sorted(got) == sorted(arrays)
    for k, v in arrays.items():
        assert got[k].shape == np.asarray(v).shape
        assert np.array_equal(got[k], np.asarray(v))


def test_reader_rejects_what_it_cannot_read(tmp_path):
    p = tmp_path / "not_a_zip.npz"
    p.write_bytes(b"hello world, definitely not a zip archive........")
    with pytest.raises(RuntimeError):
        cxx.npz_load(str(p))
    with pytest.raises(RuntimeError):
        cxx.npz_load(str(tmp_path / "missing.npz"))
    q = tmp_path / "fortran.npz"
    np.savez(q, f=np.asfortranarray(np.ones((3, 4), np.float32)))
    with pytest.raises(RuntimeError):
        cxx.npz_load(str(q))


def test_converter_layout_of_a_small_bert(tmp_path):
    hf = synthetic.make_hf_bert("bert-tiny", 0)
    arrays = bert_state_to_arrays(hf)
    H, F = hf.config.hidden_size, hf.config.intermediate_size
    assert arrays["encoder.layer.0.attention.qkv.weight"].shape == (H, 3 * H)
    assert arrays["encoder.layer.0.attention.qkv.bias"].shape == (3 * H,)
    assert arrays["encoder.layer.1.intermediate.dense.weight"].shape == (H, F)
    assert arrays["encoder.layer.1.output.dense.weight"].shape == (F, H)
    assert arrays["pooler.dense.weight"].shape == (H, H)
    sd = hf.state_dict()
    assert np.array_equal(arrays["encoder.layer.0.attention.qkv.weight"][:, H:2 * H], sd["encoder.layer.0.attention.self.key.weight"].numpy().T)
    assert not any(".attention.self." in k for k in arrays)
    path = tmp_path / "m.npz"
    np.savez_compressed(path, **arrays)
    got = read_back(path)
    assert all(np.array_equal(got[k], v) for k, v in arrays.items())
