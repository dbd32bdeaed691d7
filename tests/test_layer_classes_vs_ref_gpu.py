"""The C++ layer classes that have no golden fixture, each against the same class of the compiled reference CPU code
(oracle/_ref) on identical seeded weights and inputs; the numpy restatement stands in when that build is absent:

  AlbertLayer            layers/albert_layer.cpp:31-50
  DistrillFFN            layers/positionwise_ffn.cpp:79-123
  FusedAddBiasGELU       layers/addbias_act.cpp:20-23
  FusedAddBiasLayerNorm  layers/addbias_layernorm.cpp:20-24

fp32 within 2e-4, fp16 within 2e-2 (outputs are layer-normalised, order one).
"""
import numpy as np
import pytest
import torch

import turbotransformers_b200 as tt
from oracle import ref_driver, restate

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
cxx = tt._cxx_module
DT = {"f32": (torch.float32, 2e-4), "f16": (torch.float16, 2e-2)}
HAVE_REF = ref_driver.available()


def ours(a, dtype):
    """numpy fp32 -> this library's Tensor on the GPU in `dtype` (a private copy)."""
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype).contiguous()
    return cxx.Tensor.from_dlpack(torch.utils.dlpack.to_dlpack(t))


def back(t):
    return torch.utils.dlpack.from_dlpack(t.to_dlpack()).float().cpu().numpy()


def ffn_weights(hidden, ffn, seed):
    r = np.random.default_rng(seed)
    return {"w1": (r.standard_normal((hidden, ffn)) * 0.05).astype(np.float32), "b1": (r.standard_normal(ffn) * 0.02).astype(np.float32),
            "w2": (r.standard_normal((ffn, hidden)) * 0.05).astype(np.float32), "b2": (r.standard_normal(hidden) * 0.02).astype(np.float32),
            "g": (1.0 + 0.1 * r.standard_normal(hidden)).astype(np.float32), "b": (0.1 * r.standard_normal(hidden)).astype(np.float32),
            "x": r.standard_normal((3, 40, hidden)).astype(np.float32)}


def restate_post_ln_ffn(w):
    inter = restate.add_bias_act(restate.mat_mul(w["x"], False, w["w1"], False), w["b1"], "gelu")
    out = restate.mat_mul(inter, False, w["w2"], False).reshape(w["x"].shape)
    return inter.reshape(w["x"].shape[:-1] + (-1, )), restate.add_bias_layer_norm(w["x"], w["b2"], w["g"], w["b"], out, 1e-12)


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_albert_layer_against_reference_class(dt):
    w = ffn_weights(256, 1024, 21)
    if HAVE_REF:
        T, E = ref_driver.T, ref_driver.E
        ref = ref_driver.load().AlbertLayer(T(w["w1"]), T(w["b1"]), T(w["w2"]), T(w["b2"]), T(w["g"]), T(w["b"]))
        hid, out = E(), E()
        ref(T(w["x"]), hid, out)
        want_hid, want = ref_driver.back(hid).numpy(), ref_driver.back(out).numpy()
    else:
        want_hid, want = restate_post_ln_ffn(w)
    dtype, tol = DT[dt]
    layer = cxx.AlbertLayer(*(ours(w[k], dtype) for k in ("w1", "b1", "w2", "b2", "g", "b")))
    hid, out = cxx.Tensor.create_empty(), cxx.Tensor.create_empty()
    layer(ours(w["x"], dtype), hid, out)
    assert np.abs(back(hid) - want_hid).max() < tol
    assert np.abs(back(out) - want).max() < tol


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("is_trans", [False, True])
def test_distill_ffn_against_reference_class(dt, is_trans):
    w = ffn_weights(256, 1024, 22)
    w1, w2 = (np.ascontiguousarray(w[k].T) if is_trans else w[k] for k in ("w1", "w2"))
    if HAVE_REF:
        T, E = ref_driver.T, ref_driver.E
        ref = ref_driver.load().DistrillFFN(T(w1), T(w["b1"]), T(w2), T(w["b2"]), T(w["g"]), T(w["b"]))
        out = E()
        ref(T(w["x"]), out, is_trans)
        want = ref_driver.back(out).numpy()
    else:
        want = restate_post_ln_ffn(w)[1]
    dtype, tol = DT[dt]
    layer = cxx.DistrillFFN(ours(w1, dtype), ours(w["b1"], dtype), ours(w2, dtype), ours(w["b2"], dtype), ours(w["g"], dtype),
                            ours(w["b"], dtype))
    out = cxx.Tensor.create_empty()
    layer(ours(w["x"], dtype), out, is_trans)
    assert np.abs(back(out) - want).max() < tol


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_fused_add_bias_gelu_and_layernorm_against_reference_classes(dt):
    r = np.random.default_rng(23)
    H, F = 256, 1024
    proj = r.standard_normal((2, 37, F)).astype(np.float32)          # a projection computed elsewhere, bias not yet added
    bias_f = (r.standard_normal(F) * 0.5).astype(np.float32)
    out0 = r.standard_normal((2, 37, H)).astype(np.float32)
    resid = r.standard_normal((2, 37, H)).astype(np.float32)
    bias_h = (r.standard_normal(H) * 0.5).astype(np.float32)
    g = (1.0 + 0.1 * r.standard_normal(H)).astype(np.float32)
    b = (0.1 * r.standard_normal(H)).astype(np.float32)
    if HAVE_REF:
        T = ref_driver.T
        ref = ref_driver.load()
        t = T(proj)
        ref.FusedAddBiasGELU(T(bias_f))(t)
        want_gelu = ref_driver.back(t).numpy()
        o = T(out0)
        ref.FusedAddBiasLayerNorm(T(bias_h), T(g), T(b))(T(resid), o)
        want_ln = ref_driver.back(o).numpy()
    else:
        want_gelu = restate.add_bias_act(proj.copy(), bias_f, "gelu")
        want_ln = restate.add_bias_layer_norm(resid, bias_h, g, b, out0.copy(), 1e-12)
    dtype, tol = DT[dt]
    t = ours(proj, dtype)
    cxx.FusedAddBiasGELU(ours(bias_f, dtype))(t)
    assert np.abs(back(t) - want_gelu).max() < tol
    o = ours(out0, dtype)
    cxx.FusedAddBiasLayerNorm(ours(bias_h, dtype), ours(g, dtype), ours(b, dtype))(ours(resid, dtype), o)
    assert np.abs(back(o) - want_ln).max() < tol
