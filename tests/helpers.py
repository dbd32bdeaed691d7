"""Shared helpers of the GPU parity tests (numpy oracle in, torch device tensors out)."""
import numpy as np
import torch

from turbotransformers_b200 import _capi

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
# tolerance (max-abs) for values of order one, per storage type
ATOL = {"f32": 1e-4, "f16": 4e-3, "bf16": 3e-2}


def dev(a, dt="f32"):
    """numpy array -> contiguous cuda tensor of the storage type `dt` ('f32'|'f16'|'bf16'|torch dtype)."""
    t = torch.from_numpy(np.ascontiguousarray(a))
    if t.is_floating_point():
        t = t.to(TORCH_DT[dt] if isinstance(dt, str) else dt)
    return t.cuda().contiguous()


def host(t):
    return t.detach().float().cpu().numpy()


def rounded(a, dt):
    """fp32 numpy array rounded through the storage type, so oracle and kernel see the same inputs."""
    if dt == "f32":
        return np.asarray(a, np.float32)
    return torch.from_numpy(np.asarray(a, np.float32)).to(TORCH_DT[dt]).float().numpy()


def code(dt):
    return _capi.dtype_code(TORCH_DT[dt])


def rng(seed):
    return np.random.default_rng(seed)


def maxdiff(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max()) if np.size(a) else 0.0
