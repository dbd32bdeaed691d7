"""Tensor hand-off helpers (python/turbo_transformers/layers/utils.py:21-54 of the reference)."""
from typing import Optional, Union

import numpy as np
import torch
import torch.utils.dlpack as dlpack

from .._cxx import cxx

__all__ = ['try_convert', 'convert2tt_tensor', 'to_param_dict_convert_tt', 'to_param_dict', 'create_empty_if_none', 'AnyTensor',
           'use_current_stream']

AnyTensor = Union[cxx.Tensor, torch.Tensor]


def convert2tt_tensor(t: torch.Tensor):
    """Zero-copy alias of a torch tensor (the layer never writes it)."""
    return cxx.Tensor.from_dlpack(dlpack.to_dlpack(t.detach()))


def try_convert(t, device: Optional[torch.device] = None):
    if isinstance(t, torch.Tensor):
        return convert2tt_tensor(t)
    if isinstance(t, np.ndarray):
        on_gpu = device is None or "cuda" in str(getattr(device, "type", device))
        return cxx.nparray2tensor(t, "GPU" if on_gpu else "CPU")
    return t


def to_param_dict_convert_tt(torch_module: torch.nn.Module):
    return {k: convert2tt_tensor(v) for k, v in torch_module.named_parameters()}


def to_param_dict(torch_module: torch.nn.Module):
    return {k: v for k, v in torch_module.named_parameters()}


def create_empty_if_none(output):
    return output if output is not None else cxx.Tensor.create_empty()


def use_current_stream(t=None):
    """Point the device's kernel stream at torch's current stream so both stay ordered."""
    dev = t.device.index if isinstance(t, torch.Tensor) and t.is_cuda else torch.cuda.current_device()
    cxx.set_stream(dev, torch.cuda.current_stream(dev).cuda_stream)
    return dev
