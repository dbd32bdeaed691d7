"""python/turbo_transformers/layers/return_type.py:27-45 of the reference."""
import enum
from typing import Optional

import torch
import torch.utils.dlpack as dlpack

from .._cxx import cxx

__all__ = ['ReturnType', 'convert_returns_as_type']


class ReturnType(enum.Enum):
    turbo_transformers = 0
    TORCH = 1
    NUMPY = 2


def convert_returns_as_type(tensor, rtype: Optional[ReturnType]):
    """A cxx.Tensor as the requested type. TORCH hands the storage over through DLPack (the cxx.Tensor
    becomes null, as in the reference); NUMPY copies to the host (fp32 tensors only)."""
    if rtype is None:
        rtype = ReturnType.TORCH
    if rtype == ReturnType.turbo_transformers:
        return tensor
    if rtype == ReturnType.TORCH:
        return dlpack.from_dlpack(tensor.to_dlpack())
    if rtype == ReturnType.NUMPY:
        if tensor.dtype() == "float32":
            return cxx.tensor2nparrayf(tensor)
        return dlpack.from_dlpack(tensor.to_dlpack()).float().cpu().numpy()
    raise NotImplementedError()
