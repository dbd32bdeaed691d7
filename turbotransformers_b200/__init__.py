"""B200-native transformer-layer runtime with the Python surface of `turbo_transformers`.

    import turbotransformers_b200 as turbo_transformers
    tt_model = turbo_transformers.BertModel.from_torch(hf_bert.half(), torch.device("cuda:0"))
    sequence_output, pooled = tt_model(input_ids)

Everything computes on the GPU through hand-written sm_100a kernels; importing the package on a machine
without the built native libraries raises.
"""
from .layers import *  # noqa: F401,F403
from .utils import *  # noqa: F401,F403
from ._cxx import cxx as _cxx_module

config = _cxx_module.config
