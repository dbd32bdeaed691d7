"""HuggingFace BertModel -> the `.npz` archive the C++ API loads (the role of the reference's
tools/convert_huggingface_bert_pytorch_to_npz.py:23-74).

    python -m turbotransformers_b200.tools.convert_huggingface_bert_pytorch_to_npz MODEL_DIR_OR_NAME OUT.npz [--stored]

Archive layout (what `BertModel(filename, ...)` in csrc/host/bert_model.cpp and the `from_npz` loaders read):
    embeddings.{word,position,token_type}_embeddings.weight, embeddings.LayerNorm.{weight,bias}
    encoder.layer.N.attention.qkv.{weight [H,3H] columns q|k|v, bias [3H]}
    encoder.layer.N.attention.output.dense.{weight [H,H] as [in,out], bias}, ...output.LayerNorm.{weight,bias}
    encoder.layer.N.intermediate.dense.{weight [H,F] as [in,out], bias}
    encoder.layer.N.output.dense.{weight [F,H] as [in,out], bias}, encoder.layer.N.output.LayerNorm.{weight,bias}
    pooler.dense.{weight [H,H] as [in,out], bias}
Every Linear weight is stored [in, out] (torch keeps [out, in]); members are float32; the archive is deflated unless --stored.
"""
import sys

import numpy as np
import torch


def bert_state_to_arrays(model: torch.nn.Module) -> dict:
    """name -> float32 numpy array in the archive layout, from a HuggingFace-style BertModel module."""
    sd = {k: v.detach().float().cpu() for k, v in model.state_dict().items() if v.dtype.is_floating_point}
    out = {}
    linear_suffixes = ("attention.output.dense.weight", "intermediate.dense.weight", "output.dense.weight", "pooler.dense.weight")
    for name, w in sd.items():
        if name.endswith("attention.self.query.weight"):
            pre = name[:-len("self.query.weight")]
            qkv = torch.cat([sd[pre + "self.query.weight"], sd[pre + "self.key.weight"], sd[pre + "self.value.weight"]], 0)  # [3H, H]
            out[pre + "qkv.weight"] = qkv.t().contiguous().numpy()
            out[pre + "qkv.bias"] = torch.cat([sd[pre + "self.query.bias"], sd[pre + "self.key.bias"], sd[pre + "self.value.bias"]], 0).numpy()
        elif ".attention.self." in name:
            continue  # folded into qkv above
        elif name.endswith(linear_suffixes):
            out[name] = w.t().contiguous().numpy()
        else:
            out[name] = w.contiguous().numpy()
    return out


def save_bert_npz(model: torch.nn.Module, path: str, compressed: bool = True) -> None:
    arrays = bert_state_to_arrays(model)
    (np.savez_compressed if compressed else np.savez)(path, **arrays)


def main(argv):
    if len(argv) not in (3, 4) or (len(argv) == 4 and argv[3] != "--stored"):
        print(__doc__)
        return 2
    from transformers import BertModel
    torch.set_grad_enabled(False)
    save_bert_npz(BertModel.from_pretrained(argv[1]), argv[2], compressed=len(argv) == 3)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
