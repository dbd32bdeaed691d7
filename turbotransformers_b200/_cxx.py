"""Loads the in-tree pybind module (C++ layer classes over libttb.so). There is no fallback: if the
module cannot be imported it is built once from source, and a failure to build or load raises."""
import importlib
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def _load():
    try:
        return importlib.import_module("turbotransformers_b200.turbo_transformers_cxx")
    except ImportError as first:
        from . import build
        try:
            build.build_all()
        except Exception as e:
            raise ImportError("turbo_transformers_cxx is not built and building it failed: %s (import error: %s)" % (e, first))
        return importlib.import_module("turbotransformers_b200.turbo_transformers_cxx")


cxx = _load()

# classes the Python layer subclasses: a module built from older sources lacks some of them
_missing = [n for n in ("BertAttention", "DistrillFFN", "AlbertLayer", "NpzBertModel", "npz_load", "arena_begin") if not hasattr(cxx, n)]
if _missing:
    raise ImportError("turbo_transformers_cxx was built from older sources (no %s): rebuild with `python %s`"
                      % (", ".join(_missing), os.path.join(_HERE, "build.py")))
