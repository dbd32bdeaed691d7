"""ctypes binding of libttb.so (include/ttb.h). Loading is strict: a missing library or symbol raises.

This module is plumbing for tests, the benchmark and the no-torch users of the C ABI; the C++ layer
classes link the same library directly.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libttb.so")

OK = 0
F32, F16, BF16, I8 = 0, 1, 2, 3
ACT_GELU, ACT_TANH, ACT_RELU = 0, 1, 2
POOL_FIRST, POOL_LAST, POOL_MEAN, POOL_MAX = 0, 1, 2, 3
EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_BIAS_TANH = 0, 1, 2, 3, 4
ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_OOM, ERR_DEVICE_WAIT, ERR_BAD_INDEX = 1, 2, 3, 4, 5, 6

p, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

class LinearArgs(C.Structure):
    """ttb_linear_args of include/ttb.h."""
    _fields_ = [("dtype", i32), ("out_dtype", i32), ("A", p), ("A2", p), ("lda", i64), ("W", p), ("W2", p), ("bias", p),
                ("residual", p), ("ldr", i64), ("M", i64), ("N", i64), ("K", i64), ("epilogue", i32), ("out", p), ("out_lo", p),
                ("ldo", i64)]


# name -> (restype, argtypes); must list every function declared in include/ttb.h
SIGNATURES = {
    "ttb_ctx_create": (i32, [i32, p, C.POINTER(p)]),
    "ttb_ctx_destroy": (i32, [p]),
    "ttb_ctx_set_stream": (i32, [p, p]),
    "ttb_ctx_stream": (p, [p]),
    "ttb_ctx_device": (i32, [p]),
    "ttb_ctx_sync": (i32, [p]),
    "ttb_last_error": (C.c_char_p, [p]),
    "ttb_device_status": (i32, [p]),
    "ttb_launch_count": (C.c_uint64, [p]),
    "ttb_version": (C.c_char_p, []),
    "ttb_alloc": (i32, [p, sz, C.c_char_p, C.POINTER(p)]),
    "ttb_free": (i32, [p, p, C.c_char_p]),
    "ttb_pool_stats": (i32, [p, C.POINTER(sz), C.POINTER(sz), C.POINTER(C.c_uint64)]),
    "ttb_pool_set_limit": (i32, [p, sz]),
    "ttb_plan_activations": (i32, [p, i64, i64, i64, i64, i64, i64, i32, C.POINTER(sz)]),
    "ttb_memcpy_h2d": (i32, [p, p, p, sz]),
    "ttb_memcpy_d2h": (i32, [p, p, p, sz]),
    "ttb_copy_2d": (i32, [p, p, sz, p, sz, sz, sz]),
    "ttb_arena_begin": (i32, [p, sz]),
    "ttb_arena_end": (i32, [p, p, p]),
    "ttb_arena_release": (i32, [p, p]),
    "ttb_bytes_allocated_total": (i32, [p, p]),
    "ttb_kv_cache_append": (i32, [p, i32, p, i64, i64, i64, i64, p, p, i64]),
    "ttb_attention_decode": (i32, [p, i32, p, i64, i64, i64, i64, p, p, i64, f32, p]),
    "ttb_matmul": (i32, [p, i32, p, i32, p, i32, i64, i64, i64, f32, f32, p]),
    "ttb_batch_matmul": (i32, [p, i32, p, i32, p, i32, i64, i64, i64, i64, f32, f32, p]),
    "ttb_split_add_bias_transpose": (i32, [p, i32, p, p, i64, i64, i64, i64, p, p, p]),
    "ttb_transpose_for_score": (i32, [p, i32, p, i64, i64, i64, i64, p]),
    "ttb_add_bias_transpose_for_score": (i32, [p, i32, p, p, i64, i64, i64, i64, p]),
    "ttb_split_add_bias_transpose_pad": (i32, [p, i32, p, p, p, i64, i64, i64, i64, p, p, p]),
    "ttb_transpose_for_score_pad": (i32, [p, i32, p, p, i64, i64, i64, i64, p]),
    "ttb_add_bias_transpose_for_score_pad": (i32, [p, i32, p, p, p, i64, i64, i64, i64, p]),
    "ttb_mask_softmax": (i32, [p, i32, p, p, i64, i64, i64, i64, f32, i32]),
    "ttb_add_bias_layernorm": (i32, [p, i32, p, p, p, p, p, i64, i64, f32]),
    "ttb_layernorm": (i32, [p, i32, p, p, p, p, i64, i64, f32]),
    "ttb_layernorm_planes": (i32, [p, i32, i32, p, p, p, p, p, p, i64, i64, f32]),
    "ttb_embedding_ln_planes": (i32, [p, i32, p, p, p, p, i64, i64, i64, p, p, p, p, p, i64, i64, i64, i64, f32, p, p, p]),
    "ttb_add_bias_act": (i32, [p, i32, p, p, i64, i64, i32]),
    "ttb_lookup_embedding": (i32, [p, i32, p, p, p, i64, i64, i64, i32]),
    "ttb_add_bias": (i32, [p, i32, p, p, i64, i64]),
    "ttb_add_input_bias": (i32, [p, i32, p, p, p, i64, i64, p]),
    "ttb_seq_pool": (i32, [p, i32, p, i64, i64, i64, i32, p]),
    "ttb_seq_pool_varlen": (i32, [p, i32, p, p, i64, i64, i32, p]),
    "ttb_prepare_bert_masks": (i32, [p, i64, i64, p, p, p, p, p]),
    "ttb_prepack_weight": (i32, [p, i32, p, i32, i64, i64, i32, p]),
    "ttb_prepack_weight_int8": (i32, [p, i32, p, i32, i64, i64, p, p]),
    "ttb_linear": (i32, [p, i32, p, i64, p, p, p, i64, i64, i64, i64, i32, p, i64]),
    "ttb_linear_ex": (i32, [p, C.POINTER(LinearArgs)]),
    "ttb_split_tf32": (i32, [p, p, i64, p, p]),
    "ttb_linear_layernorm": (i32, [p, i32, p, i64, p, p, p, i64, p, p, f32, i64, i64, i64, p, i64]),
    "ttb_prepack_weight_int8_affine": (i32, [p, i32, p, i32, i64, i64, p, p, p]),
    "ttb_quantize_tensor_affine": (i32, [p, i32, p, i64, i64, p, p]),
    "ttb_linear_int8_affine": (i32, [p, i32, p, p, p, p, p, p, p, i64, i64, i64, i64, i32, p, i64]),
    "ttb_linear_int8": (i32, [p, i32, p, p, p, p, p, p, i64, i64, i64, i64, i32, p, i64]),
    "ttb_linear_int8_dynamic_noalloc": (i32, [p, i32, p, p, p, p, p, i64, i64, i64, i64, i32, p, i64]),
    "ttb_quantize_rows_int8": (i32, [p, i32, p, i64, i64, p, p]),
    "ttb_linear_int8_rowmax": (i32, [p, i32, p, p, p, p, p, p, i64, i64, i64, i64, i32, p, i64, p]),
    "ttb_quantize_rows_int8_given_max": (i32, [p, i32, p, i64, i64, p, p, p]),
    "ttb_layernorm_quant_int8": (i32, [p, i32, p, p, p, p, p, p, i64, i64, f32]),
    "ttb_attention_fwd": (i32, [p, i32, p, i64, p, i64, i64, i64, i64, p, i64, i64, i32, f32, p]),
    "ttb_embedding_ln": (i32, [p, i32, p, p, p, p, i64, i64, i64, p, p, p, p, p, i64, i64, i64, i64, f32, p]),
    "ttb_build_cu_seqlens": (i32, [p, p, i64, p]),
    "ttb_selftest_bounded_wait": (i32, [p, i64, p]),
}

_lib = None


class TTBError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"ttb status {code}: {msg}")
        self.code = code


def lib():
    """The loaded library. Raises if libttb.so has not been built (python -m turbotransformers_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m turbotransformers_b200.build`; "
                               "there is no fallback path")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def dtype_code(torch_dtype):
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int8: I8}[torch_dtype]


class Context:
    """A ttb_ctx bound to a device and (by default) torch's current stream on it."""

    def __init__(self, device=0, stream="torch"):
        import torch
        self.device = int(device)
        if stream == "torch":
            stream = torch.cuda.current_stream(self.device).cuda_stream
        h = p()
        s = lib().ttb_ctx_create(self.device, p(stream) if stream else None, C.byref(h))
        if s != OK:
            raise TTBError(s, "ttb_ctx_create failed")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            lib().ttb_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, status):
        if status != OK:
            raise TTBError(status, lib().ttb_last_error(self.h).decode())

    def call(self, name, *args):
        """Call ttb_<name>(ctx, *args); torch tensors are passed as their data pointers."""
        conv = [p(a.data_ptr()) if hasattr(a, "data_ptr") else a for a in args]
        self.check(getattr(lib(), "ttb_" + name)(self.h, *conv))

    def linear_ex(self, dtype, out_dtype, A, W, M, N, K, epilogue, out, A2=None, W2=None, bias=None, residual=None, out_lo=None,
                  lda=None, ldr=None, ldo=None):
        """ttb_linear_ex with the argument block filled from tensors (None = NULL)."""
        ptr = lambda t: (t.data_ptr() if t is not None else None)
        a = LinearArgs(dtype, out_dtype, ptr(A), ptr(A2), lda or K, ptr(W), ptr(W2), ptr(bias), ptr(residual), ldr or N, M, N, K,
                       epilogue, ptr(out), ptr(out_lo), ldo or N)
        self.check(lib().ttb_linear_ex(self.h, C.byref(a)))

    def set_stream(self, cuda_stream):
        """Queue what follows on this cudaStream_t (an int; 0 = the legacy default stream)."""
        self.check(lib().ttb_ctx_set_stream(self.h, p(cuda_stream) if cuda_stream else None))

    def device_status(self):
        return lib().ttb_device_status(self.h)

    def launches(self):
        return int(lib().ttb_launch_count(self.h))
