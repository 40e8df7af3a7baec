"""ctypes binding of libkiln_cuda.so — the one place the C ABI of include/kiln_cuda.h is mirrored.

There is no fallback: if the shared library is missing or fails to load, importing the symbols
raises. A CPU path does not exist in this package.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libkiln_cuda.so"

# status codes (include/kiln_cuda.h)
KC_OK, KC_ERR_INVALID, KC_ERR_CUDA, KC_ERR_OOM, KC_ERR_UNSUPPORTED, KC_ERR_TIMEOUT, KC_ERR_CAPACITY = range(7)
# dtype tags
KC_BOOL, KC_U8, KC_U16, KC_U32, KC_I32, KC_F16, KC_BF16, KC_F32 = range(1, 9)
KC_ARCH_LLAMA, KC_ARCH_QWEN2, KC_ARCH_GEMMA2 = 0, 1, 2
KC_ROPE_DEFAULT, KC_ROPE_LINEAR, KC_ROPE_LLAMA3 = 0, 1, 2


class KcModelDesc(C.Structure):
    _fields_ = [
        ("arch", C.c_int32), ("hidden_size", C.c_int32), ("num_layers", C.c_int32), ("num_heads", C.c_int32),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("intermediate_size", C.c_int32),
        ("vocab_size", C.c_int32), ("bits", C.c_int32), ("group_size", C.c_int32),
        ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("rope_traditional", C.c_int32),
        ("rope_scaling", C.c_int32), ("rope_factor", C.c_float), ("rope_low_freq_factor", C.c_float),
        ("rope_high_freq_factor", C.c_float), ("rope_original_max_position", C.c_float),
        ("tie_word_embeddings", C.c_int32), ("attn_logit_softcapping", C.c_float),
        ("final_logit_softcapping", C.c_float), ("query_pre_attn_scalar", C.c_float),
        ("sliding_window", C.c_int32), ("max_step_tokens", C.c_int32), ("max_step_seqs", C.c_int32),
        ("tp_rank", C.c_int32), ("tp_world", C.c_int32),
    ]


class KcTensorView(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * 4), ("on_device", C.c_int32)]


class KcSeqStep(C.Structure):
    _fields_ = [("len", C.c_int32), ("offset", C.c_int32), ("sample_rows", C.c_int32), ("n_blocks", C.c_int32),
                ("blocks", C.POINTER(C.c_uint32))]


_P = C.c_void_p
_SIGNATURES = {
    "kc_ctx_create": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "kc_ctx_destroy": (None, [_P]),
    "kc_last_error": (C.c_char_p, []),
    "kc_live_objects": (C.c_int64, []),
    "kc_sync": (C.c_int, [_P]),
    "kc_ctx_stream": (_P, [_P]),
    "kc_device_status": (C.c_int, [_P, C.POINTER(C.c_uint32)]),
    "kc_launch_count": (C.c_int64, [_P]),
    "kc_last_step_ms": (C.c_double, [_P]),
    "kc_profile_enable": (C.c_int, [_P, C.c_int32]),
    "kc_profile_read": (C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
    "kc_model_load": (C.c_int, [_P, C.POINTER(KcModelDesc), C.POINTER(KcTensorView), C.c_size_t, C.POINTER(_P)]),
    "kc_model_free": (None, [_P]),
    "kc_envelope": (C.c_int, [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "kc_model_weight_bytes": (C.c_int64, [_P]),
    "kc_kv_create": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(_P)]),
    "kc_kv_free": (None, [_P]),
    "kc_kv_copy_block": (C.c_int, [_P, C.c_uint32, C.c_uint32]),
    "kc_kv_read_block": (C.c_int, [_P, C.c_uint32, _P, C.c_size_t]),
    "kc_kv_write_block": (C.c_int, [_P, C.c_uint32, _P, C.c_size_t]),
    "kc_kv_block_bytes": (C.c_int64, [_P]),
    "kc_kv_allocated_bytes": (C.c_int64, [_P]),
    "kc_kv_reset": (C.c_int, [_P]),
    "kc_forward_step": (C.c_int, [_P, _P, C.POINTER(C.c_uint32), C.c_int32, C.POINTER(KcSeqStep), C.c_int32, C.c_int32,
                                  C.POINTER(_P), C.POINTER(C.c_int32)]),
    "kc_greedy_rows": (C.c_int, [_P, _P, C.c_int32, C.c_int32, C.c_int32, _P]),
    "kc_verify_accept": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_int32, C.c_int32, _P, _P, _P]),
    "kc_verify_step": (C.c_int, [_P, _P, C.POINTER(C.c_uint32), C.c_int32, C.POINTER(KcSeqStep), C.c_int32,
                                 C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "kc_decode_launch": (C.c_int, [_P, _P, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.POINTER(KcSeqStep), C.c_int32,
                                   C.POINTER(C.c_uint64)]),
    "kc_decode_collect": (C.c_int, [_P, C.c_uint64, C.POINTER(C.c_uint32), C.c_int32]),
    "kc_draft_stats": (C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int32]),
    "kc_draft_chain": (C.c_int, [_P, _P, C.c_uint32, C.c_int32, C.POINTER(C.c_uint32), C.c_int32, C.c_int32,
                                 C.POINTER(C.c_uint32)]),
    "kc_qweight_create": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(_P)]),
    "kc_qweight_free": (None, [_P]),
    "kc_quantized_matmul": (C.c_int, [_P, _P, _P, C.c_int32, _P]),
    "kc_quantized_matmul_stream": (C.c_int, [_P, _P, _P, C.c_int32, _P]),
    "kc_quantized_matmul_gemv": (C.c_int, [_P, _P, _P, C.c_int32, _P]),
    "kc_tp_export": (C.c_int, [_P, _P]),
    "kc_tp_attach": (C.c_int, [_P, _P]),
    "kc_model_set_stream_lane": (C.c_int, [_P, C.c_int32]),
    "kc_quantized_matmul_static": (C.c_int, [_P, _P, _P, C.c_int32, _P]),
    "kc_static_scratch_bytes": (C.c_int64, []),
    "kc_rms_norm": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, C.c_float, _P]),
    "kc_paged_attention": (C.c_int, [_P, _P, C.c_int32, _P, C.c_int32, C.c_int32, C.POINTER(KcSeqStep), C.c_int32,
                                     C.c_float, C.c_float, C.c_int32, _P]),
    "kc_rope_kv_write": (C.c_int, [_P, _P, C.c_int32, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32,
                                   C.POINTER(KcSeqStep), C.c_int32, _P]),
    "kc_tp_init": (C.c_int, [_P, _P, C.c_int32, C.c_int32]),
    "kc_tp_unique_id": (C.c_int, [_P]),
}

_lib = None


def exported_symbols() -> list[str]:
    """Every entry point include/kiln_cuda.h declares."""
    return sorted(_SIGNATURES)


def lib() -> C.CDLL:
    """Loads libkiln_cuda.so once; raises if it is absent (run ``python -m kiln_b200.build``)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m kiln_b200.build` "
                               "(there is no CPU or PyTorch fallback for the verify path)")
        # libkiln_cuda.so needs libnccl.so.2. torch bundles a newer NCCL under the same soname, so torch is
        # imported first: whichever copy is loaded first serves both, and torch's own symbols need the newer one.
        import torch  # noqa: F401
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class KcError(RuntimeError):
    """A non-zero status from the C ABI; carries the code and the library's message."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[kc status {code}] {message}")
        self.code = code
        self.message = message


def check(code: int) -> None:
    if code != KC_OK:
        raise KcError(code, lib().kc_last_error().decode("utf-8", "replace"))
