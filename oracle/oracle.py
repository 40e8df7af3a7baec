"""ctypes wrapper of the CPU oracle (oracle/kiln_oracle.cpp). TEST INFRASTRUCTURE.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may
import this module. Floating-point parity is unpinned (see the header of kiln_oracle.cpp).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

from kiln_b200 import _lib as L
from kiln_b200.api import ModelConfig, SeqStep, StepBatch, _PackedStep, tensor_views

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libkiln_oracle.so"
_P = C.c_void_p
_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "kiln_oracle.cpp"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B" if force else "-s", "all"], check=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        h = C.CDLL(str(LIB_PATH))
        h.ko_last_error.restype = C.c_char_p
        h.ko_model_load.argtypes = [C.POINTER(L.KcModelDesc), C.POINTER(L.KcTensorView), C.c_size_t, C.POINTER(_P)]
        h.ko_model_free.argtypes = [_P]
        h.ko_model_set_layer_limit.argtypes = [_P, C.c_int]
        h.ko_kv_create.argtypes = [C.c_int] * 5 + [C.POINTER(_P)]
        h.ko_kv_free.argtypes = [_P]
        h.ko_kv_data.argtypes = [_P]
        h.ko_kv_data.restype = _P
        h.ko_kv_copy_block.argtypes = [_P, C.c_uint32, C.c_uint32]
        h.ko_forward_step.argtypes = [_P, _P, C.POINTER(C.c_uint32), C.c_int32, C.POINTER(L.KcSeqStep), C.c_int32, _P,
                                      C.POINTER(C.c_int32)]
        h.ko_greedy_rows.argtypes = [_P, C.c_int, C.c_int, C.c_int, _P]
        h.ko_quantized_matmul.argtypes = [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P]
        h.ko_rms_norm.argtypes = [_P, _P, C.c_int, C.c_int, C.c_float, _P]
        h.ko_paged_attention.argtypes = [_P, C.c_int, _P, C.c_int, C.c_int, C.POINTER(L.KcSeqStep), C.c_int, C.c_float,
                                         C.c_float, C.c_int, _P]
        _lib = h
    return _lib


def set_threads(n: int) -> int:
    """Sets the OpenMP thread count of the oracle (0: leave as is) and returns the count in force."""
    return int(lib().ko_set_threads(int(n)))


def set_weight_class(cls: int) -> None:
    """0 = MLX's row-vector (qmv) arithmetic class, 1 = its tile (qmm) class; see kiln_oracle.cpp."""
    lib().ko_set_weight_class(int(cls))


def _bf16_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _bf16_t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


class OracleKv:
    def __init__(self, layers: int, kv_heads: int, head_dim: int, num_blocks: int, block_size: int):
        self.shape = (layers, 2, num_blocks, kv_heads, block_size, head_dim)
        self._h = _P()
        lib().ko_kv_create(layers, kv_heads, head_dim, num_blocks, block_size, C.byref(self._h))

    def array(self) -> np.ndarray:
        """uint16 view (bf16 bits) of the pools [layers, 2, num_blocks, kv_heads, block_size, head_dim]."""
        n = int(np.prod(self.shape))
        buf = (C.c_uint16 * n).from_address(lib().ko_kv_data(self._h))
        return np.ctypeslib.as_array(buf).reshape(self.shape)

    def copy_block(self, src: int, dst: int) -> None:
        lib().ko_kv_copy_block(self._h, src, dst)

    def __del__(self):
        try:
            if self._h:
                lib().ko_kv_free(self._h)
                self._h = _P()
        except Exception:  # interpreter shutdown
            pass


class OracleModel:
    def __init__(self, config: ModelConfig, tensors: Dict[str, torch.Tensor]):
        self.config = config
        host = {k: v.detach().cpu().contiguous() for k, v in tensors.items()}
        arr, keep = tensor_views(host)
        desc = config.to_desc(1 << 20, 1 << 20)
        self._h = _P()
        if lib().ko_model_load(C.byref(desc), arr, len(host), C.byref(self._h)) != 0:
            raise RuntimeError(lib().ko_last_error().decode())
        del keep

    def set_layer_limit(self, layers: int) -> None:
        lib().ko_model_set_layer_limit(self._h, layers)

    def forward_step(self, batch: StepBatch, kv: OracleKv, want_logits: bool = True) -> Optional[torch.Tensor]:
        p = _PackedStep(batch)
        ns = sum(s.sample_rows for s in batch.seqs)
        out = np.zeros((max(ns, 1), self.config.vocab_size), dtype=np.uint16) if want_logits else None
        n_s = C.c_int32(0)
        rc = lib().ko_forward_step(self._h, kv._h, p.ids_p, p.n, p.seq_arr, p.n_seqs,
                                   out.ctypes.data if out is not None else None, C.byref(n_s))
        if rc != 0:
            raise RuntimeError(lib().ko_last_error().decode())
        if ns == 0 or out is None:
            return None
        return _bf16_t(out[:ns])

    def __del__(self):
        try:
            if self._h:
                lib().ko_model_free(self._h)
                self._h = _P()
        except Exception:  # interpreter shutdown
            pass


def greedy_rows(logits: torch.Tensor, normalize: bool = True) -> np.ndarray:
    a = _bf16_np(logits)
    out = np.zeros(a.shape[0], dtype=np.uint32)
    lib().ko_greedy_rows(a.ctypes.data, a.shape[0], a.shape[1], int(normalize), out.ctypes.data)
    return out


def quantized_matmul(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group: int) -> torch.Tensor:
    xa, sa, ba = _bf16_np(x), _bf16_np(scales), _bf16_np(biases)
    wa = w.detach().cpu().contiguous().numpy().view(np.uint32)
    m, k = xa.shape
    n = wa.shape[0]
    y = np.zeros((m, n), dtype=np.uint16)
    lib().ko_quantized_matmul(xa.ctypes.data, wa.ctypes.data, sa.ctypes.data, ba.ctypes.data, m, n, k, bits, group, y.ctypes.data)
    return _bf16_t(y)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xa, wa = _bf16_np(x), _bf16_np(w)
    y = np.zeros_like(xa)
    lib().ko_rms_norm(xa.ctypes.data, wa.ctypes.data, xa.shape[0], xa.shape[1], eps, y.ctypes.data)
    return _bf16_t(y)


def paged_attention(kv: OracleKv, layer: int, q: torch.Tensor, seqs: List[SeqStep], scale: float, softcap: float = 0.0,
                    window: int = 0) -> torch.Tensor:
    qa = _bf16_np(q)
    n, heads, hd = qa.shape
    p = _PackedStep(StepBatch([0] * n, seqs))
    out = np.zeros((n, heads * hd), dtype=np.uint16)
    lib().ko_paged_attention(kv._h, layer, qa.ctypes.data, n, heads, p.seq_arr, p.n_seqs, scale, softcap, window, out.ctypes.data)
    return _bf16_t(out)
