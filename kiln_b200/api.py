"""Host-side mirror of the reference's device boundary for the verify path, over the C ABI.

Names and argument meaning follow the reference (paths inside ikematta/kiln):
  SeqStep / StepBatch        crates/kiln-engine/src/step.rs:14-75
  StepModel.forward_step     crates/kiln-engine/src/step.rs:85-96
  PagedKv / KvSpec           crates/kiln-engine/src/paged.rs:28-386
  ModelConfig                crates/kiln-models/src/config.rs (mlx-lm config.json fields)

torch appears here only as a holder of host/device memory; every computation is a call into
libkiln_cuda.so. Nothing in this module has a CPU code path.
"""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _lib as L
from ._lib import KcError, check  # noqa: F401  (re-exported)


# --------------------------------------------------------------------------------------
# configuration
# --------------------------------------------------------------------------------------

@dataclass
class ModelConfig:
    """Geometry of one model, in mlx-lm ``config.json`` vocabulary (config.rs)."""
    model_type: str = "llama"          # "llama" | "qwen2" | "gemma2"
    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    bits: int = 4                      # quantization.bits        (config.rs:138-148)
    group_size: int = 64               # quantization.group_size
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_traditional: bool = False     # config.rs:172-173
    rope_scaling: Optional[dict] = None
    tie_word_embeddings: bool = False
    attn_logit_softcapping: float = 0.0
    final_logit_softcapping: float = 0.0
    query_pre_attn_scalar: float = 0.0
    sliding_window: int = 0
    qkv_bias: bool = False             # qwen2: q/k/v carry .bias (nn.rs:56)

    @property
    def arch(self) -> int:
        return {"llama": L.KC_ARCH_LLAMA, "qwen2": L.KC_ARCH_QWEN2, "gemma2": L.KC_ARCH_GEMMA2}[self.model_type]

    @classmethod
    def from_mlx_config(cls, cfg: dict) -> "ModelConfig":
        """Reads the fields the reference reads from config.json (config.rs: LlamaConfig, Qwen2Config, Gemma2Config)."""
        mt = cfg["model_type"]
        if mt not in ("llama", "qwen2", "gemma2"):
            raise ValueError(f"unsupported model_type {mt!r}")
        q = cfg.get("quantization") or {}
        if q.get("bits", 4) not in (4, 8) or q.get("group_size", 64) not in (32, 64, 128):
            raise ValueError(f"unsupported quantization {q}")  # config.rs:735-760
        heads = cfg["num_attention_heads"]
        c = cls(
            model_type=mt, hidden_size=cfg["hidden_size"], num_hidden_layers=cfg["num_hidden_layers"],
            num_attention_heads=heads, num_key_value_heads=cfg.get("num_key_value_heads", heads),
            head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
            intermediate_size=cfg["intermediate_size"], vocab_size=cfg["vocab_size"],
            bits=q.get("bits", 4), group_size=q.get("group_size", 64),
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-6 if mt != "llama" else 1e-5),
            rope_theta=cfg.get("rope_theta", 1e6 if mt == "qwen2" else 10000.0),
            rope_traditional=bool(cfg.get("rope_traditional", False)),
            rope_scaling=cfg.get("rope_scaling"),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", mt == "gemma2")),
            qkv_bias=(mt == "qwen2"),
        )
        if mt == "qwen2":
            c.head_dim = cfg["hidden_size"] // heads   # no override field (qwen2.rs:5-8)
        if mt == "gemma2":
            c.attn_logit_softcapping = float(cfg.get("attn_logit_softcapping", 50.0))
            c.final_logit_softcapping = float(cfg.get("final_logit_softcapping", 30.0))
            c.query_pre_attn_scalar = float(cfg.get("query_pre_attn_scalar", c.head_dim))
            c.tie_word_embeddings = True
        return c

    def to_desc(self, max_step_tokens: int, max_step_seqs: int, tp_rank: int = 0, tp_world: int = 1) -> L.KcModelDesc:
        d = L.KcModelDesc()
        d.arch = self.arch
        d.hidden_size, d.num_layers = self.hidden_size, self.num_hidden_layers
        d.num_heads, d.num_kv_heads, d.head_dim = self.num_attention_heads, self.num_key_value_heads, self.head_dim
        d.intermediate_size, d.vocab_size = self.intermediate_size, self.vocab_size
        d.bits, d.group_size = self.bits, self.group_size
        d.rms_norm_eps, d.rope_theta = self.rms_norm_eps, self.rope_theta
        d.rope_traditional = int(self.rope_traditional)
        rs = self.rope_scaling or {}
        kind = rs.get("rope_type", rs.get("type", "default"))
        if kind == "llama3":
            d.rope_scaling = L.KC_ROPE_LLAMA3
            d.rope_factor = float(rs["factor"])
            d.rope_low_freq_factor = float(rs.get("low_freq_factor", 1.0))
            d.rope_high_freq_factor = float(rs.get("high_freq_factor", 4.0))
            d.rope_original_max_position = float(rs.get("original_max_position_embeddings", 8192))
        elif kind == "linear":
            d.rope_scaling = L.KC_ROPE_LINEAR
            d.rope_factor = float(rs["factor"])
        elif kind == "default":
            d.rope_scaling = L.KC_ROPE_DEFAULT
        else:
            raise ValueError(f"rope_scaling {kind!r} is outside this path (nn.rs:1478 yarn is used by no target config)")
        d.tie_word_embeddings = int(self.tie_word_embeddings)
        d.attn_logit_softcapping = self.attn_logit_softcapping
        d.final_logit_softcapping = self.final_logit_softcapping
        d.query_pre_attn_scalar = self.query_pre_attn_scalar
        d.sliding_window = self.sliding_window
        d.max_step_tokens, d.max_step_seqs = max_step_tokens, max_step_seqs
        d.tp_rank, d.tp_world = tp_rank, tp_world
        return d

    def kv_bytes_per_token(self) -> int:
        return self.num_hidden_layers * 2 * self.num_key_value_heads * self.head_dim * 2


# --------------------------------------------------------------------------------------
# step description (step.rs)
# --------------------------------------------------------------------------------------

@dataclass
class SeqStep:
    """One sequence's contribution to a step (step.rs:14-37)."""
    len: int
    offset: int
    sample_rows: int
    blocks: Sequence[int]


@dataclass
class StepBatch:
    """One forward pass: ids are the concatenation of every segment, in seqs order (step.rs:62-75)."""
    ids: Sequence[int]
    seqs: List[SeqStep]
    pad_rows: int = 0

    def num_tokens(self) -> int:
        return len(self.ids)


class _PackedStep:
    """ctypes view of a StepBatch; keeps the arrays alive for the duration of the call."""

    def __init__(self, batch: StepBatch):
        self.ids = np.ascontiguousarray(np.asarray(batch.ids, dtype=np.uint32))
        self.n = int(self.ids.shape[0])
        self.n_seqs = len(batch.seqs)
        self.seq_arr = (L.KcSeqStep * max(1, self.n_seqs))()
        self._keep = []
        for i, s in enumerate(batch.seqs):
            blocks = np.ascontiguousarray(np.asarray(s.blocks, dtype=np.uint32))
            self._keep.append(blocks)
            self.seq_arr[i].len = int(s.len)
            self.seq_arr[i].offset = int(s.offset)
            self.seq_arr[i].sample_rows = int(s.sample_rows)
            self.seq_arr[i].n_blocks = int(blocks.shape[0])
            self.seq_arr[i].blocks = blocks.ctypes.data_as(C.POINTER(C.c_uint32))
        self.ids_p = self.ids.ctypes.data_as(C.POINTER(C.c_uint32))


# --------------------------------------------------------------------------------------
# device objects
# --------------------------------------------------------------------------------------

class _DevView:
    """Exposes a device pointer through __cuda_array_interface__ so torch can alias it."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


def _alias_bf16(ptr: int, shape, device: int) -> torch.Tensor:
    t = torch.as_tensor(_DevView(ptr, shape, "<i2"), device=f"cuda:{device}")
    return t.view(torch.bfloat16)


def _ptr(t) -> int:
    if isinstance(t, torch.Tensor):
        return t.data_ptr()
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    raise TypeError(type(t))


class Context:
    """One device + stream; the counterpart of kiln_mlx::init + Stream::gpu()."""

    def __init__(self, device: int = 0):
        self.device = device
        self._h = C.c_void_p()
        # handles created on this context: closed before the context itself, whatever order the interpreter
        # drops the Python objects in (a library handle must not outlive its context)
        self._children = weakref.WeakSet()
        check(L.lib().kc_ctx_create(device, C.byref(self._h)))

    def _adopt(self, child) -> None:
        self._children.add(child)

    def sync(self) -> None:
        check(L.lib().kc_sync(self._h))

    @staticmethod
    def tp_unique_id() -> bytes:
        """The 128 bytes of an NCCL unique id, to be created on rank 0 and handed to every rank's tp_init."""
        buf = (C.c_uint8 * 128)()
        check(L.lib().kc_tp_unique_id(buf))
        return bytes(buf)

    def tp_init(self, unique_id: bytes, rank: int, world: int) -> None:
        """Joins the tensor-parallel communicator (before any model of that world is loaded on this context)."""
        assert len(unique_id) == 128
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        check(L.lib().kc_tp_init(self._h, buf, rank, world))

    @property
    def stream(self) -> int:
        return int(L.lib().kc_ctx_stream(self._h) or 0)

    def device_status(self) -> int:
        st = C.c_uint32(0)
        check(L.lib().kc_device_status(self._h, C.byref(st)))
        return st.value

    def draft_stats(self, reset: bool = False):
        """(milliseconds inside kc_draft_chain, tokens proposed, calls) since creation or the last reset."""
        ms, tok, calls = C.c_double(0), C.c_int64(0), C.c_int64(0)
        check(L.lib().kc_draft_stats(self._h, C.byref(ms), C.byref(tok), C.byref(calls), int(reset)))
        return float(ms.value), int(tok.value), int(calls.value)

    def launch_count(self) -> int:
        return int(L.lib().kc_launch_count(self._h))

    def last_step_ms(self) -> float:
        """Device milliseconds of the most recent verify_step (CUDA events on the context's stream)."""
        return float(L.lib().kc_last_step_ms(self._h))

    PROFILE_CLASSES = ("gemm", "gemm_reduce", "attention", "rowwise", "sampling")

    def profile_enable(self, on: bool) -> None:
        check(L.lib().kc_profile_enable(self._h, int(on)))

    def profile_read(self) -> dict:
        """{class: (milliseconds, launches)} since the previous read (synchronises the stream)."""
        ms = (C.c_double * 5)()
        n = (C.c_int64 * 5)()
        check(L.lib().kc_profile_read(self._h, ms, n))
        return {k: (ms[i], int(n[i])) for i, k in enumerate(self.PROFILE_CLASSES)}

    def close(self) -> None:
        if self._h:
            for child in list(self._children):
                child.close()
            L.lib().kc_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def live_objects() -> int:
    return int(L.lib().kc_live_objects())


@dataclass
class KvSpec:
    """Static dimensions of one paged pool set (paged.rs:28-59)."""
    layers: int
    kv_heads: int
    head_dim: int
    num_blocks: int
    block_size: int

    def bytes_per_block(self, element_size: int = 2) -> int:
        return element_size * 2 * self.layers * self.kv_heads * self.block_size * self.head_dim


class PagedKv:
    """Per-layer K/V pools on the device (paged.rs:77-386). Writes happen inside forward_step."""

    def __init__(self, ctx: Context, spec: KvSpec):
        self.ctx, self.spec = ctx, spec
        self._h = C.c_void_p()
        check(L.lib().kc_kv_create(ctx._h, spec.layers, spec.kv_heads, spec.head_dim, spec.num_blocks,
                                   spec.block_size, L.KC_BF16, C.byref(self._h)))
        ctx._adopt(self)

    def copy_block(self, src: int, dst: int) -> None:
        check(L.lib().kc_kv_copy_block(self._h, src, dst))

    def read_block_bytes(self, block: int) -> bytes:
        n = int(L.lib().kc_kv_block_bytes(self._h))
        buf = (C.c_uint8 * n)()
        check(L.lib().kc_kv_read_block(self._h, block, buf, n))
        return bytes(buf)

    def write_block_bytes(self, block: int, data: bytes) -> None:
        buf = (C.c_uint8 * len(data)).from_buffer_copy(data)
        check(L.lib().kc_kv_write_block(self._h, block, buf, len(data)))

    def bytes_per_block(self) -> int:
        return int(L.lib().kc_kv_block_bytes(self._h))

    def allocated_bytes(self) -> int:
        return int(L.lib().kc_kv_allocated_bytes(self._h))

    def reset(self) -> None:
        check(L.lib().kc_kv_reset(self._h))

    def close(self) -> None:
        if self._h:
            L.lib().kc_kv_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_DTYPE_TAG = {torch.bfloat16: L.KC_BF16, torch.int32: L.KC_U32, torch.float32: L.KC_F32, torch.float16: L.KC_F16}


def tensor_views(tensors: Dict[str, torch.Tensor]):
    """kc_tensor_view array over a name -> tensor dict (packed weights as int32 holding the u32 bits)."""
    arr = (L.KcTensorView * len(tensors))()
    keep = []
    for i, (name, t) in enumerate(tensors.items()):
        t = t.contiguous()
        keep.append(t)
        nb = name.encode()
        keep.append(nb)
        arr[i].name = nb
        arr[i].data = t.data_ptr()
        arr[i].dtype = _DTYPE_TAG[t.dtype]
        arr[i].ndim = t.dim()
        for k in range(t.dim()):
            arr[i].shape[k] = t.shape[k]
        arr[i].on_device = int(t.is_cuda)
    return arr, keep


class CudaModel:
    """A loaded model; implements the StepModel contract (step.rs:85-96) on libkiln_cuda.so."""

    def __init__(self, ctx: Context, config: ModelConfig, tensors: Dict[str, torch.Tensor], max_step_tokens: int = 512,
                 max_step_seqs: int = 64, tp_rank: int = 0, tp_world: int = 1):
        self.ctx, self.config = ctx, config
        self._h = C.c_void_p()
        desc = config.to_desc(max_step_tokens, max_step_seqs, tp_rank, tp_world)
        if any(t.is_cuda for t in tensors.values()):
            torch.cuda.synchronize()
        arr, keep = tensor_views(tensors)
        check(L.lib().kc_model_load(ctx._h, C.byref(desc), arr, len(tensors), C.byref(self._h)))
        del keep
        ctx._adopt(self)

    # --- StepModel -----------------------------------------------------------------
    def forward_step(self, batch: StepBatch, kv: PagedKv) -> Optional[torch.Tensor]:
        """Logits ``[n_sampled, vocab]`` bf16 for the sampled positions in seqs order, or None (step.rs:86-95).

        The tensor aliases a buffer the model owns: it is valid until the next call and is only ordered
        with the context's stream (call ``ctx.sync()`` before reading it from another stream).
        """
        p = _PackedStep(batch)
        logits = C.c_void_p()
        ns = C.c_int32(0)
        check(L.lib().kc_forward_step(self._h, kv._h, p.ids_p, p.n, p.seq_arr, p.n_seqs, batch.pad_rows,
                                      C.byref(logits), C.byref(ns)))
        if ns.value == 0:
            return None
        return _alias_bf16(logits.value, (ns.value, self.config.vocab_size), self.ctx.device)

    def verify_step(self, batch: StepBatch, kv: PagedKv):
        """One verify round with host buffers: (row_tokens[n_sampled], n_committed[n_seqs], n_accepted[n_seqs])."""
        p = _PackedStep(batch)
        n_sampled = sum(s.sample_rows for s in batch.seqs)
        rows = np.zeros(max(1, n_sampled), dtype=np.uint32)
        ncom = np.zeros(p.n_seqs, dtype=np.int32)
        nacc = np.zeros(p.n_seqs, dtype=np.int32)
        check(L.lib().kc_verify_step(self._h, kv._h, p.ids_p, p.n, p.seq_arr, p.n_seqs,
                                     rows.ctypes.data_as(C.POINTER(C.c_uint32)),
                                     ncom.ctypes.data_as(C.POINTER(C.c_int32)),
                                     nacc.ctypes.data_as(C.POINTER(C.c_int32))))
        return rows[:n_sampled], ncom, nacc

    def decode_launch(self, batch: StepBatch, kv: PagedKv, feed: Sequence[int]) -> int:
        """Queues one pipelined decode step (engine.rs:1656-1744) and returns its ticket; feed[i] >= 0 takes sequence
        i's input id from that row of the previous launch, still on the device."""
        p = _PackedStep(batch)
        f = np.ascontiguousarray(np.asarray(feed, dtype=np.int32))
        if f.shape[0] != p.n_seqs:
            raise ValueError("a decode step has one feed entry per sequence")
        t = C.c_uint64(0)
        check(L.lib().kc_decode_launch(self._h, kv._h, p.ids_p, f.ctypes.data_as(C.POINTER(C.c_int32)), p.seq_arr, p.n_seqs,
                                       C.byref(t)))
        return int(t.value)

    def decode_collect(self, ticket: int, n: int) -> List[int]:
        """Waits for the launch with that ticket and returns its n greedy tokens (engine.rs:1748-1766)."""
        out = np.zeros(max(1, n), dtype=np.uint32)
        check(L.lib().kc_decode_collect(self._h, int(ticket), out.ctypes.data_as(C.POINTER(C.c_uint32)), int(n)))
        return [int(x) for x in out[:n]]

    def draft_chain(self, kv: PagedKv, first_token: int, offset: int, blocks: Sequence[int], gamma: int) -> List[int]:
        """gamma chained greedy decode forwards for one sequence (draft.rs:354-388)."""
        b = np.ascontiguousarray(np.asarray(blocks, dtype=np.uint32))
        out = np.zeros(gamma, dtype=np.uint32)
        check(L.lib().kc_draft_chain(self._h, kv._h, int(first_token), int(offset), b.ctypes.data_as(C.POINTER(C.c_uint32)),
                                     int(b.shape[0]), int(gamma), out.ctypes.data_as(C.POINTER(C.c_uint32))))
        return [int(x) for x in out]

    TP_EXPORT_BYTES = 192

    def tp_connect(self, all_gather) -> None:
        """Switches this tensor-parallel slice's exchange from NCCL to peer memory (kc_tp_export / kc_tp_attach).
        ``all_gather(b: bytes) -> list[bytes]`` must return every rank's bytes in rank order (for instance through
        torch.distributed.all_gather_object); every rank calls this at the same point."""
        buf = (C.c_uint8 * self.TP_EXPORT_BYTES)()
        check(L.lib().kc_tp_export(self._h, buf))
        everyone = all_gather(bytes(buf))
        blob = b"".join(everyone)
        if len(blob) != self.TP_EXPORT_BYTES * len(everyone):
            raise ValueError("tp_connect: every rank must contribute TP_EXPORT_BYTES bytes")
        arr = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(L.lib().kc_tp_attach(self._h, arr))

    def set_stream_lane(self, on: bool = True, every_weight: bool = False) -> None:
        """Forwards of at most 8 rows take the weight-streaming kernels (kc_model_set_stream_lane): for draft models.
        By default only weights of at least 24 MB stream; ``every_weight`` streams all of them."""
        check(L.lib().kc_model_set_stream_lane(self._h, (2 if every_weight else 1) if on else 0))

    def envelope(self):
        """(max_gamma, max_key_len or 0 = unbounded, deterministic width) as the backend provides them."""
        g, k, w = C.c_int32(), C.c_int32(), C.c_int32()
        check(L.lib().kc_envelope(self._h, C.byref(g), C.byref(k), C.byref(w)))
        return g.value, k.value, w.value

    def weight_bytes(self) -> int:
        return int(L.lib().kc_model_weight_bytes(self._h))

    def kv_spec(self, num_blocks: int, block_size: int, tp_world: int = 1) -> KvSpec:
        c = self.config
        return KvSpec(c.num_hidden_layers, c.num_key_value_heads // tp_world, c.head_dim, num_blocks, block_size)

    def close(self) -> None:
        if self._h:
            L.lib().kc_model_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# --------------------------------------------------------------------------------------
# single ops (the kiln_mlx::ops / fast call sites), device tensors in and out
# --------------------------------------------------------------------------------------

def greedy_rows(ctx: Context, logits: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """Greedy token per row (engine.rs:899-900 + sampler.rs:100-104; raw argmax when normalize=False)."""
    assert logits.is_cuda and logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.is_contiguous()
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    torch.cuda.current_stream().synchronize()
    check(L.lib().kc_greedy_rows(ctx._h, logits.data_ptr(), logits.shape[0], logits.shape[1], int(normalize), out.data_ptr()))
    ctx.sync()
    return out


def verify_accept(ctx: Context, row_tokens: torch.Tensor, row_offsets: torch.Tensor, draft: torch.Tensor,
                  draft_offsets: torch.Tensor, draft_len: torch.Tensor, max_commit: int):
    n = row_offsets.shape[0]
    dev = row_tokens.device
    committed = torch.zeros(n * max_commit, dtype=torch.int32, device=dev)
    ncom = torch.zeros(n, dtype=torch.int32, device=dev)
    nacc = torch.zeros(n, dtype=torch.int32, device=dev)
    torch.cuda.current_stream().synchronize()
    check(L.lib().kc_verify_accept(ctx._h, row_tokens.data_ptr(), row_offsets.data_ptr(), draft.data_ptr(),
                                   draft_offsets.data_ptr(), draft_len.data_ptr(), n, max_commit, committed.data_ptr(),
                                   ncom.data_ptr(), nacc.data_ptr()))
    ctx.sync()
    return committed.view(n, max_commit), ncom, nacc


class QuantizedWeight:
    """One mlx affine-quantised weight re-tiled for the GEMM (ops.rs:362-388 operand)."""

    def __init__(self, ctx: Context, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group_size: int):
        self.ctx = ctx
        self.out_features = w.shape[0]
        self.in_features = w.shape[1] * 32 // bits
        self._h = C.c_void_p()
        w, scales, biases = w.contiguous(), scales.contiguous(), biases.contiguous()
        on_dev = int(w.is_cuda)
        if on_dev:
            torch.cuda.synchronize()
        check(L.lib().kc_qweight_create(ctx._h, w.data_ptr(), scales.data_ptr(), biases.data_ptr(), self.out_features,
                                        self.in_features, bits, group_size, on_dev, C.byref(self._h)))
        ctx._adopt(self)

    def matmul(self, x: torch.Tensor) -> torch.Tensor:
        """y = x · dequant(W)ᵀ; x bf16 [m, in] on the device."""
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == self.in_features
        m = x.shape[0]
        rows = (m + 15) // 16 * 16
        xp = torch.zeros(rows, self.in_features, dtype=torch.bfloat16, device=x.device)
        xp[:m] = x
        y = torch.empty(m, self.out_features, dtype=torch.bfloat16, device=x.device)
        torch.cuda.current_stream().synchronize()
        check(L.lib().kc_quantized_matmul(self.ctx._h, self._h, xp.data_ptr(), m, y.data_ptr()))
        self.ctx.sync()
        return y

    def matmul_stream(self, x: torch.Tensor) -> torch.Tensor:
        """The same product for at most 8 rows through the weight-streaming lane (kc_quantized_matmul_stream)."""
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == self.in_features
        x = x.contiguous()
        y = torch.empty(x.shape[0], self.out_features, dtype=torch.bfloat16, device=x.device)
        torch.cuda.current_stream().synchronize()
        check(L.lib().kc_quantized_matmul_stream(self.ctx._h, self._h, x.data_ptr(), x.shape[0], y.data_ptr()))
        self.ctx.sync()
        return y

    def matmul_gemv(self, x: torch.Tensor) -> torch.Tensor:
        """The same product for at most 8 rows through the small-weight lane (kc_quantized_matmul_gemv)."""
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == self.in_features
        x = x.contiguous()
        y = torch.empty(x.shape[0], self.out_features, dtype=torch.bfloat16, device=x.device)
        torch.cuda.current_stream().synchronize()
        check(L.lib().kc_quantized_matmul_gemv(self.ctx._h, self._h, x.data_ptr(), x.shape[0], y.data_ptr()))
        self.ctx.sync()
        return y

    def matmul_static(self, xp: torch.Tensor, m: int, y: torch.Tensor) -> None:
        """kc_quantized_matmul_static on caller-owned buffers: xp bf16 [round_up(m, 16), in], y bf16 [m, out], both
        on the device. This wrapper allocates nothing either; the caller synchronises (Context.sync)."""
        assert xp.is_cuda and xp.dtype == torch.bfloat16 and xp.is_contiguous() and xp.shape[1] == self.in_features
        assert xp.shape[0] >= (m + 15) // 16 * 16 and y.is_cuda and y.dtype == torch.bfloat16 and y.is_contiguous()
        assert tuple(y.shape) == (m, self.out_features)
        check(L.lib().kc_quantized_matmul_static(self.ctx._h, self._h, xp.data_ptr(), m, y.data_ptr()))

    def close(self) -> None:
        if self._h:
            L.lib().kc_qweight_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def rms_norm(ctx: Context, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    y = torch.empty_like(x)
    torch.cuda.current_stream().synchronize()
    check(L.lib().kc_rms_norm(ctx._h, x.data_ptr(), weight.data_ptr(), x.shape[0], x.shape[1], eps, y.data_ptr()))
    ctx.sync()
    return y


def paged_attention(ctx: Context, kv: PagedKv, layer: int, q: torch.Tensor, seqs: List[SeqStep], scale: float,
                    softcap: float = 0.0, window: int = 0) -> torch.Tensor:
    """q bf16 [n, heads, head_dim] post-RoPE → bf16 [n, heads*head_dim] (paged.rs:191-225 + nn.rs:800-817)."""
    n, heads, hd = q.shape
    p = _PackedStep(StepBatch([0] * n, seqs))
    out = torch.empty(n, heads * hd, dtype=torch.bfloat16, device=q.device)
    torch.cuda.current_stream().synchronize()
    check(L.lib().kc_paged_attention(ctx._h, kv._h, layer, q.contiguous().data_ptr(), n, heads, p.seq_arr, p.n_seqs,
                                     scale, softcap, window, out.data_ptr()))
    ctx.sync()
    return out


def rope_kv_write(ctx: Context, kv: PagedKv, layer: int, qkv: torch.Tensor, inv_freq: torch.Tensor, heads: int,
                  seqs: List[SeqStep], traditional: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RoPE at per-sequence offsets + KV write (nn.rs:760-769, paged.rs:147-187); returns q bf16 [n, heads, hd]."""
    n = qkv.shape[0]
    hd = kv.spec.head_dim
    p = _PackedStep(StepBatch([0] * n, seqs))
    q = torch.empty(n, heads, hd, dtype=torch.bfloat16, device=qkv.device)
    torch.cuda.current_stream().synchronize()
    check(L.lib().kc_rope_kv_write(ctx._h, kv._h, layer, qkv.contiguous().data_ptr(), bias.data_ptr() if bias is not None else None,
                                   inv_freq.data_ptr(), n, heads, int(traditional), p.seq_arr, p.n_seqs, q.data_ptr()))
    ctx.sync()
    return q
