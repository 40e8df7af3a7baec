"""ctypes binding of libkiln_host.so: the C++ scheduler pieces of the verify path.

Class and method names follow the reference (paths inside ikematta/kiln):
  BlockManager, BlockTable   crates/kiln-engine/src/block.rs
  RadixCache                 crates/kiln-engine/src/radix.rs
  Engine, EngineConfig       crates/kiln-engine/src/engine.rs
  ScriptedDrafter, DraftModel   Drafter implementations (drafter.rs:125-147, crates/kiln-models/src/draft.rs)
All logic lives in the shared library; this file only marshals arguments.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import numpy as np

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libkiln_host.so"
_P = C.c_void_p
_U32P = C.POINTER(C.c_uint32)
_lib = None

ERR_NAMES = {1: "OutOfBlocks", 2: "NotAllocated", 3: "RefcountOverflow", 4: "InvalidBlockSize", 5: "InvalidCapacity",
             6: "TokenCountOverflow", 7: "MisalignedAdoption", 20: "Model", 21: "Argument"}


class KhSeqStep(C.Structure):
    _fields_ = [("len", C.c_int32), ("offset", C.c_int32), ("sample_rows", C.c_int32), ("n_blocks", C.c_int32),
                ("blocks", _U32P)]


VERIFY_FN = C.CFUNCTYPE(C.c_int, _P, _P, _U32P, C.c_int32, C.POINTER(KhSeqStep), C.c_int32, _U32P,
                        C.POINTER(C.c_int32), C.POINTER(C.c_int32))
COPY_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint32, C.c_uint32)
BEGIN_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint64, _U32P, C.c_int32)
PROPOSE_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint64, _U32P, C.c_int32, C.c_int32, _U32P, C.POINTER(C.c_int32))
RELEASE_FN = C.CFUNCTYPE(None, _P, C.c_uint64)


class KhDrafterMemory(C.Structure):
    _fields_ = [("weights_bytes", C.c_uint64), ("kv_allocated_bytes", C.c_uint64), ("kv_used_bytes", C.c_uint64)]


MEMORY_FN = C.CFUNCTYPE(None, _P, C.POINTER(KhDrafterMemory))
CHAIN_FN = C.CFUNCTYPE(C.c_int, _P, _P, C.c_uint32, C.c_int32, _U32P, C.c_int32, C.c_int32, _U32P)


LAUNCH_FN = C.CFUNCTYPE(C.c_int, _P, _P, _U32P, C.POINTER(C.c_int32), C.POINTER(KhSeqStep), C.c_int32, C.POINTER(C.c_uint64))
COLLECT_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint64, _U32P, C.c_int32)


class KhDecodePipeline(C.Structure):
    _fields_ = [("launch", LAUNCH_FN), ("collect", COLLECT_FN)]


class KhStepModel(C.Structure):
    _fields_ = [("model", _P), ("kv", _P), ("verify_step", VERIFY_FN), ("copy_block", COPY_FN), ("vocab", C.c_int32)]


class KhDrafter(C.Structure):
    _fields_ = [("user", _P), ("begin", BEGIN_FN), ("propose", PROPOSE_FN), ("release", RELEASE_FN), ("memory", MEMORY_FN)]


class KhDraftBackend(C.Structure):
    _fields_ = [("model", _P), ("kv", _P), ("forward", VERIFY_FN), ("chain", CHAIN_FN), ("max_chunk", C.c_int32),
                ("weights_bytes", C.c_uint64), ("kv_allocated_bytes", C.c_uint64), ("kv_block_bytes", C.c_uint64)]


class KhSlabGeometry(C.Structure):
    _fields_ = [("layers", C.c_uint32), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("block_size", C.c_uint32)]


BLOCK_READ_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint32, _P, C.c_size_t)
BLOCK_WRITE_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint32, _P, C.c_size_t)


class KhBlockIo(C.Structure):
    _fields_ = [("read", BLOCK_READ_FN), ("write", BLOCK_WRITE_FN), ("dtype_tag", C.c_uint32), ("dtype_size", C.c_uint32)]


class KhSsdStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("blocks_stored", "bytes_stored", "reads_total", "writes_total", "writes_failed_total",
                                          "fingerprint_rejects_total", "flush_queue_depth", "ssd_hits_total")]


class KhFlushAck(C.Structure):
    _fields_ = [("node", C.c_uint64), ("generation", C.c_uint64), ("hash", C.c_uint8 * 32), ("ok", C.c_int32)]


class KhEngineConfig(C.Structure):
    _fields_ = [("block_size", C.c_int32), ("num_blocks", C.c_int32), ("max_batch_tokens", C.c_int32),
                ("prefill_chunk", C.c_int32), ("prefill_fine_chunk", C.c_int32), ("prefix_cache", C.c_int32),
                ("deterministic_decode_width", C.c_int32), ("gamma", C.c_int32), ("spec_max_batch", C.c_int32),
                ("spec_min_acceptance", C.c_double), ("max_key_len", C.c_int32), ("batch_verify", C.c_int32)]


class KhSpecStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("rounds_total", "proposed_total", "accepted_total", "rollback_rounds_total",
                                          "rollback_tokens_total", "rollback_nanos_total", "draft_errors_total",
                                          "standdowns_total")]


_U64, _I64, _I32 = C.c_uint64, C.c_int64, C.c_int32
_SIGNATURES = {
    "kh_last_error": (C.c_char_p, []),
    "kh_last_out_of_blocks": (None, [C.POINTER(_U64), C.POINTER(_U64)]),
    "kh_bm_create": (C.c_int, [_U64, _U64, C.POINTER(_P)]), "kh_bm_free": (None, [_P]),
    "kh_bm_block_size": (_U64, [_P]), "kh_bm_capacity": (_U64, [_P]), "kh_bm_num_free": (_U64, [_P]),
    "kh_bm_refcount": (_I64, [_P, C.c_uint32]), "kh_bm_allocate": (C.c_int, [_P, _U32P]),
    "kh_bm_retain": (C.c_int, [_P, C.c_uint32]), "kh_bm_release": (C.c_int, [_P, C.c_uint32]),
    "kh_bm_copy_on_write": (C.c_int, [_P, C.c_uint32, C.POINTER(_I32), _U32P, _U32P]),
    "kh_bm_free_list": (_U64, [_P, _U32P, _U64]),
    "kh_bt_create": (C.c_int, [C.POINTER(_P)]), "kh_bt_free": (None, [_P]), "kh_bt_num_tokens": (_U64, [_P]),
    "kh_bt_blocks": (_U64, [_P, _U32P, _U64]),
    "kh_bt_append_tokens": (C.c_int, [_P, _P, _U64, C.POINTER(_I32), _U32P, _U32P, _U32P, _U64, C.POINTER(_U64)]),
    "kh_bt_push_full_block": (C.c_int, [_P, C.c_uint32, _U64]),
    "kh_bt_push_partial_block": (C.c_int, [_P, C.c_uint32, _U64, _U64]),
    "kh_bt_truncate": (C.c_int, [_P, _P, _U64]), "kh_bt_fork": (C.c_int, [_P, _P, C.POINTER(_P)]),
    "kh_bt_release": (C.c_int, [_P, _P]),
    "kh_spec_gamma_at_width": (_U64, [_U64, _U64, _U64]), "kh_canonical_prefill_len": (_U64, [_U64, _U64, _U64, _U64]),
    "kh_radix_create": (C.c_int, [_U64, C.c_char_p, C.POINTER(_P)]), "kh_radix_free": (None, [_P]),
    "kh_radix_child": (_I64, [_P, _U64, _U32P, _U64]),
    "kh_radix_chain_hash_of": (None, [_P, _U64, _U32P, _U64, C.c_char_p]), "kh_radix_node_hash": (None, [_P, _U64, C.c_char_p]),
    "kh_radix_node_block": (_I64, [_P, _U64]), "kh_radix_node_rows": (_U64, [_P, _U64]),
    "kh_radix_node_is_partial": (_I32, [_P, _U64]), "kh_radix_node_generation": (_U64, [_P, _U64]),
    "kh_radix_is_live": (_I32, [_P, _U64, _U64]), "kh_radix_insert_child": (_U64, [_P, _U64, _U32P, _U64]),
    "kh_radix_insert_partial_child": (_U64, [_P, _U64, _U32P, _U64]),
    "kh_radix_upgrade_partial": (_I64, [_P, _U64, _U32P, _U64, C.c_uint32]),
    "kh_radix_set_resident": (None, [_P, _U64, C.c_uint32]), "kh_radix_touch": (None, [_P, _U64]),
    "kh_radix_set_on_ssd": (None, [_P, _U64]), "kh_radix_node_on_ssd": (_I32, [_P, _U64]),
    "kh_radix_evict_candidate": (_I64, [_P, _P]), "kh_radix_evict": (_I64, [_P, _P, _U64]),
    "kh_radix_prune_subtree": (None, [_P, _P, _U64]), "kh_radix_resident_blocks": (_U64, [_P]), "kh_radix_reset": (None, [_P]),
    "kh_engine_default_config": (None, [C.POINTER(KhEngineConfig)]),
    "kh_engine_create": (C.c_int, [C.POINTER(KhEngineConfig), C.POINTER(KhStepModel), C.POINTER(_P)]),
    "kh_engine_set_pipeline": (C.c_int, [_P, C.POINTER(KhDecodePipeline)]),
    "kh_engine_pipelined_steps": (C.c_uint64, [_P]),
    "kh_engine_free": (None, [_P]), "kh_engine_set_drafter": (C.c_int, [_P, C.POINTER(KhDrafter)]),
    "kh_engine_drafter_memory": (C.c_int, [_P, C.POINTER(KhDrafterMemory)]),
    "kh_engine_submit": (C.c_int, [_P, _U32P, _U64, _U64, _U32P, _U64, C.POINTER(_U64)]),
    "kh_engine_cancel": (C.c_int, [_P, _U64]), "kh_engine_step": (C.c_int, [_P]),
    "kh_engine_num_running": (_U64, [_P]), "kh_engine_num_waiting": (_U64, [_P]), "kh_engine_iterations": (_U64, [_P]),
    "kh_engine_forwards": (_U64, [_P]), "kh_engine_last_error": (C.c_char_p, [_P]),
    "kh_engine_take_output": (C.c_int, [_P, _U64, _U32P, _U64, C.POINTER(_U64), C.POINTER(_I32)]),
    "kh_engine_seq_state": (C.c_int, [_P, _U64, _U32P, _U64, C.POINTER(_U64), C.POINTER(_U64), C.POINTER(_U64),
                                      _U32P, _U32P, C.POINTER(_I32), _U32P]),
    "kh_engine_spec_stats": (None, [_P, C.POINTER(KhSpecStats)]), "kh_engine_block_manager": (_P, [_P]),
    "kh_engine_cache_stats": (None, [_P, C.POINTER(_U64), C.POINTER(_U64), C.POINTER(_U64)]),
    "kh_engine_set_ssd": (C.c_int, [_P, C.c_char_p, C.c_char_p, C.POINTER(KhSlabGeometry), _U64, C.POINTER(KhBlockIo)]),
    "kh_engine_ssd_sync": (None, [_P]), "kh_engine_ssd_stats": (None, [_P, C.POINTER(KhSsdStats)]),
    "kh_ssd_open": (C.c_int, [C.c_char_p, C.c_char_p, C.POINTER(KhSlabGeometry), _U64, C.POINTER(_P)]), "kh_ssd_close": (None, [_P]),
    "kh_ssd_contains": (C.c_int, [_P, C.c_char_p]),
    "kh_ssd_enqueue_write": (C.c_int, [_P, _U64, _U64, C.c_char_p, _U32P, _U64, C.c_char_p, _U64, C.c_uint32, C.c_uint32]),
    "kh_ssd_drain_acks": (_U64, [_P, C.POINTER(KhFlushAck), _U64]), "kh_ssd_sync": (_U64, [_P, C.POINTER(KhFlushAck), _U64]),
    "kh_ssd_read": (_I64, [_P, C.c_char_p, _U32P, _U64, _I64, C.c_char_p, _U64, C.POINTER(C.c_uint32)]),
    "kh_ssd_get_stats": (None, [_P, C.POINTER(KhSsdStats)]),
    "kh_scripted_create": (C.c_int, [C.c_double, _U64, C.c_uint32, C.POINTER(_P)]), "kh_scripted_free": (None, [_P]),
    "kh_scripted_set_continuation": (C.c_int, [_P, _U64, _U32P, _U64]), "kh_scripted_vtable": (None, [_P, C.POINTER(KhDrafter)]),
    "kh_draft_model_create": (C.c_int, [C.POINTER(KhDraftBackend), _U64, _U64, C.POINTER(_P)]),
    "kh_draft_model_free": (None, [_P]), "kh_draft_model_vtable": (None, [_P, C.POINTER(KhDrafter)]),
    "kh_draft_model_block_manager": (_P, [_P]), "kh_draft_model_live_sequences": (_U64, [_P]),
}


def exported_symbols() -> List[str]:
    return sorted(_SIGNATURES)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m kiln_b200.build`")
        h = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(h, name)
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


class HostError(RuntimeError):
    """A non-zero code from libkiln_host.so. ``kind`` names the reference's BlockError variant."""

    def __init__(self, code: int, message: str, info: Optional[dict] = None):
        super().__init__(f"[{ERR_NAMES.get(code, code)}] {message}")
        self.code, self.kind, self.message, self.info = code, ERR_NAMES.get(code, str(code)), message, info or {}


def _check(code: int) -> None:
    if code == 0:
        return
    info = {}
    if code == 1:
        cap, need = _U64(0), _U64(0)
        lib().kh_last_out_of_blocks(C.byref(cap), C.byref(need))
        info = {"capacity": cap.value, "needed": need.value}
    raise HostError(code, lib().kh_last_error().decode(), info)


def _u32(seq: Sequence[int]):
    a = np.ascontiguousarray(np.asarray(seq, dtype=np.uint32))
    return a, a.ctypes.data_as(_U32P)


# --------------------------------------------------------------------------------------
# block.rs
# --------------------------------------------------------------------------------------

class BlockManager:
    def __init__(self, capacity: int, block_size: int, _borrowed: Optional[int] = None):
        self._owned = _borrowed is None
        if _borrowed is not None:
            self._h = _P(_borrowed)
        else:
            self._h = _P()
            _check(lib().kh_bm_create(capacity, block_size, C.byref(self._h)))

    block_size = property(lambda self: int(lib().kh_bm_block_size(self._h)))
    capacity = property(lambda self: int(lib().kh_bm_capacity(self._h)))
    num_free = property(lambda self: int(lib().kh_bm_num_free(self._h)))

    def refcount(self, bid: int) -> Optional[int]:
        r = int(lib().kh_bm_refcount(self._h, bid))
        return None if r < 0 else r

    def allocate(self) -> int:
        out = C.c_uint32(0)
        _check(lib().kh_bm_allocate(self._h, C.byref(out)))
        return out.value

    def retain(self, bid: int) -> None:
        _check(lib().kh_bm_retain(self._h, bid))

    def release(self, bid: int) -> None:
        _check(lib().kh_bm_release(self._h, bid))

    def copy_on_write(self, bid: int) -> Tuple[str, int, int]:
        copied, src, dst = _I32(0), C.c_uint32(0), C.c_uint32(0)
        _check(lib().kh_bm_copy_on_write(self._h, bid, C.byref(copied), C.byref(src), C.byref(dst)))
        return ("copied" if copied.value else "writable", src.value, dst.value)

    def free_list(self) -> List[int]:
        n = self.num_free
        buf = (C.c_uint32 * max(n, 1))()
        lib().kh_bm_free_list(self._h, buf, n)
        return list(buf[:n])

    def __del__(self):
        try:
            if self._owned and self._h:
                lib().kh_bm_free(self._h)
                self._h = _P()
        except Exception:
            pass


@dataclass
class AppendPlan:
    cow: Optional[Tuple[int, int]]
    appended: List[int]


class BlockTable:
    def __init__(self, _h: Optional[int] = None):
        self._h = _P(_h) if _h is not None else _P()
        if _h is None:
            _check(lib().kh_bt_create(C.byref(self._h)))

    num_tokens = property(lambda self: int(lib().kh_bt_num_tokens(self._h)))

    @property
    def blocks(self) -> List[int]:
        n = int(lib().kh_bt_blocks(self._h, None, 0))
        buf = (C.c_uint32 * max(n, 1))()
        lib().kh_bt_blocks(self._h, buf, n)
        return list(buf[:n])

    def append_tokens(self, mgr: BlockManager, n: int) -> AppendPlan:
        cap = n // max(mgr.block_size, 1) + 2
        has, src, dst, na = _I32(0), C.c_uint32(0), C.c_uint32(0), _U64(0)
        buf = (C.c_uint32 * cap)()
        _check(lib().kh_bt_append_tokens(self._h, mgr._h, n, C.byref(has), C.byref(src), C.byref(dst), buf, cap, C.byref(na)))
        return AppendPlan((src.value, dst.value) if has.value else None, list(buf[:na.value]))

    def push_full_block(self, bid: int, block_size: int) -> None:
        _check(lib().kh_bt_push_full_block(self._h, bid, block_size))

    def push_partial_block(self, bid: int, rows: int, block_size: int) -> None:
        _check(lib().kh_bt_push_partial_block(self._h, bid, rows, block_size))

    def truncate(self, mgr: BlockManager, keep_tokens: int) -> None:
        _check(lib().kh_bt_truncate(self._h, mgr._h, keep_tokens))

    def fork(self, mgr: BlockManager) -> "BlockTable":
        out = _P()
        _check(lib().kh_bt_fork(self._h, mgr._h, C.byref(out)))
        return BlockTable(out.value)

    def release(self, mgr: BlockManager) -> None:
        _check(lib().kh_bt_release(self._h, mgr._h))

    def __del__(self):
        try:
            if self._h:
                lib().kh_bt_free(self._h)
                self._h = _P()
        except Exception:
            pass


def spec_gamma_at_width(gamma: int, spec_max_batch: int, width: int) -> int:
    return int(lib().kh_spec_gamma_at_width(gamma, spec_max_batch, width))


def canonical_prefill_len(at: int, limit: int, prefill_chunk: int, fine: int) -> int:
    return int(lib().kh_canonical_prefill_len(at, limit, prefill_chunk, fine))


# --------------------------------------------------------------------------------------
# radix.rs
# --------------------------------------------------------------------------------------

ROOT = 0


class RadixCache:
    def __init__(self, block_size: int, seed: bytes = bytes(32)):
        self._h = _P()
        _check(lib().kh_radix_create(block_size, seed, C.byref(self._h)))

    def child(self, node: int, chunk: Sequence[int]) -> Optional[int]:
        a, p = _u32(chunk)
        r = int(lib().kh_radix_child(self._h, node, p, len(a)))
        return None if r < 0 else r

    def chain_hash_of(self, node: int, chunk: Sequence[int]) -> bytes:
        a, p = _u32(chunk)
        out = C.create_string_buffer(32)
        lib().kh_radix_chain_hash_of(self._h, node, p, len(a), out)
        return out.raw

    def node_hash(self, node: int) -> bytes:
        out = C.create_string_buffer(32)
        lib().kh_radix_node_hash(self._h, node, out)
        return out.raw

    def node_block(self, node: int) -> Optional[int]:
        r = int(lib().kh_radix_node_block(self._h, node))
        return None if r < 0 else r

    def node_rows(self, node: int) -> int:
        return int(lib().kh_radix_node_rows(self._h, node))

    def node_is_partial(self, node: int) -> bool:
        return bool(lib().kh_radix_node_is_partial(self._h, node))

    def node_generation(self, node: int) -> int:
        return int(lib().kh_radix_node_generation(self._h, node))

    def is_live(self, node: int, generation: int) -> bool:
        return bool(lib().kh_radix_is_live(self._h, node, generation))

    def insert_child(self, parent: int, chunk: Sequence[int]) -> int:
        a, p = _u32(chunk)
        return int(lib().kh_radix_insert_child(self._h, parent, p, len(a)))

    def insert_partial_child(self, parent: int, tokens: Sequence[int]) -> int:
        a, p = _u32(tokens)
        return int(lib().kh_radix_insert_partial_child(self._h, parent, p, len(a)))

    def upgrade_partial(self, node: int, tokens: Sequence[int], block: int) -> Optional[int]:
        a, p = _u32(tokens)
        r = int(lib().kh_radix_upgrade_partial(self._h, node, p, len(a), block))
        return None if r < 0 else r

    def set_resident(self, node: int, block: int) -> None:
        lib().kh_radix_set_resident(self._h, node, block)

    def touch(self, node: int) -> None:
        lib().kh_radix_touch(self._h, node)

    def set_on_ssd(self, node: int) -> None:
        lib().kh_radix_set_on_ssd(self._h, node)

    def node_on_ssd(self, node: int) -> bool:
        return bool(lib().kh_radix_node_on_ssd(self._h, node))

    def evict_candidate(self, mgr: BlockManager) -> Optional[int]:
        r = int(lib().kh_radix_evict_candidate(self._h, mgr._h))
        return None if r < 0 else r

    def evict(self, mgr: BlockManager, node: int) -> Optional[int]:
        r = int(lib().kh_radix_evict(self._h, mgr._h, node))
        return None if r < 0 else r

    def prune_subtree(self, mgr: BlockManager, node: int) -> None:
        lib().kh_radix_prune_subtree(self._h, mgr._h, node)

    def resident_blocks(self) -> int:
        return int(lib().kh_radix_resident_blocks(self._h))

    def reset(self) -> None:
        lib().kh_radix_reset(self._h)

    def __del__(self):
        try:
            if self._h:
                lib().kh_radix_free(self._h)
                self._h = _P()
        except Exception:
            pass


# --------------------------------------------------------------------------------------
# engine.rs / drafter.rs / draft.rs
# --------------------------------------------------------------------------------------

@dataclass
class EngineConfig:
    """EngineConfig (engine.rs:239-306) plus the backend-provided envelope. Defaults are the reference's."""
    block_size: int = 32
    num_blocks: int = 512
    max_batch_tokens: int = 8192
    prefill_chunk: int = 2048
    prefill_fine_chunk: int = 128
    prefix_cache: bool = True
    deterministic_decode_width: int = 4
    gamma: int = 4
    spec_max_batch: int = 4
    spec_min_acceptance: float = 0.125
    max_key_len: int = 1023
    batch_verify: bool = False

    def to_c(self) -> KhEngineConfig:
        c = KhEngineConfig()
        for f in ("block_size", "num_blocks", "max_batch_tokens", "prefill_chunk", "prefill_fine_chunk",
                  "deterministic_decode_width", "gamma", "spec_max_batch", "max_key_len"):
            setattr(c, f, int(getattr(self, f)))
        c.prefix_cache, c.batch_verify = int(self.prefix_cache), int(self.batch_verify)
        c.spec_min_acceptance = float(self.spec_min_acceptance)
        return c


def default_engine_config() -> EngineConfig:
    c = KhEngineConfig()
    lib().kh_engine_default_config(C.byref(c))
    return EngineConfig(c.block_size, c.num_blocks, c.max_batch_tokens, c.prefill_chunk, c.prefill_fine_chunk,
                        bool(c.prefix_cache), c.deterministic_decode_width, c.gamma, c.spec_max_batch,
                        c.spec_min_acceptance, c.max_key_len, bool(c.batch_verify))


class StepModel:
    """The StepModel seam (step.rs:85-96) as the engine sees it: one call = forward + greedy rows on the host.

    ``from_cuda`` points the table straight at kc_verify_step / kc_kv_copy_block, so no Python runs on the
    hot path; ``from_python`` wraps a Python callable for fake models (the reference's RecordingMock pattern,
    crates/kiln-engine/tests/deterministic_partition.rs:41-125).
    """

    def __init__(self, c_struct: KhStepModel, keep, pipeline: Optional[KhDecodePipeline] = None):
        self.c, self._keep, self.pipeline = c_struct, keep, pipeline

    @classmethod
    def from_cuda(cls, model, kv) -> "StepModel":
        from . import _lib as L
        cl = L.lib()
        s = KhStepModel()
        s.model, s.kv = model._h, kv._h
        s.verify_step = C.cast(cl.kc_verify_step, VERIFY_FN)
        s.copy_block = C.cast(cl.kc_kv_copy_block, COPY_FN)
        s.vocab = model.config.vocab_size
        pipe = KhDecodePipeline(C.cast(cl.kc_decode_launch, LAUNCH_FN), C.cast(cl.kc_decode_collect, COLLECT_FN))
        return cls(s, (model, kv), pipe)

    @classmethod
    def from_python(cls, fn, vocab: int, copy_block=None, pipelined: bool = False) -> "StepModel":
        """fn(ids: list[int], seqs: list[(len, offset, sample_rows, blocks)]) -> list[int] row tokens.

        ``pipelined`` adds the launch/collect pair: launch runs fn at once on ids resolved through the previous launch's
        tokens (what the device does in stream order) and keeps the result under a ticket; collect hands it out."""
        launched = {"ticket": 0, "tokens": {}, "log": []}

        def _launch(_m, _kv, ids, feed, seqs, n_seqs, ticket):
            try:
                prev = launched["tokens"].get(launched["ticket"], [])
                py_ids = [prev[feed[i]] if feed[i] >= 0 else ids[i] for i in range(n_seqs)]
                py_seqs = [(seqs[i].len, seqs[i].offset, seqs[i].sample_rows, [seqs[i].blocks[b] for b in range(seqs[i].n_blocks)])
                           for i in range(n_seqs)]
                launched["ticket"] += 1   # like the device, only the two most recent launches stay collectable
                launched["tokens"] = {launched["ticket"] - 1: prev, launched["ticket"]: [int(t) for t in fn(py_ids, py_seqs)]}
                launched["log"].append(("launch", launched["ticket"], [int(feed[i]) for i in range(n_seqs)]))
                ticket[0] = launched["ticket"]
                return 0
            except Exception:
                return 2

        def _collect(_m, ticket, rows, n):
            toks = launched["tokens"].get(int(ticket))
            if toks is None or len(toks) != n:
                return 2
            for i, t in enumerate(toks):
                rows[i] = t
            launched["log"].append(("collect", int(ticket)))
            return 0

        def _verify(_m, _kv, ids, n, seqs, n_seqs, rows, ncom, nacc):
            try:
                py_ids = [ids[i] for i in range(n)]
                py_seqs = [(seqs[i].len, seqs[i].offset, seqs[i].sample_rows, [seqs[i].blocks[b] for b in range(seqs[i].n_blocks)])
                           for i in range(n_seqs)]
                out = fn(py_ids, py_seqs)
                for i, t in enumerate(out):
                    rows[i] = int(t)
                return 0
            except Exception:
                return 2

        def _copy(_kv, src, dst):
            if copy_block:
                copy_block(src, dst)
            return 0

        v, cp = VERIFY_FN(_verify), COPY_FN(_copy)
        s = KhStepModel()
        s.model, s.kv, s.verify_step, s.copy_block, s.vocab = None, None, v, cp, vocab
        pipe = KhDecodePipeline(LAUNCH_FN(_launch), COLLECT_FN(_collect)) if pipelined else None
        out = cls(s, (v, cp, fn, copy_block, pipe), pipe)
        out.pipeline_log = launched["log"]
        return out


class Drafter:
    """A kh_drafter table (trait Drafter, drafter.rs:125-147)."""

    def __init__(self, c_struct: KhDrafter, keep):
        self.c, self._keep = c_struct, keep

    @classmethod
    def from_python(cls, begin, propose, release, memory=None) -> "Drafter":
        """begin(seq, prompt) ; propose(seq, committed, gamma) -> list[int] (raise = DraftError) ; release(seq) ;
        memory() -> (weights_bytes, kv_allocated_bytes, kv_used_bytes), optional (Drafter::memory)."""
        def _b(_u, seq, p, n):
            try:
                begin(seq, [p[i] for i in range(n)])
                return 0
            except Exception:
                return 1

        def _p(_u, seq, c, nc, gamma, out, n_out):
            try:
                toks = propose(seq, [c[i] for i in range(nc)], gamma)
                toks = list(toks)[:gamma]
                for i, t in enumerate(toks):
                    out[i] = int(t)
                n_out[0] = len(toks)
                return 0
            except Exception:
                return 1

        def _r(_u, seq):
            release(seq)

        def _m(_u, out):
            out[0].weights_bytes, out[0].kv_allocated_bytes, out[0].kv_used_bytes = (int(v) for v in memory())

        b, p, r = BEGIN_FN(_b), PROPOSE_FN(_p), RELEASE_FN(_r)
        m = MEMORY_FN(_m) if memory is not None else MEMORY_FN()
        d = KhDrafter()
        d.user, d.begin, d.propose, d.release, d.memory = None, b, p, r, m
        return cls(d, (b, p, r, m, begin, propose, release, memory))


class ScriptedDrafter(Drafter):
    """Seeded acceptance injection: proposal position j = the registered continuation with probability p."""

    def __init__(self, p: float, seed: int, vocab: int):
        self._h = _P()
        _check(lib().kh_scripted_create(p, seed, vocab, C.byref(self._h)))
        d = KhDrafter()
        lib().kh_scripted_vtable(self._h, C.byref(d))
        super().__init__(d, None)

    def set_continuation(self, seq: int, tokens: Sequence[int]) -> None:
        a, p = _u32(tokens)
        _check(lib().kh_scripted_set_continuation(self._h, seq, p, len(a)))

    def __del__(self):
        try:
            if self._h:
                lib().kh_scripted_free(self._h)
                self._h = _P()
        except Exception:
            pass


class DraftModel(Drafter):
    """DraftModel (draft.rs:109-122): a second model with its own pool, block manager and tables."""

    def __init__(self, model, kv, num_blocks: int, block_size: int, max_chunk: int = 2048):
        from . import _lib as L
        cl = L.lib()
        b = KhDraftBackend()
        b.model, b.kv = model._h, kv._h
        b.forward = C.cast(cl.kc_verify_step, VERIFY_FN)
        b.chain = C.cast(cl.kc_draft_chain, CHAIN_FN)
        b.max_chunk = max_chunk
        b.weights_bytes = int(cl.kc_model_weight_bytes(model._h))
        b.kv_allocated_bytes = int(cl.kc_kv_allocated_bytes(kv._h))
        b.kv_block_bytes = int(cl.kc_kv_block_bytes(kv._h))
        self._h = _P()
        _check(lib().kh_draft_model_create(C.byref(b), num_blocks, block_size, C.byref(self._h)))
        d = KhDrafter()
        lib().kh_draft_model_vtable(self._h, C.byref(d))
        super().__init__(d, (model, kv))

    def block_manager(self) -> BlockManager:
        return BlockManager(0, 0, _borrowed=lib().kh_draft_model_block_manager(self._h))

    def live_sequences(self) -> int:
        return int(lib().kh_draft_model_live_sequences(self._h))

    def __del__(self):
        try:
            if self._h:
                lib().kh_draft_model_free(self._h)
                self._h = _P()
        except Exception:
            pass


class SsdStore:
    """SsdStore (ssd.rs:159-586) on its own: slab files under `directory`, index rebuilt from their headers on open."""

    def __init__(self, directory: str, fingerprint: bytes, layers: int, kv_heads: int, head_dim: int, block_size: int,
                 max_bytes: int = 1 << 40):
        assert len(fingerprint) == 32
        self.geometry = KhSlabGeometry(layers, kv_heads, head_dim, block_size)
        self._h = _P()
        _check(lib().kh_ssd_open(str(directory).encode(), bytes(fingerprint), C.byref(self.geometry), max_bytes, C.byref(self._h)))

    def payload_bytes(self, dtype_size: int) -> int:
        g = self.geometry
        return g.layers * 2 * g.kv_heads * g.block_size * g.head_dim * dtype_size

    def contains(self, chain_hash: bytes) -> bool:
        return bool(lib().kh_ssd_contains(self._h, bytes(chain_hash)))

    def enqueue_write(self, node: int, generation: int, chain_hash: bytes, tokens: Sequence[int], payload: bytes, dtype_tag: int = 7,
                      dtype_size: int = 2) -> None:
        a, p = _u32(tokens)
        _check(lib().kh_ssd_enqueue_write(self._h, node, generation, bytes(chain_hash), p, len(a), bytes(payload), len(payload),
                                          dtype_tag, dtype_size))

    def _acks(self, fn):
        buf = (KhFlushAck * 256)()
        n = fn(self._h, buf, 256)
        return [(int(buf[i].node), int(buf[i].generation), bytes(buf[i].hash), bool(buf[i].ok)) for i in range(n)]

    def drain_acks(self):
        return self._acks(lib().kh_ssd_drain_acks)

    def sync(self):
        return self._acks(lib().kh_ssd_sync)

    def read(self, chain_hash: bytes, expected_tokens: Sequence[int], pool_dtype_tag: int = -1, dtype_size: int = 2):
        """(payload, dtype tag) or None when the slot is missing or fails verification."""
        a, p = _u32(expected_tokens)
        cap = self.payload_bytes(8)
        buf = C.create_string_buffer(cap)
        tag = C.c_uint32(0)
        n = lib().kh_ssd_read(self._h, bytes(chain_hash), p, len(a), pool_dtype_tag, buf, cap, C.byref(tag))
        return None if n < 0 else (buf.raw[:n], int(tag.value))

    def stats(self) -> dict:
        s = KhSsdStats()
        lib().kh_ssd_get_stats(self._h, C.byref(s))
        return {n: int(getattr(s, n)) for n, _ in KhSsdStats._fields_}

    def close(self) -> None:
        if self._h:
            lib().kh_ssd_close(self._h)
            self._h = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


FINISH_KINDS = {0: None, 1: "stop", 2: "length", 3: "error", 4: "cancelled"}


@dataclass
class SeqState:
    blocks: List[int]
    num_tokens: int
    generated: int
    spec_proposed: int
    spec_accepted: int
    standdown: int
    cached_tokens: int


class Engine:
    """Engine::{new, submit, step, set_drafter, spec_stats} (engine.rs:1006-1407)."""

    def __init__(self, config: EngineConfig, model: StepModel, pipelined: bool = True):
        """``pipelined``: use the model's launch/collect pair (when it has one) for steady-state plain decode
        (engine.rs:1428-1475); the reference always does."""
        self.config, self._model, self._drafter = config, model, None
        self._h = _P()
        c = config.to_c()
        _check(lib().kh_engine_create(C.byref(c), C.byref(model.c), C.byref(self._h)))
        if pipelined and model.pipeline is not None:
            _check(lib().kh_engine_set_pipeline(self._h, C.byref(model.pipeline)))

    def set_drafter(self, drafter: Drafter) -> None:
        self._drafter = drafter
        _check(lib().kh_engine_set_drafter(self._h, C.byref(drafter.c)))

    def drafter_memory(self):
        """Engine::drafter_memory (engine.rs:1128-1132): dict of the attached drafter's footprint, or None."""
        m = KhDrafterMemory()
        if not lib().kh_engine_drafter_memory(self._h, C.byref(m)):
            return None
        return {"weights_bytes": int(m.weights_bytes), "kv_allocated_bytes": int(m.kv_allocated_bytes),
                "kv_used_bytes": int(m.kv_used_bytes)}

    def set_ssd(self, directory: str, fingerprint: bytes, layers: int, kv_heads: int, head_dim: int, max_bytes: int = 1 << 40,
                read_block=None, write_block=None, kv=None, dtype_tag: int = 7, dtype_size: int = 2) -> None:
        """Attaches the SSD tier (kh_engine_set_ssd). With ``kv`` (an api.PagedKv) the block IO is kc_kv_read_block /
        kc_kv_write_block on the model's pool; otherwise read_block(block) -> bytes and write_block(block, bytes) are
        Python callables (fake models)."""
        g = KhSlabGeometry(layers, kv_heads, head_dim, self.config.block_size)
        io = KhBlockIo()
        if kv is not None:
            from . import _lib as L
            cl = L.lib()
            io.read, io.write = C.cast(cl.kc_kv_read_block, BLOCK_READ_FN), C.cast(cl.kc_kv_write_block, BLOCK_WRITE_FN)
            self._ssd_keep = (kv,)
        else:
            def _r(_kv, block, dst, n):
                try:
                    data = read_block(int(block))
                    if len(data) != n:
                        return 2
                    C.memmove(dst, data, n)
                    return 0
                except Exception:
                    return 2

            def _w(_kv, block, src, n):
                try:
                    write_block(int(block), C.string_at(src, n))
                    return 0
                except Exception:
                    return 2
            io.read, io.write = BLOCK_READ_FN(_r), BLOCK_WRITE_FN(_w)
            self._ssd_keep = (io.read, io.write, read_block, write_block)
        io.dtype_tag, io.dtype_size = dtype_tag, dtype_size
        _check(lib().kh_engine_set_ssd(self._h, str(directory).encode(), bytes(fingerprint), C.byref(g), max_bytes, C.byref(io)))

    def ssd_sync(self) -> None:
        lib().kh_engine_ssd_sync(self._h)

    def ssd_stats(self) -> dict:
        s = KhSsdStats()
        lib().kh_engine_ssd_stats(self._h, C.byref(s))
        return {n: int(getattr(s, n)) for n, _ in KhSsdStats._fields_}

    def set_pipelined(self, on: bool) -> None:
        """Turns pipelined plain decode on (the model must offer launch/collect) or off."""
        if on and self._model.pipeline is None:
            raise ValueError("this step model has no launch/collect pair")
        _check(lib().kh_engine_set_pipeline(self._h, C.byref(self._model.pipeline) if on else None))

    def submit(self, prompt: Sequence[int], max_tokens: int, stop_tokens: Sequence[int] = ()) -> int:
        a, p = _u32(prompt)
        s, sp = _u32(stop_tokens)
        out = _U64(0)
        _check(lib().kh_engine_submit(self._h, p, len(a), max_tokens, sp, len(s), C.byref(out)))
        return out.value

    def cancel(self, arrival: int) -> None:
        lib().kh_engine_cancel(self._h, arrival)

    def step(self) -> None:
        rc = lib().kh_engine_step(self._h)
        if rc != 0:
            msg = lib().kh_engine_last_error(self._h).decode()
            try:   # the step ran on this thread: the device library's own message names the failing call
                from . import _lib as _cuda
                detail = _cuda.lib().kc_last_error().decode("utf-8", "replace")
                if detail:
                    msg += f" ({detail})"
            except Exception:
                pass
            raise HostError(rc, msg)

    num_running = property(lambda self: int(lib().kh_engine_num_running(self._h)))
    num_waiting = property(lambda self: int(lib().kh_engine_num_waiting(self._h)))
    iterations = property(lambda self: int(lib().kh_engine_iterations(self._h)))
    forwards = property(lambda self: int(lib().kh_engine_forwards(self._h)))
    pipelined_steps = property(lambda self: int(lib().kh_engine_pipelined_steps(self._h)))

    def take_output(self, arrival: int, cap: int = 4096) -> Tuple[List[int], Optional[str]]:
        buf = (C.c_uint32 * cap)()
        n, fk = _U64(0), _I32(0)
        _check(lib().kh_engine_take_output(self._h, arrival, buf, cap, C.byref(n), C.byref(fk)))
        return list(buf[:n.value]), FINISH_KINDS[fk.value]

    def seq_state(self, arrival: int) -> SeqState:
        nb = _U64(0)
        _check(lib().kh_engine_seq_state(self._h, arrival, None, 0, C.byref(nb), None, None, None, None, None, None))
        buf = (C.c_uint32 * max(nb.value, 1))()
        nt, gen, sp, sa, sd, ct = _U64(0), _U64(0), C.c_uint32(0), C.c_uint32(0), _I32(0), C.c_uint32(0)
        _check(lib().kh_engine_seq_state(self._h, arrival, buf, nb.value, C.byref(nb), C.byref(nt), C.byref(gen),
                                         C.byref(sp), C.byref(sa), C.byref(sd), C.byref(ct)))
        return SeqState(list(buf[:nb.value]), nt.value, gen.value, sp.value, sa.value, sd.value, ct.value)

    def spec_stats(self) -> dict:
        s = KhSpecStats()
        lib().kh_engine_spec_stats(self._h, C.byref(s))
        return {n: int(getattr(s, n)) for n, _ in KhSpecStats._fields_}

    def block_manager(self) -> BlockManager:
        return BlockManager(0, 0, _borrowed=lib().kh_engine_block_manager(self._h))

    def cache_stats(self) -> dict:
        h, t, r = _U64(0), _U64(0), _U64(0)
        lib().kh_engine_cache_stats(self._h, C.byref(h), C.byref(t), C.byref(r))
        return {"hits_total": h.value, "tokens_reused_total": t.value, "resident_blocks": r.value}

    def run_to_completion(self, arrivals: Sequence[int], max_steps: int = 100000) -> dict:
        """Steps until every listed request has finished; returns arrival -> (tokens, finish kind)."""
        out = {a: ([], None) for a in arrivals}
        for _ in range(max_steps):
            pending = [a for a in arrivals if out[a][1] is None]
            if not pending:
                return out
            self.step()
            for a in pending:
                toks, fk = self.take_output(a)
                out[a] = (out[a][0] + toks, fk)
        raise RuntimeError("engine did not finish within max_steps")

    def __del__(self):
        try:
            if self._h:
                lib().kh_engine_free(self._h)
                self._h = _P()
        except Exception:
            pass
