"""The C ABI without a GPU: both shared libraries load, every entry point the headers declare is exported, the
Python signature tables cover exactly the declared set, and argument validation that needs no device answers
with a status and a message (never an abort), like kiln-mlx's error contract (crates/kiln-mlx/src/error.rs:54-72)."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared(header: str, macro: str):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(macro + r"\s+[^;(]*?\b(k[ch]_[a-z0-9_]+)\s*\(", text)))


def test_cuda_library_exports_every_declared_symbol():
    from kiln_b200 import _lib
    names = declared("kiln_cuda.h", "KC_API")
    assert len(names) >= 30
    handle = _lib.lib()
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert names == _lib.exported_symbols(), "kiln_b200/_lib.py signature table and include/kiln_cuda.h disagree"


def test_host_library_exports_every_declared_symbol():
    from kiln_b200 import host
    names = declared("kiln_host.h", "KH_API")
    handle = C.CDLL(str(host.LIB_PATH))
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert names == host.exported_symbols(), "kiln_b200/host.py signature table and include/kiln_host.h disagree"


def test_errors_are_statuses_with_messages():
    import torch
    from kiln_b200 import _lib as L
    lib = L.lib()
    h = C.c_void_p()
    assert lib.kc_ctx_create(0, None) == L.KC_ERR_INVALID
    assert b"NULL" in lib.kc_last_error()
    if not torch.cuda.is_available():
        rc = lib.kc_ctx_create(0, C.byref(h))
        assert rc == L.KC_ERR_CUDA and b"no CUDA device" in lib.kc_last_error()
    assert lib.kc_sync(None) == L.KC_ERR_INVALID
    assert lib.kc_live_objects() >= 0
    assert lib.kc_kv_create(None, 1, 1, 64, 1, 16, L.KC_BF16, C.byref(h)) == L.KC_ERR_INVALID


def test_no_cpu_fallback_in_the_product():
    """The package never imports the oracle and never computes on the host: the product path fails loudly instead."""
    for f in (ROOT / "kiln_b200").glob("*.py"):
        text = f.read_text()
        assert "import oracle" not in text and "from oracle" not in text, f"{f.name} reaches into oracle/"
    for f in list((ROOT / "kiln_b200" / "csrc").rglob("*.c*")) + list((ROOT / "include").glob("*.h")):
        assert "oracle/" not in f.read_text().replace("oracle/ ", ""), f"{f.name} references oracle/"
