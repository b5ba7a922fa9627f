"""The C-ABI library loads and exports every symbol include/whirl_b200.h declares.  No GPU, no compute calls."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "whirl_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(whirl_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from whirl_llm_b200 import build
    path = build.build()
    lib = ctypes.CDLL(path)
    syms = declared_symbols()
    assert len(syms) >= 14
    for s in syms:
        assert hasattr(lib, s), f"{s} is declared in include/whirl_b200.h but not exported"


def test_bindings_cover_the_header():
    from whirl_llm_b200 import api
    assert sorted(api.DECLARED) == declared_symbols()
    assert api.lib.whirl_version() >= 100
    assert api.lib.whirl_status_string(0) == b"ok"
    # argument checks that need no device
    assert api.workspace_bytes(1024, 262144) > 0
    assert api.lib.whirl_topk_rows(None, 0, 1, 8, 4, 1.0, None, None, None, None, None, 0, None) == 1  # WHIRL_ERR_INVALID
    assert b"topk_rows" in api.lib.whirl_last_error()


def test_no_product_import_of_the_oracle():
    # the shipped package must not import, load or execute anything under oracle/
    pkg = os.path.join(ROOT, "whirl_llm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".hpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("no CPU or PyTorch fallback", ""), f"{f} mentions the oracle"
