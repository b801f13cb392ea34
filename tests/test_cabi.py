"""The C ABI: the shared library loads without a GPU and exports every symbol that
include/bamboo_b200.h declares; the Python binding mirrors the descriptor struct."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bamboo_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from bamboo_b200 import lib
    handle = lib.load()
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(handle, name), name
    assert handle.bb_version() >= 100


def test_gemm_descriptor_layout_matches_header():
    from bamboo_b200 import lib
    text = open(os.path.join(ROOT, "include", "bamboo_b200.h")).read()
    body = text[text.index("typedef struct bb_gemm_desc"):text.index("} bb_gemm_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"(?:const\s+)?(?:void\*|long long|int)\s+([A-Za-z0-9_, ]+);", body)
    flat = [f.strip() for group in fields for f in group.split(",")]
    assert flat == [name for name, _ in lib.GemmDesc._fields_]
    assert ctypes.sizeof(lib.GemmDesc) % 8 == 0


def test_argument_errors_do_not_need_a_gpu():
    from bamboo_b200 import lib
    handle = lib.load()
    rc = handle.bb_gemm_bf16(None, None)
    assert rc == -1 and b"bb_gemm_bf16" in handle.bb_last_error()
