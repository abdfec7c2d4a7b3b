"""The C-ABI library without a GPU: it builds, loads, exports every declared symbol, and
rejects bad arguments with error codes before any CUDA work."""
import ctypes as C
import re
from pathlib import Path

from loopfuse_b200 import _native

HEADER = Path(__file__).resolve().parents[1] / "include" / "lf_sm100.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(lf_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol(native_lib):
    names = declared_functions()
    assert set(names) == set(_native.EXPORTS)
    for name in names:
        assert hasattr(native_lib, name), name


def test_strerror(native_lib):
    assert native_lib.lf_strerror(0) == b"ok"
    assert b"workspace" in native_lib.lf_strerror(-4)
    assert native_lib.lf_strerror(-999) == b"unknown status"


def test_workspace_bytes(native_lib):
    assert native_lib.lf_decode_workspace_bytes(64, 32, 1, 128, 1) == 0
    assert native_lib.lf_decode_workspace_bytes(64, 32, 1, 128, 4) == 64 * 32 * 4 * 130 * 4
    assert native_lib.lf_decode_workspace_bytes(64, 8, 4, 128, 8) == 64 * 8 * 4 * 8 * 130 * 4


def test_argument_validation_needs_no_gpu(native_lib):
    a = _native.LfPrefillArgs()
    assert native_lib.lf_prefill_bf16(C.byref(a), None) == -1       # null pointers
    a.q = a.k = a.v = a.out = 0x1000
    a.B, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = 1, 4, 3, 128, 128, 128
    assert native_lib.lf_prefill_bf16(C.byref(a), None) == -1       # Hq % Hkv
    a.Hkv = 4
    a.D = 96
    assert native_lib.lf_prefill_bf16(C.byref(a), None) == -2       # unsupported head dim
    a.D = 128
    a.q = 0x1008
    assert native_lib.lf_prefill_bf16(C.byref(a), None) == -3       # misaligned pointer

    d = _native.LfDecodeArgs()
    assert native_lib.lf_decode_bf16(C.byref(d), None) == -1
    d.q = d.k = d.v = d.out = 0x1000
    d.B, d.Hkv, d.G, d.Skv, d.D = 2, 2, 3, 512, 128
    assert native_lib.lf_decode_bf16(C.byref(d), None) == -2        # G not in {1,2,4,8}
    d.G = 4
    d.splits = 2
    for i, s in enumerate((8192, 4096, 128)):
        d.q_stride[i] = d.o_stride[i] = s
        d.k_stride[i] = d.v_stride[i] = s
    assert native_lib.lf_decode_bf16(C.byref(d), None) == -4        # no workspace
    d.splits = 33
    assert native_lib.lf_decode_bf16(C.byref(d), None) == -7        # more than 32 splits
    d.splits = 2
    assert native_lib.lf_decode_paged_bf16(C.byref(d), None) == -1  # no block table


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", tmp_path / "nope.so")
    try:
        _native.load()
    except RuntimeError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("load() must raise when the library is missing")


def test_build_fingerprint_covers_every_included_file():
    """Every file a .cu under csrc/ #includes from the source tree is part of the rebuild
    fingerprint, so editing any of them rebuilds the library."""
    import re
    from loopfuse_b200 import build as B
    covered = {p.resolve() for p in B.fingerprint_files()}
    seen, todo = set(), [p for p in B.CSRC.glob("*.cu")]
    while todo:
        f = todo.pop()
        if f in seen:
            continue
        seen.add(f)
        for inc in re.findall(r'#include\s+"([^"]+)"', f.read_text()):
            target = (f.parent / inc).resolve()
            assert target.exists(), f"{f.name} includes missing {inc}"
            assert target in covered, f"{target} is not in the build fingerprint"
            todo.append(target)
    assert any(p.name == "lf_prefill_wide.cuh" for p in seen)
