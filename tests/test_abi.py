"""The C-ABI library loads without a GPU or a driver and exports every symbol include/eider_b200.h declares; the ctypes
table in eider_b200/_lib.py lists the same set.  No compute call is made here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "eider_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"EIDER_B200_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from eider_b200 import build, _lib
    build.build()  # no-op when the in-tree library is current
    names = _declared()
    assert len(names) >= 40
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(_lib.SIGNATURES) == names
    _lib.load()


def test_host_only_entry_points():
    from eider_b200 import _lib
    lib = _lib.load()
    # pure host arithmetic: crates/eider-cuda/src/format.rs:520-527
    assert lib.eider_b200_nvfp4_scale_layout_len(128, 128) == 1024
    assert lib.eider_b200_nvfp4_scale_layout_len(130, 80) == 2048
    assert lib.eider_b200_nvfp4_gemm_tn_supported(512, 27648, 5120) == 1
    assert lib.eider_b200_nvfp4_gemm_tn_supported(512, 27648, 5136) == 0
    assert lib.eider_b200_nvfp4_grouped_gemm_supported(1536, 4096, 2048, 128) == 1
    assert lib.eider_b200_nvfp4_grouped_gemm_supported(1500, 4096, 2048, 128) == 0
    assert lib.eider_b200_moe_sort_scratch_bytes(32768, 128) == 128 * 128 * 4


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    from eider_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        _lib.load()
    except RuntimeError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must fail loudly")
