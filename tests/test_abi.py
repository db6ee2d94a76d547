"""The C-ABI library loads on a machine without a GPU and exports what include/xlstm_cuda.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "xlstm_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xlstm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from xlstm_cuda import _lib
    lib = _lib.load()
    names = declared_symbols()
    assert "xlstm_mlstm_step" in names and "xlstm_mlstm_chunkwise_fwd" in names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(names) == set(_lib.exported_symbols()), "ctypes signature table out of sync with the header"


def test_version_and_status_strings_without_a_gpu():
    from xlstm_cuda import _lib
    lib = _lib.load()
    assert lib.xlstm_version() >= 100
    assert lib.xlstm_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert len(lib.xlstm_strerror(code)) > 3
    # argument checks run before any CUDA call
    assert lib.xlstm_softcap(None, None, 5, 15.0, 0, None) == -1
    assert lib.xlstm_mlstm_chunkwise_workspace_bytes(1, 1, 64, 64, 64, 64, 0) == 0


def test_no_product_module_imports_the_oracle():
    pkg = ROOT / "xlstm-metal_b200"
    for path in pkg.rglob("*.py"):
        src = path.read_text()
        assert "oracle" not in src.replace("# oracle", ""), f"{path} mentions the oracle"
