"""Place the reference's own CPU implementation of the decode path under ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY.

The reference is Python: nothing is compiled.  Its recurrent mLSTM cell is one torch-only file
(``xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py`` in the
reference project) that imports on any machine with torch.  This recipe copies that file, unmodified,
from the reference checkout into ``oracle/_ref/`` (git-ignored: it never enters the history, but it
travels to the GPU machine with the working tree, like a compiled reference library would) so that
the benchmark's reference arm can time the reference's own class on the host cores there.  Where
the checkout is absent the recipe does nothing and the arm falls back to the C restatement.
"""
from __future__ import annotations

import importlib.util
import os
import shutil
from pathlib import Path

_HERE = Path(__file__).resolve().parent
REF_DIR = _HERE / "_ref"
CELL_REL = "xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py"
CELL_FILE = REF_DIR / "mlstm_recurrent_kernel_cell.py"


def build(reference_root: str | None = None) -> Path | None:
    """Copy the cell file if the reference checkout is present; return its path (or None).  The checkout is looked
    for at ``reference_root``, else at ``$XLSTM_REFERENCE_ROOT``, else in a ``reference`` folder beside the repository."""
    root = reference_root or os.environ.get("XLSTM_REFERENCE_ROOT") or str(_HERE.parent.parent / "reference")
    src = Path(root) / CELL_REL
    if src.exists():
        REF_DIR.mkdir(parents=True, exist_ok=True)
        if not CELL_FILE.exists() or CELL_FILE.read_bytes() != src.read_bytes():
            shutil.copyfile(src, CELL_FILE)
    return CELL_FILE if CELL_FILE.exists() else None


def load_cell_class():
    """``mLSTMRecurrentKernelCell`` of the reference, imported from ``oracle/_ref`` (None if absent)."""
    if not CELL_FILE.exists():
        return None
    spec = importlib.util.spec_from_file_location("xlstm_ref_recurrent_cell", CELL_FILE)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.mLSTMRecurrentKernelCell


if __name__ == "__main__":
    print(build())
