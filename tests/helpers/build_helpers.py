"""Build the CUDA test helpers next to their sources (in-tree, like the library itself)."""
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent.parent / "xlstm-metal_b200" / "csrc"
INCLUDE = HERE.parent.parent / "include"


def build(force: bool = False) -> Path:
    src, out = HERE / "timeout_probe.cu", HERE / "libtimeout_probe.so"
    deps = [src, CSRC / "tcgen05.cuh"]
    if out.exists() and not force and all(out.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return out
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler",
           "-fPIC", "-I", str(CSRC), "-I", str(INCLUDE), str(src), "-o", str(out)]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build())
