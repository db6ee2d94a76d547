"""Deterministic parameter fill shared by the fixture generator and the tests.

Values come from numpy's PCG64 stream (stable across numpy / torch versions) in sorted
parameter-name order, so the reference modules (when the fixtures are made) and the CUDA-backed
modules (when the tests run) hold identical weights without shipping them.
"""
import numpy as np
import torch


def fill_parameters(named: dict, seed: int) -> None:
    rng = np.random.default_rng(seed)
    with torch.no_grad():
        for name in sorted(named):
            p = named[name]
            shape = tuple(p.shape)
            if name.endswith("fgate_proj.bias") or name.endswith("W_f.bias"):
                val = np.linspace(3.0, 6.0, shape[0])
            elif "norm" in name and name.endswith("weight"):
                val = 1.0 + 0.1 * rng.standard_normal(shape)
            elif name.endswith("bias"):
                val = 0.1 * rng.standard_normal(shape)
            elif name.startswith("embedding") or ".R_" in name or name.startswith("R_"):
                val = 0.3 * rng.standard_normal(shape)
            else:
                val = 0.06 * rng.standard_normal(shape)
            p.copy_(torch.from_numpy(np.asarray(val, np.float32)).to(p.dtype))
