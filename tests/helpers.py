"""Shared helpers for the tests: golden-fixture loading and dtype plumbing."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
# max-abs gates stated by the benchmark definition: fp32 1e-6, fp16 / bf16 2e-3
TOL = {torch.float32: 1e-6, torch.float16: 2e-3, torch.bfloat16: 2e-3}


def golden_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def _t(a: np.ndarray, dt: torch.dtype) -> torch.Tensor:
    if dt == torch.float32:
        return torch.from_numpy(a.copy())
    return torch.from_numpy(a.view(np.int16).copy()).view(dt)


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    dt = DTYPES[bytes(z["dtype"]).decode()]
    steps = []
    i = 0
    while f"q{i}" in z:
        steps.append(tuple(_t(z[f"{k}{i}"], dt) for k in ("q", "k", "v", "out")))
        i += 1
    return {"dtype": dt, "K": _t(z["K"], dt), "V": _t(z["V"], dt), "scale": float(z["scale"]),
            "prompt": int(z["prompt"]), "steps": steps}
