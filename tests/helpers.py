"""Shared helpers for the tests: golden-fixture loading and dtype plumbing."""
import glob
import os

import numpy as np
import torch

# lines the tests want shown after the run (measured errors, timing tables): printed by conftest's terminal summary
REPORT = []


def report(line: str) -> None:
    REPORT.append(line)


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


ULP = {torch.float32: 2.0 ** -23, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


def max_err(a, b):
    return (a.double().cpu() - b.double().cpu()).abs().max().item()


def assert_close_ulp(got, ref64, dtype, what, ulps=1.0, floor=None):
    """|got - ref| <= ulps * ulp(|ref|) + floor, element-wise; ref is the fp64 value."""
    floor = floor if floor is not None else {torch.float32: 1e-6, torch.float16: 2e-4, torch.bfloat16: 2e-4}[dtype]
    err = (got.double().cpu() - ref64).abs()
    bound = ulps * ULP[dtype] * ref64.abs() + floor
    bad = err > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} elements off, worst {err.max().item():.3e}"


def same_dtype_gate(got, same, ref64, dtype, what):
    """The stated gate against the same-dtype torch function, widened only by that
    function's own measured distance from the fp64 value of the same inputs."""
    noise = max_err(same, ref64)
    err = max_err(got, same)
    assert err <= max(TOL[dtype], 1.25 * noise + ULP[dtype] * ref64.abs().max().item()), \
        f"{what}: err vs same-dtype torch {err:.3e}, oracle noise {noise:.3e}"
    return err, noise
