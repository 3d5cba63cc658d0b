"""Generates tests/golden/*.npz by EXECUTING the reference's own contract function.

Run where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/FastForwardAttention

example.py cannot be imported (its module body needs a GPU and the compiled extension), so
the text of ``torch_attn_func`` (example.py:6-7) is cut out of the file with ``ast`` and
executed as is; nothing of it is stored in this repository.  Each case drives the function
the way example.py:30-46 does (concatenate the new k/v row, evaluate on the whole prefix) on
seeded N(0,1) inputs and stores inputs and outputs.  16-bit floats are stored as their uint16
bit patterns because numpy has no bfloat16.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, dtype, B, H, Dh, prompt, steps, seed
CASES = [
    ("f32_d64", torch.float32, 2, 3, 64, 37, 4, 11),
    ("f16_d64", torch.float16, 2, 3, 64, 37, 4, 12),
    ("bf16_d128", torch.bfloat16, 2, 2, 128, 70, 3, 13),
    ("f16_d80", torch.float16, 1, 3, 80, 19, 3, 14),
    ("f32_d80", torch.float32, 1, 2, 80, 33, 2, 15),
    ("f16_d256", torch.float16, 1, 2, 256, 130, 3, 16),
    ("f32_d128", torch.float32, 1, 2, 128, 65, 2, 17),
    ("bf16_d64_noprompt", torch.bfloat16, 1, 2, 64, 0, 3, 18),
]


def load_reference_function(ref_root: str):
    src = open(os.path.join(ref_root, "example.py")).read()
    tree = ast.parse(src)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "torch_attn_func")
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "example.py", "exec"), ns)
    return ns["torch_attn_func"]


def to_np(x: torch.Tensor) -> np.ndarray:
    if x.dtype == torch.float32:
        return x.numpy()
    return x.contiguous().view(torch.int16).numpy().view(np.uint16)


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "..", "..", "..", "reference")
    fn = load_reference_function(ref_root)
    torch.set_num_threads(1)
    for name, dt, B, H, Dh, Lp, steps, seed in CASES:
        g = torch.Generator().manual_seed(seed)
        K = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
        V = torch.randn(B, H, Lp, Dh, generator=g).to(dt)
        scale = 1.0 / (Dh ** 0.5)
        rec = {"K": to_np(K), "V": to_np(V), "scale": np.float64(scale), "prompt": np.int64(Lp),
               "dtype": np.bytes_(str(dt).split(".")[-1])}
        Kc, Vc = K, V
        for i in range(steps):
            q = torch.randn(B, H, 1, Dh, generator=g).to(dt)
            k = torch.randn(B, H, 1, Dh, generator=g).to(dt)
            v = torch.randn(B, H, 1, Dh, generator=g).to(dt)
            t = Lp + i
            Kc = torch.cat([Kc, k], axis=-2)
            Vc = torch.cat([Vc, v], axis=-2)
            out = fn(q.view(B * H, 1, Dh), Kc.view(B * H, t + 1, Dh), Vc.view(B * H, t + 1, Dh), scale)
            rec[f"q{i}"], rec[f"k{i}"], rec[f"v{i}"] = to_np(q), to_np(k), to_np(v)
            rec[f"out{i}"] = to_np(out.view(B, H, Dh))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        print("wrote", name)


if __name__ == "__main__":
    main()
