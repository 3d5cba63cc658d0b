"""CPU oracle for the decoder masked multi-head attention step.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is the
checker used by the tests, by the smoke check and by the CPU-baseline leg of the benchmark.

Two things are restated here, each from the reference file and lines it follows:

* ``torch_attn_func`` -- the reference's own torch statement of the attention contract
  (example.py:6-7, README.md:29-30), driven step by step exactly as example.py:40-42 drives
  it (append the new k/v row, then evaluate on the whole prefix).  The arithmetic lives in
  PyTorch (the reference pins no version; this image has torch 2.11).  Pinned by the golden
  vectors under tests/golden, which are produced by executing the reference's function text.
* the pruning rule of the reference's CUDA kernel (attention.cu:1108-1126 softmax incl. the
  left-padding mask, :1184-1191 threshold and skip, :461-469 ``leq``, :1227-1256 new token is
  always kept).  The reference has no test that passes p > 0 and no CPU implementation of the
  rule, so no reference TEST pins it.  It is pinned instead against the reference itself:
  (a) the fp16 comparison quirk, exhaustively, against the CUDA toolkit's own host
  implementation of the same expression (oracle/half_leq_host.cu, tests/test_oracle.py);
  (b) the whole rule against the reference's own CUDA kernel, compiled unmodified into
  oracle/_ref and run on a GPU, whose kept set is read off its output with one-hot value rows
  (tests/test_reference_kernel_gpu.py): identical in fp32, identical in fp16 outside a band
  of the reference's own fp16 score noise around the threshold.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------------------
# The contract function (example.py:6-7).
# --------------------------------------------------------------------------------------
def torch_attn_func(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, softmax_temp: float) -> torch.Tensor:
    """softmax(Q K^T * temp) V on [N, Lq, Dh] x [N, L, Dh] operands, in the operands' dtype."""
    scores = torch.bmm(Q, K.transpose(1, 2)) * softmax_temp
    probs = torch.nn.functional.softmax(scores, dim=-1)
    return torch.bmm(probs, V)


class DecodeOracle:
    """Iterative decode driven like example.py:30-46, on pre-allocated buffers.

    example.py grows K and V with ``torch.cat`` every step (:40-41) and calls the contract
    function on the views ``[B*H, t+1, Dh]`` (:42).  Here the rows are written into buffers of
    the final length and the same call is made on a prefix view; the operands, and therefore
    the arithmetic, are identical, but nothing is reallocated.
    """

    def __init__(self, K: torch.Tensor, V: torch.Tensor, max_len: int, compute_dtype: Optional[torch.dtype] = None):
        B, H, Lp, Dh = K.shape
        assert V.shape == K.shape and max_len >= Lp
        self.B, self.H, self.Dh, self.Lmax = B, H, Dh, max_len
        self.in_dtype = K.dtype
        self.dtype = compute_dtype or K.dtype
        self.K = torch.zeros(B * H, max_len, Dh, dtype=self.dtype)
        self.V = torch.zeros(B * H, max_len, Dh, dtype=self.dtype)
        self.K[:, :Lp] = K.reshape(B * H, Lp, Dh).to(self.dtype)
        self.V[:, :Lp] = V.reshape(B * H, Lp, Dh).to(self.dtype)

    def append(self, k: torch.Tensor, v: torch.Tensor, t: int) -> None:
        self.K[:, t] = k.reshape(self.B * self.H, self.Dh).to(self.dtype)
        self.V[:, t] = v.reshape(self.B * self.H, self.Dh).to(self.dtype)

    def step(self, q, k, v, softmax_scale: float, t: int) -> torch.Tensor:
        """Append row t and return the attention over rows 0..t, shape [B, H, Dh]."""
        assert 0 <= t < self.Lmax
        self.append(k, v, t)
        N = self.B * self.H
        out = torch_attn_func(q.reshape(N, 1, self.Dh).to(self.dtype), self.K[:, : t + 1], self.V[:, : t + 1],
                              softmax_scale)
        return out.view(self.B, self.H, self.Dh)


def attention_reference(q, K, V, softmax_scale: float, dtype: torch.dtype, chunk: int = 64) -> torch.Tensor:
    """The contract function evaluated in ``dtype`` (float32 / float64 up-cast of the same
    inputs), chunked over the (batch*head) axis so that a long cache need not be up-cast at
    once.  q: [N, 1, Dh]; K, V: [N, L, Dh].  Returns [N, Dh] in ``dtype``."""
    outs = []
    for i in range(0, q.shape[0], chunk):
        outs.append(torch_attn_func(q[i:i + chunk].to(dtype), K[i:i + chunk].to(dtype), V[i:i + chunk].to(dtype),
                                    softmax_scale)[:, 0])
    return torch.cat(outs, 0)


# --------------------------------------------------------------------------------------
# The pruning rule (attention.cu:1108-1126, 1184-1191, 461-469, 1227-1256).
# --------------------------------------------------------------------------------------
def half_bits_as_number_rn(bits: np.ndarray) -> np.ndarray:
    """What ``__half(unsigned short)`` makes of a raw bit pattern.

    The reference's ``leq(uint16_t, uint16_t)`` hands two raw fp16 bit patterns to ``__hle``
    (attention.cu:466-469).  The implicit ``unsigned short -> __half`` conversion is the numeric
    constructor (round-to-nearest-even of the INTEGER value, ``__ushort2half_rn``), not a bit
    cast, so the numbers that get compared are the patterns themselves rounded to 11
    significant bits.  uint16 -> float32 is exact and float32 -> float16 rounds to nearest
    even, which is the same operation.
    """
    with np.errstate(over="ignore"):  # patterns above 65519 become +inf, as in the toolkit
        return bits.astype(np.uint16).astype(np.float32).astype(np.float16)


def leq_reference(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``leq(a, b)`` of attention.cu:461-469 for a tensor ``a`` and a scalar/broadcast ``b``.

    float32: plain ``a <= b`` (:461-464).  float16: the bit-pattern comparison described in
    :func:`half_bits_as_number_rn` (:466-469).  bfloat16 does not exist in the reference; the
    engine defines it as the plain value comparison, and so does this function.
    """
    if a.dtype == torch.float16:
        an = half_bits_as_number_rn(a.contiguous().view(torch.int16).numpy().view(np.uint16))
        bn = half_bits_as_number_rn(b.contiguous().view(torch.int16).numpy().view(np.uint16))
        return torch.from_numpy(an <= bn)
    return a <= b


def pruned_attention(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, softmax_scale: float, p: float,
                     first_key: Optional[torch.Tensor] = None, eps: float = 1e-6
                     ) -> Tuple[torch.Tensor, torch.Tensor, dict]:
    """One decode step under the reference's pruning rule.

    q: [N, Dh]; K, V: [N, t+1, Dh] with the new token already in row t; all in the storage
    dtype T (float32 / float16 / bfloat16).  ``first_key``: optional [N] int tensor, keys below
    it are masked (the left-padding overload, attention.cu:814-817, 1054, 1112-1113).

    Follows the kernel:
      s_i   = scale * (q . K_i)                              fp32           (:1053)
      m     = max over unmasked i                                            (:1072, 1081-1106)
      e_i   = exp(s_i - m), 0 where masked                                   (:1112-1113)
      inv   = 1 / (sum_i e_i + eps)                                          (:1122)
      P_i   = cvt_T(e_i * inv)                                               (:1124-1126)
      Theta = cvt_T(p * inv)                                                 (:1184-1185)
      cached position i < t is skipped iff leq(P_i, Theta)                   (:1188-1191)
      the new token t is always kept                                         (:1227-1256)
      out   = sum_{kept} P_i * V_i, NOT renormalised
    Deliberate differences from the kernel's shortcuts, none of which is part of the rule:
    exp and the division are evaluated exactly (the kernel uses __expf and __fdividef) and the
    weighted sum is accumulated in fp32 and rounded once (the kernel's fp16 path accumulates
    in fp16).  Positions whose P_i lies within one rounding step of Theta can therefore differ
    from a run of the kernel; ``info['borderline']`` counts them.

    Returns (out [N, Dh] in T, kept [N, t+1] bool, info).
    """
    T = q.dtype
    N, L, Dh = K.shape
    t = L - 1
    qf, Kf = q.to(torch.float32), K.to(torch.float32)
    s = torch.einsum("nd,nld->nl", qf, Kf) * softmax_scale
    masked = torch.zeros(N, L, dtype=torch.bool)
    if first_key is not None:
        masked = torch.arange(L)[None, :] < first_key.to(torch.int64)[:, None]
    m = s.masked_fill(masked, -float("inf")).max(dim=1, keepdim=True).values
    e = torch.exp(s - m).masked_fill(masked, 0.0)
    inv = 1.0 / (e.sum(dim=1, keepdim=True) + eps)
    P = (e * inv).to(T)
    theta = (p * inv).to(torch.float32).to(T)
    skip = leq_reference(P, theta)
    skip[:, t] = False
    kept = ~skip
    Pk = P.to(torch.float32) * kept
    out = torch.einsum("nl,nld->nd", Pk, V.to(torch.float32)).to(T)

    # Borderline census: positions whose decision flips if P_i moves by one unit in the last
    # place of T (fp32: by a relative 1e-5, the size of the kernel's exp shortcut plus the
    # summation-order noise of a 64..256-term fp32 dot product in the exponent).
    if T in (torch.float32, torch.float64):
        lo, hi = (e * inv) * (1 - 1e-5), (e * inv) * (1 + 1e-5)
        flips = (lo <= theta) != (hi <= theta)
    else:
        bits = P.contiguous().view(torch.int16).to(torch.int32)
        up = (bits + 1).to(torch.int16).view(T)
        dn = torch.clamp(bits - 1, min=0).to(torch.int16).view(T)
        flips = leq_reference(up, theta) != leq_reference(dn, theta)
    flips[:, t] = False
    info = {"borderline": int(flips.sum()), "kept_fraction": float(kept[:, :t].float().mean()) if t else 1.0}
    return out, kept, info


def torch_rounding_points(q, K, V, softmax_scale: float) -> torch.Tensor:
    """The contract function's four rounding points, restated in fp32 arithmetic.

    torch evaluates ``bmm(softmax(bmm(Q, K^T) * scale), V)`` on fp16/bf16 operands as: scores
    accumulated in fp32 and rounded to T; times scale in fp32, rounded to T; softmax in fp32,
    rounded to T; weighted sum accumulated in fp32, rounded to T (example.py:6-7 as executed by
    torch's CPU kernels).  This is what the engine's ``round_like_torch`` mode reproduces; the
    function exists so the test can separate rounding-placement error from arithmetic error.
    q: [N, Dh]; K, V: [N, L, Dh].  Returns [N, Dh] in T.
    """
    T = q.dtype
    s = torch.einsum("nd,nld->nl", q.float(), K.float()).to(T)
    s = (s.float() * softmax_scale).to(T)
    P = torch.softmax(s.float(), dim=-1).to(T)
    return torch.einsum("nl,nld->nd", P.float(), V.float()).to(T)


def algorithmic_bytes(elem_size: int, B: int, H: int, Dh: int, t: int, kept_rows: Optional[int] = None) -> int:
    """HBM bytes one decode step must move: K and V rows 0..t-1 read once, q/k/v read, rows t of
    both caches written, out written.  With pruning only the kept V rows are read."""
    if kept_rows is None:
        return elem_size * B * H * Dh * (2 * t + 6)
    return elem_size * B * H * Dh * (t + 6) + elem_size * Dh * kept_rows


def softmax_scale_for(Dh: int) -> float:
    return 1.0 / math.sqrt(Dh)
