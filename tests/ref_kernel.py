"""Driver for the reference's own CUDA kernel, built unmodified into oracle/_ref/libffa_ref.so
by `make -C oracle ref` (test infrastructure; see oracle/ref_shim.cu).  Used on a GPU box to
pin the restated pruning rule against what the reference kernel actually does."""
import ctypes as C
import os

import torch

SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libffa_ref.so")


def available():
    return os.path.exists(SO)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class ReferenceKernel:
    """fp32 or fp16 only, like the reference (torch_ffa_api.cpp:60-101)."""

    def __init__(self, K, V, max_len, launch="optimized"):
        assert K.dtype in (torch.float32, torch.float16)
        self.L = C.CDLL(SO)
        self.L.ffa_ref_attention.argtypes = [C.c_int] * 5 + [C.c_float, C.c_int] + [C.c_void_p] * 7 + [C.c_float] + [C.c_int] * 4
        B, H, Lp, Dh = K.shape
        self.B, self.H, self.Dh, self.Lmax, self.dt = B, H, Dh, max_len, K.dtype
        self.es = K.element_size()
        dev = torch.device("cuda:0")
        x = 16 // self.es
        self.k_cache = torch.zeros(B, H, Dh // x, max_len, x, dtype=K.dtype, device=dev)
        self.v_cache = torch.zeros(B, H, max_len, Dh, dtype=K.dtype, device=dev)
        Kd, Vd = K.to(dev).contiguous(), V.to(dev).contiguous()
        torch.cuda.synchronize()
        if Lp > 0:
            rc = self.L.ffa_ref_cache_init(self.es, _p(self.k_cache), _p(self.v_cache), _p(Kd), _p(Vd), B, Lp, max_len, Dh, H)
            assert rc == 0, rc
        torch.cuda.synchronize()
        fp16 = K.dtype == torch.float16
        if launch == "optimized":
            # what get_launch_params returns with use_default_ft = false: its arg-min loop keeps the
            # LAST candidate (kernel_launch_utils.h:171-172), i.e. tpb 256, tpk 4, tpv 8 (fp16) / 1 (fp32)
            self.tpb, self.tpk, self.tpv = 256, 4, (8 if fp16 else 1)
        else:
            # FasterTransformer's static rule (kernel_launch_utils.h:137-154)
            self.tpv = 8 if fp16 else 4
            self.tpb, self.tpk = (64, 4) if Lp < 32 else (128, 2) if Lp < 2048 else (256, 1)

    def attention(self, q, k, v, scale, t, p=0.0, seq_lengths=None, right_or_no_padding=True):
        dev = self.k_cache.device
        q, k, v = (x.to(dev).contiguous() for x in (q, k, v))
        out = torch.zeros(self.B, self.H, self.Dh, dtype=self.dt, device=dev)
        sl = seq_lengths.to(dev).to(torch.int32).contiguous() if seq_lengths is not None else None
        torch.cuda.synchronize()
        rc = self.L.ffa_ref_attention(self.es, self.B, self.H, self.Dh, self.Lmax, float(scale), int(t), _p(q), _p(k), _p(v),
                                      _p(self.k_cache), _p(self.v_cache), _p(out), _p(sl), float(p), self.tpv, self.tpk,
                                      self.tpb, int(right_or_no_padding))
        torch.cuda.synchronize()
        assert rc == 0, f"reference kernel launch failed: cuda error {rc}"
        return out
