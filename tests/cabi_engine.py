"""Test-side driver of the C ABI: torch owns the device memory, every computation goes
through libffa_b200.so with raw pointers (the way a non-torch host would call it)."""
import ctypes as C

import torch

from fastforwardattention_b200 import capi

CODE = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class CAbiEngine:
    def __init__(self, K, V, max_len, use_default=False, with_scores=True, device="cuda:0"):
        self.L = capi.lib()
        self.dev = torch.device(device)
        B, H, Lp, Dh = K.shape
        self.B, self.H, self.Dh, self.Lmax, self.dtype = B, H, Dh, max_len, K.dtype
        code = CODE[K.dtype]
        kb, vb = C.c_size_t(), C.c_size_t()
        capi.check(self.L.ffa_cache_bytes(code, B, H, max_len, Dh, C.byref(kb), C.byref(vb)))
        es = K.element_size()
        assert kb.value == B * H * max_len * Dh * es
        self.k_cache = torch.empty(B, H, max_len, Dh, dtype=K.dtype, device=self.dev)
        self.v_cache = torch.empty(B, H, max_len, Dh, dtype=K.dtype, device=self.dev)
        # canaries: rows the engine must never touch are checked by the tests
        self.k_cache.fill_(777.0)
        self.v_cache.fill_(777.0)
        Kd, Vd = K.to(self.dev).contiguous(), V.to(self.dev).contiguous()
        capi.check(self.L.ffa_cache_init(code, B, H, Lp, max_len, Dh, _ptr(Kd), _ptr(Vd), _ptr(self.k_cache),
                                         _ptr(self.v_cache), _stream()))
        self.plan = C.c_void_p()
        capi.check(self.L.ffa_plan_create(code, B, H, Dh, max_len, int(use_default), self.dev.index or 0,
                                          C.byref(self.plan)))
        n = self.L.ffa_workspace_bytes(self.plan, int(with_scores))
        self.ws = torch.empty(n, dtype=torch.uint8, device=self.dev)
        capi.check(self.L.ffa_workspace_bind(self.plan, _ptr(self.ws), n, _stream()))
        self.mask = torch.zeros(B, H, (max_len + 31) // 32, dtype=torch.int32, device=self.dev)
        torch.cuda.synchronize()

    def close(self):
        if self.plan:
            self.L.ffa_plan_destroy(self.plan)
            self.plan = None

    def __del__(self):
        self.close()

    def set_mode(self, mode):
        capi.check(self.L.ffa_plan_set_mode(self.plan, mode))

    def set_prune_path(self, path):
        capi.check(self.L.ffa_plan_set_prune_path(self.plan, path))

    def set_launch(self, tile_rows=0, stages=0, consumer_warps=0, ctas_per_sm=0, grid=0):
        l = capi.Launch(tile_rows, stages, consumer_warps, ctas_per_sm, grid, 0, 0)
        capi.check(self.L.ffa_plan_set_launch(self.plan, C.byref(l)))

    def launch_shape(self, t):
        l = capi.Launch()
        capi.check(self.L.ffa_plan_get_launch(self.plan, t, C.byref(l)))
        return {n: getattr(l, n) for n, _ in capi.Launch._fields_}

    def attention(self, q, k, v, scale, t, p=0.0, seq_lengths=None, right_or_no_padding=True, want_mask=False):
        q, k, v = (x.to(self.dev).contiguous() for x in (q, k, v))
        out = torch.empty(self.B, self.H, self.Dh, dtype=self.dtype, device=self.dev)
        sl = seq_lengths.to(self.dev).to(torch.int32).contiguous() if seq_lengths is not None else None
        capi.check(self.L.ffa_attention(self.plan, _ptr(q), _ptr(k), _ptr(v), _ptr(self.k_cache), _ptr(self.v_cache),
                                        _ptr(out), float(scale), int(t), _ptr(sl), int(right_or_no_padding), float(p),
                                        _ptr(self.mask) if want_mask else None, _stream()))
        return out

    def status(self):
        s = C.c_int(0)
        self.L.ffa_device_status(self.plan, _stream(), C.byref(s))
        return s.value

    def kept(self, t):
        """[B*H, t+1] bool from the packed mask."""
        m = self.mask.cpu().view(self.B * self.H, -1).to(torch.int64) & 0xFFFFFFFF
        bits = (m[:, :, None] >> torch.arange(32)[None, None, :]) & 1
        return bits.reshape(self.B * self.H, -1)[:, : t + 1].bool()
