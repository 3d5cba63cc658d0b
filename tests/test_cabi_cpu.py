"""CPU-side checks of the boundary: the library loads, exports every symbol the header
declares, and rejects bad arguments without touching a GPU."""
import ctypes as C
import os
import re

import pytest

from fastforwardattention_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ffa_c_api.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ffa_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = capi.lib()
    names = declared_symbols()
    assert len(names) >= 13
    for n in names:
        assert hasattr(L, n), n
    assert sorted(capi.SYMBOLS) == [n for n in names if n in capi.SYMBOLS]
    assert set(names) >= set(capi.SYMBOLS)


def test_argument_validation_without_gpu():
    L = capi.lib()
    kb, vb = C.c_size_t(), C.c_size_t()
    assert L.ffa_cache_bytes(capi.BF16, 32, 32, 32768, 128, C.byref(kb), C.byref(vb)) == 0
    assert kb.value == vb.value == 32 * 32 * 32768 * 128 * 2
    assert L.ffa_cache_bytes(capi.F32, 1, 32, 1000, 64, C.byref(kb), C.byref(vb)) == 0
    assert kb.value == 32 * 1000 * 64 * 4
    assert L.ffa_cache_bytes(7, 1, 1, 8, 64, C.byref(kb), C.byref(vb)) == -1
    assert L.ffa_cache_bytes(capi.F16, 1, 1, 8, 96, C.byref(kb), C.byref(vb)) == -2
    assert b"head_dim" in L.ffa_last_error()
    assert L.ffa_cache_bytes(capi.F16, 0, 1, 8, 64, C.byref(kb), C.byref(vb)) == -3
    assert L.ffa_cache_init(capi.F16, 1, 1, 9, 8, 64, None, None, None, None, None) == -3
    assert L.ffa_attention(None, None, None, None, None, None, None, 1.0, 0, None, 1, 0.0, None, None) == -4
    assert L.ffa_workspace_bytes(None, 0) == 0
    assert L.ffa_peer_push_target(None, None) == -4
    assert L.ffa_static_scratch_status(None, None) == -4
    assert L.ffa_launch_count() == 0


def test_python_module_fails_loudly_when_extension_is_missing(monkeypatch):
    import importlib

    import fastforwardattention_b200 as pkg

    def boom(name, package=None):
        raise ImportError("no module")

    monkeypatch.setattr(importlib, "import_module", boom)
    with pytest.raises(ImportError, match="compiled extension is missing"):
        pkg.FastForwardAttn


def test_extension_class_surface():
    from ff_attention import FastForwardAttn

    for name in ("attention", "get_cache", "set_mode", "launch_shape", "device_status"):
        assert hasattr(FastForwardAttn, name)
    import torch

    with pytest.raises(RuntimeError, match="CUDA tensors"):
        FastForwardAttn(torch.zeros(1, 1, 4, 64), torch.zeros(1, 1, 4, 64), 8, False)


def test_header_is_plain_c_and_links(tmp_path):
    """include/ffa_c_api.h must be usable from C (no C++, no CUDA headers): compile a C99
    translation unit against it, link the shared library, call one entry point."""
    import subprocess

    src = tmp_path / "use_header.c"
    src.write_text('#include "ffa_c_api.h"\n'
                   "int main(void) { size_t a, b; if (ffa_cache_bytes(FFA_DTYPE_F16, 2, 3, 8, 64, &a, &b) != FFA_OK) return 1;\n"
                   "  return (a == 2u * 3u * 8u * 64u * 2u && a == b && ffa_last_error() != 0) ? 0 : 2; }\n")
    exe = tmp_path / "use_header"
    libdir = os.path.dirname(capi.LIB_PATH)
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"), str(src),
                    "-L", libdir, "-lffa_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_peer_gather_arguments_without_gpu():
    """Buffer sizing and argument checks of the peer-memory gather need no device."""
    L = capi.lib()
    p = C.c_void_p()
    capi.check(L.ffa_plan_create_offline(capi.BF16, 32, 4, 128, 32768, 0, 148, 232448, 233472, C.byref(p)))
    half = 32 * 8 * 4 * 128 * 2                              # [B][world][H * Dh] bf16
    assert L.ffa_peer_gather_bytes(p, 8) == 2 * half + 256   # two halves + arrival flags
    assert L.ffa_peer_gather_bytes(p, 9) == 0 and L.ffa_peer_gather_bytes(p, 0) == 0
    assert L.ffa_peer_gather_bytes(None, 2) == 0
    need = L.ffa_peer_gather_bytes(p, 2)
    bufs = (C.c_void_p * 2)(0x10000, 0x20000)
    assert L.ffa_peer_gather_attach(p, 2, 2, bufs, need) == -3 and b"rank" in L.ffa_last_error()
    assert L.ffa_peer_gather_attach(p, 9, 0, bufs, need) == -3
    assert L.ffa_peer_gather_attach(p, 2, 0, bufs, need - 1) == -6 and b"need" in L.ffa_last_error()
    assert L.ffa_peer_gather_attach(p, 2, 0, (C.c_void_p * 2)(0x10000, 0), need) == -4
    assert L.ffa_peer_gather_attach(p, 2, 0, (C.c_void_p * 2)(0x10000, 0x20010), need) == -4
    assert L.ffa_peer_gather_attach(p, 2, 0, None, need) == -4
    assert L.ffa_peer_gather(p, 0x30000, 0x40000, 3, 100, None) == -4 and b"attach" in L.ffa_last_error()
    assert L.ffa_peer_gather_attach(p, 2, 1, bufs, need) == 0
    assert L.ffa_peer_gather(p, 0x30000, 0x40000, 3, 100, None) == -6       # no workspace: nothing is launched
    assert L.ffa_peer_gather_attach(p, 0, 0, None, 0) == 0                   # detach
    assert L.ffa_peer_gather(p, 0x30000, 0x40000, 3, 100, None) == -4
    g = C.c_void_p()
    assert L.ffa_peer_mem_alloc(0, C.byref(g), C.create_string_buffer(64)) == -4
    assert L.ffa_peer_mem_open(None, C.byref(g)) == -4
    assert L.ffa_peer_mem_close(None) == 0 and L.ffa_peer_mem_free(None) == 0
    L.ffa_plan_destroy(p)
