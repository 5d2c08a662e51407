"""The allocation-free decode-attention entry point, called the way a host without
torch's allocator would call it: through its exported C symbol, with raw device
pointers.  Some callers of this library cannot allocate device memory at all (a
plugin inside a server whose pool owns the GPU, a decode loop where cudaMalloc
would stall the device), so this variant keeps its split-KV partials in an 8 MiB
array built into the library instead of a caller-provided workspace.

Checked here: two calls in a row give the same result as the regular,
workspace-taking entry point (the shared array keeps the first call's contents,
the second call must not be disturbed by them), and a request larger than the
built-in array is refused with a clear message instead of being launched.
This file sorts last on purpose: a stop-at-first-failure run has then already
executed every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    import penny_cpp
    lib = ctypes.CDLL(penny_cpp.__file__)
    fn = lib.penny_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p,
                                                                ctypes.c_size_t]
    return fn


def _call(fn, qkv, kc, vc, pos, out, Hq, Hkv, splits, scale):
    err = ctypes.create_string_buffer(256)
    rc = fn(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), out.data_ptr(), qkv.shape[0], Hq, Hkv,
            kc.shape[2], splits, scale, torch.cuda.current_stream().cuda_stream, err, len(err))
    return rc, err.value.decode()


def test_no_alloc_entry_matches_workspace_entry_twice():
    from penny_b200._ext import ops
    fn = _entry()
    torch.manual_seed(11)
    B, Hq, Hkv, D, L = 6, 8, 2, 128, 700
    scale = 1.0 / math.sqrt(D)
    kc = torch.randn(B, Hkv, L, D, device="cuda").bfloat16()
    vc = torch.randn(B, Hkv, L, D, device="cuda").bfloat16()
    for call, (splits, seed) in enumerate([(4, 1), (3, 2)]):
        g = torch.Generator(device="cuda").manual_seed(seed)
        qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda", generator=g).bfloat16()
        pos = torch.randint(0, L - 1, (B,), device="cuda", generator=g).to(torch.int32)
        want = torch.empty(B, Hq * D, device="cuda", dtype=torch.bfloat16)
        ws = torch.empty(ops.decode_attn_workspace_bytes(B, Hq, splits), dtype=torch.uint8, device="cuda")
        ops.decode_attention(qkv, kc, vc, pos, want, ws, Hq, Hkv, splits, scale)
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc, msg = _call(fn, qkv, kc, vc, pos, got, Hq, Hkv, splits, scale)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.cuda.memory_allocated() == before
        # same kernels, same inputs: the tolerance the attention tests use
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_no_alloc_entry_rejects_oversized_request():
    fn = _entry()
    B, Hq, Hkv, D, L = 64, 32, 8, 128, 64
    qkv = torch.zeros(B, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(B, Hkv, L, D, device="cuda", dtype=torch.bfloat16)
    pos = torch.zeros(B, dtype=torch.int32, device="cuda")
    out = torch.zeros(B, Hq * D, device="cuda", dtype=torch.bfloat16)
    rc, msg = _call(fn, qkv, kc, kc, pos, out, Hq, Hkv, 16, 0.1)  # 64*32*16*520 B = 17 MB > 8 MiB
    assert rc == 2 and "too large" in msg
    rc, msg = _call(fn, qkv, kc, kc, pos, out, Hq, 5, 1, 0.1)     # Hq not a multiple of Hkv
    assert rc == 1 and "bad shape" in msg
