"""The allocation-free attention-backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory where they call it (fixed memory
pools, a step recovering from an out-of-memory error, host frameworks that forbid allocator calls on
the hot path). ``nb_flash_bwd_noalloc`` serves them by keeping its scratch in a fixed device array.
This test checks that it produces what the regular entry point produces, twice in a row (the
scratch is shared and keeps the previous call's contents), and that it refuses oversized problems.
It sits last in collection order so that a run stopping at the first failure has already run
everything else, and it passes both on its own and after the other tests.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(q, k, v, o, do, lse, delta, dqkv, seg, H, hd, status):
    from nestor_b200.ops import _lib
    rows, inner = q.shape[0], H * hd
    a = _lib.FlashBwdArgs()
    a.Q, a.K, a.V, a.ld_qkv = q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0)
    a.O, a.ld_o, a.dO, a.ld_do = o.data_ptr(), o.stride(0), do.data_ptr(), do.stride(0)
    a.lse, a.delta = lse.data_ptr(), (delta.data_ptr() if delta is not None else None)
    a.dQ, a.dK, a.dV = dqkv.data_ptr(), dqkv.data_ptr() + inner * 2, dqkv.data_ptr() + 2 * inner * 2
    a.ld_dqkv = dqkv.stride(0)
    a.seg_start, a.nseg = seg.data_ptr(), seg.numel() - 1
    a.rows, a.H, a.hd, a.scale = rows, H, hd, 1.0 / hd
    a.status = status.data_ptr()
    a.max_tiles = -(-rows // 128) + seg.numel() - 1
    return a


def test_noalloc_entry_point_matches_regular_entry_point():
    from nestor_b200.ops import _lib, flash
    L = _lib.lib()
    L.nb_flash_bwd.argtypes = [C.POINTER(_lib.FlashBwdArgs), C.c_void_p]
    L.nb_flash_bwd.restype = C.c_int
    L.nb_flash_bwd_noalloc.argtypes = [C.POINTER(_lib.FlashBwdArgs), C.c_void_p]
    L.nb_flash_bwd_noalloc.restype = C.c_int
    L.nb_flash_bwd_noalloc_error.restype = C.c_char_p
    dev = torch.device("cuda")
    status = _lib.status_word(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (H, hd, lens) in enumerate([(5, 40, [300, 1, 129, 700]), (3, 64, [512, 64, 200])]):
        torch.manual_seed(call)
        rows, inner = sum(lens), H * hd
        qkv = torch.randn(rows, 3 * inner, device=dev).to(torch.bfloat16)
        seg = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
        q, k, v = qkv[:, :inner], qkv[:, inner:2 * inner], qkv[:, 2 * inner:]
        o, lse = flash.flash_fwd(q, k, v, seg, H, hd, 1.0 / hd)
        do = torch.randn(rows, inner, device=dev).to(torch.bfloat16)
        want = torch.full((rows, 3 * inner), float("nan"), device=dev, dtype=torch.bfloat16)
        got = torch.full_like(want, float("nan"))
        delta = torch.empty(rows, H, dtype=torch.float32, device=dev)
        assert L.nb_flash_bwd(C.byref(_args(q, k, v, o, do, lse, delta, want, seg, H, hd, status)), stream) == 0
        rc = L.nb_flash_bwd_noalloc(C.byref(_args(q, k, v, o, do, lse, None, got, seg, H, hd, status)), stream)
        assert rc == 0, L.nb_flash_bwd_noalloc_error()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        assert torch.isfinite(got.float()).all()
        rel = ((got.float() - want.float()).norm() / want.float().norm()).item()
        assert rel < 2e-2, (call, rel)
    # a problem beyond the built-in scratch is refused with a message, and nothing is launched
    big = _args(q, k, v, o, do, lse, None, got, seg, H, hd, status)
    big.rows = (1 << 20) // H + 1
    assert L.nb_flash_bwd_noalloc(C.byref(big), stream) == -100
    assert b"exceeds the built-in scratch" in L.nb_flash_bwd_noalloc_error()
