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


def _oracle(qkv, do, lens, H, hd):
    """fp32 PyTorch statement of the op: causal softmax attention per segment, gradients by autograd."""

    inner = H * hd
    x = qkv.float().requires_grad_()
    outs, b = [], 0
    for n in lens:
        q, k, v = (x[b:b + n, i * inner:(i + 1) * inner].view(n, H, hd).transpose(0, 1) for i in range(3))
        s = (q @ k.transpose(1, 2)) / hd
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool, device=x.device).triu(1), float("-inf"))
        outs.append((s.softmax(-1) @ v).transpose(0, 1).reshape(n, inner))
        b += n
    torch.cat(outs).backward(do.float())
    return x.grad


def test_args_struct_has_the_size_the_library_expects():
    from nestor_b200.ops import _lib
    L = _lib.lib()
    L.nb_flash_bwd_args_size.restype = C.c_int
    L.nb_flash_args_size.restype = C.c_int
    assert L.nb_flash_bwd_args_size() == C.sizeof(_lib.FlashBwdArgs)
    assert L.nb_flash_args_size() == C.sizeof(_lib.FlashArgs)


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
        exact = _oracle(qkv, do, lens, H, hd)
        rel = ((got.float() - exact).norm() / exact.norm()).item()
        assert rel < 2e-2, ("against the fp32 statement of the op", call, rel)
    # a problem beyond the built-in scratch is refused with a message, and nothing is launched
    big = _args(q, k, v, o, do, lse, None, got, seg, H, hd, status)
    big.rows = (1 << 20) // H + 1
    assert L.nb_flash_bwd_noalloc(C.byref(big), stream) == -100
    assert b"exceeds the built-in scratch" in L.nb_flash_bwd_noalloc_error()


def test_noalloc_entry_point_on_a_second_device():
    """The scratch symbol is resolved per device; a call on device 1 uses device 1's copy."""

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two devices")
    from nestor_b200.ops import _lib, flash
    L = _lib.lib()
    L.nb_flash_bwd_noalloc.argtypes = [C.POINTER(_lib.FlashBwdArgs), C.c_void_p]
    L.nb_flash_bwd_noalloc.restype = C.c_int
    L.nb_flash_bwd_noalloc_error.restype = C.c_char_p
    dev = torch.device("cuda", 1)
    with torch.cuda.device(dev):
        torch.manual_seed(3)
        H, hd, lens = 2, 40, [260, 130]
        rows, inner = sum(lens), H * hd
        status = _lib.status_word(dev)
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        qkv = torch.randn(rows, 3 * inner, device=dev).to(torch.bfloat16)
        seg = torch.tensor([0, 260, 390], dtype=torch.int32, device=dev)
        q, k, v = qkv[:, :inner], qkv[:, inner:2 * inner], qkv[:, 2 * inner:]
        o, lse = flash.flash_fwd(q, k, v, seg, H, hd, 1.0 / hd)
        do = torch.randn(rows, inner, device=dev).to(torch.bfloat16)
        got = torch.full((rows, 3 * inner), float("nan"), device=dev, dtype=torch.bfloat16)
        rc = L.nb_flash_bwd_noalloc(C.byref(_args(q, k, v, o, do, lse, None, got, seg, H, hd, status)), stream)
        assert rc == 0, L.nb_flash_bwd_noalloc_error()
        torch.cuda.synchronize(dev)
        _lib.check_status(dev)
        exact = _oracle(qkv, do, lens, H, hd)
        rel = ((got.float() - exact).norm() / exact.norm()).item()
        assert rel < 2e-2, rel
