"""Host-side logic of the kernel front ends that needs no GPU: tile-width choice, activation buffer pitch, and the
ctypes mirrors of the argument blocks against the sizes the built library reports."""

import ctypes as C
from pathlib import Path

import pytest
import torch

from nestor_b200.ops import gemm as G

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("mult", [16, 64, 128])
@pytest.mark.parametrize("n", [8, 40, 64, 120, 216, 256, 344, 640, 1000, 1920, 4096])
def test_tile_width_is_a_legal_multiple_and_never_wastes_a_whole_tile(n, mult):
    bn = G.pick_bn(n, mult=mult)
    assert bn % mult == 0 and mult <= bn <= 256
    tiles = -(-n // bn)
    assert tiles * bn - n < bn                      # the last tile holds at least one real column
    if n % 256 == 0:
        assert bn == 256                            # exact fits take the widest tile


def test_tile_width_examples():
    assert G.pick_bn(640, mult=64) == 256           # three wide tiles beat five of 128 for MN-major B (fixed cost per tile)
    assert G.pick_bn(128) == 128 and G.pick_bn(48) == 48
    assert G.pick_bn(1920, mult=16) in (240, 256)


@pytest.mark.parametrize("cols", [8, 64, 100, 168, 344, 1024])
def test_rows_buffer_pitch_covers_whole_64_column_atoms(cols):
    buf = G.rows_buffer(10, cols, torch.bfloat16, "cpu")
    assert buf.shape == (10, cols) and buf.stride(1) == 1
    assert buf.stride(0) % 64 == 0 and buf.stride(0) >= cols and buf.stride(0) - cols < 64


def test_argument_blocks_match_the_built_library():
    """The Python mirrors of the attention argument blocks have the size the compiled library reports (a stale binary
    or an edited struct would misread raw pointers). Skipped when the library has not been built on this machine."""

    if not (ROOT / "nestor_b200" / "_C" / "libnestor_b200.so").is_file():
        pytest.skip("kernel library not built")
    from nestor_b200.ops import _lib
    L = _lib.lib()
    L.nb_flash_bwd_args_size.restype = C.c_int
    L.nb_flash_args_size.restype = C.c_int
    assert L.nb_flash_bwd_args_size() == C.sizeof(_lib.FlashBwdArgs)
    assert L.nb_flash_args_size() == C.sizeof(_lib.FlashArgs)
    for name in ("nb_gemm", "nb_flash_fwd", "nb_flash_bwd", "nb_flash_bwd_noalloc", "nb_depth_read_norm",
                 "nb_allreduce_push", "nb_param_push", "nb_ns_prepare", "nb_bias_update", "nb_route_fwd"):
        assert hasattr(L, name), name              # the entry points the front ends bind
