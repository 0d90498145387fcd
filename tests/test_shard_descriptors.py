"""Host-side arithmetic of the rank-sharded expert banks (no GPU): which operands are gathered, and the
arena / staging offsets handed to the fused all-gather GEMM."""

import torch

from nestor_b200.ops import _lib
from nestor_b200.ops import gemm as G
from nestor_b200.parallel.shard import ShardedBanks


def _arena(n):
    return torch.zeros(n, dtype=torch.bfloat16)


def test_spec_only_for_bank_views_of_the_arena_whose_experts_divide_the_world():
    E, d, h = 8, 64, 24
    arena = _arena(64 + 3 * E * d * h)
    sb = ShardedBanks(arena, [arena.data_ptr(), arena.data_ptr() + 2, 0, 0][:2], rank=1)
    wg = arena[64 : 64 + E * d * h].view(E, d, h)
    wu = arena[64 + E * d * h : 64 + 2 * E * d * h].view(E, d, h)
    spec = sb.spec(wg, wu)
    assert spec is not None and spec.groups_per_rank == E // 2 and spec.arena_ptr == arena.data_ptr()
    assert spec.stage.numel() == 2 * E * d * h and sb.gathered_bytes == 2 * E * d * h * 2
    assert sb.spec(wg) is not None and sb.stage.numel() == 2 * E * d * h          # the staging buffer only grows
    assert sb.spec(torch.zeros(E, d, h, dtype=torch.bfloat16)) is None             # not a view of the arena
    assert sb.spec(arena[64 : 64 + 7 * d * h].view(7, d, h)) is None               # 7 experts over 2 ranks
    assert sb.spec(wg.float()) is None and sb.spec(wg[0]) is None                  # wrong dtype / not a bank
    assert sb.spec(wg, wu[:, :, : h // 2]) is None                                 # second operand of another shape
    assert ShardedBanks(arena, [arena.data_ptr()], rank=0).spec(wg) is None        # one rank: nothing to gather


def test_stage_descriptor_offsets_and_strided_groups():
    E, a, b, gap = 4, 16, 24, 64
    arena = _arena(128 + E * (a * b + gap) + E * a * b)
    B = torch.as_strided(arena, (E, a, b), (a * b + gap, b, 1), 128)           # groups at a stride wider than a group
    raw = torch.empty(2 * E * a * b + 128, dtype=torch.bfloat16)
    skip = (-raw.data_ptr() % 256) // 2                    # the front end insists on a 256-byte aligned staging buffer
    stage = raw[skip : skip + 2 * E * a * b]
    assert stage.data_ptr() % 256 == 0
    flags = torch.zeros(E + 1, dtype=torch.int32)
    spec = G.Gather(src=[arena.data_ptr(), arena.data_ptr()], arena_ptr=arena.data_ptr(), stage=stage, flags=flags,
                    groups_per_rank=2)
    args = _lib.GemmArgs()
    sB, sB2 = G._stage_for_gather(args, spec, B, None)
    assert sB2 is None and sB.shape == B.shape and sB.is_contiguous() and sB.data_ptr() == stage.data_ptr()
    assert args.gather_seg_src_off[0] == 128 * 2 and args.gather_seg_dst_off[0] == 0
    assert args.gather_group_bytes == a * b * 2 and args.gather_group_stride_src == (a * b + gap) * 2
    assert (args.gather_nseg, args.gather_groups_per_rank, args.gather_on) == (1, 2, 1)
    assert (args.gather_chunk, args.gather_nbuf, args.gather_lanes) == (8192, 4, 1)
