"""Verify that an adapted checkpoint kept every router of its starting checkpoint bit-identical.

Compares all router weights and balancing biases between two checkpoints of the same experiment
(reference ``scripts/check_frozen_routers.py:60-99``). Exit status 1 on any difference.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

ROUTER_MARKERS = ("group_router.", "public_router.", "private_routers.", "expert_router.")


def router_keys(state: dict) -> list[str]:
    return sorted(k for k in state if any(m in k for m in ROUTER_MARKERS))


def compare(before: dict, after: dict) -> list[str]:
    changed = []
    for k in router_keys(before):
        if k not in after or not torch.equal(before[k], after[k]):
            changed.append(k)
    return changed


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("before", type=Path); ap.add_argument("after", type=Path)
    a = ap.parse_args(argv)
    b = torch.load(a.before, map_location="cpu", weights_only=False)["model"]
    c = torch.load(a.after, map_location="cpu", weights_only=False)["model"]
    changed = compare(b, c)
    print(f"{len(router_keys(b))} router tensors compared, {len(changed)} changed")
    for k in changed[:20]:
        print("  changed:", k)
    return 1 if changed else 0


if __name__ == "__main__":
    sys.exit(main())
