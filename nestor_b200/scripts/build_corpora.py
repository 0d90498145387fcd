"""Build the derived corpora of the continued-training protocols.

``seen-subset``: the window set an equal-token run consumed (optionally the multiset for a longer
equal-FLOP run). ``replay-mix``: a target corpus with a share of replayed extension data. Reference:
``scripts/build_seen_subset.py``, ``scripts/build_replay_mix.py``.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

from nestor_b200.data.corpora import build_replay_mix, build_seen_subset_bin


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("seen-subset")
    s.add_argument("--source", type=Path, required=True); s.add_argument("--output", type=Path, required=True)
    s.add_argument("--block-size", type=int, required=True); s.add_argument("--cpt-tokens", type=int, default=500_000_000)
    s.add_argument("--tokens-per-step", type=int, default=1_048_576); s.add_argument("--seed", type=int, default=0)
    s.add_argument("--multiset-steps", type=int, default=None); s.add_argument("--multiset-seed", type=int, default=1)
    r = sub.add_parser("replay-mix")
    r.add_argument("--target", type=Path, required=True); r.add_argument("--replay", type=Path, required=True)
    r.add_argument("--output", type=Path, required=True); r.add_argument("--block-size", type=int, required=True)
    r.add_argument("--target-share-pct", type=int, default=75); r.add_argument("--mix-tokens", type=int, default=504_000_000)
    r.add_argument("--tokens-per-step", type=int, default=1_048_576); r.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.cmd == "seen-subset":
        meta = build_seen_subset_bin(a.source, a.output, block_size=a.block_size, cpt_tokens=a.cpt_tokens,
                                     tokens_per_step=a.tokens_per_step, seed=a.seed, multiset_steps=a.multiset_steps,
                                     multiset_seed=a.multiset_seed)
    else:
        meta = build_replay_mix(a.target, a.replay, a.output, block_size=a.block_size, target_share_pct=a.target_share_pct,
                                mix_tokens=a.mix_tokens, tokens_per_step=a.tokens_per_step, seed=a.seed)
    print(json.dumps(meta, indent=2))


if __name__ == "__main__":
    main()
