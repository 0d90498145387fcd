"""Continued-training protocols as environment emitters: the context-length ladder and domain adaptation.

A protocol object describes one continued-training run of a registered cell and turns it into the
``DCLM_*`` / ``NESTOR_*`` environment a launcher exports before ``nestor_cli --experiment <cell>``.

Length extension (reference ``nestor/continual/extension.py``): 4k -> 8k/16k/32k/64k, 1,048,576
tokens per step, an equal-token budget of 477 steps (500M tokens), RoPE base raised per length, peak
learning rates a quarter of pretraining, 10 % warmup. The two equal-FLOP settings (Nestor only) run
``ceil(500M / r / 1,048,576)`` steps where ``r`` is the cell's forward FLOPs per token relative to the
baseline of its rung, with the learning rates scaled by ``r``; the "repeated" variant trains on the
equal-token run's window multiset. Domain adaptation (``nestor/continual/adaptation.py``): 477 steps
at 32k on one of four target corpora with 0 or 25 % replay of extension data; routed families train
with frozen routers.

``python -m nestor_b200.continual.protocols {extension,adaptation} ...`` prints the ``export`` lines.
"""

from __future__ import annotations

import argparse
import dataclasses as dc
import math
import shlex
from pathlib import Path

from nestor_b200.continual.flops import flop_ratio, split_experiment_name

PRETRAIN_LENGTH = 4096
LENGTHS = (8192, 16384, 32768, 65536)
ROPE_BASE = {4096: 10_000, 8192: 500_000, 16384: 1_000_000, 32768: 2_000_000, 65536: 5_000_000}
TOKENS_PER_STEP = 1_048_576
EXTENSION_TOKENS = 500_000_000
EXTENSION_STEPS = math.ceil(EXTENSION_TOKENS / TOKENS_PER_STEP)     # 477
WARMUP_FRACTION = 0.1
LR_MUON, LR_ADAMW = 0.0025, 7.5e-5
HELDOUT_DOCUMENTS = {8192: 200, 16384: 200, 32768: 200, 65536: 100}
SETTINGS = ("equal_tokens", "equal_flops_new", "equal_flops_repeated")
REFERENCE_FAMILY = "moe"

ADAPTATION_LENGTH = 32768
ADAPTATION_STEPS = EXTENSION_STEPS
PAPER_EXPERIMENTS = ("nestor_500m", "moe_500m", "dense_1b")
PAPER_REPLAY_PCTS = (0, 25)
MIX_TOKENS = 504_000_000
EVAL_SEQUENCES = 200
FROZEN_ROUTER_FAMILIES = ("moe", "nestor")


def extension_corpus_name(seq_len: int) -> str:
    return f"dclm_longdoc_ge{seq_len}_train.bin"


def heldout_corpus_name(seq_len: int) -> str:
    return f"dclm_longdoc_ge{seq_len}_val.bin"


def repeated_corpus_name(seq_len: int, steps: int) -> str:
    return f"dclm_longdoc_ge{seq_len}_train_repeated_T{steps}.bin"


def extension_flop_ratio(experiment: str, seq_len: int, reference: str = REFERENCE_FAMILY) -> float:
    """``r(S)``: the cell's causal body FLOPs per token over those of ``<reference>_<scale>``."""

    return flop_ratio(experiment, f"{reference}_{split_experiment_name(experiment)[1]}", seq_len=seq_len)


def equal_flop_steps(ratio: float) -> int:
    return math.ceil(EXTENSION_TOKENS / ratio / TOKENS_PER_STEP)


def resolve_checkpoint(path: Path) -> Path:
    """A checkpoint file, or the newest ``model_final.pt`` under a run directory."""

    if path.is_file():
        return path
    found = sorted(path.rglob("model_final.pt"), key=lambda p: p.stat().st_mtime)
    if not found:
        raise FileNotFoundError(f"no model_final.pt under {path}")
    return found[-1]


@dc.dataclass(frozen=True)
class ExtensionRun:
    experiment: str
    seq_len: int
    setting: str = "equal_tokens"
    reference: str = REFERENCE_FAMILY

    def __post_init__(self) -> None:
        family, _ = split_experiment_name(self.experiment)
        if self.seq_len not in LENGTHS:
            raise ValueError(f"seq_len must be one of {LENGTHS}, got {self.seq_len}")
        if self.setting not in SETTINGS:
            raise ValueError(f"setting must be one of {SETTINGS}, got {self.setting!r}")
        if self.reference not in ("moe", "dense"):
            raise ValueError(f"reference must be 'moe' or 'dense', got {self.reference!r}")
        if self.setting != "equal_tokens" and family != "nestor":
            raise ValueError(f"{self.setting!r} is a Nestor setting; the baselines run at equal tokens")

    family = property(lambda self: split_experiment_name(self.experiment)[0])
    scale = property(lambda self: split_experiment_name(self.experiment)[1])

    @property
    def flop_ratio(self) -> float:
        return 1.0 if self.setting == "equal_tokens" else extension_flop_ratio(self.experiment, self.seq_len, self.reference)

    steps = property(lambda self: equal_flop_steps(self.flop_ratio))
    warmup_steps = property(lambda self: int(self.steps * WARMUP_FRACTION))
    lr_muon = property(lambda self: LR_MUON * self.flop_ratio)
    lr_adamw = property(lambda self: LR_ADAMW * self.flop_ratio)
    rope_base = property(lambda self: ROPE_BASE[self.seq_len])
    seqs_per_step = property(lambda self: TOKENS_PER_STEP // self.seq_len)
    tokens = property(lambda self: self.steps * TOKENS_PER_STEP)
    run_suffix = property(lambda self: f"ext{self.seq_len}_{self.setting}")

    def corpus(self, data_dir: Path) -> Path:
        if self.setting == "equal_flops_repeated":
            return data_dir / repeated_corpus_name(self.seq_len, self.steps)
        return data_dir / extension_corpus_name(self.seq_len)

    def heldout(self, data_dir: Path) -> Path:
        return data_dir / heldout_corpus_name(self.seq_len)

    def env(self, *, data_dir: Path, init_checkpoint: Path | None, output_root: Path = Path("outputs")) -> dict[str, str]:
        env = {
            "DCLM_BLOCK_SIZE": str(self.seq_len),
            "DCLM_ROPE_BASE": str(self.rope_base),
            "DCLM_DATA_PATH": str(self.corpus(data_dir)),
            "DCLM_MAX_STEPS": str(self.steps),
            "DCLM_WARMUP_STEPS": str(self.warmup_steps),
            "DCLM_LR_MUON": f"{self.lr_muon:.6g}",
            "DCLM_LR_ADAMW": f"{self.lr_adamw:.6g}",
            "DCLM_RUN_SUFFIX": self.run_suffix,
            "NESTOR_OUTPUT_ROOT": str(output_root / "continual" / f"{self.experiment}_{self.run_suffix}"),
            "NESTOR_GATHERED_CAP_BUCKET": str(self.seq_len // 32),
            "CONTINUAL_SEQS_PER_STEP": str(self.seqs_per_step),
            "CONTINUAL_HELDOUT": str(self.heldout(data_dir)),
            "CONTINUAL_HELDOUT_DOCUMENTS": str(HELDOUT_DOCUMENTS[self.seq_len]),
        }
        if init_checkpoint is not None:
            env["DCLM_INIT_CHECKPOINT"] = str(resolve_checkpoint(init_checkpoint))
        return env

    def describe(self) -> str:
        return (f"{self.experiment} -> {self.seq_len // 1024}k {self.setting}: r={self.flop_ratio:.4f} steps={self.steps} "
                f"warmup={self.warmup_steps} tokens={self.tokens:,} lr_muon={self.lr_muon:.6g} "
                f"lr_adamw={self.lr_adamw:.6g} rope={self.rope_base}")


@dc.dataclass(frozen=True)
class Corpus:
    name: str
    title: str
    train_bin: str
    test_bin: str
    eval_mode: str     # "documents" (score whole documents) or "packed" (contiguous windows)


CORPORA = {c.name: c for c in (
    Corpus("pg19", "PG-19 (books)", "pg19_train.bin", "pg19_test.bin", "documents"),
    Corpus("owm", "OpenWebMath (mathematics)", "owm_train.bin", "owm_test.bin", "packed"),
    Corpus("algstack", "AlgebraicStack (code)", "algstack_train.bin", "algstack_test.bin", "packed"),
    Corpus("fw2de", "FineWeb-2 German", "fw2de_train.bin", "fw2de_test.bin", "packed"),
)}
REPLAY_SOURCE = extension_corpus_name(ADAPTATION_LENGTH)
FORGETTING_HELDOUT = heldout_corpus_name(ADAPTATION_LENGTH)


def replay_mix_name(corpus: str, replay_pct: int) -> str:
    return f"{corpus}_replay{replay_pct}.bin"


def freezes_routers(experiment: str) -> bool:
    return split_experiment_name(experiment)[0] in FROZEN_ROUTER_FAMILIES


@dc.dataclass(frozen=True)
class AdaptationRun:
    experiment: str
    corpus: str
    replay_pct: int = 0

    def __post_init__(self) -> None:
        split_experiment_name(self.experiment)
        if self.corpus not in CORPORA:
            raise ValueError(f"corpus must be one of {tuple(CORPORA)}, got {self.corpus!r}")
        if not 0 <= self.replay_pct < 100:
            raise ValueError(f"replay_pct must be in [0, 100), got {self.replay_pct}")

    extension = property(lambda self: ExtensionRun(self.experiment, ADAPTATION_LENGTH, "equal_tokens"))
    freeze_routers = property(lambda self: freezes_routers(self.experiment))

    @property
    def run_suffix(self) -> str:
        base = f"adapt_{self.corpus}"
        return f"{base}_replay{self.replay_pct}" if self.replay_pct else base

    def training_corpus(self, data_dir: Path) -> Path:
        return data_dir / (replay_mix_name(self.corpus, self.replay_pct) if self.replay_pct else CORPORA[self.corpus].train_bin)

    def target_test(self, data_dir: Path) -> Path:
        return data_dir / CORPORA[self.corpus].test_bin

    def forgetting_heldout(self, data_dir: Path) -> Path:
        return data_dir / FORGETTING_HELDOUT

    def env(self, *, data_dir: Path, init_checkpoint: Path | None, output_root: Path = Path("outputs")) -> dict[str, str]:
        env = self.extension.env(data_dir=data_dir, init_checkpoint=None, output_root=output_root)
        env.update({
            "DCLM_DATA_PATH": str(self.training_corpus(data_dir)),
            "DCLM_RUN_SUFFIX": self.run_suffix,
            "NESTOR_OUTPUT_ROOT": str(output_root / "continual" / f"{self.experiment}_{self.run_suffix}"),
            "CONTINUAL_TARGET_TEST": str(self.target_test(data_dir)),
            "CONTINUAL_TARGET_EVAL_MODE": CORPORA[self.corpus].eval_mode,
        })
        if self.freeze_routers:
            env["NESTOR_FREEZE_ROUTERS"] = "1"
        if init_checkpoint is not None:
            env["DCLM_INIT_CHECKPOINT"] = str(resolve_checkpoint(init_checkpoint))
        return env

    def describe(self) -> str:
        who = "frozen routers" if self.freeze_routers else "all parameters"
        e = self.extension
        return (f"{self.experiment} on {CORPORA[self.corpus].title}, {self.replay_pct} % replay, {who}: {ADAPTATION_STEPS} steps x "
                f"{e.seqs_per_step} x {ADAPTATION_LENGTH} tokens, lr_muon={e.lr_muon:.6g} lr_adamw={e.lr_adamw:.6g} rope={e.rope_base}")


def extension_paper_runs() -> list[ExtensionRun]:
    runs = []
    for scale in ("100m", "200m", "500m", "1b"):
        for seq_len in LENGTHS:
            for family in ("dense", "moe", "nestor"):
                runs.append(ExtensionRun(f"{family}_{scale}", seq_len))
            for setting in SETTINGS[1:]:
                runs.append(ExtensionRun(f"nestor_{scale}", seq_len, setting, "dense" if scale == "200m" else "moe"))
    return runs


def adaptation_paper_runs() -> list[AdaptationRun]:
    return [AdaptationRun(e, c, r) for e in PAPER_EXPERIMENTS for c in CORPORA for r in PAPER_REPLAY_PCTS]


def format_env(env: dict[str, str]) -> str:
    return "\n".join(f"export {k}={shlex.quote(v)}" for k, v in env.items())


def main(argv: list[str] | None = None) -> None:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = p.add_subparsers(dest="kind", required=True)
    e = sub.add_parser("extension")
    e.add_argument("--experiment", required=True); e.add_argument("--seq-len", type=int, required=True)
    e.add_argument("--setting", default="equal_tokens", choices=SETTINGS); e.add_argument("--reference", default=REFERENCE_FAMILY)
    a = sub.add_parser("adaptation")
    a.add_argument("--experiment", required=True); a.add_argument("--corpus", required=True, choices=tuple(CORPORA))
    a.add_argument("--replay-pct", type=int, default=0)
    for s in (e, a):
        s.add_argument("--data-dir", type=Path, default=Path("data")); s.add_argument("--init-checkpoint", type=Path, default=None)
        s.add_argument("--output-root", type=Path, default=Path("outputs"))
    args = p.parse_args(argv)
    run = (ExtensionRun(args.experiment, args.seq_len, args.setting, args.reference) if args.kind == "extension"
           else AdaptationRun(args.experiment, args.corpus, args.replay_pct))
    print(f"# {run.describe()}")
    print(format_env(run.env(data_dir=args.data_dir, init_checkpoint=args.init_checkpoint, output_root=args.output_root)))


if __name__ == "__main__":
    main()
