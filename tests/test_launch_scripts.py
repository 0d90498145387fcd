"""The shell launchers parse, and the memory recipe picks the documented rung for each scale and length."""

import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SCRIPTS = sorted((ROOT / "launch").glob("*.sh"))


@pytest.mark.parametrize("script", SCRIPTS, ids=lambda p: p.name)
def test_launcher_parses(script):
    assert subprocess.run(["bash", "-n", str(script)], capture_output=True).returncode == 0


@pytest.mark.parametrize("experiment,length,want", [
    ("nestor_200m", 4096, (0, 0, 0)),
    ("nestor_200m", 32768, (1, 0, 0)),
    ("nestor_500m", 8192, (0, 0, 0)),
    ("nestor_500m", 16384, (1, 0, 0)),
    ("nestor_500m", 65536, (1, 1, 0)),
    ("nestor_1b", 4096, (1, 0, 0)),
    ("nestor_1b", 16384, (1, 1, 0)),
    ("nestor_1b", 32768, (1, 1, 4)),
    ("dense_100m", 65536, (1, 0, 0)),
])
def test_memory_recipe_rungs(experiment, length, want):
    """``memory_recipe.sh <experiment> <length>`` exports the recompute flags of that rung; a preset flag wins."""

    env = {k: v for k, v in os.environ.items() if not k.startswith("NESTOR_")}
    probe = ('source launch/memory_recipe.sh "$1" "$2" >/dev/null; '
             'echo "$NESTOR_ACTIVATION_CHECKPOINT $NESTOR_ACTIVATION_CHECKPOINT_SPLIT $NESTOR_EXPERT_HALF_CHUNKS $NESTOR_FUSED_HEAD_CE"')
    out = subprocess.run(["bash", "-c", probe, "probe", experiment, str(length)], cwd=ROOT, env=env,
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    ckpt, split, chunks, fused = (int(v) for v in out.stdout.split())
    assert (ckpt, split, chunks) == want and fused == 1
    env["NESTOR_ACTIVATION_CHECKPOINT"] = "0"
    out = subprocess.run(["bash", "-c", probe, "probe", experiment, str(length)], cwd=ROOT, env=env,
                         capture_output=True, text=True)
    assert out.stdout.split()[0] == "0"


def test_every_flag_the_launchers_export_is_known_to_the_package():
    """A flag exported by ``launch/*.sh`` is either read somewhere in the package or listed in the catalogue of
    reference flags that have no effect here: no launcher line can silently go stale."""

    import re
    from nestor_b200.utils.flags import DIFFERENT, NO_EFFECT
    read = set()
    for f in (ROOT / "nestor_b200").rglob("*.py"):
        read |= set(re.findall(r'"((?:NESTOR|DCLM|WANDB|CONTINUAL)_[A-Z0-9_]+)"', f.read_text()))
    read |= set(re.findall(r'"((?:NESTOR|DCLM)_[A-Z0-9_]+)"', (ROOT / "bench.py").read_text()))
    known = read | set(NO_EFFECT) | {name for name, _, _ in DIFFERENT}
    exported = set()
    for script in SCRIPTS:
        exported |= set(re.findall(r"^\s*export\s+((?:NESTOR|DCLM)_[A-Z0-9_]+)=", script.read_text(), flags=re.M))
    assert exported, "the launchers export their flags with `export NAME=...`"
    unknown = sorted(exported - known)
    assert not unknown, unknown
