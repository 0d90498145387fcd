"""The run directory and its sidecars: config.json, git revision, source snapshot, and the experiment tracker's run id
that a resumed run continues (against a stand-in for the tracker package)."""

import dataclasses as dc
import json
import sys
import types
import zipfile


from nestor_b200.pipelines import RunContext


class _Run:
    def __init__(self, run_id):
        self.id, self.logged, self.finished = run_id, [], False

    def log(self, payload, step):
        self.logged.append((step, payload))

    def finish(self):
        self.finished = True


def _job(tmp_path, monkeypatch, project="proj"):
    from nestor_b200.experiments.tiny import nestor_tiny
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "out"))
    exp = nestor_tiny()
    exp.jobs[0] = dc.replace(exp.jobs[0], wandb_project=project, wandb_run_name="tiny", wandb_tags=["a", "b"])
    return exp, exp.jobs[0]


def test_run_directory_sidecars(tmp_path, monkeypatch):
    exp, job = _job(tmp_path, monkeypatch)
    ctx = RunContext(job, exp)
    assert ctx.run_dir.parent == tmp_path / "out" / "nestor_tiny" and ctx.run_dir.name.endswith("__nestor_tiny_train")
    cfg = json.loads((ctx.run_dir / "config.json").read_text())
    assert cfg["job"]["max_steps"] == job.max_steps
    assert cfg["job"]["model"]["backbone_config"]["block_residual_mode"] == "attn_res_column"
    with zipfile.ZipFile(ctx.run_dir / "source_snapshot.zip") as z:
        names = z.namelist()
    assert any(n.endswith("nestor_b200/models/nestor.py") for n in names)
    # nothing from the scratch folders the repository ignores, and no built artefacts
    from pathlib import Path
    ignore = (Path(__file__).resolve().parent.parent / ".gitignore").read_text().splitlines()
    scratch = [line.strip().strip("/") for line in ignore if line.strip().endswith("/") and not line.startswith("#")]
    assert scratch and not any(f"{d}/" in n for d in scratch for n in names if d not in ("build",))
    assert not any(n.endswith(".so") for n in names)
    ctx.close()


def test_tracker_run_id_is_stored_and_continued(tmp_path, monkeypatch):
    exp, job = _job(tmp_path, monkeypatch)
    calls = []

    def init(**kw):
        calls.append(kw)
        return _Run(kw.get("id") or "fresh123")

    monkeypatch.setitem(sys.modules, "wandb", types.SimpleNamespace(init=init))
    monkeypatch.setenv("WANDB_MODE", "online")
    first = RunContext(job, exp)
    first.init_wandb()
    assert calls[-1]["project"] == "proj" and calls[-1]["id"] is None and calls[-1]["resume"] is None
    assert calls[-1]["tags"] == ["a", "b"] and calls[-1]["config"]["max_steps"] == job.max_steps
    assert (first.run_dir / "wandb_run_id.txt").read_text().strip() == "fresh123"
    ckpt = first.run_dir / "checkpoints" / "model_00000002.pt"
    ckpt.parent.mkdir()
    ckpt.touch()
    run = first.wandb_run
    first.close()
    assert run.finished

    second = RunContext(job, exp)
    second.init_wandb(resume_from=ckpt)                      # the id beside the resumed run is continued
    assert calls[-1]["id"] == "fresh123" and calls[-1]["resume"] == "allow"
    second.close()

    # the tracker never stops a run: a failing init is logged and training goes on without it
    def broken(**kw):
        raise RuntimeError("no network")

    monkeypatch.setitem(sys.modules, "wandb", types.SimpleNamespace(init=broken))
    third = RunContext(job, exp)
    third.init_wandb()
    assert third.wandb_run is None
    third.close()
    # disabled by mode or by configuration: the package is not even consulted
    monkeypatch.setenv("WANDB_MODE", "disabled")
    n = len(calls)
    monkeypatch.setitem(sys.modules, "wandb", types.SimpleNamespace(init=init))
    fourth = RunContext(job, exp)
    fourth.init_wandb()
    fifth = RunContext(dc.replace(job, wandb_project=None), exp)
    monkeypatch.setenv("WANDB_MODE", "online")
    fifth.init_wandb()
    assert len(calls) == n
