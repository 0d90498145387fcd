"""Trainer details: fused head + cross-entropy against materialised logits, the weight average (EMA) and its
checkpoint entry, explicit positions against the default, private routers batched against one-by-one."""

import dataclasses as dc

import pytest
import torch

from nestor_b200.models import Model
from nestor_b200.ops import reference as R


def _tokens(seed, shape=(2, 64)):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 100_263, shape, generator=g)


def test_fused_head_loss_equals_the_loss_on_materialised_logits(tiny_scale):
    """``fused_head``: the model hands the loss the normalised hidden state and the head weight, and the chunked
    head + cross-entropy op never holds ``[B*S, V]`` logits; loss and every gradient equal the plain path's."""

    from nestor_b200.train.losses import CausalLMLoss
    cfg = tiny_scale.build_experiment("moe", "tiny").jobs[0].model
    torch.manual_seed(0)
    m = Model.from_config(cfg).eval()
    ids = _tokens(1)
    grads = {}
    for fused in (False, True):
        m.zero_grad(set_to_none=True)
        m.fused_head = fused
        out = m(ids)
        loss = CausalLMLoss()(out.pred, ids, out.aux).total
        loss.backward()
        grads[fused] = (float(loss), {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None})
    assert abs(grads[True][0] - grads[False][0]) < 1e-5
    assert set(grads[True][1]) == set(grads[False][1])
    for n, g in grads[False][1].items():
        assert torch.allclose(grads[True][1][n], g, atol=1e-6, rtol=1e-4), n


def test_explicit_positions_equal_the_default(tiny_scale):
    """Token tensors come with no mask and implicit positions ``0..S-1`` (the trivial-mask contract of the text
    adapter, reference nestor/adapters/text.py:167-170); passing those positions explicitly changes nothing, shifted
    positions do (RoPE)."""

    cfg = tiny_scale.build_experiment("nestor", "tiny").jobs[0].model
    torch.manual_seed(0)
    m = Model.from_config(cfg).eval()
    ids = _tokens(2, (2, 32))
    pos = torch.arange(32).unsqueeze(0).expand(2, -1)
    with torch.no_grad():
        a, b, c = m(ids).pred, m(ids, pos=pos).pred, m(ids, pos=pos + 5).pred
    assert torch.equal(a, b)
    assert not torch.allclose(a, c)


@pytest.mark.parametrize("gate_mode", ["renorm", "switch"])
def test_private_routers_batched_equal_one_router_at_a_time(gate_mode):
    """``route_selected`` routes every (token, selected column) pair through that column's private router in one
    batched call; the result is what each column's own top-k router gives for its members (reference
    nestor/backbones/batched_router.py:140-240)."""

    torch.manual_seed(0)
    T, G, Q, kc, k = 40, 5, 6, 3, 2
    scores = torch.randn(T, G, Q)
    bias = torch.randn(G, Q) * 0.3
    cols = torch.stack([torch.randperm(G)[:kc] for _ in range(T)])
    col_gates = torch.rand(T, kc)
    ids, w, idx = R.route_selected(scores, bias, cols, col_gates, k, gate_mode, torch.float32)
    assert ids.shape == (T, kc * k) and w.shape == (T, kc * k) and idx.shape == (T, kc, k)
    for g in range(G):
        members = (cols == g).nonzero()                       # (token, slot) pairs of column g
        if members.numel() == 0:
            continue
        t, slot = members[:, 0], members[:, 1]
        want_idx, want_gate = R.route_topk(scores[t, g], bias[g], k, gate_mode)
        assert torch.equal(idx[t, slot], want_idx)
        got = w.view(T, kc, k)[t, slot]
        assert torch.allclose(got, want_gate * col_gates[t, slot].unsqueeze(-1), atol=1e-6)
        assert torch.equal(ids.view(T, kc, k)[t, slot], g * Q + want_idx)


def test_weight_average_follows_the_masters_and_is_checkpointed(tmp_path, monkeypatch):
    """``ema_decay``: after every optimizer step the shadow moves ``1 - decay`` of the way to the fp32 masters; the
    checkpoint carries it by parameter name and a resumed trainer continues from it."""

    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.train.trainer import Trainer
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    torch.manual_seed(0)
    job = dc.replace(nestor_tiny().jobs[0], ema_decay=0.9)
    tr = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"), run_dir=tmp_path)
    assert tr.ema is not None and torch.equal(tr.ema["flat"], tr.arena.master)
    shadow = tr.arena.master.clone()
    for step in range(2):
        ids = _tokens(10 + step)
        loss, counts = tr.train_step((ids, ids))
        tr.update_weights(counts)
        shadow = shadow + (tr.arena.master - shadow) * (1.0 - 0.9)
        assert torch.allclose(tr.ema["flat"], shadow, atol=1e-7)
    assert not torch.equal(tr.ema["flat"], tr.arena.master)
    tr.global_step = 2
    tr.save_checkpoint()
    path = tr.checkpoint_path()
    payload = torch.load(path, weights_only=False)
    name, p = next(iter(tr.model.named_parameters()))
    slot = tr.arena.slot(p)
    assert torch.equal(payload["ema"][slot.name].reshape(-1), tr.ema["flat"][slot.offset : slot.offset + slot.numel])
    torch.manual_seed(1)
    other = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"), run_dir=tmp_path)
    other.resume(path)
    assert other.global_step == 2 and torch.equal(other.ema["flat"], tr.ema["flat"])
    assert torch.equal(other.arena.master, tr.arena.master)


_NEUTRAL_FLAGS = [
    {"NESTOR_NO_DEPTH_KEY_CACHE": "1"},                 # every read recomputes its key scales
    {"NESTOR_CE_CHUNK_ROWS": "48"},                     # smaller head + cross-entropy chunks
    {"NESTOR_FUSED_HEAD_CE": "0"},                      # materialised logits
    {"NESTOR_RUNAHEAD": "0"},                           # the host waits for every step
    {"NESTOR_LOSSFREE_GLOBAL_COUNTS": "1"},             # one rank: the global counts are the local ones
    {"NESTOR_MUON_SHARD": "1", "NESTOR_ZERO1": "1"},    # one rank owns everything
    {"NESTOR_ACTIVATION_OFFLOAD": "1"},                 # nothing to spill without a GPU
    {"NESTOR_EMA_DECAY": "0.99"},                       # the shadow never feeds back
    {"NESTOR_ACTIVATION_CHECKPOINT": "1", "NESTOR_ACTIVATION_CHECKPOINT_SPLIT": "1", "NESTOR_EXPERT_HALF_CHUNKS": "2"},
]


def _two_steps(monkeypatch, flags):
    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.train.trainer import Trainer
    for k, v in flags.items():
        monkeypatch.setenv(k, v)
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    torch.manual_seed(0)
    job = nestor_tiny().jobs[0]
    tr = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"))
    tr.model.train()
    for blk in tr.model.backbone.blocks:
        blk.freeze_routing_noise = True
    losses = []
    for step in range(2):
        ids = _tokens(20 + step)
        loss, counts = tr.train_step((ids, ids))
        tr.update_weights(counts)
        losses.append(float(loss.total))
    for k in flags:
        monkeypatch.delenv(k)
    return losses, tr.arena.master.clone()


@pytest.fixture(scope="module")
def _plain_run():
    threads = torch.get_num_threads()
    torch.set_num_threads(1)                             # one thread: CPU reductions are then repeatable to the bit
    mp = pytest.MonkeyPatch()
    try:
        yield _two_steps(mp, {})
    finally:
        mp.undo()
        torch.set_num_threads(threads)


@pytest.mark.parametrize("flags", _NEUTRAL_FLAGS, ids=lambda f: "+".join(sorted(f)))
def test_execution_flags_leave_the_training_trajectory_unchanged(flags, _plain_run, monkeypatch):
    """Flag twins: the knobs that choose HOW a step is executed (caching, chunking, recomputation, sharding of state,
    host synchronisation, offload, weight averaging) give the same losses and the same weights after two optimizer
    steps as the plain run. Bit for bit, except where the flag changes a summation order (chunked cross-entropy,
    materialised logits, recomputed halves, per-read key scales), where the weights agree to rounding."""

    want_losses, want = _plain_run
    losses, got = _two_steps(monkeypatch, flags)
    assert all(abs(a - b) < 2e-6 for a, b in zip(losses, want_losses)), (losses, want_losses)
    reordered = {"NESTOR_CE_CHUNK_ROWS", "NESTOR_FUSED_HEAD_CE", "NESTOR_ACTIVATION_CHECKPOINT",
                 "NESTOR_NO_DEPTH_KEY_CACHE"} & set(flags)          # (shared vs per-read scale nodes: another backward order)
    if reordered:
        moved = float((want - got).norm() / want.norm())
        assert moved < 1e-4, moved
    else:
        assert torch.equal(got, want), float((got - want).abs().max())


def test_evaluation_during_training_and_eval_job_submission(tmp_path, monkeypatch):
    """A train job with an eval suite scores it every ``NESTOR_EVAL_FREQ`` steps (JSON per evaluation under
    ``evals/``, training mode restored afterwards); ``eval_submit_scripts`` hands each new checkpoint to the
    scheduler, and a missing ``sbatch`` only logs a warning."""

    import json
    import subprocess
    from nestor_b200.configs import DataLoaderConfig, DclmDatasetConfig, EvalSuiteConfig, LanguageModelingEvalConfig
    from nestor_b200.data.datasets import write_synthetic_bin
    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.pipelines import TrainPipeline
    data = write_synthetic_bin(tmp_path / "train.bin", 64 * 40, 100_277, doc_len_range=(16, 64))
    held = write_synthetic_bin(tmp_path / "held.bin", 64 * 8, 100_277, seed=4, doc_len_range=(16, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    monkeypatch.setenv("DCLM_MAX_STEPS", "2")
    monkeypatch.setenv("DCLM_CKPT_FREQ", "1")
    monkeypatch.setenv("NESTOR_EVAL_FREQ", "1")
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "out"))
    exp = nestor_tiny(); exp.name = "nestor_tiny"
    suite = EvalSuiteConfig(evals=[LanguageModelingEvalConfig(
        name="held_out", dataset_config=DclmDatasetConfig(data_path=held, block_size=64),
        dataloader_config=DataLoaderConfig(batch_size=2, num_workers=0))])
    script = tmp_path / "eval_job.sh"
    script.write_text("#!/bin/bash\n")
    exp.jobs[0] = dc.replace(exp.jobs[0], eval_suite=suite, eval_submit_scripts=[(script, 1)])
    submitted = []

    real_run = subprocess.run

    def fake_run(cmd, **kw):
        if cmd[0] != "sbatch":
            return real_run(cmd, **kw)
        submitted.append(cmd)
        if len(submitted) == 2:
            raise FileNotFoundError("sbatch")                 # no scheduler on this machine: a warning, not an error
        return subprocess.CompletedProcess(cmd, 0, b"", b"")

    monkeypatch.setattr(subprocess, "run", fake_run)
    pipe = TrainPipeline.from_config(job_config=exp.jobs[0], experiment_config=exp)
    trainer = pipe.setup()
    trainer.train()
    assert trainer.model.training and trainer.global_step == 2
    files = sorted((pipe.ctx.run_dir / "evals").glob("eval_step_*.json"))
    assert [f.name for f in files] == ["eval_step_00000001.json", "eval_step_00000002.json"]
    metrics = json.loads(files[-1].read_text())["held_out"]
    assert 5.0 < metrics["cross_entropy"] < 13.0 and metrics["tokens"] > 0
    assert len(submitted) == 2 and submitted[0][0] == "sbatch" and submitted[0][1] == str(script)
    assert submitted[0][2].endswith("model_00000001.pt") and submitted[1][2].endswith("model_00000002.pt")
    pipe.ctx.close()


def test_throughput_and_utilisation_metrics(monkeypatch):
    """The step metrics follow from tokens per step, FLOPs per token, the step time and the peak: tokens/s is the
    whole job's, TFLOP/s and the utilisation are per GPU, the running average excludes the first (warm-up) step when a
    steady-state clock exists; ``NESTOR_MFU_FLOPS_PER_STEP`` pins the FLOPs of one rank's micro-batch."""

    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.train.trainer import Trainer
    from nestor_b200.train import trainer as T
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    job = dc.replace(nestor_tiny().jobs[0], grad_accum_steps=4)
    tr = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"))
    tr.tokens_per_micro = 2 * 64
    tr.world = 8                                                 # as if eight ranks ran this step
    m: dict = {}
    flops_tok, peak, dt = 3.0e6, 2.0e12, 0.5
    t0 = T.PROCESS_START                                         # the process clock the run average is measured on
    tr._add_mfu(m, flops_tok, peak, dt, now=t0 + 110.0, steps=5, t_steady=t0 + 100.0)
    tokens_step = 128 * 4 * 8
    assert m["tokens_per_sec"] == tokens_step / dt and m["samples_per_sec"] == m["tokens_per_sec"] / 2
    per_gpu = flops_tok * tokens_step / 8
    assert m["tflops_per_gpu"] == pytest.approx(per_gpu / dt / 1e12) and m["mfu_instant"] == pytest.approx(per_gpu / dt / peak)
    assert m["mfu_runavg_excl_init"] == pytest.approx(per_gpu * 4 / 10.0 / peak)          # four steps in ten seconds
    assert m["mfu_runavg_incl_init"] == pytest.approx(per_gpu * 5 / 110.0 / peak) and "mem_peak_alloc_gib" not in m
    first: dict = {}
    tr._add_mfu(first, flops_tok, peak, dt, now=t0 + 100.0, steps=1, t_steady=t0 + 100.0)
    assert "mfu_runavg_excl_init" not in first                   # nothing but the warm-up step so far
    tr.tokens_per_micro = 0
    empty: dict = {}
    tr._add_mfu(empty, flops_tok, peak, dt, now=1.0, steps=1, t_steady=None)
    assert empty == {}
