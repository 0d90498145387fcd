"""Optimizer math, schedules, checkpoint format and the CPU training loop."""

import math
from pathlib import Path

import pytest
import torch
from torch import nn

from nestor_b200.configs import CosineAnnealingConfig, MuonAdamWConfig, PowerLawConfig, WSDConfig
from nestor_b200.data.datasets import write_synthetic_bin
from nestor_b200.models.tags import ADAMW_DECAY, ADAMW_NO_DECAY, ParamTag, muon_matrix, tag
from nestor_b200.ops import reference as R
from nestor_b200.parallel.arena import ParamArena
from nestor_b200.pipelines import TrainPipeline, find_latest_checkpoint, resolve_resume_checkpoint
from nestor_b200.train import checkpoint as ck
from nestor_b200.train.optim import MuonAdamW, build_optimizer, build_param_groups, build_scheduler


class Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = tag(nn.Parameter(torch.randn(12, 20)), muon_matrix(12, 20))
        self.bank = tag(nn.Parameter(torch.randn(3, 20, 8)), muon_matrix(8, 20))
        self.emb = tag(nn.Parameter(torch.randn(30, 20)), ADAMW_DECAY)
        self.gain = tag(nn.Parameter(torch.ones(20)), ADAMW_NO_DECAY)
        self.readout = tag(nn.Parameter(torch.randn(4, 20)), ParamTag("adamw", lr_mul=0.5 / 20))


def test_param_groups_follow_tags():
    cfg = MuonAdamWConfig(lr_muon=0.01, lr_adamw=3e-4, weight_decay=0.1)
    groups = build_param_groups(cfg, Toy())
    muon = [g for g in groups if g["method"] == "muon"]
    adam = [g for g in groups if g["method"] == "adamw"]
    assert [round(g["lr"], 8) for g in muon] == sorted(round(0.01 * math.sqrt(s), 8) for s in (8 / 20, 12 / 20))
    assert {(round(g["lr"], 10), g["weight_decay"]) for g in adam} == {
        (3e-4, 0.1), (3e-4, 0.0), (round(3e-4 * 0.025, 10), 0.1)}


def test_muon_and_adamw_steps_match_manual_math():
    torch.manual_seed(0)
    m = Toy()
    cfg = MuonAdamWConfig(lr_muon=0.02, lr_adamw=1e-3, weight_decay=0.1, betas=(0.9, 0.95))
    opt = build_optimizer(cfg, m)
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    grads = {n: torch.randn_like(p) for n, p in m.named_parameters()}
    for n, p in m.named_parameters():
        p.grad = grads[n].clone()
    opt.step()
    lr = 0.02 * math.sqrt(12 / 20)
    g = grads["a"]
    want = before["a"] * (1 - lr * 0.1) - lr * R.newton_schulz(g + 0.95 * g, 5)      # buf = g on the first step
    assert torch.allclose(m.a, want, atol=1e-5)
    lrb = 0.02 * math.sqrt(8 / 20)
    gb = grads["bank"]
    wantb = before["bank"] * (1 - lrb * 0.1) - lrb * R.newton_schulz(gb * 1.95, 5)
    assert torch.allclose(m.bank, wantb, atol=1e-5)
    ge = grads["emb"]
    m1, m2 = 0.1 * ge, 0.05 * ge * ge
    upd = (m1 / 0.1) / ((m2 / 0.05).sqrt() + 1e-8)
    assert torch.allclose(m.emb, before["emb"] * (1 - 1e-3 * 0.1) - 1e-3 * upd, atol=1e-6)
    assert torch.allclose(m.gain, before["gain"] - 1e-3 * torch.sign(grads["gain"]), atol=1e-5)   # no decay


def test_contiguous_ownership_covers_the_arena():
    m = Toy()
    arena = ParamArena(m)
    opt = MuonAdamW(build_param_groups(MuonAdamWConfig(), m), arena=arena, shard=False)
    opt.world, opt.owned = 3, [[], [], []]
    opt.owner.clear()
    opt._assign_owners()
    cuts = opt.owner_cuts
    assert cuts[0] == 0 and cuts[-1] == arena.numel and cuts == sorted(cuts) and len(cuts) == 4
    for p, o in opt.owner.items():
        off = arena.slot(p).offset
        assert cuts[o] <= off < cuts[o + 1]


def test_schedules():
    p = [nn.Parameter(torch.zeros(1))]
    opt = torch.optim.SGD(p, lr=1.0)
    s = build_scheduler(CosineAnnealingConfig(T_max=100, warmup_steps=10, eta_min=0.1), opt)
    lrs = []
    for _ in range(60):
        lrs.append(opt.param_groups[0]["lr"]); opt.step(); s.step()
    assert lrs[0] == 0.0 and abs(lrs[5] - 0.5) < 1e-9 and abs(lrs[10] - 1.0) < 1e-9 and lrs[59] < lrs[11]
    opt = torch.optim.SGD(p, lr=1.0)
    s = build_scheduler(WSDConfig(total_steps=100, warmup_steps=10, decay_steps=20, eta_min=0.1, decay_shape="linear"), opt)
    vals = []
    for _ in range(101):
        vals.append(opt.param_groups[0]["lr"]); opt.step(); s.step()
    assert vals[50] == 1.0 and abs(vals[90] - (0.1 + 0.9 * 0.5)) < 1e-9 and abs(vals[100] - 0.1) < 1e-9
    opt = torch.optim.SGD(p, lr=0.01)
    s = build_scheduler(PowerLawConfig(warmup_steps=5, base_lr=0.01), opt)
    for _ in range(10):
        opt.step(); s.step()
    assert 0 < opt.param_groups[0]["lr"] <= 0.01


def test_arena_views_and_stack(tiny_scale):
    from nestor_b200.models import Model
    m = Model.from_config(tiny_scale.build_experiment("nestor", "tiny").jobs[0].model)
    before = {k: v.clone() for k, v in m.state_dict().items()}
    arena = ParamArena(m)
    for k, v in m.state_dict().items():
        assert torch.equal(v, before[k]), k
    layer = m.backbone.blocks[0].layers[0]
    p = layer.attention_groups[0].q_proj.weight
    assert p.data_ptr() == arena.master[arena.slot(p).offset:].data_ptr()
    p.grad.fill_(2.0)
    s = arena.slot(p)
    assert float(arena.grad[s.offset:s.offset + s.numel].sum()) == 2.0 * s.numel
    arena.zero_grad()
    assert float(p.grad.abs().sum()) == 0.0
    w = layer.qkv_weight()
    assert w.shape == (8, 3 * p.shape[0], p.shape[1])
    assert torch.equal(w[3, p.shape[0]:2 * p.shape[0]], layer.attention_groups[3].k_proj.weight)


def test_checkpoint_key_conversions():
    E, d, h = 3, 4, 6
    stacked = {"x.expert_pool.stacked_public.w_up": torch.randn(E, d, h), "x.expert_pool.stacked_public.w_gate": torch.randn(E, d, h),
               "x.expert_pool.stacked_public.w_down": torch.randn(E, h, d), "x.other": torch.randn(2)}
    un = ck.unstack_expert_banks(stacked)
    assert "x.expert_pool.public_experts.1.layers.0.weight" in un and un["x.expert_pool.public_experts.1.layers.0.weight"].shape == (h, d)
    back = ck.stack_expert_banks(un, set(stacked))
    assert all(torch.equal(back[k], stacked[k]) for k in stacked)
    legacy = {"l.group_specific_experts.0.0.layers.0.weight": torch.zeros(1)}
    assert "l.shared_experts.0.layers.0.weight" in ck.remap_legacy_bank_keys(legacy, {"l.shared_experts.0.layers.0.weight"})
    cur = {"a": torch.zeros(2), "b": torch.zeros(3)}
    with pytest.raises(RuntimeError):
        ck.filter_init_state({"a": torch.zeros(2)}, cur, {"a", "b"})
    kept, skipped = ck.filter_init_state({"a": torch.zeros(2), "b": torch.zeros(4), "c": torch.zeros(1)}, cur, {"a", "b"}, allow_partial=True)
    assert set(kept) == {"a"} and skipped == {"b", "c"}


def test_resume_policy(tmp_path):
    assert resolve_resume_checkpoint(explicit=Path("e"), explicit_strict=True, latest_own=Path("l")) == (Path("e"), True, "explicit")
    assert resolve_resume_checkpoint(explicit=Path("e"), explicit_strict=False, latest_own=Path("l")) == (Path("l"), True, "auto")
    assert resolve_resume_checkpoint(explicit=Path("e"), explicit_strict=False, latest_own=None) == (Path("e"), False, "init")
    assert resolve_resume_checkpoint(explicit=None, explicit_strict=True, latest_own=None)[2] == "none"
    for run, steps in (("r1", (2, 4)), ("r2", (6,))):
        d = tmp_path / run / "checkpoints"; d.mkdir(parents=True)
        for s in steps:
            (d / f"model_{s:08d}.pt").write_bytes(b"x")
        (d / "model_final.pt").write_bytes(b"x")
    best, step = find_latest_checkpoint(tmp_path)
    assert step == 6 and best.parent.parent.name == "r2"
    assert find_latest_checkpoint(tmp_path, exclude_run_dir=tmp_path / "r2")[1] == 4


def test_cli_train_checkpoint_and_auto_resume(tmp_path, monkeypatch):
    """Tiny experiment end to end on CPU: train, checkpoint format, then a second launch resumes and fast-forwards."""

    data = write_synthetic_bin(tmp_path / "train.bin", 256 * 40, 100_277, doc_len_range=(32, 256))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "out"))
    monkeypatch.setenv("DCLM_MAX_STEPS", "2")
    monkeypatch.setenv("DCLM_CKPT_FREQ", "1")
    monkeypatch.setenv("DCLM_GRAD_ACCUM", "2")
    from nestor_b200.cli import main
    assert main(["--experiment", "nestor_tiny"]) == 0
    run_dirs = list((tmp_path / "out" / "nestor_tiny").iterdir())
    assert len(run_dirs) == 1 and (run_dirs[0] / "config.json").is_file()
    payload = torch.load(run_dirs[0] / "checkpoints" / "model_00000002.pt", weights_only=False)
    assert {"model", "step", "epoch", "git_sha", "optimizer", "scheduler"} <= set(payload)
    assert payload["step"] == 2 and all(v.dtype == torch.float32 for v in payload["model"].values() if v.is_floating_point())
    assert any("momentum_buffer" in s for s in payload["optimizer"]["state"].values())
    monkeypatch.setenv("DCLM_MAX_STEPS", "3")
    import time; time.sleep(1.1)                 # run directories are second-stamped
    from nestor_b200.experiments.tiny import nestor_tiny
    exp = nestor_tiny(); exp.name = "nestor_tiny"
    pipe = TrainPipeline.from_config(job_config=exp.jobs[0], experiment_config=exp)
    trainer = pipe.setup()
    assert trainer.global_step == 2
    model_state = {k: v for k, v in trainer.model.state_dict().items()}
    assert all(torch.allclose(model_state[k].float().cpu(), payload["model"][k]) for k in payload["model"])
    trainer.train()
    assert trainer.global_step == 3
    pipe.ctx.close()


def test_update_weights_raises_when_a_collective_reported_a_timeout(tiny_scale, tmp_path, monkeypatch):
    """A nonzero device status word (a bounded peer wait that gave up) must surface as ``PeerTimeout`` out of the
    optimizer step instead of letting training continue on unreduced gradients."""

    from nestor_b200.models import Model
    from nestor_b200.parallel.symm import PeerTimeout
    from nestor_b200.train.trainer import Trainer
    data = write_synthetic_bin(tmp_path / "train.bin", 64 * 40, 100_277, doc_len_range=(16, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    job = tiny_scale.build_experiment("nestor", "tiny").jobs[0]
    trainer = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"))
    ids = torch.randint(0, 1000, (2, 64))
    trainer.model.train()
    trainer.train_step((ids, ids))
    trainer.update_weights({})                      # no status source on a single CPU process: nothing to check
    trainer.peer_status = torch.zeros(1, dtype=torch.int32)
    trainer.train_step((ids, ids))
    trainer.update_weights({})                      # clean status: the probe is queued and passes
    trainer.check_peer_status()
    trainer.train_step((ids, ids))
    trainer.update_weights({})
    trainer.peer_status.fill_(5)                    # what a timed-out in-kernel barrier leaves behind
    trainer._probe_peer_status()
    trainer.train_step((ids, ids))
    with pytest.raises(PeerTimeout, match="status 5"):
        trainer.update_weights({})
    assert int(trainer.peer_status.item()) == 0     # cleared, so a caller that recovers can carry on


def test_drop_mup_puts_every_parameter_in_one_adamw_group(tiny_scale, monkeypatch):
    from nestor_b200.models import Model
    from nestor_b200.train.optim import build_param_groups

    job = tiny_scale.build_experiment("nestor", "tiny").jobs[0]
    m = Model.from_config(job.model)
    assert len(build_param_groups(job.optimizer, m)) > 2
    monkeypatch.setenv("NESTOR_DROP_MUP", "1")
    groups = build_param_groups(job.optimizer, m)
    assert len(groups) == 1 and groups[0]["method"] == "adamw" and groups[0]["lr"] == job.optimizer.lr_adamw
    assert sum(p.numel() for p in groups[0]["params"]) == sum(p.numel() for p in m.parameters() if p.requires_grad)


_TRAIN_VARIANTS = {
    # column-resolved sublayer reads, one block merged, per-source head queries, mass-conserving gains
    "wide_reads": dict(block_column_head_only=False, block_column_blocks=[0], block_column_gain_init=1.0,
                       block_column_mass_lambda=0.5, block_column_head_query_per_source=True),
    # banks of pointwise experts whose size changes with depth, single-column blocks, merged depth reads
    "pointwise_banks": dict(
        block_residual_mode="attn_res_kimi", block_column_include_aggregate=False, block_column_gain_init=1.0,
        block_column_head_only=False, block_column_deviation_sources=False, num_groups=[1, 1],
        num_groups_per_token=[1, 1], block_num_layers=[2, 1], block_layer_num_experts=[[3, 5], [4]],
        router_num_shared_experts=[2, 4], router_num_experts_per_group_per_token=[2, 2],
        block_mlp_activations="gelu", block_mlp_hidden_dims=[[96]] * 2, router_num_dense_shared_experts=1,
        block_expert_pool_public_experts=[0, 0], block_expert_pool_private_experts=[0, 0]),
}


@pytest.mark.parametrize("variant", list(_TRAIN_VARIANTS))
def test_configuration_variants_train_and_checkpoint(variant, tmp_path, monkeypatch):
    """Models outside the registered cells go through the whole pipeline on CPU: parameter arena, Muon + AdamW
    groups, three optimizer steps with finite weights, balancing-bias updates, a checkpoint that holds the final state."""

    import dataclasses as dc
    data = write_synthetic_bin(tmp_path / "train.bin", 64 * 40, 100_277, doc_len_range=(16, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "out"))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    monkeypatch.setenv("DCLM_MAX_STEPS", "3")
    monkeypatch.setenv("DCLM_CKPT_FREQ", "3")
    from nestor_b200.experiments.tiny import nestor_tiny
    exp = nestor_tiny(); exp.name = f"nestor_tiny_{variant}"
    job = exp.jobs[0]
    job = dc.replace(job, model=dc.replace(job.model, backbone_config=dc.replace(
        job.model.backbone_config, **_TRAIN_VARIANTS[variant])))
    exp.jobs[0] = job
    pipe = TrainPipeline.from_config(job_config=job, experiment_config=exp)
    trainer = pipe.setup()
    trainer.train()
    assert trainer.global_step == 3
    state = {k: v.detach().float().cpu().clone() for k, v in trainer.model.state_dict().items()}
    assert all(torch.isfinite(v).all() for v in state.values() if v.is_floating_point())
    pipe.ctx.close()
    (ckpt,) = list((tmp_path / "out").glob("*/*/checkpoints/model_00000003.pt"))
    payload = torch.load(ckpt, weights_only=False)
    assert payload["step"] == 3 and set(payload["model"]) == set(state)
    assert all(torch.allclose(payload["model"][k].float(), state[k]) for k in state if state[k].is_floating_point())


@pytest.mark.parametrize("family", ["nestor", "moe"])
def test_bf16_compute_copy_routes_gradients_into_the_fp32_arena(family, tiny_scale):
    """The bf16 compute copy on CPU: strided stack / fused / concatenated views of the copy feed the ops, and their
    gradients come back through the views into the fp32 gradient arena. With masters that are exactly representable
    in bf16 this is the same computation as an fp32 arena whose ops round the weights per use, so loss and gradients
    agree to the last bits; the copy follows the masters on ``refresh_compute``."""

    from nestor_b200.models import Model
    from nestor_b200.train.losses import CausalLMLoss
    cfg = tiny_scale.build_experiment(family, "tiny").jobs[0].model
    ids = torch.randint(0, 100263, (2, 48))
    results = {}
    for mode in ("copy", "per_use"):
        torch.manual_seed(0)
        m = Model.from_config(cfg).eval()
        with torch.no_grad():
            for n, p in m.named_parameters():
                if "query" in n:
                    p.normal_(0, 0.3)
                p.copy_(p.to(torch.bfloat16).float())                 # masters on the bf16 grid
        m.compute_dtype, m.fused_head = torch.bfloat16, False
        arena = ParamArena(m, compute_dtype=torch.bfloat16 if mode == "copy" else torch.float32)
        if mode == "copy":
            assert arena.compute is not arena.master and arena.compute.dtype == torch.bfloat16
            assert torch.equal(arena.compute.float(), arena.master)
            layer = m.backbone.blocks[0].layers[0]
            w = layer.qkv_weight()                                    # a strided view of the copy, not a new tensor
            first = arena.slot(layer.attention_groups[0].q_proj.weight)
            assert w.dtype == torch.bfloat16 and w._nb_grad.dtype == torch.float32
            assert w.untyped_storage().data_ptr() == arena.compute.untyped_storage().data_ptr()
            assert w.storage_offset() == first.offset
        out = m(ids)
        loss = CausalLMLoss()(out.pred, ids, out.aux).total
        loss.backward()
        results[mode] = (float(loss), arena.grad.clone(), arena)
    (la, ga, arena), (lb, gb, _) = results["copy"], results["per_use"]
    assert abs(la - lb) < 1e-6
    assert float(ga.norm()) > 0 and float((ga - gb).norm() / gb.norm()) < 1e-5
    arena.master.mul_(0.5)
    arena.refresh_compute()
    assert torch.equal(arena.compute.float(), arena.master.to(torch.bfloat16).float())
    assert sum(n for _, n in arena.buckets(1000)) == arena.numel and max(n for _, n in arena.buckets(1000)) <= 1000
