"""Data pipeline, derived corpora, evaluation helpers and continued-training protocols."""

import json

import numpy as np
import pytest
import torch
from torch.utils.data.distributed import DistributedSampler

from nestor_b200.configs import DataLoaderConfig, DclmDatasetConfig
from nestor_b200.continual import protocols as C
from nestor_b200.data.corpora import build_replay_mix, build_seen_subset_bin, multiset_extra_indices, seen_window_indices
from nestor_b200.data.datasets import DclmTokenDataset, PinnedWindowLoader, epoch_permutation, write_synthetic_bin
from nestor_b200.data.documents import document_spans, load_document, select_documents
from nestor_b200.eval.long_context import PerPositionLoss, binned_mean, moving_average, sequence_nll, token_nll
from nestor_b200.eval.metrics import load_balance, routing_metrics


def test_dataset_windows_and_remap(tmp_path):
    tok = np.arange(100, dtype=np.uint32); tok[7] = 100257
    p = tmp_path / "t.bin"; tok.tofile(p)
    (tmp_path / "t.bin.meta.json").write_text(json.dumps({"token_dtype": "uint32", "num_tokens": 100}))
    ds = DclmTokenDataset(DclmDatasetConfig(data_path=p, block_size=16, token_remap={100257: 100261}))
    assert len(ds) == 6
    a, b = ds[0]
    assert a.dtype == torch.int64 and a[7] == 100261 and torch.equal(a, b) and ds[2][0][0] == 32
    (tmp_path / "t.bin.meta.json").write_text(json.dumps({"num_tokens": 99}))
    with pytest.raises(ValueError):
        DclmTokenDataset(DclmDatasetConfig(data_path=p, block_size=16))


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_loader_order_is_the_distributed_sampler_order(tmp_path, world):
    p = write_synthetic_bin(tmp_path / "s.bin", 8 * 53, 1000)
    ds = DclmTokenDataset(DclmDatasetConfig(data_path=p, block_size=8))
    for rank in range(world):
        sampler = DistributedSampler(ds, num_replicas=world, rank=rank, shuffle=True, seed=0, drop_last=True)
        sampler.set_epoch(0)
        mine = epoch_permutation(len(ds), 0, 0, world, rank, True, True)
        assert list(sampler) == mine.tolist()
    loader = PinnedWindowLoader(ds, DataLoaderConfig(batch_size=2 * world), rank=0, world=world, seed=0, pin=False)
    rows = [b[0].clone() for b in loader]
    order = epoch_permutation(len(ds), 0, 0, world, 0, True, True)
    assert len(rows) == len(loader) == (len(ds) // world) // 2
    assert torch.equal(rows[1][0], ds[int(order[2])][0])


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_seen_subset_is_the_union_over_ranks(world):
    n, steps, seqs = 1000, 7, 16
    seen = set(seen_window_indices(n, steps, seqs).tolist())
    per_rank = steps * seqs // world
    union = set()
    for r in range(world):
        union |= set(epoch_permutation(n, 0, 0, world, r, True, True)[:per_rank].tolist())
    assert union == seen and len(seen) == steps * seqs
    with pytest.raises(ValueError):
        seen_window_indices(10, 2, 8)
    extra = multiset_extra_indices(np.array(sorted(seen)), 20)
    assert len(extra) == 20 and set(extra.tolist()) <= seen and len(set(extra.tolist())) == 20


def test_documents_and_corpora(tmp_path):
    eot = 100257
    tok = np.array([1, 2, eot, 3, eot, eot, 4, 5, 6, eot, 7], dtype=np.uint32)
    spans = document_spans(tok, eot, chunk_tokens=4)
    assert spans.tolist() == [[0, 2], [3, 4], [5, 5], [6, 9]]
    assert select_documents(spans, min_tokens=2).tolist() == [[0, 2], [6, 9]]
    assert load_document(tok, spans[3], max_tokens=2).tolist() == [4, 5]
    src = write_synthetic_bin(tmp_path / "src.bin", 16 * 200, 500)
    meta = build_seen_subset_bin(src, tmp_path / "seen.bin", block_size=16, cpt_tokens=16 * 8 * 5, tokens_per_step=16 * 8,
                                 multiset_steps=7)
    assert meta["steps"] == 5 and meta["unique_windows"] == 40 and meta["extra_windows"] == 16
    assert (tmp_path / "seen.bin").stat().st_size == meta["num_tokens"] * 4
    mix = build_replay_mix(src, src, tmp_path / "mix.bin", block_size=16, target_share_pct=75, mix_tokens=16 * 8 * 8,
                           tokens_per_step=16 * 8)
    assert [p["steps"] for p in mix["sources"]] == [6, 2] and mix["num_windows"] == 64


def test_protocol_budgets_and_env(tmp_path):
    assert C.EXTENSION_STEPS == 477
    eq = C.ExtensionRun("nestor_200m", 32768, "equal_flops_new", "dense")
    assert eq.steps == 570 and C.ExtensionRun("nestor_200m", 65536, "equal_flops_new", "dense").steps == 592
    assert C.ExtensionRun("nestor_200m", 32768, "equal_flops_new", "moe").steps == 571
    base = C.ExtensionRun("moe_500m", 16384)
    assert base.steps == 477 and base.warmup_steps == 47 and base.seqs_per_step == 64 and base.rope_base == 1_000_000
    with pytest.raises(ValueError):
        C.ExtensionRun("dense_200m", 8192, "equal_flops_new")
    ck = tmp_path / "run" / "checkpoints"; ck.mkdir(parents=True); (ck / "model_final.pt").write_bytes(b"x")
    env = eq.env(data_dir=tmp_path, init_checkpoint=tmp_path / "run")
    assert env["DCLM_BLOCK_SIZE"] == "32768" and env["DCLM_INIT_CHECKPOINT"].endswith("model_final.pt")
    assert float(env["DCLM_LR_MUON"]) == pytest.approx(0.0025 * eq.flop_ratio, rel=1e-5)
    ad = C.AdaptationRun("nestor_500m", "pg19", 25)
    e2 = ad.env(data_dir=tmp_path, init_checkpoint=None)
    assert e2["NESTOR_FREEZE_ROUTERS"] == "1" and e2["DCLM_DATA_PATH"].endswith("pg19_replay25.bin")
    assert "NESTOR_FREEZE_ROUTERS" not in C.AdaptationRun("dense_1b", "owm").env(data_dir=tmp_path, init_checkpoint=None)
    assert len(C.adaptation_paper_runs()) == 3 * 4 * 2


def test_per_position_loss_and_smoothing():
    acc = PerPositionLoss(8)
    acc.add(np.array([1.0, 2.0, 3.0]), start=1); acc.add(torch.tensor([3.0, 4.0]), start=1)
    assert acc.tokens == 5 and acc.cross_entropy() == pytest.approx(13 / 5)
    m = acc.mean_by_position()
    assert np.isnan(m[0]) and m[1] == 2.0 and m[3] == 3.0
    assert np.allclose(moving_average(np.array([1.0, np.nan, 3.0]), 3), [1.0, 2.0, 3.0])
    assert binned_mean(acc.sums, acc.counts, 4)[0]["tokens"] == 5
    with pytest.raises(ValueError):
        moving_average(np.zeros(3), 2)
    assert set(acc.to_dict(ma_window=3, bin_size=4)) >= {"cross_entropy", "mean_by_position", "moving_average", "bins"}


def test_routing_metrics():
    even, skew = torch.full((4,), 10.0), torch.tensor([40.0, 0, 0, 0])
    assert load_balance(even) == pytest.approx(1.0) and load_balance(skew) == pytest.approx(0.0, abs=1e-6)
    m = routing_metrics({"blocks.0.group_router": even, "blocks.0.layers.0.expert_pool.private_routers.1": skew})
    assert m["routing/blocks.0.group_router/frac/c2"] == 0.25 and m["routing/group/mean_balance"] == pytest.approx(1.0)
    assert m["routing/private/mean_max_frac"] == 1.0


def test_long_context_nll_and_frozen_routers(tiny_scale):
    from nestor_b200.models import Model
    from nestor_b200.train.frozen_routers import freeze_routers, routers_are_frozen
    torch.manual_seed(0)
    m = Model.from_config(tiny_scale.build_experiment("nestor", "tiny").jobs[0].model).eval()
    ids = torch.randint(0, 100263, (1, 48))
    nll, _ = sequence_nll(m, ids, head_chunk=7)
    part, _ = token_nll(m, ids, target_start=5, target_end=20)
    assert nll.shape == (47,) and torch.allclose(nll[4:19], part, atol=1e-5)
    logits = m(ids).pred[0, :-1]
    assert torch.allclose(nll, torch.nn.functional.cross_entropy(logits, ids[0, 1:], reduction="none"), atol=1e-4)
    assert not routers_are_frozen(m)
    assert freeze_routers(m) > 0 and routers_are_frozen(m)
    m.train()
    a = m(ids).aux["blocks"][0]["group_idx"]; b = m(ids).aux["blocks"][0]["group_idx"]
    assert torch.equal(a, b)                                        # no exploration noise once frozen


def test_source_snapshot_keeps_sources_and_prunes_the_rest(tmp_path):
    import zipfile
    from nestor_b200.utils.snapshot import snapshot_sources, source_files
    root = tmp_path / "repo"
    for rel, text in {"pkg/a.py": "x = 1", "pkg/csrc/k.cu": "__global__ void k(){}", "pkg/_C/lib.so": "bin",
                      "pkg/__pycache__/a.pyc": "", "outputs/run/model.pt": "w", "data/train.bin": "t", ".git/HEAD": "ref",
                      "README.md": "# hi", "pkg/notes.ckpt": "c", "big.txt": "y" * 64}.items():
        f = root / rel
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text(text)
    names = {p.as_posix() for p in source_files(root)}
    assert names == {"pkg/a.py", "pkg/csrc/k.cu", "README.md", "big.txt"}
    out = snapshot_sources(root, tmp_path / "run" / "source_snapshot", max_file_bytes=32)
    assert out.suffix == ".zip" and set(zipfile.ZipFile(out).namelist()) == names - {"big.txt"}


def test_pinned_window_loader_keeps_a_batch_intact_for_depth_more_draws(tmp_path):
    """A consumer that copies asynchronously may still be reading batch i while it draws later ones: the ring must not
    refill batch i's buffer before ``depth`` further batches have been drawn."""

    import time

    import torch

    from nestor_b200.configs import DataLoaderConfig, DclmDatasetConfig
    from nestor_b200.data.datasets import DclmTokenDataset, PinnedWindowLoader, write_synthetic_bin

    path = tmp_path / "tokens.bin"
    write_synthetic_bin(path, 64 * 40 + 1, 1000, seed=3)
    ds = DclmTokenDataset(DclmDatasetConfig(data_path=path, block_size=64))
    loader = PinnedWindowLoader(ds, DataLoaderConfig(batch_size=2, num_workers=0, shuffle=False), depth=3, pin=False)
    held = []
    for i, (x, _) in enumerate(loader):
        held.append((x, x.clone()))
        time.sleep(0.01)                      # let the producer thread run as far ahead as the queue allows
        for j in range(max(0, i - 3), i + 1):   # the last depth + 1 batches drawn are all still what they were
            assert torch.equal(held[j][0], held[j][1]), (i, j)
        if i >= 14:
            break
