"""The command-line tools end to end on small files: text -> token file, corpus builders, held-out and long-context
evaluation of a checkpoint, and the frozen-router verifier across a router-frozen continuation."""

import gzip
import json
import time

import pytest
import torch

from nestor_b200.data.datasets import write_synthetic_bin
from nestor_b200.data.documents import document_spans, open_token_bin, read_bin_meta


def test_text_to_token_file_offline(tmp_path, capsys):
    """``preprocess_text_bin --tokenizer bytes``: jsonl, gzipped jsonl and plain text in one call; every kept document
    is followed by the end-of-text id, short documents are dropped, long ones cut, and the sidecar describes the file."""

    from nestor_b200.scripts import preprocess_text_bin
    docs = ["alpha beta gamma", "x", "delta " * 20, "épsilon ζ"]
    (tmp_path / "in").mkdir()
    (tmp_path / "in" / "a.jsonl").write_text("\n".join(json.dumps({"text": d}) for d in docs[:2]) + "\n")
    with gzip.open(tmp_path / "in" / "b.jsonl.gz", "wt", encoding="utf-8") as f:
        f.write(json.dumps({"text": docs[2]}) + "\n")
    (tmp_path / "in" / "c.txt").write_text(docs[3], encoding="utf-8")
    out = tmp_path / "tokens.bin"
    preprocess_text_bin.main([str(tmp_path / "in"), "--output", str(out), "--tokenizer", "bytes", "--workers", "2",
                              "--min-doc-tokens", "2", "--max-doc-tokens", "40", "--batch-docs", "2"])
    assert "3 documents" in capsys.readouterr().out
    tokens, eot = open_token_bin(out)
    meta = read_bin_meta(out)
    assert eot == 256 and meta["tokenizer"] == "bytes" and meta["num_docs"] == 3
    assert meta["num_tokens"] == len(tokens)
    spans = document_spans(tokens, eot)
    texts = [bytes(int(t) for t in tokens[a:b]).decode("utf-8") for a, b in spans]
    assert texts == [docs[0], (docs[2])[:40], docs[3]]                   # the one-byte document is gone, the long one is cut
    assert all(int(tokens[b]) == 256 for _, b in spans)


def test_corpus_builders_from_the_command_line(tmp_path, capsys):
    from nestor_b200.scripts import build_corpora
    src = write_synthetic_bin(tmp_path / "src.bin", 64 * 200, 50_000, doc_len_range=(16, 64))
    build_corpora.main(["seen-subset", "--source", str(src), "--output", str(tmp_path / "seen.bin"), "--block-size", "64",
                        "--cpt-tokens", str(64 * 40), "--tokens-per-step", str(64 * 4)])
    meta = json.loads(capsys.readouterr().out)
    seen, _ = open_token_bin(tmp_path / "seen.bin")
    assert len(seen) == meta["num_tokens"] == 64 * 40 and len(seen) % 64 == 0
    target = write_synthetic_bin(tmp_path / "target.bin", 64 * 100, 50_000, seed=3, doc_len_range=(16, 64))
    build_corpora.main(["replay-mix", "--target", str(target), "--replay", str(tmp_path / "seen.bin"), "--output",
                        str(tmp_path / "mix.bin"), "--block-size", "64", "--target-share-pct", "75",
                        "--mix-tokens", str(64 * 32), "--tokens-per-step", str(64 * 4)])
    mix_meta = json.loads(capsys.readouterr().out)
    mix, _ = open_token_bin(tmp_path / "mix.bin")
    assert len(mix) == mix_meta["num_tokens"] == 64 * 32


def _train(tmp_path, monkeypatch, root, steps):
    from nestor_b200.cli import main
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / root))
    monkeypatch.setenv("DCLM_MAX_STEPS", str(steps))
    assert main(["--experiment", "nestor_tiny"]) == 0
    return sorted((tmp_path / root / "nestor_tiny").glob("*/checkpoints/model_final.pt"))[-1]


def test_evaluation_tools_and_the_frozen_router_check(tmp_path, monkeypatch, capsys):
    """Train two steps; score the checkpoint with the held-out and the long-context tools; continue from it with the
    routers frozen (``NESTOR_FREEZE_ROUTERS=1``) and without, and let the verifier tell the two apart."""

    from nestor_b200.scripts import check_frozen_routers, eval_heldout, eval_long_context
    data = write_synthetic_bin(tmp_path / "train.bin", 64 * 60, 100_277, doc_len_range=(16, 64))
    held = write_synthetic_bin(tmp_path / "held.bin", 64 * 16, 100_277, seed=9, doc_len_range=(48, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    monkeypatch.setenv("DCLM_CKPT_FREQ", "100")
    base = _train(tmp_path, monkeypatch, "base", 2)
    capsys.readouterr()

    eval_heldout.main(["--experiment", "nestor_tiny", "--checkpoint", str(base), "--data", str(held), "--block-size", "64",
                       "--batch", "2", "--max-windows", "6", "--output", str(tmp_path / "heldout.json")])
    res = json.loads((tmp_path / "heldout.json").read_text())
    assert res["windows"] == 6 and res["tokens"] == 6 * 63 and 5.0 < res["cross_entropy"] < 13.0
    assert json.loads(capsys.readouterr().out)["cross_entropy"] == res["cross_entropy"]

    eval_long_context.main(["--experiment", "nestor_tiny", "--checkpoint", str(base), "--data", str(held), "--seq-len", "48",
                            "--documents", "4", "--head-chunk", "16", "--output", str(tmp_path / "long.json")])
    long = json.loads((tmp_path / "long.json").read_text())
    assert long and 5.0 < float(long.get("cross_entropy", long.get("mean_nll", 0.0)) or 0.0) < 13.0

    # continue from the checkpoint, once with frozen routers and once without
    monkeypatch.setenv("DCLM_INIT_CHECKPOINT", str(base))
    monkeypatch.setenv("NESTOR_FREEZE_ROUTERS", "1")
    time.sleep(1.1)
    frozen = _train(tmp_path, monkeypatch, "frozen", 2)
    monkeypatch.delenv("NESTOR_FREEZE_ROUTERS")
    time.sleep(1.1)
    free = _train(tmp_path, monkeypatch, "free", 2)
    capsys.readouterr()
    assert check_frozen_routers.main([str(base), str(frozen)]) == 0
    assert ", 0 changed" in capsys.readouterr().out
    assert check_frozen_routers.main([str(base), str(free)]) == 1
    assert "changed:" in capsys.readouterr().out
    # the frozen continuation did train everything else
    a = torch.load(base, weights_only=False)["model"]
    b = torch.load(frozen, weights_only=False)["model"]
    assert any(not torch.equal(a[k], b[k]) for k in a if "attention_groups" in k)


def test_dclm_shard_tree_to_token_file(tmp_path, capsys):
    """``preprocess_dclm`` walks ``global-shard_*/local-shard_*/shard_*.jsonl.zst`` in sorted order, reads only the
    chosen global shards and stops at the token target; zstd streams are read with the ``zstandard`` package or, when
    that is missing, through Arrow's codec."""

    pa = pytest.importorskip("pyarrow")
    from nestor_b200.scripts import preprocess_dclm
    root = tmp_path / "dclm"
    texts = {}
    for g in (1, 2):
        for l in (0, 1):
            d = root / f"global-shard_{g:02d}_of_10" / f"local-shard_{l}_of_10"
            d.mkdir(parents=True)
            body = "".join(json.dumps({"text": f"g{g} l{l} doc{i} " + "w" * 10}) + "\n" for i in range(3))
            texts[(g, l)] = body
            with pa.CompressedOutputStream(pa.OSFile(str(d / "shard_00000000_processed.jsonl.zst"), "wb"), "zstd") as f:
                f.write(body.encode("utf-8"))
    out = tmp_path / "dclm.bin"
    preprocess_dclm.main(["--dclm-root", str(root), "--out", str(out), "--global-shards", "2", "--tokenizer", "bytes",
                          "--workers", "1"])
    tokens, eot = open_token_bin(out)
    spans = document_spans(tokens, eot)
    docs = [bytes(int(t) for t in tokens[a:b]).decode() for a, b in spans]
    assert len(docs) == 6 and all(d.startswith("g2 ") for d in docs)          # only global shard 2, both local shards
    assert docs[0].startswith("g2 l0 doc0") and docs[3].startswith("g2 l1 doc0")
    capsys.readouterr()
    preprocess_dclm.main(["--dclm-root", str(root), "--out", str(out), "--tokenizer", "bytes", "--workers", "1",
                          "--target-tokens", "30"])
    assert read_bin_meta(out)["num_tokens"] >= 30                              # (checked once per batch of documents)
    with pytest.raises(SystemExit):
        preprocess_dclm.main(["--dclm-root", str(tmp_path / "nothing"), "--out", str(out)])


def test_describe_an_experiment_without_running_it(capsys, monkeypatch):
    """``scripts.describe`` builds the model on the meta device and reports geometry, parameter counts by optimizer,
    tokens per step, FLOPs per token and the per-GPU footprint; the numbers are those of the registry tests."""

    from nestor_b200.scripts import describe
    monkeypatch.delenv("DCLM_BLOCK_SIZE", raising=False)
    info = describe.describe("nestor_200m", world=8)
    assert info["parameters"]["total"] == 761_788_781 and info["tokens_per_step"] == 524_288
    assert sum(info["parameters"]["by_optimizer"].values()) == info["parameters"]["trainable"]
    assert [b["columns_per_token"] for b in info["blocks"]] == [3, 4, 5, 6, 6, 7, 8]
    assert [b["exports"] for b in info["blocks"]] == [4, 5, 6, 7, 7, 8, 9]
    assert info["flops_per_token"]["training"] == 3 * info["flops_per_token"]["forward"]
    assert abs(info["per_gpu_gib"]["parameter_arenas"] - 761_788_781 * 10 / 2**30) < 0.01
    one = describe.describe("nestor_200m", world=1)["per_gpu_gib"]["optimizer_state"]
    assert abs(one / 8 - info["per_gpu_gib"]["optimizer_state"]) < 0.01
    assert describe.main(["--experiment", "dense_100m"]) == 0
    text = capsys.readouterr().out
    assert "dense MLP" in text and "attn_res_kimi" in text and "141,011,709" in text
    assert describe.main(["--experiment", "moe_100m", "--json"]) == 0
    out = capsys.readouterr().out
    assert json.loads(out[out.index("{"):])["blocks"][0]["experts"].startswith("bank: ")


def test_checkpoint_layout_conversion_round_trip(tmp_path, monkeypatch, capsys):
    """Stacked banks -> one weight set per expert -> stacked again is the identity; the per-expert file has the key
    names of the reference's unstacked layout and loads into a fresh model; optimizer state is dropped."""

    from nestor_b200.eval.loading import load_experiment_checkpoint
    from nestor_b200.scripts import convert_checkpoint
    data = write_synthetic_bin(tmp_path / "train.bin", 64 * 40, 100_277, doc_len_range=(16, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    base = _train(tmp_path, monkeypatch, "base", 1)
    capsys.readouterr()
    per, back = tmp_path / "per_expert.pt", tmp_path / "stacked.pt"
    assert convert_checkpoint.main(["--experiment", "nestor_tiny", "--checkpoint", str(base), "--output", str(per),
                                    "--to", "per-expert"]) == 0
    assert convert_checkpoint.main(["--experiment", "nestor_tiny", "--checkpoint", str(per), "--output", str(back),
                                    "--to", "stacked"]) == 0
    a = torch.load(base, weights_only=False)
    b = torch.load(per, weights_only=False)
    c = torch.load(back, weights_only=False)
    assert "optimizer" in a and "optimizer" not in b and b["step"] == a["step"]
    assert not any(".stacked_" in k for k in b["model"])
    assert "backbone.blocks.0.layers.0.expert_pool.private_experts.3.1.gate.weight" in b["model"]
    assert "backbone.blocks.0.layers.0.expert_pool.public_experts.2.layers.1.weight" in b["model"]
    assert set(c["model"]) == set(a["model"]) and all(torch.equal(c["model"][k], a["model"][k]) for k in a["model"])
    model, info = load_experiment_checkpoint("nestor_tiny", per)          # either layout loads
    assert info["stacked"] is False and not info["skipped"]
    want = a["model"]["backbone.blocks.0.layers.0.expert_pool.stacked_private.w_up"]
    assert torch.equal(model.state_dict()["backbone.blocks.0.layers.0.expert_pool.stacked_private.w_up"], want)
    with pytest.raises(ValueError, match="already"):
        convert_checkpoint.convert(a, "nestor_tiny", "stacked")


def test_heldout_evaluation_of_the_weight_average(tmp_path, monkeypatch, capsys):
    """A run with ``NESTOR_EMA_DECAY`` stores the averaged weights beside the live ones; ``eval_heldout --ema`` scores
    the average (a different number), in either bank layout."""

    from nestor_b200.scripts import eval_heldout
    data = write_synthetic_bin(tmp_path / "train.bin", 64 * 40, 100_277, doc_len_range=(16, 64))
    held = write_synthetic_bin(tmp_path / "held.bin", 64 * 8, 100_277, seed=2, doc_len_range=(32, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    monkeypatch.setenv("NESTOR_EMA_DECAY", "0.5")
    ckpt = _train(tmp_path, monkeypatch, "ema", 3)
    capsys.readouterr()
    payload = torch.load(ckpt, weights_only=False)
    assert set(payload["ema"]) == {k for k, v in payload["model"].items() if k in payload["ema"]}
    assert any(not torch.equal(payload["ema"][k], payload["model"][k]) for k in payload["ema"])
    scores = {}
    for flag in ((), ("--ema",)):
        eval_heldout.main(["--experiment", "nestor_tiny", "--checkpoint", str(ckpt), "--data", str(held),
                           "--block-size", "64", "--max-windows", "4", *flag])
        out = capsys.readouterr().out
        scores[flag] = json.loads(out[out.index("{"):])["cross_entropy"]
    assert scores[()] != scores[("--ema",)] and all(5.0 < v < 13.0 for v in scores.values())
