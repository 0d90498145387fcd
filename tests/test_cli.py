"""The command line: registry listing, error paths, the .env file, and an experiment of a train job followed by an
eval job that reads the checkpoint the train job wrote."""

import json
import os
from pathlib import Path


from nestor_b200.data.datasets import write_synthetic_bin


def test_listing_and_error_paths(capsys):
    from nestor_b200.cli import main
    assert main(["--list-experiments"]) == 0
    out = capsys.readouterr().out
    assert "nestor_200m" in out and "dense_1b" in out and "nestor_tiny" in out
    assert main([]) == 1 and "--experiment is required" in capsys.readouterr().out
    assert main(["--experiment", "no_such_cell"]) == 1 and "Error" in capsys.readouterr().out


def test_dotenv_fills_in_without_overriding(tmp_path, monkeypatch):
    from nestor_b200.cli import _load_dotenv
    env = tmp_path / ".env"
    env.write_text("# comment\nexport NB_TEST_A='from file'\nNB_TEST_B=\"quoted\"\nnot a pair\nNB_TEST_C = spaced \n")
    monkeypatch.setenv("NB_TEST_A", "already set")
    for k in ("NB_TEST_B", "NB_TEST_C"):
        monkeypatch.delenv(k, raising=False)
    _load_dotenv(env)
    try:
        assert os.environ["NB_TEST_A"] == "already set"          # the environment wins over the file
        assert os.environ["NB_TEST_B"] == "quoted" and os.environ["NB_TEST_C"] == "spaced"
    finally:
        os.environ.pop("NB_TEST_B", None); os.environ.pop("NB_TEST_C", None)
    _load_dotenv(tmp_path / "absent.env")                        # a missing file is not an error


def test_train_job_then_eval_job(tmp_path, monkeypatch):
    """A train experiment writes ``model_final.pt``; an experiment with an eval job builds the same model, loads that
    file, scores a held-out token file and writes ``eval_results.json`` / ``.md`` into its own run directory. Both
    go through ``nestor_cli``."""

    from nestor_b200.cli import main
    from nestor_b200.configs import (DataLoaderConfig, DclmDatasetConfig, EvalJobConfig, EvalSuiteConfig,
                                     ExperimentConfig, LanguageModelingEvalConfig)
    from nestor_b200.experiments import register_experiment
    from nestor_b200.experiments import registry as reg
    from nestor_b200.experiments.tiny import nestor_tiny
    train_bin = write_synthetic_bin(tmp_path / "train.bin", 64 * 40, 100_277, doc_len_range=(16, 64))
    held_bin = write_synthetic_bin(tmp_path / "held.bin", 64 * 12, 100_277, seed=5, doc_len_range=(16, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(train_bin))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    monkeypatch.setenv("DCLM_MAX_STEPS", "1")
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "out"))
    assert main(["--experiment", "nestor_tiny"]) == 0
    (ckpt,) = list((tmp_path / "out" / "nestor_tiny").glob("*/checkpoints/model_final.pt"))

    def held_out_eval():
        return ExperimentConfig(output_root=tmp_path / "out", jobs=[EvalJobConfig(
            name="held_out", model=nestor_tiny().jobs[0].model, model_checkpoint_path=ckpt,
            eval_suite=EvalSuiteConfig(evals=[LanguageModelingEvalConfig(
                name="held_out", dataset_config=DclmDatasetConfig(data_path=held_bin, block_size=64),
                dataloader_config=DataLoaderConfig(batch_size=2, num_workers=0))]))])

    register_experiment(held_out_eval)
    try:
        assert main(["--experiment", "held_out_eval"]) == 0
    finally:
        reg._CELLS.pop("held_out_eval", None)
    results = list((tmp_path / "out" / "held_out_eval").glob("*__held_out/eval_results.json"))
    assert len(results) == 1
    metrics = json.loads(results[0].read_text())["held_out"]
    assert 5.0 < metrics["cross_entropy"] < 13.0 and metrics["tokens"] > 0
    assert (results[0].parent / "eval_results.md").read_text().startswith("| eval | metric | value |")


def test_reference_flags_are_reported_at_start_up(caplog):
    """A launcher written for the reference exports its fast-path switches; here they select nothing, and the start-up
    report says so (and warns about values that ask for a mode with a different equivalent)."""

    import logging
    from nestor_b200.utils.flags import NO_EFFECT, classify, report_reference_flags
    env = {"NESTOR_TRITON_PACKED_ATTN": "1", "NESTOR_COMPILE": "0", "NESTOR_MOE_GROUPED_MM": "1", "NESTOR_DDP": "0",
           "NESTOR_MUON_SHARD": "1", "NESTOR_STACKED_EXPERT_BANKS": "1", "NESTOR_COLUMN_SLOT_UPDATES": ""}
    found = classify(env)
    assert set(found["no_effect"]) == {"NESTOR_TRITON_PACKED_ATTN", "NESTOR_COMPILE", "NESTOR_MOE_GROUPED_MM"}
    assert set(found["different"]) == {"NESTOR_DDP=0"}
    logger = logging.getLogger("nestor_b200.test_flags")
    logger.propagate = True
    with caplog.at_level(logging.INFO, logger="nestor_b200.test_flags"):
        report_reference_flags(logger, env)
    text = caplog.text
    assert "NESTOR_TRITON_PACKED_ATTN" in text and "no effect here" in text and "ZeRO-1" in text
    assert classify({}) == {"no_effect": {}, "different": {}}
    # nothing this package reads is listed as having no effect
    import re
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent / "nestor_b200"
    read = set()
    for f in root.rglob("*.py"):
        if f.name != "flags.py":
            read |= set(re.findall(r'"(NESTOR_[A-Z0-9_]+)"', f.read_text()))
    # (two are named elsewhere without being acted on: the trainer's note about the bf16 mode, and the variable the
    # long-context protocol exports for launchers of the reference)
    assert not (read & set(NO_EFFECT)) - {"NESTOR_BF16_MASTER", "NESTOR_GATHERED_CAP_BUCKET"}
