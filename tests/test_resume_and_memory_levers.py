"""Resume continuity (a resumed run sees the batches and reaches the weights of an uninterrupted one), the host-copy
cache behind activation offload, and the once-only out-of-memory snapshot."""

import pickle
import time

import torch

from nestor_b200.data.datasets import write_synthetic_bin
from nestor_b200.pipelines import TrainPipeline


class _Tap:
    """A loader that notes the first tokens of every batch it hands out."""

    def __init__(self, inner, log):
        self.inner, self.log = inner, log

    def __len__(self):
        return len(self.inner)

    def set_epoch(self, epoch):
        if hasattr(self.inner, "set_epoch"):
            self.inner.set_epoch(epoch)

    def __iter__(self):
        for batch in self.inner:
            self.log.append(tuple(int(v) for v in batch[0].reshape(-1)[:4]))
            yield batch


def _launch(monkeypatch, steps):
    """Run the tiny experiment until ``steps`` optimizer steps are done; the schedule always spans four."""

    import dataclasses as dc
    monkeypatch.setenv("DCLM_MAX_STEPS", "4")
    from nestor_b200.experiments.tiny import nestor_tiny
    exp = nestor_tiny(); exp.name = "nestor_tiny"
    exp.jobs[0] = dc.replace(exp.jobs[0], max_steps=steps)
    pipe = TrainPipeline.from_config(job_config=exp.jobs[0], experiment_config=exp)
    trainer = pipe.setup()
    for blk in trainer.model.backbone.blocks:       # no exploration noise: the runs differ only in where they start
        blk.freeze_routing_noise = True
    log = []
    trainer.train_loader = _Tap(trainer.train_loader, log)
    trainer.train()
    state = trainer.arena.master.clone()
    step = trainer.global_step
    pipe.ctx.close()
    return log, state, step


def test_resumed_run_continues_where_the_data_and_the_weights_were(tmp_path, monkeypatch):
    """Four steps in one go against two steps, a checkpoint, and a second launch that resumes to four: the resumed
    launch skips exactly the micro-batches already trained on ((step x accumulation) mod batches per epoch), trains
    on the same remaining ones, restores optimizer and scheduler state, and ends with the same weights."""

    # one thread: multi-threaded CPU reductions differ in the last bit from run to run, and Newton-Schulz in bf16
    # amplifies that; single-threaded, a resumed run is bit-identical to an uninterrupted one
    threads = torch.get_num_threads()
    torch.set_num_threads(1)
    try:
        _resume_case(tmp_path, monkeypatch)
    finally:
        torch.set_num_threads(threads)


def _resume_case(tmp_path, monkeypatch):
    data = write_synthetic_bin(tmp_path / "train.bin", 64 * 60, 100_277, doc_len_range=(16, 64))
    monkeypatch.setenv("DCLM_DATA_PATH", str(data))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    monkeypatch.setenv("DCLM_GRAD_ACCUM", "2")
    monkeypatch.setenv("DCLM_CKPT_FREQ", "2")
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "straight"))
    straight_log, straight_state, step = _launch(monkeypatch, 4)
    assert step == 4 and len(straight_log) >= 8      # (the loop may draw one batch ahead of the step that ends the run)
    straight_log = straight_log[:8]

    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "resumed"))
    first_log, _, step = _launch(monkeypatch, 2)
    assert step == 2 and first_log[:4] == straight_log[:4]
    time.sleep(1.1)                                   # run directories are second-stamped
    second_log, resumed_state, step = _launch(monkeypatch, 4)
    assert step == 4
    # the second launch draws the four trained batches again only to skip them, then the four new ones
    assert second_log[:8] == straight_log
    assert torch.equal(resumed_state, straight_state), float((resumed_state - straight_state).abs().max())

    # NESTOR_RESUME_NO_FASTFORWARD=1 restarts the epoch instead (and therefore trains on the first batches again)
    monkeypatch.setenv("NESTOR_RESUME_NO_FASTFORWARD", "1")
    monkeypatch.setenv("NESTOR_OUTPUT_ROOT", str(tmp_path / "resumed2"))
    _launch(monkeypatch, 2)
    time.sleep(1.1)
    again_log, _, _ = _launch(monkeypatch, 4)
    assert again_log[:4] == straight_log[:4]


def test_host_copy_cache_is_keyed_by_storage_and_version():
    from nestor_b200.train.activation_offload import HostCopyCache, _HostCopy, ActivationOffloadStats, activation_offload
    base = torch.arange(64.0)
    a, b = base[:32], base[32:]                       # two views of one storage
    cache = HostCopyCache()
    assert cache.key(a) == cache.key(b) and cache.get(a) is None
    copy = _HostCopy(base.clone(), base.device, None)
    cache.put(a, copy)
    assert cache.get(b) is copy                       # the other view finds the same host copy
    assert cache.get(torch.arange(64.0)) is None      # another storage does not
    base.add_(1.0)                                    # an in-place write makes the copy stale: new version, new key
    assert cache.get(a) is None
    cache.put(a, copy)
    del copy
    import gc; gc.collect()
    assert cache.get(a) is None                       # entries die with their last referencing save
    # without a GPU the context changes nothing and counts nothing
    x = torch.randn(8, 8, requires_grad=True)
    with activation_offload() as stats:
        y = (x @ x).sum()
    y.backward()
    assert isinstance(stats, ActivationOffloadStats) and stats.packed == 0 and "nothing moved" in stats.summary()
    assert x.grad is not None


def test_oom_snapshot_is_written_once_and_never_masks_the_error(tmp_path, monkeypatch):
    from nestor_b200.train import oom_snapshot as O
    calls = []
    monkeypatch.setattr(torch.cuda.memory, "_snapshot", lambda: calls.append(1) or {"segments": [], "device_traces": []})
    d = O.OomSnapshotDumper(tmp_path / "diag" / "diag_oom_rank0.pickle")
    d.suspended = True                                 # deliberate probing (batch-size calibration) is muted
    d(0, 1 << 30, 2 << 30, 123)
    assert not d.path.exists() and not d.dumped
    d.suspended = False
    d(0, 1 << 30, 2 << 30, 123)
    d(0, 5, 6, 7)                                      # later failures are ignored
    assert len(calls) == 1 and d.dumped
    with open(d.path, "rb") as f:
        payload = pickle.load(f)
    assert payload["requested_bytes"] == 1 << 30 and payload["device_free"] == 123 and "snapshot" in payload
    # a failing snapshot must not raise out of the allocator's callback
    monkeypatch.setattr(torch.cuda.memory, "_snapshot", lambda: (_ for _ in ()).throw(RuntimeError("no history")))
    e = O.OomSnapshotDumper(tmp_path / "diag" / "other.pickle")
    e(0, 1, 2, 3)
    assert e.dumped and not e.path.exists()
    if not torch.cuda.is_available():
        assert O.install_oom_snapshot(tmp_path) is None
