"""Headline benchmark: nestor_200m pretraining throughput (tokens/s) on N GPUs of one node.

Config (both arms): the registered ``nestor_200m`` cell — 7 blocks / 17 layers, d=640, 8
columns on the k=(3..8) schedule, hybrid expert pool, 100,263-token vocabulary, 4096-token
context — 4 sequences per GPU per micro-batch, gradient accumulation 32/N so every
optimizer step is the rung's 524,288 tokens (strong scaling), bf16 compute with fp32
masters, Muon (sharded over ranks) + AdamW, gradient clipping, loss-free router-bias
updates. Data: a synthetic token ``.bin`` (uniform ids, documents with log-uniform lengths
in [64, 4096] separated by end-of-text), random-init weights.

``python bench.py --gpus N --steps K --warmup W`` (under ``torch.distributed.run`` for N>1)
prints ONE JSON line from rank 0. Two timed regions of K optimizer steps each, both
bracketed by barrier + ``torch.cuda.synchronize()`` and timed with CUDA events (max over
ranks): ``value`` uses micro-batches already resident on the device; ``e2e`` goes through
``Trainer.train_step`` / ``update_weights`` with every micro-batch copied from pinned host
memory and the step's loss read back to the host. Inputs per step (4 x 4096 x 8 B x accum)
are tiny next to the 126 MB L2, but the working set of one micro-batch (several GB of
activations and 3 GB of parameters) is far larger than L2, so no explicit flush is needed.

``--experiment`` takes any registered cell (``{dense,moe,nestor}_{100m,200m,500m,1b}``); the accumulation follows the
cell's tokens per optimizer step (``nestor_1b``: 2,097,152 tokens, accumulation 128/N; run it with
``NESTOR_ACTIVATION_CHECKPOINT=1``, and the reference arm with ``NESTOR_DDP=0`` as well, for the FSDP2 configuration).

``--impl reference`` runs the unmodified reference package installed under
``baseline/_ref`` through its own ``TrainPipeline`` with its launcher's speed-stack flags.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
EXPERIMENT = "nestor_200m"
SEQ_LEN = 4096
SEQS_PER_GPU = 4
TOKENS_PER_STEP = 524_288       # the 200m rung; other rungs: see tokens_per_step()
_RUNG_TOKENS = {"100m": 262_144, "200m": 524_288, "500m": 1_048_576, "1b": 2_097_152}


def tokens_per_step(experiment: str) -> int:
    """Tokens per optimizer step of an experiment's scale rung (the registries of both arms insist on it)."""

    return _RUNG_TOKENS.get(experiment.rsplit("_", 1)[-1], TOKENS_PER_STEP)

VOCAB = 100_263
BASELINE_TOKENS_PER_SEC = None  # the reference publishes no throughput figure

_CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def _args() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--experiment", default=EXPERIMENT)
    return p.parse_args()


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """``nvidia-smi`` clock/throttle sampling in the background (read-only queries)."""

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.path = Path(tempfile.mkstemp(prefix="clocks_", suffix=".csv")[1])

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except FileNotFoundError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.path.unlink(missing_ok=True)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _data_path(world: int, rank: int, steps_total: int, step_tokens: int = TOKENS_PER_STEP) -> Path:
    """Synthetic corpus shared by all ranks (rank 0 writes, others wait for the sidecar)."""

    path = Path(tempfile.gettempdir()) / f"nestor_bench_{VOCAB}_{SEQ_LEN}.bin"
    need = max(2 * steps_total * step_tokens, 16 * 1024 * 1024)
    meta = Path(f"{path}.meta.json")
    if rank == 0:
        ok = meta.is_file() and json.loads(meta.read_text()).get("num_tokens", 0) >= need
        if not ok:
            sys.path.insert(0, str(ROOT))
            from nestor_b200.data.datasets import write_synthetic_bin
            tmp = path.with_suffix(".tmp")
            write_synthetic_bin(tmp, need, VOCAB, seed=0, doc_len_range=(64, SEQ_LEN))
            tmp.replace(path)
            Path(f"{tmp}.meta.json").replace(meta)
    return path


def _max_over_ranks(ms: float, device) -> float:
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _bracket(device) -> None:
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize(device)


# ----------------------------------------------------------------------------- ours
def run_ours(a: argparse.Namespace) -> dict:
    sys.path.insert(0, str(ROOT))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    step_tokens = tokens_per_step(a.experiment)
    accum = max(1, step_tokens // (SEQS_PER_GPU * SEQ_LEN * world))
    os.environ["DCLM_GLOBAL_BATCH"] = str(SEQS_PER_GPU * world)
    os.environ["DCLM_GRAD_ACCUM"] = str(accum)
    os.environ["DCLM_MAX_STEPS"] = str(10_000)
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    import torch
    from nestor_b200.utils.distributed import barrier, init_distributed
    device = init_distributed(enabled=True)
    if device.type != "cuda":
        raise SystemExit("bench.py needs a CUDA device")
    path = _data_path(world, rank, a.steps * 2 + a.warmup + 2, step_tokens)
    barrier()
    os.environ["DCLM_DATA_PATH"] = str(path)

    from nestor_b200 import ops
    from nestor_b200.data.datasets import DclmTokenDataset, PinnedWindowLoader
    from nestor_b200.experiments import discover_experiments, get_experiment
    from nestor_b200.models import Model
    from nestor_b200.train.trainer import Trainer
    from nestor_b200.utils.seed import set_seed

    discover_experiments()
    job = get_experiment(a.experiment)().jobs[0]
    set_seed(job.seed)
    loader = PinnedWindowLoader(DclmTokenDataset(job.train_dataset), job.train_dataloader, rank=rank, world=world,
                                seed=0)
    model = Model.from_config(job.model)
    trainer = Trainer(job, model, loader, device=device, run_dir=None)
    model.train()
    batches = iter(loader)

    def step_e2e() -> float:
        counts: dict = {}
        total = None
        for _ in range(accum):
            loss, c = trainer.train_step(next(batches))
            total = loss.total.detach() if total is None else total + loss.total.detach()
            counts = trainer.add_counts(counts, c)
        trainer.update_weights(counts)
        return float(total.item()) / accum       # device -> host read of the step's loss

    resident = [tuple(t.to(device) for t in next(batches)) for _ in range(accum)]

    def step_resident() -> None:
        counts: dict = {}
        for b in resident:
            _, c = trainer.train_step((b[0], b[0]))
            counts = trainer.add_counts(counts, c)
        trainer.update_weights(counts)

    for _ in range(max(3, a.warmup)):
        step_e2e()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    launches0 = ops.launch_count()
    _bracket(device)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step_resident()
    e1.record()
    _bracket(device)
    launches = ops.launch_count() - launches0
    ms_dev = _max_over_ranks(e0.elapsed_time(e1), device)

    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last_loss = 0.0
    for _ in range(a.steps):
        last_loss = step_e2e()
    f1.record()
    _bracket(device)
    clocks = sampler.stop() if rank == 0 else {}
    ms_e2e = _max_over_ranks(f0.elapsed_time(f1), device)

    # Where a step's time goes beyond its micro-batches (untimed extra steps): the micro-batch alone, then one step
    # with an event at every phase boundary of the optimizer step. "exposed" = step - accum x micro-batch.
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _bracket(device)
    g0.record()
    for b in resident:
        trainer.train_step((b[0], b[0]))
    g1.record()
    _bracket(device)
    ms_micro = _max_over_ranks(g0.elapsed_time(g1), device) / accum
    trainer.phase_events = []
    trainer.update_weights({})
    phases = {k: _max_over_ranks(v, device) for k, v in trainer.phase_times_ms().items()}
    trainer.phase_events = None
    comm_ms = phases.get("grad_reduce", 0.0) + phases.get("param_push", 0.0)
    exposed = ms_dev / a.steps - accum * ms_micro

    # Kernel census of one untimed eager micro-batch (a replayed graph shows up as one item to the profiler): how many
    # of the launches are kernels of the in-tree library (namespaces nb / nbr / nbo / nbm) and how many come from
    # PyTorch (copies, fills, the embedding, small reductions).
    census = None
    if rank == 0:
        try:
            from torch.profiler import ProfilerActivity, profile
            saved, trainer._graph_enabled = trainer._graph_enabled, False
            trainer.train_step((resident[0][0], resident[0][0]))
            torch.cuda.synchronize(device)
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                trainer.train_step((resident[0][0], resident[0][0]))
                torch.cuda.synchronize(device)
            trainer._graph_enabled = saved
            trainer.arena.zero_grad()
            ev = [e for e in prof.key_averages() if e.device_type == torch.autograd.DeviceType.CUDA]
            own = [e for e in ev if e.key.replace("void ", "").startswith(("nb::", "nbr::", "nbo::", "nbm::"))]
            census = {"own_launches": sum(e.count for e in own), "other_launches": sum(e.count for e in ev) - sum(e.count for e in own),
                      "own_device_ms": sum(e.device_time_total for e in own) / 1e3,
                      "other_device_ms": (sum(e.device_time_total for e in ev) - sum(e.device_time_total for e in own)) / 1e3}
        except Exception as exc:      # the census is informative only
            census = {"error": f"{type(exc).__name__}: {exc}"[:160]}
    _bracket(device)      # every rank leaves together (rank 0 alone ran the census)

    tokens = step_tokens * a.steps
    value = tokens / (ms_dev / 1e3)
    h2d = accum * SEQS_PER_GPU * SEQ_LEN * 8
    return {
        "metric": f"{a.experiment} train tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": ms_dev / a.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None if BASELINE_TOKENS_PER_SEC is None else value / BASELINE_TOKENS_PER_SEC,
        "dtype": "bf16", "data": "synthetic uniform token ids in log-uniform-length documents; random-init weights",
        "impl": "ours",
        "config": {"model": a.experiment, "global_batch": SEQS_PER_GPU * world, "grad_accum": accum,
                   "tokens_per_step": step_tokens, "seq_len": SEQ_LEN, "parallelism": f"dp{world}",
                   "optimizer": "sharded Muon + AdamW, clip 1.0", "l2": "working set >> L2 (no flush needed)"},
        "stack": {"kernels": "in-tree sm_100a library (tcgen05 / TMA), CUDA-graph micro-batch",
                  "grad_transport": os.environ.get("NESTOR_B200_GRAD_TRANSPORT", "fused")},
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": last_loss},
        "gpu_launches": launches, "clocks": clocks, "micro_batch_kernel_census": census,
        "step_breakdown_ms": {"micro_batch": ms_micro, "outside_micro_batches": exposed, "exposed_comm_ms": comm_ms if world > 1 else 0.0,
                              **{f"update_{k}": v for k, v in phases.items()}},
    }


# ------------------------------------------------------------------------ reference
def _install_varlen_causal_shim() -> str | None:
    """Let the reference's ``varlen_attn(..., is_causal=True)`` calls run on a torch whose ``varlen_attn`` spells
    causal masking as ``window_size=(-1, 0)``.

    The reference (``nestor/backbones/nestor.py:3462,6213,6357``) was written against a torch whose
    ``torch.nn.attention.varlen.varlen_attn`` takes ``is_causal``; later releases replaced the keyword by
    ``window_size`` and derive ``is_causal = window_size == (-1, 0)`` before calling the same flash kernel. The
    wrapper below is installed on the torch module attribute only (the reference package stays byte-identical)
    and forwards every other argument untouched, so the reference's packed-varlen fast path runs with its
    speed-stack flags at 1. Returns ``None`` when the fast path is usable (natively or through the wrapper),
    else one line saying why it had to be switched off.
    """

    try:
        import inspect
        from torch.nn.attention import varlen
    except ImportError:
        return "torch.nn.attention.varlen is missing in this torch; packed-varlen attention flags are off"
    params = inspect.signature(varlen.varlen_attn).parameters
    if "is_causal" in params:
        return None
    if "window_size" not in params:
        return ("this torch's varlen_attn has neither is_causal nor window_size; NESTOR_ATTN_PACKED_VARLEN / "
                "NESTOR_TRITON_PACKED_ATTN / NESTOR_GATHERED_VARLEN are off")
    stock = varlen.varlen_attn

    def varlen_attn(query, key, value, cu_seq_q, cu_seq_k, max_q, max_k, *args, is_causal: bool = False, **kwargs):
        if is_causal:
            kwargs["window_size"] = (-1, 0)
        return stock(query, key, value, cu_seq_q, cu_seq_k, max_q, max_k, *args, **kwargs)

    varlen_attn.__wrapped__ = stock
    try:   # one two-segment case against per-segment causal SDPA before trusting the encoding
        import torch
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        g = torch.Generator(device=dev).manual_seed(0)
        q, k, v = (torch.randn(96, 2, 40, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(3))
        cu = torch.tensor([0, 40, 96], device=dev, dtype=torch.int32)
        got = varlen_attn(q, k, v, cu, cu, 56, 56, is_causal=True).float()
        want = torch.cat([torch.nn.functional.scaled_dot_product_attention(
            q[a:b].transpose(0, 1).float(), k[a:b].transpose(0, 1).float(), v[a:b].transpose(0, 1).float(),
            is_causal=True).transpose(0, 1) for a, b in ((0, 40), (40, 96))])
        err = float((got - want).abs().max())
        if not err < 3e-2:
            return (f"varlen_attn(window_size=(-1, 0)) differs from per-segment causal SDPA by {err:.3g}; "
                    "packed-varlen attention flags are off")
    except Exception as exc:  # the check itself could not run: keep the stock fallback arm
        return f"varlen_attn causal check failed ({type(exc).__name__}: {exc})"[:200] + "; packed-varlen flags are off"
    varlen.varlen_attn = varlen_attn
    return None


class _BenchDone(Exception):
    pass


def run_reference(a: argparse.Namespace) -> dict:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "nestor").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref)"}
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    step_tokens = tokens_per_step(a.experiment)
    accum = max(1, step_tokens // (SEQS_PER_GPU * SEQ_LEN * world))
    warm = max(3, a.warmup)
    # The launcher's speed stack (scripts/lib/speed_stack.sh of the reference), verbatim defaults.
    stack = dict(
        NESTOR_DDP="1", NESTOR_COMPILE=os.environ.get("NESTOR_COMPILE", "1"), NESTOR_BF16="1",
        NESTOR_DENSE_NO_ROUTER="1", NESTOR_RUNAHEAD="0", NESTOR_DDP_BROADCAST_BUFFERS="1",
        NESTOR_DDP_STATIC_GRAPH="0", NESTOR_GATHERED_CAUSAL_FLASH="1", NESTOR_GATHERED_VARLEN="1",
        NESTOR_MOE_GROUPED_MM="1", NESTOR_CE_CHUNK_ROWS="4096", NESTOR_COLUMN_SLOT_UPDATES="1",
        NESTOR_DENSE_TAIL_ATTN="1", NESTOR_GROUPED_MM_FUSED_GATE="1", NESTOR_ATTN_PACKED_VARLEN="1",
        NESTOR_DDP_NO_SYNC="1", NESTOR_MUON_SHARD="1", NESTOR_STACKED_EXPERT_BANKS="1",
        NESTOR_BATCHED_ROUTERS="1", NESTOR_TRITON_PACKED_ATTN="1", NESTOR_TRITON_INDEX_BUILD="1",
        NESTOR_TRITON_EXPERT_DISPATCH="1")
    adjusted = _install_varlen_causal_shim()
    if adjusted is not None:
        for k in ("NESTOR_ATTN_PACKED_VARLEN", "NESTOR_TRITON_PACKED_ATTN", "NESTOR_GATHERED_VARLEN"):
            stack[k] = "0"
    for k, v in stack.items():
        os.environ.setdefault(k, v)
    os.environ.update(
        WANDB_MODE="disabled", DCLM_GLOBAL_BATCH=str(SEQS_PER_GPU * world), DCLM_GRAD_ACCUM=str(accum),
        DCLM_MAX_STEPS=str(warm + a.steps + 1), DCLM_WARMUP_STEPS="2", DCLM_CKPT_FREQ="1000000",
        DCLM_LOG_FREQ="1000000", DCLM_NUM_WORKERS="2",
        NESTOR_OUTPUT_ROOT=str(Path(tempfile.gettempdir()) / "nestor_ref_out"))
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29533"), ("RANK", "0"), ("WORLD_SIZE", "1"),
                 ("LOCAL_RANK", "0")):
        os.environ.setdefault(k, v)   # a bare `python bench.py` run still gets an env:// rendezvous
    path = _data_path(world, rank, a.steps + warm + 2, step_tokens)
    os.environ["DCLM_DATA_PATH"] = str(path)
    sys.path.insert(0, str(ref))
    try:
        import torch
        import nestor.cli as ref_cli  # noqa: F401  (imports timing first, like the console script)
        from nestor.experiments.registry import get_experiment
        from nestor.pipelines.train import TrainPipeline
        from nestor.train.trainer import Trainer as RefTrainer
        from nestor.utils.distributed import cleanup_distributed
        ref_cli._discover_experiments()
        if world > 1:
            time.sleep(2.0 if rank else 0.0)  # rank 0 wrote the corpus above; give the file system a beat
        experiment = get_experiment(a.experiment)()
        experiment.name = a.experiment
        experiment.save_source_snapshot = False
        job = experiment.jobs[0]
    except Exception as exc:  # missing dependency of the reference in this image
        return {"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"[:300]}

    events: list = []
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    stock_update = RefTrainer._update_weights

    def timed_update(self, *args, **kwargs):
        out = stock_update(self, *args, **kwargs)
        if len(events) == warm - 1 and rank == 0:
            sampler.start()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        events.append(ev)
        if len(events) >= warm + a.steps:
            raise _BenchDone()
        return out

    RefTrainer._update_weights = timed_update  # timing probe only: stock step body runs unchanged
    device = None
    try:
        pipe = TrainPipeline.from_config(job_config=job, experiment_config=experiment)
        device = pipe.device
        try:
            pipe.run()
        except _BenchDone:
            pass
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else {}
        ms = _max_over_ranks(events[warm - 1].elapsed_time(events[warm + a.steps - 1]), torch.device(device))
        tokens = step_tokens * a.steps
        value = tokens / (ms / 1e3)
        out = {
            "metric": f"{a.experiment} train tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": a.steps, "warmup": warm, "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic uniform token ids in log-uniform-length documents; random-init weights",
            "config": {"model": a.experiment, "global_batch": SEQS_PER_GPU * world, "grad_accum": accum,
                       "tokens_per_step": step_tokens, "seq_len": SEQ_LEN, "parallelism": f"dp{world}",
                       "optimizer": "sharded Muon + AdamW, clip 1.0", "l2": "working set >> L2 (no flush needed)"},
            "stack": {"speed_stack": {k: os.environ[k] for k in stack}, "speed_stack_adjusted": adjusted},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": accum * SEQS_PER_GPU * SEQ_LEN * 16,
                    "d2h_bytes_per_step": 8 * accum,
                    "note": "the reference's stock loop already copies every batch from its pinned DataLoader "
                            "and reads num_tokens back per micro-batch; the same region is reported for both"},
            "gpu_launches": None, "clocks": clocks,
        }
    except Exception as exc:
        out = {"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {exc}"[:400]}
    finally:
        RefTrainer._update_weights = stock_update
        try:
            cleanup_distributed()
        except Exception:
            pass
    return out


def main() -> int:
    a = _args()
    result = run_reference(a) if a.impl == "reference" else run_ours(a)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(result), flush=True)
    if a.impl == "ours":
        from nestor_b200.utils.distributed import cleanup_distributed
        cleanup_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
