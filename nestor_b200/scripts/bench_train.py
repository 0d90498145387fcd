"""Timed training steps of any registered experiment under chosen run knobs (one process per GPU).

``python -m nestor_b200.scripts.bench_train --experiment nestor_200m --block-size 16384 --seqs-per-gpu 1 --accum 8``
builds the experiment with the given context length, per-GPU micro-batch and accumulation, runs ``--warmup``
untimed optimizer steps and ``--steps`` timed ones on synthetic token ids through ``Trainer.train_step`` /
``update_weights`` (CUDA events, barrier + synchronise on both sides, max over ranks) and prints one JSON line
with tokens/s and peak memory. Environment flags (``NESTOR_FREEZE_ROUTERS``, ``NESTOR_ACTIVATION_OFFLOAD``,
``NESTOR_ACTIVATION_CHECKPOINT``, ...) apply as in a real run. Launch with torchrun for several GPUs.
"""

from __future__ import annotations

import argparse
import json
import os


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--experiment", default="nestor_200m")
    ap.add_argument("--block-size", type=int, default=4096)
    ap.add_argument("--seqs-per-gpu", type=int, default=4)
    ap.add_argument("--accum", type=int, default=4)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kernel-table", type=int, default=0, metavar="ROWS",
                    help="after the timed steps, run one more step under torch.profiler and print the ROWS kernels "
                         "with the most device time (use with NESTOR_B200_CUDA_GRAPH=0: a replayed graph shows as one item)")
    a = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ["DCLM_BLOCK_SIZE"] = str(a.block_size)
    if a.block_size != 4096:          # at the series context length the registry insists on the scale's tokens/step
        os.environ["DCLM_GLOBAL_BATCH"] = str(a.seqs_per_gpu * world)
        os.environ["DCLM_GRAD_ACCUM"] = str(a.accum)
    os.environ.setdefault("DCLM_DATA_PATH", "/tmp/unused.bin")
    os.environ.setdefault("DCLM_MAX_STEPS", "10000")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    import torch
    import torch.distributed as dist

    from nestor_b200 import ops
    from nestor_b200.experiments import discover_experiments, get_experiment
    from nestor_b200.models import Model
    from nestor_b200.train.trainer import Trainer
    from nestor_b200.utils.distributed import init_distributed
    from nestor_b200.utils.seed import set_seed

    device = init_distributed(enabled=True)
    discover_experiments()
    import dataclasses as dc
    job = dc.replace(get_experiment(a.experiment)().jobs[0], grad_accum_steps=a.accum)   # the loss is scaled by 1/accum
    set_seed(job.seed)
    model = Model.from_config(job.model)
    trainer = Trainer(job, model, [], device=device, run_dir=None)
    model.train()
    vocab = int(getattr(job.model.head_config, "vocab_size", 0) or 100263)
    gen = torch.Generator(device=device).manual_seed(1234 + int(os.environ.get("RANK", "0")))

    def step() -> None:
        counts: dict = {}
        for _ in range(a.accum):
            ids = torch.randint(0, vocab, (a.seqs_per_gpu, a.block_size), device=device, generator=gen)
            _, c = trainer.train_step((ids, ids))
            counts = trainer.add_counts(counts, c)
        trainer.update_weights(counts)

    def bracket() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(a.warmup):
        step()
    bracket()
    torch.cuda.reset_peak_memory_stats(device)
    n0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    bracket()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tokens = a.seqs_per_gpu * world * a.accum * a.block_size
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({
            "experiment": a.experiment, "n_gpus": world, "block_size": a.block_size, "seqs_per_gpu": a.seqs_per_gpu,
            "grad_accum": a.accum, "tokens_per_step": tokens, "ms_per_step": float(ms.item()),
            "tokens_per_s": tokens / float(ms.item()) * 1e3,
            "peak_mem_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30,
            "gpu_launches_per_step": (ops.launch_count() - n0) / a.steps,
            "flags": {k: v for k, v in os.environ.items() if k.startswith("NESTOR_")}}), flush=True)
    if a.kernel_table > 0 and int(os.environ.get("RANK", "0")) == 0:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize(device)
        events = [e for e in prof.key_averages() if e.device_type == torch.autograd.DeviceType.CUDA]
        events.sort(key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in events)
        ours = sum(e.device_time_total for e in events if "nb" in e.key.split("(")[0])
        print(f"device time of one step: {total / 1e3:.2f} ms in {sum(e.count for e in events)} launches; "
              f"{ours / max(total, 1):.1%} in the in-tree kernels", flush=True)
        for e in events[: a.kernel_table]:
            print(f"{e.device_time_total / 1e3:9.3f} ms {e.device_time_total / max(total, 1):6.1%} {e.count:6d} x "
                  f"{e.device_time_total / max(e.count, 1):8.1f} us  {e.key[:110]}", flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
