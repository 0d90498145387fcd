"""The training loop.

One optimizer step = ``grad_accum_steps`` micro-batches of forward+backward into the
gradient arena, one data-parallel reduction, gradient clipping on the flat buffer, the
Muon/AdamW step, a refresh of the compute copy, the scheduler step and the loss-free
router-bias nudge. Behaviour parity with the reference's ``Trainer``
(``nestor/train/trainer.py``): loss is scaled by ``1/accum`` per micro-batch (``:835-866``);
clipping precedes the step (``:906-911``); bias nudges use the whole window's selections
(``:1026-1128``); resume fast-forwards the loader by ``(step * accum) % batches_per_epoch``
micro-batches (``:362-395``); ``NESTOR_RUNAHEAD`` bounds host run-ahead (``:467-479``);
EMA shadow (``:960-1000``); MFU/throughput metrics (``:761-816``); per-phase wall timers
under ``NESTOR_TRAIN_PROFILE`` and a ``torch.profiler`` window under ``NESTOR_TORCH_PROFILE``.

What differs by design: gradients are never synchronised per micro-batch (there is no
``no_sync`` context to manage), host<->device traffic is one pinned async copy in and one
scalar out per logged step, and step timing is taken with CUDA events.
"""

from __future__ import annotations

import collections
import contextlib
import logging
import math
import os
import subprocess
import time
from pathlib import Path
from typing import Any, Iterable

import torch
from torch import Tensor, nn

from nestor_b200.configs import TrainJobConfig
from nestor_b200.models.nestor import RouterCounts, add_router_counts, apply_bias_updates, router_counts
from nestor_b200.parallel.arena import ParamArena
from nestor_b200.parallel.grad_sync import GradReducer
from nestor_b200.train import checkpoint as ckpt
from nestor_b200.train.flops import train_flops_per_token
from nestor_b200.train.losses import LossOutput, build_loss
from nestor_b200.train.optim import build_optimizer, build_scheduler
from nestor_b200.utils.distributed import barrier, get_rank, get_world_size, is_main_process
from nestor_b200.utils.batches import split_supervised_batch
from nestor_b200.utils.logging import get_logger, log_metrics
from nestor_b200.utils.timing import PROCESS_START


def _env_flag(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default) == "1"


class Trainer:
    def __init__(self, config: TrainJobConfig, model: nn.Module, train_loader: Iterable, *,
                 device: torch.device, run_dir: Path | None = None, eval_suite: Any = None,
                 logger: logging.Logger | None = None) -> None:
        self.config, self.model, self.train_loader = config, model, train_loader
        self.device, self.run_dir, self.eval_suite = device, run_dir, eval_suite
        self.logger = logger or get_logger("nestor_b200.train")
        self.world, self.rank = get_world_size(), get_rank()
        bf16 = config.use_amp and device.type == "cuda" and os.environ.get("NESTOR_BF16", "1") == "1"
        self.compute_dtype = torch.bfloat16 if bf16 else torch.float32
        model.to(device)
        model.compute_dtype = self.compute_dtype
        model.fused_head = os.environ.get("NESTOR_FUSED_HEAD_CE", "1") == "1"
        if _env_flag("NESTOR_FREEZE_ROUTERS"):
            from nestor_b200.train.frozen_routers import freeze_routers
            freeze_routers(model)
        transport = os.environ.get("NESTOR_B200_GRAD_TRANSPORT", "fused" if device.type == "cuda" else "gloo")
        fused = self.world > 1 and device.type == "cuda" and transport == "fused"
        self.arena = ParamArena(model, compute_dtype=self.compute_dtype, device=device, symmetric=fused)
        self.reducer = GradReducer(self.arena, transport=transport)
        self.reducer.sync_buffers(model)
        self.loss_fn = build_loss(config.loss)
        self.optimizer = build_optimizer(config.optimizer, model)
        self.scheduler = build_scheduler(config.scheduler, self.optimizer)
        self.param_push = None
        if fused and getattr(self.optimizer, "sharded", False) and getattr(self.optimizer, "owner_cuts", None):
            from nestor_b200.parallel.symm import ParamPush
            self.param_push = ParamPush(self.arena.master, self.arena.compute)
            self.optimizer.param_sync = lambda opt: None      # distribution happens after the compute-copy refresh
        if device.type == "cuda":
            # expert banks read from their owner ranks by the all-gather fused into the bank GEMMs (off unless asked
            # for); always reassigned, so that a trainer never inherits the peer table of an earlier one's arena
            from nestor_b200.ops import cuda as cuda_ops
            cuda_ops.BANK_SHARDS = None
            if fused and self.param_push is not None and self.compute_dtype == torch.bfloat16 and _env_flag("NESTOR_FSDP_BANKS"):
                from nestor_b200.parallel.shard import ShardedBanks
                g = self.param_push.group
                cuda_ops.BANK_SHARDS = ShardedBanks(self.arena.compute, [int(g.peers.aux[r]) for r in range(g.world)], g.rank)
        # the pushed range carries every parameter in it; when its owner is the only one to update them (ZeRO-1 for
        # AdamW as well) it is also the only one that needs their reduced gradients: reduce-scatter
        self.zero = bool(self.param_push is not None and getattr(self.optimizer, "shard_adamw", False))
        # the push distributes the bf16 compute copy only: fp32 masters (and the EMA shadow) outside this rank's range
        # are stale between checkpoints (see gather_masters)
        self.masters_sharded = bool(self.param_push is not None and not self.param_push.push_master)
        # Device status word of the in-kernel collectives: a bounded peer wait that gave up leaves a nonzero code
        # there and the kernel returns without reducing / pushing. It is read back once per optimizer step.
        if os.environ.get("NESTOR_BF16_MASTER") == "0" and bf16:
            # the reference's NESTOR_BF16_MASTER=1 (bf16 matrices with fp32 masters in the optimizer, no cast per use)
            # is how this trainer always runs in bf16; there is no per-use-cast mode to fall back to
            self.logger.info("NESTOR_BF16_MASTER=0 has no effect: the bf16 compute copy with fp32 masters is the only bf16 mode")
        self.nvtx = _env_flag("NESTOR_NVTX")
        self.phase_events: list | None = None     # set to [] to time the phases of the next update_weights
        self.peer_status: Tensor | None = None
        self._status_host: Tensor | None = None
        self._status_event = None
        if fused:
            from nestor_b200.ops import _lib
            self.peer_status = _lib.status_word(device)
        self.global_step, self.epoch = 0, 0
        self.ema: dict[str, Tensor] | None = None
        decay = os.environ.get("NESTOR_EMA_DECAY")
        self.ema_decay = float(decay) if decay else config.ema_decay
        if self.ema_decay:
            self.ema = {"flat": self.arena.master.clone()}
        self.runahead = int(os.environ.get("NESTOR_RUNAHEAD", "0"))
        self._step_events: collections.deque = collections.deque()
        self._h2d_events: collections.deque = collections.deque()
        self.global_counts = _env_flag("NESTOR_LOSSFREE_GLOBAL_COUNTS")
        self.offload = _env_flag("NESTOR_ACTIVATION_OFFLOAD")
        self.tokens_per_micro: int | None = None
        self._graph: dict | None = None
        self._graph_warmup = 0
        self._graph_enabled = (device.type == "cuda" and _env_flag("NESTOR_B200_CUDA_GRAPH", "1") and not self.offload
                               and not _env_flag("NESTOR_TORCH_PROFILE") and not _env_flag("NESTOR_TRAIN_PROFILE"))
        self._oom_dumper = None
        if _env_flag("NESTOR_DIAG_OOM_SNAPSHOT") and run_dir is not None:
            from nestor_b200.train.oom_snapshot import install_oom_snapshot
            self._oom_dumper = install_oom_snapshot(run_dir, rank=self.rank)

    # ------------------------------------------------------------------ one micro-batch
    def _to_device(self, batch: Any) -> tuple[Tensor, Tensor]:
        inputs, targets = batch
        staged = not inputs.is_cuda
        inputs = inputs.to(self.device, non_blocking=True)
        targets = inputs if targets is batch[0] else targets.to(self.device, non_blocking=True)
        if staged:
            self._note_host_copy()
        return inputs, targets

    # A loader that stages batches in a ring of pinned buffers reuses a buffer a few batches later. The copies above are
    # asynchronous and the host runs ahead of the device (a whole optimizer step of micro-batches when nothing is read
    # back), so without a bound a buffer could be refilled before the device has read it. The host therefore never gets
    # more than ``H2D_WINDOW`` batches ahead of the last executed copy; the ring of ``PinnedWindowLoader`` is sized for it.
    H2D_WINDOW = 3

    def _note_host_copy(self) -> None:
        if self.device.type != "cuda":
            return
        ev = torch.cuda.Event()
        ev.record()
        self._h2d_events.append(ev)
        while len(self._h2d_events) > self.H2D_WINDOW:
            self._h2d_events.popleft().synchronize()

    def _activation_ctx(self):
        if self.offload and self.device.type == "cuda":
            from nestor_b200.train.activation_offload import activation_offload
            return activation_offload()
        return contextlib.nullcontext()

    @contextlib.contextmanager
    def _nvtx(self, name: str):
        """NVTX range around a phase of the step (``NESTOR_NVTX=1``): shows up in timeline profilers."""

        on = self.nvtx and self.device.type == "cuda"
        if on:
            torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            if on:
                torch.cuda.nvtx.range_pop()

    @staticmethod
    def add_counts(total: dict | None, counts: dict) -> dict:
        """Sum the router counts of successive ``train_step`` calls (one launch per micro-batch when both are packed)."""

        return add_router_counts(total, counts)

    def train_step(self, batch: Any) -> tuple[LossOutput, dict[str, Tensor]]:
        """Forward + backward of one micro-batch; gradients accumulate into the arena.

        On CUDA the whole micro-batch (forward, loss, backward, router counts) is captured once
        into a CUDA graph and replayed afterwards: every shape is static (packed layouts have
        exactly ``T*k`` rows, plans are built on the device) and nothing in the step reads
        device memory from the host, so a replay is one launch. ``NESTOR_B200_CUDA_GRAPH=0``
        keeps eager launches; activation offload and the eager profiler also disable capture.
        """

        batch = split_supervised_batch(batch)      # (inputs, targets) pairs or inputs/targets, inputs/labels, x/y mappings
        with self._nvtx("micro_batch"):
            if self._graph_enabled and self.model.training:
                return self._graphed_step(batch)
            return self._eager_step(batch)

    def _graphed_step(self, batch: Any) -> tuple[LossOutput, dict[str, Tensor]]:
        inputs, _ = batch
        g = self._graph
        if g is None or g["ids"].shape != inputs.shape:
            if self._graph_warmup < 2:
                # First calls run eagerly (lazy kernel attributes, caches) on a side stream, so that no
                # autograd node created here is tied to the default stream when capture starts.
                self._graph_warmup += 1
                side = self._side_stream = getattr(self, "_side_stream", None) or torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    out = self._eager_step(batch)
                torch.cuda.current_stream().wait_stream(side)
                return out
            ids = torch.empty(inputs.shape, dtype=inputs.dtype, device=self.device)
            ids.copy_(inputs, non_blocking=True)
            torch.cuda.synchronize()
            from nestor_b200.ops import _lib
            graph = torch.cuda.CUDAGraph()
            before = _lib.LAUNCHES
            with torch.cuda.graph(graph):
                loss, counts = self._eager_step((ids, ids), on_device=True)
            g = self._graph = {"graph": graph, "ids": ids, "loss": loss, "counts": counts,
                               "kernels": _lib.LAUNCHES - before}   # in-tree kernels recorded in the graph
            graph.replay()            # capture records without executing: run this micro-batch now
            return loss, counts
        from nestor_b200.ops import _lib
        g["ids"].copy_(inputs, non_blocking=True)
        if not inputs.is_cuda:
            self._note_host_copy()
        g["graph"].replay()
        _lib.count_launch(g["kernels"])
        return g["loss"], g["counts"]

    def _eager_step(self, batch: Any, on_device: bool = False) -> tuple[LossOutput, dict[str, Tensor]]:
        inputs, targets = batch if on_device else self._to_device(batch)
        self.tokens_per_micro = inputs.numel()
        with self._activation_ctx():
            out = self.model(inputs)
            loss = self.loss_fn(out.pred, targets, out.aux)
        (loss.total / self.config.grad_accum_steps).backward()
        # (packed: the values are views of one flat tensor, so that a step's micro-batches are summed with one launch)
        counts = RouterCounts.pack(router_counts(self.model.backbone, out.aux)) if self.model.training else {}
        # hand back values only: a live grad_fn would keep this step's autograd nodes alive
        loss = LossOutput(total=loss.total.detach(), components={k: v.detach() for k, v in loss.components.items()})
        return loss, counts

    # ----------------------------------------------------------------- optimizer step
    @torch.no_grad()
    def clip_grad_norm(self, max_norm: float) -> Tensor:
        """Global L2 clip on the flat gradient buffer (one reduction, one scale)."""

        if self.zero:
            # every rank holds the reduced gradient of its own range only: partial sums of squares, one scalar reduce
            lo, hi = self.optimizer.owned_range()
            own = self.arena.grad[lo:hi]
            sq = torch.linalg.vector_norm(own).square()
            torch.distributed.all_reduce(sq)
            norm = sq.sqrt()
            own.mul_((max_norm / (norm + 1e-6)).clamp(max=1.0))
            return norm
        norm = torch.linalg.vector_norm(self.arena.grad)
        scale = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        self.arena.grad.mul_(scale)
        return norm

    def _probe_peer_status(self) -> None:
        """Queue an asynchronous read-back of the status word behind this step's collectives."""

        st = self.peer_status
        if st is None:
            return
        if st.is_cuda:
            if self._status_host is None:
                self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._status_host.copy_(st, non_blocking=True)
            self._status_event = torch.cuda.Event()
            self._status_event.record()
        else:
            self._status_host = st

    def check_peer_status(self) -> None:
        """Raise ``PeerTimeout`` if a collective of an earlier optimizer step gave up waiting for a peer.

        Without this the step would carry on with unreduced local gradients and stale parameters, and the replicas
        would silently diverge. The value inspected is the one queued by the previous ``update_weights`` (already
        complete by the time the next step's micro-batches have been submitted), so the check costs no extra stall.
        """

        if self._status_host is None:
            return
        if self._status_event is not None:
            self._status_event.synchronize()
            self._status_event = None
        code = int(self._status_host.item())
        if code:
            from nestor_b200.parallel.symm import PeerTimeout
            if self.peer_status is not None:
                self.peer_status.zero_()
            self._status_host = None
            raise PeerTimeout(f"rank {self.rank}: an in-kernel collective reported status {code} at step "
                              f"{self.global_step} (a bounded wait on a peer gave up); gradients or parameters of "
                              "that step are not synchronised")
        if self.peer_status is not None and not self.peer_status.is_cuda:
            self._status_host = None

    def _mark(self, name: str) -> None:
        """Phase boundary of ``update_weights`` (CUDA events, only while ``phase_events`` is a list)."""

        if self.nvtx and self.device.type == "cuda":
            if name != "start":
                torch.cuda.nvtx.range_pop()
            if name != "rest":
                nxt = {"start": "grad_reduce", "grad_reduce": "clip", "clip": "optimizer", "optimizer": "param_push",
                       "param_push": "rest"}[name]
                torch.cuda.nvtx.range_push(f"update/{nxt}")
        if self.phase_events is not None and self.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_events.append((name, ev))

    def phase_times_ms(self) -> dict[str, float]:
        """Device time of each phase of the last ``update_weights`` recorded with ``phase_events = []``."""

        ev = self.phase_events or []
        if ev:
            ev[-1][1].synchronize()
        return {ev[i + 1][0]: ev[i][1].elapsed_time(ev[i + 1][1]) for i in range(len(ev) - 1)}

    def update_weights(self, window_counts: dict[str, Tensor]) -> Tensor | None:
        self.check_peer_status()
        self._mark("start")
        if self.zero:
            self.reducer.reduce_scatter(*self.optimizer.owned_range())
        else:
            self.reducer.reduce()
        self._mark("grad_reduce")
        norm = None
        if self.config.max_grad_norm is not None:
            norm = self.clip_grad_norm(self.config.max_grad_norm)
        self._mark("clip")
        if _env_flag("NESTOR_DEBUG_GRAD") and self.global_step < 5 and is_main_process():
            g = self.arena.grad
            self.logger.info("[grad] step %d norm=%s finite=%s absmax=%.3e", self.global_step,
                             None if norm is None else f"{norm.item():.4e}",
                             bool(torch.isfinite(g).all().item()), g.abs().max().item())
        self.optimizer.step()
        self._mark("optimizer")
        if self.param_push is not None:
            # each rank stores the range it owns into every replica, itself included (fp32 master + bf16 compute
            # copy); the ranges tile the arena, so this is also the refresh of the whole compute copy
            self.param_push.run(*self.optimizer.owned_range())
        else:
            self.arena.refresh_compute()
        self._mark("param_push")
        self.arena.zero_grad()
        if self.ema is not None:
            if self.masters_sharded:      # only this rank's range of the master is current; the shadow is sharded the same way
                lo, hi = self.optimizer.owned_range()
                self.ema["flat"][lo:hi].lerp_(self.arena.master[lo:hi], 1.0 - self.ema_decay)
            else:
                self.ema["flat"].lerp_(self.arena.master, 1.0 - self.ema_decay)
        if self.scheduler is not None:
            self.scheduler.step()
        apply_bias_updates(self.model.backbone, window_counts, global_counts=self.global_counts)
        if self.world > 1 and not self.global_counts and _env_flag("NESTOR_DDP_BROADCAST_BUFFERS", "1"):
            self.reducer.sync_buffers(self.model)  # rank-0 statistics win, as with DDP buffer broadcast
        self._mark("rest")
        self._probe_peer_status()
        return norm

    # --------------------------------------------------------------------------- loop
    def train(self) -> None:
        cfg = self.config
        self.model.train()
        log_every = int(os.environ.get("NESTOR_LOG_FREQ") or cfg.log_frequency)
        peak = float(os.environ.get("NESTOR_MFU_PEAK_TFLOPS", "2250")) * 1e12
        flops_tok = float(os.environ.get("NESTOR_MFU_FLOPS_PER_TOKEN", "0")) or train_flops_per_token(
            self.model.config, self._seq_len())
        pinned = float(os.environ.get("NESTOR_MFU_FLOPS_PER_STEP", "0") or 0)
        if pinned > 0:
            # FLOPs of one forward + backward micro-batch of one rank, as the reference takes it
            # (nestor/train/trainer.py:587-603); divided by the micro-batch's tokens once they are known
            loader_cfg = getattr(cfg, "train_dataloader", None)
            per_rank = max(1, int(getattr(loader_cfg, "batch_size", self.world)) // self.world)
            flops_tok = pinned / max(1, per_rank * self._seq_len())
            self.logger.info("[MFU] flops/microbatch pinned via env: %.3e", pinned)
        if _env_flag("NESTOR_MFU_CALIBRATE"):
            # cross-check of the analytic count against FlopCounterMode on the PyTorch statement of the model
            from nestor_b200.train.flops import calibrate_flops
            cal = calibrate_flops(self.model, seq_len=int(os.environ.get("NESTOR_MFU_CALIB_SEQ", "128")),
                                  batch=int(os.environ.get("NESTOR_MFU_CALIB_BATCH", "1")))
            self.logger.info("[MFU] forward FLOPs/token at the calibration length: counted %.4e, analytic %.4e (ratio %.4f)",
                             cal["counted"], cal["analytic"], cal["ratio"])
            flops_tok *= cal["ratio"]
        profile = _env_flag("NESTOR_TRAIN_PROFILE")
        tprof, tp_start, tp_n = None, int(os.environ.get("NESTOR_TORCH_PROFILE_START", "12")), \
            int(os.environ.get("NESTOR_TORCH_PROFILE_STEPS", "10"))
        if _env_flag("NESTOR_TORCH_PROFILE"):
            from torch.profiler import ProfilerActivity, profile as torch_profile
            tprof = torch_profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA])
        tp_active = False
        try:
            batches_per_epoch = len(self.train_loader)
        except TypeError:
            batches_per_epoch = 0
        skip = 0
        if self.global_step > 0 and batches_per_epoch > 0 and not _env_flag("NESTOR_RESUME_NO_FASTFORWARD"):
            skip = (self.global_step * cfg.grad_accum_steps) % batches_per_epoch
            if skip:
                self.logger.info("[resume] fast-forwarding %d micro-batches (step %d x accum %d, %d per epoch)",
                                 skip, self.global_step, cfg.grad_accum_steps, batches_per_epoch)
        self.logger.info("Starting training for %d steps", cfg.max_steps)
        loss_acc: Tensor | None = None
        comp_acc: dict[str, Tensor] = {}
        counts_acc: dict[str, Tensor] = {}
        micro = 0
        steps_done, t_steady, t_win, win_steps = 0, None, time.monotonic(), 0
        t_prev = time.perf_counter()
        while self.global_step < cfg.max_steps:
            if hasattr(self.train_loader, "set_epoch"):
                self.train_loader.set_epoch(self.epoch)
            for batch in self.train_loader:
                if skip > 0:
                    skip -= 1
                    continue
                if self.global_step >= cfg.max_steps:
                    break
                if tprof is not None:
                    if steps_done == tp_start and not tp_active:
                        tprof.__enter__()
                        tp_active = True
                    elif tp_active and steps_done >= tp_start + tp_n:
                        tprof.__exit__(None, None, None)
                        tp_active, done = False, tprof
                        tprof = None
                        if is_main_process():
                            self.logger.info("[TORCHPROF] top ops:\n%s",
                                             done.key_averages().table(sort_by="cuda_time_total", row_limit=25))
                t_data = time.perf_counter() - t_prev
                t0 = time.perf_counter()
                loss, counts = self.train_step(batch)
                if profile and self.device.type == "cuda":
                    torch.cuda.synchronize()
                t_fb = time.perf_counter() - t0
                if (self.global_step + 1) % log_every == 0:
                    d = loss.total.detach()
                    loss_acc = d if loss_acc is None else loss_acc + d
                    for k, v in loss.components.items():
                        comp_acc[k] = v.detach() if k not in comp_acc else comp_acc[k] + v.detach()
                counts_acc = add_router_counts(counts_acc, counts)
                micro += 1
                if micro < cfg.grad_accum_steps:
                    t_prev = time.perf_counter()
                    continue
                t1 = time.perf_counter()
                self.update_weights(counts_acc)
                if profile:
                    if self.device.type == "cuda":
                        torch.cuda.synchronize()
                    if is_main_process() and steps_done >= 5:
                        self.logger.info("[TPROF] data=%.3f fwd_bwd=%.3f update=%.3f", t_data, t_fb,
                                         time.perf_counter() - t1)
                self.global_step += 1
                self._bound_runahead()
                steps_done += 1
                if steps_done == 1:
                    if self.device.type == "cuda":
                        torch.cuda.synchronize()
                    t_steady = t_win = time.monotonic()
                    win_steps = steps_done
                if self.global_step % log_every == 0:
                    now = time.monotonic()
                    metrics = {"loss": (loss_acc.item() / micro) if loss_acc is not None else 0.0}
                    for k, v in comp_acc.items():
                        metrics[k] = v.item() / micro
                    if self.scheduler is not None:
                        lrs = self.scheduler.get_last_lr()
                        metrics["lr"], metrics["lr_max"] = lrs[0], max(lrs)
                    dt = (now - t_win) / max(steps_done - win_steps, 1)
                    t_win, win_steps = now, steps_done
                    self._add_mfu(metrics, flops_tok, peak, dt, now, steps_done, t_steady)
                    log_metrics(self.logger, metrics, self.global_step, prefix="train/")
                loss_acc, comp_acc, counts_acc, micro = None, {}, {}, 0
                eval_every = int(os.environ.get("NESTOR_EVAL_FREQ") or cfg.eval_frequency)
                if self.eval_suite is not None and self.global_step % eval_every == 0:
                    self.run_eval()
                if self.global_step % cfg.checkpoint_frequency == 0:
                    self.save_checkpoint()
                    self.submit_eval_jobs()
                t_prev = time.perf_counter()
            self.epoch += 1
        self.save_checkpoint(final=True)
        self.logger.info("Training complete!")

    def _bound_runahead(self) -> None:
        if self.runahead < 0 or self.device.type != "cuda":
            return
        if self.runahead == 0:
            torch.cuda.synchronize()
            self.check_peer_status()
            return
        ev = torch.cuda.Event()
        ev.record()
        self._step_events.append(ev)
        if len(self._step_events) > self.runahead:
            self._step_events.popleft().synchronize()

    def _add_mfu(self, metrics: dict, flops_tok: float, peak: float, dt: float, now: float,
                 steps: int, t_steady: float | None) -> None:
        if not self.tokens_per_micro:
            return
        tokens_step = self.tokens_per_micro * self.config.grad_accum_steps * self.world
        flops_step_gpu = flops_tok * tokens_step / self.world
        metrics["sec_per_step"] = dt
        metrics["tokens_per_sec"] = tokens_step / dt if dt > 0 else 0.0
        metrics["samples_per_sec"] = metrics["tokens_per_sec"] / max(1, self.tokens_per_micro // max(1, self._seq_len()))
        metrics["tflops_per_gpu"] = flops_step_gpu / dt / 1e12 if dt > 0 else 0.0
        metrics["mfu_instant"] = flops_step_gpu / dt / peak if dt > 0 else 0.0
        if t_steady is not None and steps > 1:
            metrics["mfu_runavg_excl_init"] = flops_step_gpu * (steps - 1) / max(now - t_steady, 1e-9) / peak
        metrics["mfu_runavg_incl_init"] = flops_step_gpu * steps / max(now - PROCESS_START, 1e-9) / peak
        if self.device.type == "cuda":
            metrics["mem_peak_alloc_gib"] = torch.cuda.max_memory_allocated() / 2**30
            metrics["mem_peak_reserved_gib"] = torch.cuda.max_memory_reserved() / 2**30

    def _seq_len(self) -> int:
        return int(getattr(self.config.train_dataset, "block_size", 0) or 1)

    # ------------------------------------------------------------------ eval / ckpt
    def run_eval(self) -> None:
        results = self.eval_suite.run(self.model)
        if is_main_process() and self.run_dir is not None:
            import json
            out = self.run_dir / "evals"
            out.mkdir(parents=True, exist_ok=True)
            (out / f"eval_step_{self.global_step:08d}.json").write_text(json.dumps(results, indent=2))
        log_metrics(self.logger, {f"{k}": v for k, v in _flatten(results).items()}, self.global_step, prefix="eval/")
        self.model.train()

    def checkpoint_path(self, final: bool = False) -> Path | None:
        if self.run_dir is None or self.config.checkpoint_dir is None:
            return None
        d = self.run_dir / self.config.checkpoint_dir
        return d / ("model_final.pt" if final else f"model_{self.global_step:08d}.pt")

    @torch.no_grad()
    def gather_masters(self) -> None:
        """Bring the fp32 masters (and the EMA shadow) of every range up to date from their owners.

        With the bf16-only parameter push each rank's fp32 state is current for its own arena range only; everything
        that reads the whole fp32 model (checkpoints, weight comparisons across ranks) calls this first. All ranks
        must call it together."""

        if not self.masters_sharded:
            return
        from nestor_b200.parallel.symm import gather_ranges
        gather_ranges(self.arena.master, self.optimizer.owner_cuts)
        if self.ema is not None:
            gather_ranges(self.ema["flat"], self.optimizer.owner_cuts)

    def save_checkpoint(self, final: bool = False) -> None:
        path = self.checkpoint_path(final)
        if path is None:
            return
        self.gather_masters()
        ema = None
        if self.ema is not None:
            ema = {s.name: self.ema["flat"][s.offset : s.offset + s.numel].view(s.shape).cpu().clone()
                   for s in self.arena.slots.values()}
        ckpt.save_checkpoint(path, self.model, self.optimizer, self.scheduler, step=self.global_step,
                             epoch=self.epoch, ema=ema)
        if is_main_process():
            self.logger.info("saved %s", path)
        # Only rank 0 writes the file. The others wait here, on the process group's long timeout, instead of inside
        # the next step's in-kernel barrier, whose wait budget is seconds.
        barrier()

    def resume(self, path: Path, *, strict: bool = True, allow_partial: bool = False) -> None:
        state = ckpt.load_checkpoint(path, self.model, self.optimizer if strict else None,
                                     self.scheduler if strict else None, strict=strict, allow_partial=allow_partial)
        self.arena.refresh_compute()
        if strict:
            self.global_step, self.epoch = int(state.get("step", 0)), int(state.get("epoch", 0))
            if self.ema is not None and state.get("ema"):
                for s in self.arena.slots.values():
                    if s.name in state["ema"]:
                        self.ema["flat"][s.offset : s.offset + s.numel].copy_(state["ema"][s.name].reshape(-1))
        self.logger.info("%s from %s at step %d", "resumed" if strict else "initialised", path, self.global_step)

    def submit_eval_jobs(self) -> None:
        """``sbatch`` the configured evaluation scripts against the checkpoint just written (rank 0)."""

        scripts = self.config.eval_submit_scripts
        path = self.checkpoint_path()
        if not scripts or not is_main_process() or path is None:
            return
        for script, every in scripts:
            if every and self.global_step % every:
                continue
            try:
                subprocess.run(["sbatch", str(script), str(path)], check=False, capture_output=True, timeout=60)
            except (FileNotFoundError, subprocess.TimeoutExpired) as exc:
                self.logger.warning("eval submission failed for %s: %s", script, exc)


def _flatten(d: dict, prefix: str = "") -> dict[str, Any]:
    out = {}
    for k, v in d.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(_flatten(v, key + "/"))
        elif isinstance(v, (int, float)):
            out[key] = v
    return out
