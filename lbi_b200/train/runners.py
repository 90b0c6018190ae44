"""Training loops for the dense and the LBI variant (reference train/runners.py:104-552).

Both variants share one loop; they differ in the *stepper* that turns a batch into an optimizer step:

* dense                      forward, ``loss.backward()``, clip, AdamW
* lbi / scan, reference_scan, autograd   ``forward_with_cache`` (graph cut at the interface states for the scan
                             engines), the chosen ``ADEngine``, clip, AdamW
* lbi / fast                 ``FastLBIEngine.step``: structured kernels end to end, fused clip + AdamW on flat buffers

Artefacts, metric rows, evaluation cadence, ablation splits, checkpoint cadence and the RNG contract (model init
under ``seed``, corpora ``seed+11/+29``, train/eval generators ``seed+101/+202``, per-evaluation generator
``seed+202+11*step``, ablation generator ``seed+303+17*step+idx``) follow the reference.  Unlike the reference the
loop reads the loss back from the device only on logging steps, so steps queue without a host sync in between.
"""
from __future__ import annotations

import json
import math
import os
import time
from contextlib import nullcontext
from pathlib import Path
from typing import Any, Dict

import torch

from ..backward import AutogradEngine, ReferenceScanEngine, ScanADEngine
from ..models.lbi_language_model import LBILanguageModel
from .checkpointing import maybe_restore_training_state, save_checkpoint
from .config import DENSE_VARIANT, LBI_VARIANT, LEGACY_DENSE_REGIME, LEGACY_LBI_REGIME, LBITrainingConfig
from .data import build_corpora, sample_batch_any
from .eval import evaluate_native, evaluate_reference, next_token_loss, resolve_eval_message_ablation_modes
from .metrics import log_row, write_run_metadata
from .model_builders import build_dense_model, build_lbi_model
from ..utils.failure import FaultInjector, Heartbeat, check_kernel_status

_EVAL_MESSAGE_ABLATION_MODES = ("zero_all", "noise", "mask")


def _lbi_cache_state_norm(cache: dict[str, Any]) -> float:
    states = cache.get("states", [])
    if not states:
        return 0.0
    return float(torch.stack([s.detach().float().norm(dim=-1).mean() for s in states]).mean().item())


def _resolve_device(cfg: LBITrainingConfig) -> torch.device:
    if cfg.device == "cpu":
        return torch.device("cpu")
    local_rank = int(os.environ.get("LOCAL_RANK", "0")) if _world_size() > 1 else None
    if cfg.device == "cuda":
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA requested but not available.")
        return torch.device("cuda") if local_rank is None else torch.device("cuda", local_rank)
    if torch.cuda.is_available():
        return torch.device("cuda") if local_rank is None else torch.device("cuda", local_rank)
    return torch.device("cpu")


def _world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def _make_comm(device: torch.device):
    """Communicator of a multi-process launch (torchrun environment): peer-memory kernels on GPUs unless
    LBI_B200_COMM=collective, library collectives otherwise and on CPU ranks; None for a single process."""
    if _world_size() <= 1:
        return None
    from ..parallel.comm import CollectiveComm, init_distributed_from_env

    init_distributed_from_env(device.type)
    if device.type == "cuda" and os.environ.get("LBI_B200_COMM", "symm") != "collective":
        try:
            from ..parallel.symm import SymmComm

            return SymmComm()
        except Exception as exc:  # no peer access between the GPUs of this job
            print(f"[lbi_b200] peer-memory plane unavailable ({exc}); using library collectives", flush=True)
    return CollectiveComm()


def _autocast_context(cfg: LBITrainingConfig, device: torch.device):
    if cfg.dtype == "bfloat16":
        return torch.autocast(device_type=device.type, dtype=torch.bfloat16)
    return nullcontext()


def _lr_multiplier(cfg: LBITrainingConfig, step: int) -> float:
    """0 at step 0, linear warm-up, then constant / cosine / linear decay towards ``min_lr_ratio``."""
    if step <= 0:
        return 0.0
    if cfg.warmup_steps > 0 and step <= cfg.warmup_steps:
        return float(step) / float(cfg.warmup_steps)
    if cfg.lr_schedule == "constant":
        return 1.0
    progress = min(1.0, max(0.0, float(step - cfg.warmup_steps) / float(max(1, cfg.steps - cfg.warmup_steps))))
    if cfg.lr_schedule == "linear":
        decay = 1.0 - progress
    elif cfg.lr_schedule == "cosine":
        decay = 0.5 * (1.0 + math.cos(math.pi * progress))
    else:
        raise ValueError(f"unsupported lr_schedule: {cfg.lr_schedule}")
    return cfg.min_lr_ratio + (1.0 - cfg.min_lr_ratio) * decay


def _scheduled_lr(cfg: LBITrainingConfig, step: int) -> float:
    return float(cfg.lr_model * _lr_multiplier(cfg, step))


def _set_optimizer_lr(optimizer, lr: float) -> None:
    for group in optimizer.param_groups:
        group["lr"] = lr


# ----------------------------------------------------------------------------------------------------- steppers
class _AutogradStepper:
    """Dense model, or an LBI model driven by one of the autograd-based engines."""

    def __init__(self, cfg, model, device, engine, lbi: bool) -> None:
        self.cfg, self.model, self.device, self.engine, self.lbi = cfg, model, device, engine, lbi
        self.optimizer = torch.optim.AdamW(model.parameters(), lr=cfg.lr_model, weight_decay=cfg.weight_decay)
        self.diagnostics: dict[str, Any] = {}
        self.cache: dict[str, Any] | None = None

    def step(self, xb, yb, lr: float, want_jacobian_stats: bool = False) -> torch.Tensor:
        cfg, model = self.cfg, self.model
        _set_optimizer_lr(self.optimizer, lr)
        engine = self.engine
        if self.lbi and isinstance(engine, ScanADEngine):
            engine = ScanADEngine.from_config(cfg, compute_interface_jacobian_stats=want_jacobian_stats)
        with _autocast_context(cfg, self.device):
            if self.lbi:
                logits, cache = model.forward_with_cache(xb, detach_states=getattr(engine, "requires_detached_states", False))
            else:
                logits, cache = model(xb), None
        loss = next_token_loss(logits, yb)
        result = engine.backward(model=model, loss=loss, cache=cache)
        self.diagnostics, self.cache = result.diagnostics, cache
        if cfg.grad_clip > 0:
            torch.nn.utils.clip_grad_norm_(model.parameters(), cfg.grad_clip)
        self.optimizer.step()
        return loss.detach()

    def message_norm(self) -> float | str:
        return _lbi_cache_state_norm(self.cache) if (self.lbi and self.cache is not None) else ""


class _FlatOptimizerView:
    """Presents the flat fused optimizer through the ``state_dict`` / ``load_state_dict`` protocol of torch.optim."""

    def __init__(self, engine, cfg) -> None:
        self.engine, self.cfg = engine, cfg
        self.param_groups = [{"lr": cfg.lr_model}]

    def _order(self) -> list[str]:
        return [name for name, p in self.engine.model.named_parameters() if p.requires_grad]

    def state_dict(self) -> dict:
        """Consolidated over ranks: every rank must call this (the moment shards are all-gathered)."""
        e = self.engine
        hyper = {"lr": self.param_groups[0]["lr"], "betas": tuple(e.betas), "eps": e.eps, "weight_decay": e.weight_decay,
                 "amsgrad": False, "maximize": False, "foreach": None, "capturable": False, "differentiable": False,
                 "fused": None}
        return e.flat.state_dict_like_torch(self._order(), hyper, comm=getattr(e, "comm", None))

    def load_state_dict(self, sd: dict) -> None:
        self.engine.flat.load_state_dict_like_torch(sd, self._order())


class _FrozenState:
    """An optimizer state dict that was already consolidated (checkpoint writer of multi-process runs)."""

    def __init__(self, sd: dict) -> None:
        self._sd = sd

    def state_dict(self) -> dict:
        return self._sd


class _FastStepper:
    def __init__(self, cfg, model, device) -> None:
        from ..parallel import FastLBIEngine

        act = torch.bfloat16 if cfg.dtype == "bfloat16" else torch.float32
        self.engine = FastLBIEngine(model, lr=cfg.lr_model, weight_decay=cfg.weight_decay, grad_clip=cfg.grad_clip,
                                    basis_chunk=max(1, cfg.jacobian_basis_chunk), act_dtype=act, comm=_make_comm(device))
        self.optimizer = _FlatOptimizerView(self.engine, cfg)
        self.diagnostics: dict[str, Any] = {"interface_scan_rms": 0.0}
        self.cfg = cfg

    def step(self, xb, yb, lr: float, want_jacobian_stats: bool = False) -> torch.Tensor:
        self.optimizer.param_groups[0]["lr"] = lr
        loss = self.engine.step(xb, yb, lr=lr)
        if want_jacobian_stats and self.engine.last.get("jacobians") is not None:
            from ..backward.suffix_scan import interface_state_jacobian_t_stats

            jac = self.engine.last["jacobians"]
            mats = [jac[:, k] for k in range(jac.shape[1] - 1)]
            if mats:
                self.diagnostics["interface_jacobian_stats"] = interface_state_jacobian_t_stats(
                    mats, include_suffix=bool(self.cfg.log_interface_jacobian_suffix))
        return loss

    def message_norm(self) -> float | str:
        return ""


class _DenseFastStepper:
    """The dense model on the structured kernels without autograd (``--variants dense --backward-engine fast``)."""

    def __init__(self, cfg, model, device) -> None:
        from ..parallel import DenseFastEngine

        act = torch.bfloat16 if cfg.dtype == "bfloat16" else torch.float32
        self.engine = DenseFastEngine(model, lr=cfg.lr_model, weight_decay=cfg.weight_decay, grad_clip=cfg.grad_clip, act_dtype=act)
        self.optimizer = _FlatOptimizerView(self.engine, cfg)
        self.diagnostics: dict[str, Any] = {}

    def step(self, xb, yb, lr: float, want_jacobian_stats: bool = False) -> torch.Tensor:
        self.optimizer.param_groups[0]["lr"] = lr
        return self.engine.step(xb, yb, lr=lr)

    def message_norm(self) -> float | str:
        return ""


def _build_stepper(cfg, model, device, variant: str):
    if _world_size() > 1 and (variant == DENSE_VARIANT or cfg.backward_engine != "fast"):
        raise ValueError("multi-process training is region-parallel: it needs the lbi variant with --backward-engine fast")
    if variant == DENSE_VARIANT:
        if cfg.backward_engine == "fast":
            return _DenseFastStepper(cfg, model, device)
        return _AutogradStepper(cfg, model, device, AutogradEngine(), lbi=False)
    if cfg.backward_engine == "fast":
        return _FastStepper(cfg, model, device)
    engine = {"scan": ScanADEngine.from_config(cfg), "reference_scan": ReferenceScanEngine(), "autograd": AutogradEngine()}[cfg.backward_engine]
    return _AutogradStepper(cfg, model, device, engine, lbi=True)


# ----------------------------------------------------------------------------------------------------- the loop
def _run_training(cfg: LBITrainingConfig, *, run_dir: Path, variant: str) -> Dict[str, Any]:
    """Runs the loop with this rank's liveness published from a background thread (multi-process runs), so that a long
    evaluation, a consolidated checkpoint save on rank 0 or a slow step never looks like a dead rank to the peers.  A rank
    that hangs inside a step is caught by its own step watchdog; one that raises reports through ``fail/<rank>``."""
    heartbeat, progress = None, {"step": -1}
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        heartbeat = Heartbeat.from_process_group(stale_after_s=float(os.environ.get("LBI_B200_HEARTBEAT_STALE_S", "120")))
        heartbeat.start_background(interval_s=float(os.environ.get("LBI_B200_HEARTBEAT_EVERY_S", "1.0")),
                                   step_fn=lambda: progress["step"])
    try:
        return _run_training_loop(cfg, run_dir=run_dir, variant=variant, heartbeat=heartbeat, progress=progress)
    finally:
        if heartbeat is not None:
            heartbeat.stop()


def _run_training_loop(cfg: LBITrainingConfig, *, run_dir: Path, variant: str, heartbeat, progress: dict) -> Dict[str, Any]:
    is_lbi = variant == LBI_VARIANT
    legacy_regime = LEGACY_LBI_REGIME if is_lbi else LEGACY_DENSE_REGIME
    device = _resolve_device(cfg)
    torch.manual_seed(cfg.seed)
    if device.type == "cuda":
        torch.cuda.manual_seed_all(cfg.seed)
    model = (build_lbi_model(cfg) if is_lbi else build_dense_model(cfg)).to(device=device, dtype=torch.float32)
    if is_lbi and not isinstance(model, LBILanguageModel):
        raise TypeError("LBI training requires LBILanguageModel")
    stepper = _build_stepper(cfg, model, device, variant)
    is_main = int(os.environ.get("RANK", "0")) == 0 or _world_size() <= 1   # rank 0 owns every file of the run
    distributed = _world_size() > 1
    train_corpus, val_corpus = build_corpora(cfg, device=device)
    if is_main:
        write_run_metadata(cfg=cfg, run_dir=run_dir, model=model, train_corpus=train_corpus, val_corpus=val_corpus)
    log_row_main = log_row if is_main else (lambda *a, **k: None)

    gen_device = device if cfg.data_mode == "synthetic" else torch.device("cpu")
    train_gen = torch.Generator(device=gen_device)
    train_gen.manual_seed(cfg.seed + 101)
    eval_gen = torch.Generator(device=gen_device)
    eval_gen.manual_seed(cfg.seed + 202)
    restore = maybe_restore_training_state(
        mode="resume" if cfg.resume_from else "init", load_from=cfg.resume_from or cfg.init_from, regime=variant, model=model,
        optimizer=stepper.optimizer, device=device, train_generator=train_gen, eval_generator=eval_gen,
    )
    if isinstance(stepper, (_FastStepper, _DenseFastStepper)):
        stepper.engine.flat.refresh_shadow()  # weights may just have been replaced by a checkpoint

    final_train = final_val = float("nan")
    best_val, best_val_step = float(restore["best_val_ce_loss"]), int(restore["best_val_step"])
    best_path = latest_path = ""
    final_ablations: Dict[str, float] = {}
    final_jac_stats: Dict[str, float] = {}
    tokens_per_step = int(cfg.batch_size * cfg.seq_len)
    total_tokens = int(restore["tokens_seen"])
    start_step = int(restore["start_step"])
    scan_rms = 0.0

    def checkpoint_extra(**more) -> dict:
        extra = {"variant": variant, "regime": variant, "legacy_regime": legacy_regime, "train_ce_loss": final_train}
        if is_lbi:
            extra.update(owned_lbi_model=True, interface_scan_rms=scan_rms, interface_jacobian_mode=cfg.interface_jacobian_mode,
                         jacobian_basis_chunk=cfg.jacobian_basis_chunk, interface_jacobian_stats=final_jac_stats,
                         region_axis=cfg.region_axis, backward_engine=cfg.backward_engine)
        extra.update(more)
        return extra

    def save(filename: str, step: int, **more) -> str:
        if distributed:  # all ranks: complete the fp32 master copy and consolidate the optimizer shards
            stepper.engine.sync_master_params()
            optimizer = _FrozenState(stepper.optimizer.state_dict())
            if not is_main:
                return ""
        else:
            optimizer = stepper.optimizer
        return str(save_checkpoint(
            run_dir=run_dir, filename=filename, model=model, optimizer=optimizer, cfg=cfg, device=device,
            train_generator=train_gen, eval_generator=eval_gen, step=step, tokens_seen=total_tokens,
            best_val_ce_loss=best_val, best_val_step=best_val_step, extra=checkpoint_extra(**more)))

    injector = FaultInjector(rank=int(os.environ.get("RANK", "0")))
    window_t0, window_steps = time.perf_counter(), 0
    for step in range(start_step + 1, cfg.steps + 1):
        # between steps: nothing of this rank is in flight, so faults are injected and peers are checked here
        injector.at_step(step, heartbeat=heartbeat, checkpoint_path=Path(latest_path) if latest_path else None)
        progress["step"] = step
        if heartbeat is not None:
            heartbeat.beat(step)
            heartbeat.check_peers()
        model.train()
        xb, yb = sample_batch_any(cfg=cfg, corpus=train_corpus, batch_size=cfg.batch_size, generator=train_gen, device=device)
        want_stats = is_lbi and cfg.log_interface_jacobian_every > 0 and (
            step % cfg.log_interface_jacobian_every == 0 or step == 1 or step == cfg.steps)
        loss = stepper.step(xb, yb, _scheduled_lr(cfg, step), want_jacobian_stats=want_stats)
        window_steps += 1
        total_tokens = int(step * tokens_per_step)
        jac_stats = stepper.diagnostics.get("interface_jacobian_stats") if is_lbi else None
        if jac_stats is not None:
            final_jac_stats = dict(jac_stats)
        logging = (step % cfg.log_every) == 0 or step == 1 or want_stats or step == cfg.steps
        if logging:
            final_train = float(loss.item())  # the only device read of a training step
            if device.type == "cuda":
                check_kernel_status(loss)
            elapsed = max(1e-9, time.perf_counter() - window_t0)
            scan_rms = float(stepper.diagnostics.get("interface_scan_rms", 0.0)) if is_lbi else 0.0
            row = {"step": step, "tokens_seen": total_tokens, "split": "train", "ce_loss": final_train,
                   "message_norm": stepper.message_norm() if is_lbi else "", "scan_align": scan_rms if is_lbi else "",
                   "tokens_per_s": float(window_steps * tokens_per_step / elapsed), "wall_time_s": float(elapsed / window_steps)}
            if jac_stats is not None:
                row.update(jac_stats)
            if (step % cfg.log_every) == 0 or step == 1 or want_stats:
                log_row_main(run_dir, row)
            window_t0, window_steps = time.perf_counter(), 0

        if (step % cfg.eval_every) == 0 or step == cfg.steps:
            if distributed:
                stepper.engine.sync_master_params()  # evaluation runs replicated on the fp32 master weights
            if is_lbi:
                step_gen = torch.Generator(device=gen_device)
                step_gen.manual_seed(cfg.seed + 202 + step * 11)
                val = evaluate_native(cfg=cfg, model=model, val_corpus=val_corpus, eval_batches=cfg.eval_batches, generator=step_gen,
                                      device=device, sample_batch_fn=sample_batch_any, autocast_context_fn=_autocast_context)
            else:
                val = evaluate_reference(cfg=cfg, model=model, val_corpus=val_corpus, eval_batches=cfg.eval_batches, generator=eval_gen,
                                         device=device, sample_batch_fn=sample_batch_any, autocast_context_fn=_autocast_context)
            final_val = float(val["ce_loss"])
            if final_val < best_val:
                best_val, best_val_step = final_val, step
                if cfg.save_checkpoints:
                    best_path = save("best.pt", step, val_ce_loss=final_val, is_best=True)
            blank = {"step": step, "tokens_seen": total_tokens, "message_norm": "", "scan_align": "", "tokens_per_s": 0.0, "wall_time_s": 0.0}
            log_row_main(run_dir, {**blank, "split": "val", "ce_loss": final_val})
            if is_lbi:
                modes = resolve_eval_message_ablation_modes(cfg, ablation_modes=_EVAL_MESSAGE_ABLATION_MODES)
                for idx, mode in enumerate(modes):
                    batch_gen = torch.Generator(device=gen_device)
                    batch_gen.manual_seed(cfg.seed + 202 + step * 11)
                    noise_gen = torch.Generator(device=device)
                    noise_gen.manual_seed(cfg.seed + 303 + step * 17 + idx)
                    ablated = evaluate_native(cfg=cfg, model=model, val_corpus=val_corpus, eval_batches=cfg.eval_batches,
                                              generator=batch_gen, device=device, sample_batch_fn=sample_batch_any,
                                              autocast_context_fn=_autocast_context, message_ablation=mode,
                                              ablation_generator=noise_gen)
                    final_ablations[f"val_{mode}"] = float(ablated["ce_loss"])
                    log_row_main(run_dir, {**blank, "split": f"val_{mode}", "ce_loss": float(ablated["ce_loss"])})
            window_t0, window_steps = time.perf_counter(), 0

        if cfg.save_checkpoints and ((step % cfg.save_every) == 0 or step == cfg.steps):
            latest_path = save("latest.pt", step)

    summary: Dict[str, Any] = {
        "variant": variant, "regime": variant, "legacy_regime": legacy_regime, "task": cfg.task, "steps": int(cfg.steps),
        "start_step": start_step, "final_train_ce_loss": final_train, "final_val_ce_loss": final_val,
        "best_val_ce_loss": best_val, "best_val_step": best_val_step, "train_tokens_per_step": tokens_per_step,
        "total_train_tokens": total_tokens, "save_checkpoints": bool(cfg.save_checkpoints),
        "best_checkpoint_path": best_path, "latest_checkpoint_path": latest_path,
        "resumed_from": str(restore["checkpoint_path"]) if cfg.resume_from else "",
        "initialized_from": str(restore["checkpoint_path"]) if cfg.init_from else "", "run_dir": str(run_dir),
    }
    if is_lbi:
        summary.update(
            interface_jacobian_mode=cfg.interface_jacobian_mode, jacobian_basis_chunk=int(cfg.jacobian_basis_chunk),
            log_interface_jacobian_every=int(cfg.log_interface_jacobian_every),
            log_interface_jacobian_suffix=bool(cfg.log_interface_jacobian_suffix),
            final_interface_jacobian_stats=final_jac_stats, final_eval_message_ablations=final_ablations,
            owned_lbi_model=True, region_axis=cfg.region_axis, backward_engine=cfg.backward_engine,
        )
    if is_main:
        (run_dir / "summary.json").write_text(json.dumps(summary, indent=2, sort_keys=True), encoding="utf-8")
    return summary


def run_dense_training(cfg: LBITrainingConfig, *, run_dir: Path) -> Dict[str, Any]:
    return _run_training(cfg, run_dir=run_dir, variant=DENSE_VARIANT)


def run_lbi_training(cfg: LBITrainingConfig, *, run_dir: Path) -> Dict[str, Any]:
    return _run_training(cfg, run_dir=run_dir, variant=LBI_VARIANT)
