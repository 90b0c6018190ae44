#!/usr/bin/env python
"""Headline benchmark: LBI training tokens/s with exact region-local backprop.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # the unmodified reference from baseline/_ref

Configs "cfg3" / "cfg5" (--config): LBI Mamba-3 130M / LBI Mamba-2 780M, on the same region-parallel engine at 1 - 8 GPUs
(--engine scan: the autograd scan engine, one GPU).  --variant dense: the dense model of the same size, either --impl.
Config "cfg4" (default): LBI Transformer, 24 layers, d_model 1024, 16 heads x 64, RoPE, RMSNorm, SwiGLU 2816,
vocab 32768, sequence 16384 split into 8 regions of 2048 tokens, interface width 128, batch 4, bf16, AdamW,
uniform-random tokens, random-init weights.  Regions are placed on the GPUs in contiguous blocks (8 regions on N
GPUs), so the global batch is fixed and scaling is strong.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

CONFIGS = {
    # name: model + data shape
    "cfg4": dict(model="lbi-transformer-350m", layers=24, dim=1024, n_heads=16, d_intermediate=2816, vocab=32768,
                 seq_len=16384, regions=8, batch=4, message_dim=128, message_hidden=1024),
    "cfg4-depth": dict(model="lbi-transformer-350m-depth-regions", layers=24, dim=1024, n_heads=16, d_intermediate=2816,
                       vocab=32768, seq_len=16384, regions=8, batch=4, message_dim=128, message_hidden=1024, axis="depth"),
    "small": dict(model="lbi-transformer-small", layers=4, dim=512, n_heads=8, d_intermediate=1408, vocab=8192,
                  seq_len=4096, regions=8, batch=2, message_dim=32, message_hidden=512),
    # cfg3 / cfg5 are the LBI Mamba-3 (~130M) and LBI Mamba-2 (~780M) shapes (region-parallel engine like cfg4).
    "cfg3": dict(model="lbi-mamba3-130m", backbone="mamba3", layers=24, dim=768, d_state=128, headdim=64, expand=2, chunk=128,
                 vocab=32768, seq_len=8192, regions=8, batch=8, message_dim=64, message_hidden=768),
    "cfg5": dict(model="lbi-mamba2-780m", backbone="mamba2", layers=48, dim=1536, d_state=128, headdim=64, expand=2, chunk=256,
                 vocab=32768, seq_len=32768, regions=32, batch=2, message_dim=256, message_hidden=1536, basis_chunk=64, recompute=True),
    # a slice of cfg5 (same widths, 4 layers, 4 regions of 1024 tokens) for per-op profiles that finish in seconds
    "cfg5-slice": dict(model="lbi-mamba2-780m-slice", backbone="mamba2", layers=4, dim=1536, d_state=128, headdim=64, expand=2, chunk=256,
                       vocab=32768, seq_len=4096, regions=4, batch=2, message_dim=256, message_hidden=1536, basis_chunk=64),
    "mamba-tiny": dict(model="lbi-mamba3-tiny", backbone="mamba3", layers=2, dim=256, d_state=128, headdim=64, expand=2, chunk=128,
                       vocab=1024, seq_len=1024, regions=4, batch=2, message_dim=16, message_hidden=64),
    "tiny": dict(model="lbi-transformer-tiny", layers=2, dim=256, n_heads=4, d_intermediate=512, vocab=1024,
                 seq_len=1024, regions=8, batch=2, message_dim=16, message_hidden=64),
}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--config", type=str, default="cfg4", choices=sorted(CONFIGS))
    p.add_argument("--basis-chunk", type=int, default=0, help="basis directions per pullback pass (0: the config's default, 16 if none)")
    p.add_argument("--recompute-forward", type=str, default="auto", choices=["auto", "on", "off"],
                   help="drop each region's cached activations after its forward and rebuild them before its pullback / local VJP")
    p.add_argument("--comm", type=str, default="auto", choices=["auto", "collective", "symm"])
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--jacobian-mode", type=str, default="recompute", choices=["recompute", "graph", "structured"],
                   help="scan-engine configs: how the interface Jacobians are materialised")
    p.add_argument("--engine", type=str, default="fast", choices=["fast", "scan"],
                   help="fast: the autograd-free region-parallel engine (every backbone); scan: ScanADEngine over autograd (Mamba configs)")
    p.add_argument("--variant", type=str, default="lbi", choices=["lbi", "dense"],
                   help="dense: the dense model of the same size (no regions, plain autograd + AdamW), for either --impl")
    p.add_argument("--profile-ops", action="store_true", help="after the timed run, time one more step op by op (stderr)")
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.proc = None
        self.gpu_index = gpu_index

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, max_clock, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        median = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": median, "sm_max_mhz": max_clock, "samples": len(clocks), "reasons": sorted(reasons)}


def physical_gpu_index(local_rank: int) -> int:
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        ids = [x for x in visible.split(",") if x.strip()]
        try:
            return int(ids[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def make_batches(cfg: dict, count: int, seed: int):
    """Pinned host batches of uniform-random tokens: (inputs [B, T], targets [B, T]) int64."""
    gen = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(count):
        seq = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq_len"] + 1), generator=gen, dtype=torch.int64)
        x, y = seq[:, :-1].contiguous(), seq[:, 1:].contiguous()
        if torch.cuda.is_available():
            x, y = x.pin_memory(), y.pin_memory()
        out.append((x, y))
    return out


def max_over_ranks(value: float, device) -> float:
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def barrier_sync():
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


# --------------------------------------------------------------------------------------------------- this framework
def run_ours(args) -> dict:
    from lbi_b200 import ops
    from lbi_b200.backbones import BackboneSpec
    from lbi_b200.interfaces import VectorMLPInterface
    from lbi_b200.models import LBILanguageModel
    from lbi_b200.parallel import CollectiveComm, FastLBIEngine, LocalComm, init_distributed_from_env

    cfg = CONFIGS[args.config]
    # strict mode: a route from a CUDA bf16 tensor to PyTorch / cuBLAS / flash_attn raises instead of running silently
    ops.dispatch.set_strict(os.environ.get("LBI_B200_STRICT", "1") != "0")
    rank, local_rank, world = init_distributed_from_env("cuda")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N > 1")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    comm = LocalComm()
    comm_name = "local"
    if world > 1:
        comm_name = "collective"
        comm = CollectiveComm()
        if args.comm in ("auto", "symm"):
            try:
                from lbi_b200.parallel.symm import SymmComm

                comm = SymmComm()
                comm_name = "symm"
            except Exception as exc:  # noqa: BLE001 - fall back to library collectives, and say so
                if args.comm == "symm":
                    raise
                if rank == 0:
                    print(f"[bench] peer-memory comm unavailable ({exc!r}); using library collectives", file=sys.stderr)

    axis = cfg.get("axis", "sequence")
    torch.manual_seed(0)
    if "backbone" in cfg:
        spec = BackboneSpec(name=cfg["backbone"], dim=cfg["dim"], layers=cfg["layers"], d_state=cfg["d_state"], headdim=cfg["headdim"],
                            expand=cfg["expand"], d_conv=4, chunk_size=cfg["chunk"])
    else:
        spec = BackboneSpec(name="transformer", dim=cfg["dim"], layers=cfg["layers"], n_heads=cfg["n_heads"], d_conv=0,
                            d_intermediate=cfg["d_intermediate"])
    iface = VectorMLPInterface(feature_dim=cfg["dim"], num_regions=cfg["regions"], interface_width=cfg["message_dim"],
                               interface_map_hidden_dim=cfg["message_hidden"])
    model = LBILanguageModel(vocab_size=cfg["vocab"], layers_per_region=max(1, cfg["layers"] // cfg["regions"]),
                             backbone_spec=spec, interface=iface, tie_embeddings=True, region_axis=axis,
                             num_sequence_regions=cfg["regions"]).to(device)
    n_params = sum(p.numel() for p in model.parameters())
    basis_chunk = args.basis_chunk or cfg.get("basis_chunk", 16)
    recompute = {"on": True, "off": False, "auto": bool(cfg.get("recompute", False)) and axis == "sequence"}[args.recompute_forward]
    engine = FastLBIEngine(model, lr=3e-4, weight_decay=0.01, grad_clip=1.0, basis_chunk=basis_chunk, comm=comm,
                           recompute_forward=recompute)

    total = args.warmup + args.steps
    host = make_batches(cfg, total, seed=1234)
    dev_batches = [(x.to(device, non_blocking=True), y.to(device, non_blocking=True)) for x, y in host]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)  # > 126 MB L2

    for i in range(args.warmup):
        engine.step(*dev_batches[i])
    barrier_sync()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = ops.dispatch.KERNEL_LAUNCHES["count"]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    loss = None
    for i in range(args.warmup, total):
        flush.zero_()
        loss = engine.step(*dev_batches[i])
    stop.record()
    barrier_sync()
    clocks = sampler.stop()
    launches = ops.dispatch.KERNEL_LAUNCHES["count"] - launches0
    ms = max_over_ranks(start.elapsed_time(stop), device) / max(1, args.steps)
    tokens = cfg["batch"] * cfg["seq_len"]
    value = tokens / (ms / 1e3)

    e2e = None
    if not args.no_e2e:
        barrier_sync()
        t0 = time.perf_counter()
        for i in range(args.steps):
            x, y = host[args.warmup + i]
            xd, yd = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
            loss_val = float(engine.step(xd, yd).item())  # device -> host read of the step's loss
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0, device)
        e2e = {"value": tokens * args.steps / dt, "unit": "tokens/s",
               "h2d_bytes_per_step": int(host[0][0].numel() * 8 + host[0][1].numel() * 8), "d2h_bytes_per_step": 4,
               "last_loss": loss_val}

    if args.profile_ops and rank == 0 or (args.profile_ops and world > 1):
        from lbi_b200.ops import profile

        profile.enable()
        profile.reset()
        engine.step(*dev_batches[-1])
        if rank == 0:
            print(profile.report(), file=sys.stderr)
        profile.disable()

    status = ops.ext().kernel_status(flush) if ops.native_available() else 0
    return {
        "metric": "train tokens/s (device-timed, max over ranks)", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
        "impl": "ours",
        "config": {"model": cfg["model"], "global_batch": cfg["batch"], "seq_len": cfg["seq_len"], "regions": cfg["regions"],
                   "region_axis": axis, "same_decomposition": axis == "depth",
                   "interface_width": cfg["message_dim"], "params": n_params,
                   "parallelism": f"rp{world}" if world > 1 else "single", "comm": comm_name,
                   "backward": "suffix-scan exact (structured pullback over basis)", "basis_chunk": basis_chunk,
                   "recompute_forward": recompute,
                   **({"kernel_chunk": 128, "chunk_note": f"the scan kernels block time in chunks of 128 tokens whatever the model's "
                       f"chunk_size ({cfg['chunk']}); the result does not depend on the blocking"} if "backbone" in cfg else {}),
                   "optimizer": "AdamW + global-norm clip in the timed region",
                   "cache": "L2 flushed (256 MB write) before every timed step; per-step working set is GBs"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": float(loss) if loss is not None else None,
        "kernel_status": int(status), "strict": bool(ops.dispatch.STRICT["enabled"]), "fallbacks": dict(ops.dispatch.FALLBACKS),
    }


def run_ours_scan_engine(args) -> dict:
    """Mamba configs: LBILanguageModel + ScanADEngine (recompute Jacobian provider over blocks of basis directions, the
    state mixers on the tcgen05 scan kernels forward and backward) + AdamW with clipping, one GPU."""
    import torch.nn.functional as F

    from lbi_b200 import ops
    from lbi_b200.backbones import BackboneSpec
    from lbi_b200.backward import ScanADEngine
    from lbi_b200.interfaces import VectorMLPInterface
    from lbi_b200.models import LBILanguageModel

    cfg = CONFIGS[args.config]
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("the Mamba configs run on one GPU (the region-parallel engine covers the Transformer backend)")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)
    spec = BackboneSpec(name=cfg["backbone"], dim=cfg["dim"], layers=cfg["layers"], d_state=cfg["d_state"], headdim=cfg["headdim"],
                        expand=cfg["expand"], d_conv=4, chunk_size=cfg["chunk"])
    iface = VectorMLPInterface(feature_dim=cfg["dim"], num_regions=cfg["regions"], interface_width=cfg["message_dim"],
                               interface_map_hidden_dim=cfg["message_hidden"])
    model = LBILanguageModel(vocab_size=cfg["vocab"], layers_per_region=max(1, cfg["layers"] // cfg["regions"]), backbone_spec=spec,
                             interface=iface, tie_embeddings=True, region_axis="sequence",
                             num_sequence_regions=cfg["regions"]).to(device)
    n_params = sum(p.numel() for p in model.parameters())
    engine = ScanADEngine(state_jacobian_mode=args.jacobian_mode, state_jacobian_basis_chunk=args.basis_chunk or 16)
    optimizer = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.01)

    def step(x, y):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, cache = model.forward_with_cache(x, detach_states=True)
        loss = F.cross_entropy(logits.float().reshape(-1, cfg["vocab"]), y.reshape(-1))
        engine.backward(model=model, loss=loss, cache=cache)
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        optimizer.step()
        return loss.detach()

    total = args.warmup + args.steps
    host = make_batches(cfg, total, seed=1234)
    dev_batches = [(x.to(device, non_blocking=True), y.to(device, non_blocking=True)) for x, y in host]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    for i in range(args.warmup):
        step(*dev_batches[i])
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    launches0 = ops.dispatch.KERNEL_LAUNCHES["count"]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    loss = None
    for i in range(args.warmup, total):
        flush.zero_()
        loss = step(*dev_batches[i])
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    launches = ops.dispatch.KERNEL_LAUNCHES["count"] - launches0
    ms = start.elapsed_time(stop) / max(1, args.steps)
    tokens = cfg["batch"] * cfg["seq_len"]
    e2e = None
    if not args.no_e2e:
        t0 = time.perf_counter()
        for i in range(args.steps):
            x, y = host[args.warmup + i]
            loss_val = float(step(x.to(device, non_blocking=True), y.to(device, non_blocking=True)).item())
        torch.cuda.synchronize()
        e2e = {"value": tokens * args.steps / (time.perf_counter() - t0), "unit": "tokens/s",
               "h2d_bytes_per_step": int(host[0][0].numel() * 8 + host[0][1].numel() * 8), "d2h_bytes_per_step": 4,
               "last_loss": loss_val}
    status = ops.ext().kernel_status(flush) if ops.native_available() else 0
    return {
        "metric": "train tokens/s (device-timed, max over ranks)", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights", "impl": "ours",
        "config": {"model": cfg["model"], "global_batch": cfg["batch"], "seq_len": cfg["seq_len"], "regions": cfg["regions"],
                   "region_axis": "sequence", "interface_width": cfg["message_dim"], "params": n_params, "parallelism": "single",
                   "backward": f"suffix-scan exact (scan engine, {args.jacobian_mode} Jacobian provider, kernel scans forward and backward)",
                   "basis_chunk": args.basis_chunk or 16, "optimizer": "AdamW + global-norm clip in the timed region",
                   "cache": "L2 flushed (256 MB write) before every timed step; per-step working set is GBs"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": float(loss) if loss is not None else None,
        "kernel_status": int(status),
    }


# --------------------------------------------------------------------------------------------------- reference arm
def reference_backbone_fields(cfg: dict) -> dict:
    """Backbone fields of the reference's LBITrainingConfig for one of CONFIGS.  Its Transformer requires d_conv >= 1; its
    Mamba-2 runs the unfused path (use_mem_eff_path=False: the fused one needs the causal_conv1d package, which this image
    does not have); Mamba-3 is its Triton SISO path."""
    if "backbone" not in cfg:
        return dict(backbone="transformer", n_heads=cfg["n_heads"], d_intermediate=cfg["d_intermediate"], d_conv=1)
    return dict(backbone=cfg["backbone"], d_state=cfg["d_state"], headdim=cfg["headdim"], expand=cfg["expand"], d_conv=4,
                chunk_size=cfg["chunk"], use_mem_eff_path=False)


def import_reference():
    """Put the unmodified reference tree (baseline/_ref) first on sys.path.  Returns an error string or None."""
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "train")):
        return ("baseline/_ref does not hold the reference tree (it has no setup.py/pyproject, pip cannot install it; copy it with "
                "baseline/install_reference.sh)")
    # The image pre-registers an unrelated namespace package called `cuda` (cuda-python); the reference's own
    # top-level `cuda` package must win, so drop the cached entry before putting the reference first on sys.path.
    for name in [m for m in sys.modules if m == "cuda" or m.startswith("cuda.")]:
        del sys.modules[name]
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    return None


def run_dense(args) -> dict:
    """The dense model of the same size (no regions): forward under bf16 autocast, next-token loss, autograd backward, global-norm
    clip and torch AdamW, for this framework (its modules run the sm_100a kernels through autograd Functions) or for the
    reference (models/dense_language_model.py:11-47 with backward/autograd.py:11-28 there).  One GPU."""
    cfg = CONFIGS[args.config]
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            return {"impl": args.impl, "variant": "dense", "unavailable": "the dense arms are single-device (no region decomposition to spread)"}
        return {}
    if args.impl == "reference":
        err = import_reference()
        if err:
            return {"impl": "reference", "unavailable": err}
        try:
            from train.config import LBITrainingConfig
            from train.eval import next_token_loss
            from train.model_builders import build_dense_model
        except Exception as exc:  # noqa: BLE001
            return {"impl": "reference", "unavailable": f"reference import failed: {exc!r}"[:300]}
        fields = reference_backbone_fields(cfg)
    else:
        from lbi_b200.train.config import LBITrainingConfig
        from lbi_b200.train.eval import next_token_loss
        from lbi_b200.train.model_builders import build_dense_model

        fields = reference_backbone_fields(cfg)
        if "backbone" not in cfg:
            fields["d_conv"] = 0
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)
    rcfg = LBITrainingConfig(variants="dense", regime="dense", device="cuda", dtype="bfloat16", vocab_size=cfg["vocab"], tie_embeddings=True,
                             seq_len=cfg["seq_len"], batch_size=cfg["batch"], layers=cfg["layers"], dim=cfg["dim"], lr_model=3e-4,
                             weight_decay=0.01, grad_clip=1.0, steps=max(1, args.steps + args.warmup), **fields)
    try:
        model = build_dense_model(rcfg).to(device=device, dtype=torch.float32)
    except Exception as exc:  # noqa: BLE001
        return {"impl": args.impl, "variant": "dense", "unavailable": f"dense model build failed: {exc!r}"[:300]}
    n_params = sum(p.numel() for p in model.parameters())
    fast = None
    if args.impl == "ours":
        # this framework's dense arm: the closed-form chain on the sm_100a kernels, flat-buffer AdamW (no autograd, no library GEMM)
        from lbi_b200.parallel import DenseFastEngine

        fast = DenseFastEngine(model, lr=rcfg.lr_model, weight_decay=rcfg.weight_decay, grad_clip=rcfg.grad_clip)
    else:
        optimizer = torch.optim.AdamW(model.parameters(), lr=rcfg.lr_model, weight_decay=rcfg.weight_decay)

    def step(xb, yb):
        if fast is not None:
            return fast.step(xb, yb)
        model.train()
        optimizer.zero_grad(set_to_none=True)
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
            logits = model(xb)
        loss = next_token_loss(logits, yb)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), rcfg.grad_clip)
        optimizer.step()
        return loss.detach()

    total = args.warmup + args.steps
    host = make_batches(cfg, total, seed=1234)
    dev_batches = [(x.to(device, non_blocking=True), y.to(device, non_blocking=True)) for x, y in host]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    launches0 = 0
    if args.impl == "ours":
        from lbi_b200 import ops

        launches0 = ops.dispatch.KERNEL_LAUNCHES["count"]
    try:
        for i in range(args.warmup):
            step(*dev_batches[i])
        torch.cuda.synchronize()
        sampler = ClockSampler(physical_gpu_index(0))
        sampler.start()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        loss = None
        for i in range(args.warmup, total):
            flush.zero_()
            loss = step(*dev_batches[i])
        stop.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = start.elapsed_time(stop) / max(1, args.steps)
        tokens = cfg["batch"] * cfg["seq_len"]
        e2e = None
        if not args.no_e2e:
            t0 = time.perf_counter()
            for i in range(args.steps):
                x, y = host[args.warmup + i]
                loss_val = float(step(x.to(device, non_blocking=True), y.to(device, non_blocking=True)).item())
            torch.cuda.synchronize()
            e2e = {"value": tokens * args.steps / (time.perf_counter() - t0), "unit": "tokens/s",
                   "h2d_bytes_per_step": int(host[0][0].numel() * 16), "d2h_bytes_per_step": 4, "last_loss": loss_val}
    except Exception as exc:  # noqa: BLE001
        return {"impl": args.impl, "variant": "dense", "unavailable": f"dense step failed: {exc!r}"[:300]}
    launches = 0
    if args.impl == "ours":
        launches = ops.dispatch.KERNEL_LAUNCHES["count"] - launches0
    return {
        "metric": "train tokens/s (device-timed, max over ranks)", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16" if fast is not None else "bf16 autocast (fp32 weights)",
        "data": "synthetic uniform-random tokens, random-init weights", "impl": args.impl, "variant": "dense",
        "config": {"model": cfg["model"] + "-dense", "global_batch": cfg["batch"], "seq_len": cfg["seq_len"], "regions": 1,
                   "params": n_params, "parallelism": "single",
                   "backward": "dense closed-form chain on the sm_100a kernels (no regions, no autograd)" if fast is not None
                   else "dense autograd (no regions)",
                   "optimizer": ("fused clip + AdamW on flat buffers" if fast is not None else "torch AdamW + global-norm clip")
                   + " in the timed region",
                   "cache": "L2 flushed (256 MB write) before every timed step; per-step working set is GBs"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": float(loss) if loss is not None else None,
    }


def run_reference(args) -> dict:
    """The unmodified reference tree under baseline/_ref, driven through its own classes on one GPU."""
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            return {"impl": "reference", "unavailable": "reference is single-device: it has no torch.distributed code path, so there is no N>1 run"}
        return {}
    err = import_reference()
    if err:
        return {"impl": "reference", "unavailable": err}
    cfg = CONFIGS[args.config]
    try:
        from backward import ScanADEngine, assign_grad_map, build_interface_pullback_provider, lbi_scan_backward_step
        from train.config import LBITrainingConfig
        from train.eval import next_token_loss
        from train.model_builders import build_lbi_model
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference import failed: {exc!r}"[:300]}

    device = torch.device("cuda", 0)
    # the reference's regions are layer ranges of equal size: 48 layers cannot give 32 regions, so the nearest split is reported
    layers_per_region = max(1, -(-cfg["layers"] // cfg["regions"]))
    ref_regions = -(-cfg["layers"] // layers_per_region)
    # The reference's recompute Jacobian mode replicates the batch `chunk` times per pass; the launcher default (32) and
    # 8 do not fit 180 GB at this configuration, so the largest chunk that fits is used and reported.
    env_chunk = os.environ.get("LBI_REF_BASIS_CHUNK")
    chunks = [int(env_chunk)] if env_chunk else [8, 4, 2, 1]
    total = args.warmup + args.steps
    host = make_batches(cfg, total, seed=1234)
    path = {"engine": "ScanADEngine.backward"}
    last_oom = ""
    for chunk in chunks:
        torch.manual_seed(0)
        rcfg = LBITrainingConfig(
            variants="lbi", regime="lbi", device="cuda", dtype="bfloat16", vocab_size=cfg["vocab"],
            tie_embeddings=True, seq_len=cfg["seq_len"], batch_size=cfg["batch"], layers=cfg["layers"], dim=cfg["dim"],
            region_size=layers_per_region, message_dim=cfg["message_dim"], message_hidden_dim=cfg["message_hidden"],
            interface_jacobian_mode="recompute", jacobian_basis_chunk=chunk, lr_model=3e-4, weight_decay=0.01, grad_clip=1.0,
            steps=max(1, args.steps + args.warmup), **reference_backbone_fields(cfg),
        )
        try:
            model = build_lbi_model(rcfg).to(device=device, dtype=torch.float32)
            optimizer = torch.optim.AdamW(model.parameters(), lr=rcfg.lr_model, weight_decay=rcfg.weight_decay)
        except Exception as exc:  # noqa: BLE001
            return {"impl": "reference", "unavailable": f"reference model build failed: {exc!r}"[:300]}
        n_params = sum(p.numel() for p in model.parameters())
        dev_batches = [(x.to(device), y.to(device)) for x, y in host]

        def step(xb, yb):
            model.train()
            with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                logits, cache = model.forward_with_cache(xb)
            loss = next_token_loss(logits, yb)
            engine = ScanADEngine.from_config(rcfg)
            try:
                engine.backward(model=model, loss=loss, cache=cache)
            except TypeError:
                # Python >= 3.12: the reference's isinstance check against its runtime-checkable Protocol raises;
                # call the function the engine wraps (same arguments, same providers).
                path["engine"] = "lbi_scan_backward_step (ScanADEngine.backward raises TypeError on Python 3.12)"
                model.zero_grad(set_to_none=True)
                result = lbi_scan_backward_step(model, ce_loss=loss, cache=cache, pullback_provider=engine.pullback_provider,
                                                local_vjp_provider=engine.local_vjp_provider)
                assign_grad_map(model, result.grad_map)
            torch.nn.utils.clip_grad_norm_(model.parameters(), rcfg.grad_clip)
            optimizer.step()
            return loss

        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
        # One reference step at the headline configuration takes about 13 minutes on a B200 (recompute chunk 1 is the only
        # one that fits), so the requested warm-up / step counts are cut to what fits LBI_REF_TIME_BUDGET_S (default 1500 s,
        # never below one warm-up and one timed step); the counts actually run are the ones reported.
        budget_s = float(os.environ.get("LBI_REF_TIME_BUDGET_S", "1500"))
        n_warm, n_steps = args.warmup, args.steps
        try:
            t_first = None
            i = 0
            while i < n_warm:
                t0 = time.perf_counter()
                step(*dev_batches[i])
                torch.cuda.synchronize()
                if t_first is None:
                    t_first = time.perf_counter() - t0
                    if t_first * (args.warmup + args.steps) > budget_s:
                        n_warm = 1
                        n_steps = max(1, min(args.steps, int((budget_s - t_first) // t_first)))
                i += 1
            total = n_warm + n_steps
            torch.cuda.synchronize()
            sampler = ClockSampler(physical_gpu_index(0))
            sampler.start()
            # A reference step takes minutes at this configuration, so the device-timed and the end-to-end figure come
            # from the same K steps: every step copies its batch from pinned host memory and reads its loss back (as the
            # reference's own training loop does); CUDA events give the device time, the wall clock the end-to-end time.
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            wall0 = time.perf_counter()
            start.record()
            for i in range(n_warm, total):
                flush.zero_()
                x, y = host[i]
                loss = step(x.to(device, non_blocking=True), y.to(device, non_blocking=True))
                loss_val = float(loss.item())
            stop.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - wall0
            clocks = sampler.stop()
            break
        except torch.OutOfMemoryError as exc:
            last_oom = str(exc)[:120]
            del model, optimizer, dev_batches, flush, step
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            continue
        except Exception as exc:  # noqa: BLE001
            # compiler errors quote the whole kernel first and say what went wrong last: keep both ends, on one line
            text = " ".join(f"{type(exc).__name__}: {exc}".split())
            if len(text) > 520:
                text = text[:200] + " ... " + text[-300:]
            return {"impl": "reference", "unavailable": f"reference step failed: {text}"}
    else:
        return {"impl": "reference", "unavailable": f"reference ran out of GPU memory at the named config for every recompute chunk in {chunks}: {last_oom}"}
    ms = start.elapsed_time(stop) / max(1, n_steps)
    tokens = cfg["batch"] * cfg["seq_len"]
    e2e = {"value": tokens * n_steps / wall, "unit": "tokens/s", "h2d_bytes_per_step": int(host[0][0].numel() * 16),
           "d2h_bytes_per_step": 4, "last_loss": loss_val, "note": "same steps as the device-timed figure (wall clock)"}
    return {
        "metric": "train tokens/s (device-timed, max over ranks)", "value": tokens / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": 1, "steps": n_steps, "warmup": n_warm, "ms_per_step": ms, "higher_is_better": True,
        "requested": {"steps": args.steps, "warmup": args.warmup, "time_budget_s": budget_s},
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 autocast (fp32 weights)",
        "data": "synthetic uniform-random tokens, random-init weights", "impl": "reference",
        "config": {"model": cfg["model"], "global_batch": cfg["batch"], "seq_len": cfg["seq_len"], "regions": ref_regions,
                   "region_axis": "depth (the reference has no sequence-axis regions)", "same_decomposition": False,
                   "same_decomposition_note": "the reference cuts depth (layer ranges over the full sequence); this framework's default "
                                              "arm cuts the sequence; `--config cfg4-depth` is this framework on the reference's cut",
                   "interface_width": cfg["message_dim"], "params": n_params, "parallelism": "single", "jacobian_mode": "recompute",
                   "basis_chunk": chunk, "backbone_fields": {k: v for k, v in reference_backbone_fields(cfg).items()},
                   "path": path["engine"]},
        "clocks": clocks, "e2e": e2e, "gpu_launches": 0, "final_loss": float(loss.detach()),
    }


def main() -> None:
    args = parse_args()
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return
    mamba = "backbone" in CONFIGS[args.config]
    if args.variant == "dense":
        result = run_dense(args)
    elif args.impl == "reference":
        result = run_reference(args)
    else:
        result = run_ours_scan_engine(args) if (mamba and args.engine == "scan") else run_ours(args)
    if int(os.environ.get("RANK", "0")) == 0 and result:
        print(json.dumps(result))
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
