"""Failure detection, host-side fault injection and restart-from-checkpoint.

Nothing here makes a GPU fault: failures are injected on the host (an exception, a process exit, a skipped
heartbeat, a truncated checkpoint file) and detected on the host:

* ``check_kernel_status``   every device-side wait in this package's kernels is bounded and reports through a status
                            word; a non-zero word becomes a ``KernelWaitTimeout`` after the step;
* ``StepWatchdog``          polls a CUDA event with ``event.query()`` and reports a step that does not finish in time;
* ``Heartbeat``             ranks publish (step, wall time) in the ``torch.distributed`` store; before launching the next
                            step a rank checks its peers and raises ``PeerFailure`` for a stale or failed one, so no
                            collective or peer-memory kernel is launched against a dead rank;
* ``FaultInjector``         ``LBI_B200_INJECT="raise@step=3,rank=1;exit@step=5;stall_heartbeat@step=2;corrupt_checkpoint@step=4"``;
* ``run_with_recovery``     re-runs a training function with ``resume_from`` pointing at the newest loadable checkpoint.

The reference is a single process without any of this (its only robustness is silent kernel fall-back,
cuda/transformer/__init__.py:143-152); recovery relies on its checkpoint format, which this package keeps.
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Any, Callable

import torch


class KernelWaitTimeout(RuntimeError):
    """A bounded device-side wait ran out; the value is the site code the kernel recorded."""


class PeerFailure(RuntimeError):
    """A peer rank reported a failure or stopped publishing heartbeats."""


class StepTimeout(RuntimeError):
    """The watchdog saw a step exceed its time limit."""


class InjectedFault(RuntimeError):
    """Raised by the fault injector."""


def check_kernel_status(like: torch.Tensor | None = None) -> None:
    """Raise if any kernel of the extension recorded a timed-out wait on this device (the word is reset)."""
    from .. import ops

    if not torch.cuda.is_available() or not ops.native_available():
        return
    ref = like if like is not None else torch.empty(0, device="cuda")
    code = int(ops.ext().kernel_status(ref))
    if code != 0:
        raise KernelWaitTimeout(f"a bounded wait inside a kernel ran out (site {code})")


# ------------------------------------------------------------------------------------------------------ watchdog
class StepWatchdog:
    """Host watchdog for one device step: ``arm(event)`` after recording ``event`` at the end of the step's stream work,
    ``wait()`` polls ``event.query()`` and raises ``StepTimeout`` when ``limit_s`` passes first.  Polling never blocks in
    the driver, so a step that is stuck leaves the host free to report and shut down cleanly."""

    def __init__(self, limit_s: float = 300.0, poll_s: float = 0.005) -> None:
        self.limit_s, self.poll_s = float(limit_s), float(poll_s)
        self._event: Any = None
        self._t0 = 0.0

    def arm(self, event: Any) -> None:
        self._event, self._t0 = event, time.monotonic()

    def wait(self) -> float:
        if self._event is None:
            return 0.0
        while not self._event.query():
            if time.monotonic() - self._t0 > self.limit_s:
                raise StepTimeout(f"step did not finish within {self.limit_s:.1f} s")
            time.sleep(self.poll_s)
        return time.monotonic() - self._t0


# ------------------------------------------------------------------------------------------------------ heartbeat
class Heartbeat:
    """Per-rank liveness through a key-value store (``dist.TCPStore`` / ``FileStore`` / ``HashStore`` or the default
    process-group store).  Keys: ``hb/<rank>`` = "<step>:<unix time>", ``fail/<rank>`` = message."""

    def __init__(self, store: Any, rank: int, world_size: int, stale_after_s: float = 30.0) -> None:
        self.store, self.rank, self.world_size, self.stale_after_s = store, int(rank), int(world_size), float(stale_after_s)
        self._muted = False
        self._born = time.time()   # a peer that has not published yet is given stale_after_s from here
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        self.beat(-1)

    @classmethod
    def from_process_group(cls, stale_after_s: float = 30.0) -> "Heartbeat":
        import torch.distributed as dist

        store = dist.distributed_c10d._get_default_store()
        return cls(store, dist.get_rank(), dist.get_world_size(), stale_after_s)

    def beat(self, step: int) -> None:
        if not self._muted:
            self.store.set(f"hb/{self.rank}", f"{int(step)}:{time.time():.3f}")

    def mute(self) -> None:
        """Stop publishing (fault injection: a rank that is alive but silent)."""
        self._muted = True

    def report_failure(self, message: str) -> None:
        self.store.set(f"fail/{self.rank}", message[:500])

    def start_background(self, interval_s: float = 1.0, step_fn: Callable[[], int] = lambda: -1) -> None:
        def loop() -> None:
            while not self._stop.wait(interval_s):
                self.beat(step_fn())

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5.0)

    def _get(self, key: str) -> str | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def peer_states(self) -> dict[int, dict[str, Any]]:
        now, out = time.time(), {}
        for r in range(self.world_size):
            hb, fail = self._get(f"hb/{r}"), self._get(f"fail/{r}")
            step, stamp = (-1, 0.0)
            if hb:
                a, b = hb.split(":")
                step, stamp = int(a), float(b)
            out[r] = {"step": step, "age_s": now - (stamp if hb else self._born), "failure": fail}
        return out

    def check_peers(self) -> None:
        """Raise ``PeerFailure`` if a peer reported a failure or has been silent for longer than ``stale_after_s``."""
        for r, st in self.peer_states().items():
            if r == self.rank:
                continue
            if st["failure"]:
                raise PeerFailure(f"rank {r} failed: {st['failure']}")
            if st["age_s"] > self.stale_after_s:
                raise PeerFailure(f"rank {r} silent for {st['age_s']:.1f} s (last step {st['step']})")


# ------------------------------------------------------------------------------------------------------ injection
@dataclass(frozen=True)
class Fault:
    """One injected fault: kind, step, optional rank, transient or not."""

    kind: str                 # raise | exit | stall_heartbeat | corrupt_checkpoint
    step: int
    rank: int | None = None
    once: bool = False        # a transient fault: fires once per process, not again when a restarted run reaches the step


class FaultInjector:
    """Host-side faults at chosen steps.  Spec: ``kind@step=N[,rank=R][,once=1]`` joined by ``;`` (environment LBI_B200_INJECT).
    ``once=1`` marks a transient fault: it is remembered for the life of the process, so a run restarted in-process passes it."""

    KINDS = {"raise", "exit", "stall_heartbeat", "corrupt_checkpoint"}
    _fired_in_process: set = set()

    def __init__(self, spec: str | None = None, rank: int = 0) -> None:
        self.rank = int(rank)
        self.faults = self.parse(spec if spec is not None else os.environ.get("LBI_B200_INJECT", ""))
        self.fired: set[Fault] = set()

    @classmethod
    def parse(cls, spec: str) -> list[Fault]:
        out = []
        for item in filter(None, (s.strip() for s in spec.split(";"))):
            kind, _, rest = item.partition("@")
            if kind not in cls.KINDS:
                raise ValueError(f"unknown fault kind {kind!r}; known: {sorted(cls.KINDS)}")
            fields = dict(kv.split("=") for kv in rest.split(",") if kv)
            out.append(Fault(kind, int(fields.get("step", 0)), int(fields["rank"]) if "rank" in fields else None,
                             fields.get("once", "0") not in ("0", "", "false")))
        return out

    @classmethod
    def reset_process_memory(cls) -> None:
        cls._fired_in_process.clear()

    def due(self, step: int, kind: str | None = None) -> list[Fault]:
        return [f for f in self.faults if f.step == step and f not in self.fired and (f.rank is None or f.rank == self.rank)
                and (kind is None or f.kind == kind) and not (f.once and (f, self.rank) in self._fired_in_process)]

    def at_step(self, step: int, *, heartbeat: Heartbeat | None = None, checkpoint_path: Path | None = None) -> None:
        """Call between steps (no kernels or collectives of this rank in flight)."""
        for f in self.due(step):
            self.fired.add(f)
            if f.once:
                self._fired_in_process.add((f, self.rank))
            if f.kind == "stall_heartbeat" and heartbeat is not None:
                heartbeat.mute()
            elif f.kind == "corrupt_checkpoint" and checkpoint_path is not None and Path(checkpoint_path).exists():
                data = Path(checkpoint_path).read_bytes()
                Path(checkpoint_path).write_bytes(data[: max(1, len(data) // 3)])
            elif f.kind == "raise":
                if heartbeat is not None:
                    heartbeat.report_failure(f"injected fault at step {step}")
                raise InjectedFault(f"injected fault at step {step} on rank {self.rank}")
            elif f.kind == "exit":
                if heartbeat is not None:
                    heartbeat.report_failure(f"injected exit at step {step}")
                os._exit(17)


# ------------------------------------------------------------------------------------------------------ recovery
def newest_loadable_checkpoint(run_dir: Path) -> Path | None:
    """latest.pt if it loads, else best.pt, else None (a truncated file counts as missing)."""
    for name in ("latest.pt", "best.pt"):
        for path in sorted(Path(run_dir).rglob(name)):
            try:
                torch.load(path, map_location="cpu", weights_only=False)
            except Exception:
                continue
            return path
    return None


def _is_device_error(exc: BaseException) -> bool:
    """True for errors raised by the accelerator runtime (never retried in-process)."""
    accel = getattr(torch, "AcceleratorError", None)
    if accel is not None and isinstance(exc, accel):
        return True
    if isinstance(exc, (KernelWaitTimeout, PeerFailure, StepTimeout, InjectedFault)):
        return False
    text = str(exc)
    return isinstance(exc, RuntimeError) and ("CUDA error" in text or "cudaError" in text or "CUBLAS_STATUS" in text
                                              or "NCCL error" in text)


def run_with_recovery(train_fn: Callable[[Any], dict], cfg: Any, *, max_restarts: int = 2,
                      retry_on: tuple[type[BaseException], ...] = (KernelWaitTimeout, PeerFailure, StepTimeout,
                                                                    InjectedFault)) -> dict:
    """Run ``train_fn(cfg)``; after a failure restart it with ``resume_from`` set to the newest loadable checkpoint of
    the run (or from scratch when there is none).  The run directory must be stable (``cfg.run_name`` set).

    Only the failures this module defines are retried by default.  A CUDA error (``torch.AcceleratorError``, a
    ``RuntimeError`` from a launch, a sticky context error after a device fault) is never retried in-process, whatever
    ``retry_on`` says: re-running the same kernels in the same context repeats the fault and hides shape or state-dict
    bugs behind restarts, so it propagates and the launcher or an operator decides."""
    if not getattr(cfg, "run_name", ""):
        raise ValueError("run_with_recovery needs cfg.run_name so that restarts find the same run directory")
    attempt, failures = 0, []
    while True:
        try:
            result = train_fn(cfg)
            result["restarts"], result["failures"] = attempt, failures
            return result
        except retry_on as exc:  # noqa: PERF203
            if _is_device_error(exc):
                raise
            failures.append(f"{type(exc).__name__}: {exc}")
            attempt += 1
            if attempt > max_restarts:
                raise
            root = Path(cfg.output_dir) / cfg.run_name
            ckpt = newest_loadable_checkpoint(root)
            cfg = replace(cfg, resume_from=str(ckpt) if ckpt is not None else "", init_from="")
