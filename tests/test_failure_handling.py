"""Failure detection and recovery, with every fault injected on the host (CPU / gloo ranks only)."""
import json
import multiprocessing as mp
import os
import time
from pathlib import Path

import pytest
import torch
import torch.distributed as dist

from lbi_b200.train.config import LBITrainingConfig
from lbi_b200.train.lbi import run_lbi_experiment
from lbi_b200.utils import failure as F


def _cfg(tmp_path, **kw):
    base = dict(variants="lbi", backbone="transformer", device="cpu", dtype="float32", output_dir=str(tmp_path / "out"), run_name="run",
                task="copy", vocab_size=32, seq_len=16, train_sequences=32, val_sequences=8, batch_size=2, steps=4, eval_every=2,
                eval_batches=1, log_every=1, save_every=1, layers=2, dim=16, n_heads=2, region_size=1, message_dim=4, message_hidden_dim=8)
    base.update(kw)
    return LBITrainingConfig(**base)


def test_fault_spec_parsing():
    faults = F.FaultInjector.parse("raise@step=3,rank=1; exit@step=5;stall_heartbeat@step=2")
    assert faults == [F.Fault("raise", 3, 1), F.Fault("exit", 5, None), F.Fault("stall_heartbeat", 2, None)]
    assert F.FaultInjector.parse("raise@step=3,once=1") == [F.Fault("raise", 3, None, True)]
    with pytest.raises(ValueError):
        F.FaultInjector.parse("explode@step=1")
    inj = F.FaultInjector("raise@step=3,rank=1", rank=0)
    inj.at_step(3)  # other rank: nothing happens
    with pytest.raises(F.InjectedFault):
        F.FaultInjector("raise@step=3,rank=1", rank=1).at_step(3)


def test_recovery_resumes_from_latest_checkpoint(tmp_path, monkeypatch):
    monkeypatch.setenv("LBI_B200_INJECT", "raise@step=3")
    calls = []

    def train(cfg):
        calls.append(cfg.resume_from)
        out = run_lbi_experiment(cfg)
        return out

    # the injector fires once per process-level spec; the restarted run must not fire again, so drop the spec after it fired
    def train_once(cfg):
        try:
            return train(cfg)
        finally:
            os.environ.pop("LBI_B200_INJECT", None)

    result = F.run_with_recovery(train_once, _cfg(tmp_path), max_restarts=2)
    assert result["restarts"] == 1 and "InjectedFault" in result["failures"][0]
    assert calls[0] == "" and calls[1].endswith("latest.pt")
    run = result["runs"][0]
    assert run["start_step"] == 2 and run["steps"] == 4
    rows = [json.loads(line) for line in (Path(run["run_dir"]) / "metrics.jsonl").read_text().splitlines()]
    assert [r["step"] for r in rows if r["split"] == "train"] == [1, 2, 3, 4]


def test_training_entry_restarts_under_the_restart_limit(tmp_path, monkeypatch):
    """The command-line route: ``run_with_restarts`` resumes after a transient injected fault and gives up beyond the limit."""
    from lbi_b200.train.lbi import run_with_restarts

    F.FaultInjector.reset_process_memory()
    monkeypatch.setenv("LBI_B200_INJECT", "raise@step=3")
    with pytest.raises(F.InjectedFault):
        run_with_restarts(_cfg(tmp_path / "none"), 0)
    with pytest.raises(F.InjectedFault):           # a fault that comes back at the same step every time exhausts the limit
        run_with_restarts(_cfg(tmp_path / "always"), 1)
    monkeypatch.setenv("LBI_B200_INJECT", "raise@step=3,once=1")
    out = run_with_restarts(_cfg(tmp_path / "one"), 2)
    assert out["restarts"] == 1 and out["runs"][0]["start_step"] >= 2 and out["runs"][0]["steps"] == 4
    import lbi_b200.train.lbi as entry

    monkeypatch.setenv("WORLD_SIZE", "2")  # multi-process runs are left to the launcher: the call goes straight through
    monkeypatch.setattr(entry, "run_lbi_experiment", lambda cfg: {"direct": True})
    assert run_with_restarts(_cfg(tmp_path / "multi"), 2) == {"direct": True}


def test_corrupt_latest_checkpoint_falls_back(tmp_path):
    cfg = _cfg(tmp_path, steps=2)
    out = run_lbi_experiment(cfg)
    run_dir = Path(out["runs"][0]["run_dir"])
    latest = run_dir / "checkpoints" / "latest.pt"
    best = run_dir / "checkpoints" / "best.pt"
    assert F.newest_loadable_checkpoint(run_dir) == latest
    F.FaultInjector("corrupt_checkpoint@step=1").at_step(1, checkpoint_path=latest)
    assert F.newest_loadable_checkpoint(run_dir) == (best if best.exists() else None)


def test_watchdog_times_out_on_an_event_that_never_completes():
    class Never:
        def query(self):
            return False

    class Done:
        def query(self):
            return True

    dog = F.StepWatchdog(limit_s=0.05, poll_s=0.005)
    dog.arm(Never())
    with pytest.raises(F.StepTimeout):
        dog.wait()
    dog.arm(Done())
    assert dog.wait() < 0.05


def _rank_main(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hb = F.Heartbeat.from_process_group(stale_after_s=1.0)
    inj = F.FaultInjector("raise@step=2,rank=1" if mode == "raise" else "stall_heartbeat@step=2,rank=1", rank=rank)
    outcome = "finished"
    try:
        for step in range(1, 6):
            inj.at_step(step, heartbeat=hb)
            hb.beat(step)
            hb.check_peers()
            if step < 2:  # a collective while everyone is alive
                t = torch.ones(1)
                dist.all_reduce(t)
            time.sleep(0.6)
    except F.PeerFailure as exc:
        outcome = f"peer_failure:{exc}"
    except F.InjectedFault:
        outcome = "injected"
    q.put((rank, outcome))
    q.close()
    q.join_thread()
    # leave without a collective: the survivor must not block on the failed rank
    os._exit(0)


@pytest.mark.parametrize("mode", ["raise", "stall"])
def test_peer_failure_is_seen_on_the_host_before_the_next_launch(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000) + (0 if mode == "raise" else 1)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert results[0].startswith("peer_failure"), results
    if mode == "raise":
        assert results[1] == "injected" and "injected fault at step 2" in results[0]
    else:
        assert "silent" in results[0]


def test_device_errors_and_plain_runtime_errors_are_not_retried(tmp_path):
    calls = []

    def cuda_fault(cfg):
        calls.append("cuda")
        raise F.KernelWaitTimeout("CUDA error: an illegal memory access was encountered")   # even a retryable class ...

    def shape_bug(cfg):
        calls.append("shape")
        raise RuntimeError("size mismatch for blocks.0.weight")

    # ... is retried only when it does not come from the device runtime; this one is one of ours, so it is retried
    with pytest.raises(F.KernelWaitTimeout):
        F.run_with_recovery(cuda_fault, _cfg(tmp_path), max_restarts=1)
    assert calls == ["cuda", "cuda"]
    calls.clear()
    with pytest.raises(RuntimeError):
        F.run_with_recovery(shape_bug, _cfg(tmp_path), max_restarts=2)
    assert calls == ["shape"]          # a plain RuntimeError is not in the default retry set
    calls.clear()

    def launch_failure(cfg):
        calls.append("launch")
        raise RuntimeError("CUDA error: unspecified launch failure")

    with pytest.raises(RuntimeError):
        F.run_with_recovery(launch_failure, _cfg(tmp_path), max_restarts=2, retry_on=(RuntimeError,))
    assert calls == ["launch"]         # never retried in-process, even when the caller widens retry_on


def test_background_heartbeat_keeps_a_slow_rank_alive():
    """A rank whose loop iteration takes longer than the staleness limit (evaluation, checkpoint save) still publishes
    through its background thread, so the peer check of another rank does not raise."""
    store = dist.HashStore()
    slow = F.Heartbeat(store, rank=0, world_size=2, stale_after_s=0.4)
    other = F.Heartbeat(store, rank=1, world_size=2, stale_after_s=0.4)
    progress = {"step": 7}
    slow.start_background(interval_s=0.05, step_fn=lambda: progress["step"])
    try:
        time.sleep(0.9)                # rank 0's main thread is "busy" for more than twice the limit
        other.check_peers()            # must not raise
        assert other.peer_states()[0]["step"] == 7
    finally:
        slow.stop()
    time.sleep(0.6)                    # thread stopped: now the silence is real
    with pytest.raises(F.PeerFailure):
        other.check_peers()
