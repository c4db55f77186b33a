"""Failure detection and recovery logic, exercised on the host only: the rerun state machine's triage of a bad
result (transient fault / persistent fault / genuine result), cross-rank consensus over Gloo, replayable data
iterators, signal handling, straggler reports, heartbeat time-outs and the simulated-fault timer (with a fake kill).
Mirrors the reference's tests/unit_tests/test_rerun_state_machine... and the fault-tolerance glue tests."""
import os
import signal
import threading
import time

import pytest
import torch

from megatron_lm_b200.training.resilience import (
    EXIT_CODE_FAILED_ON_RESULT_VALIDATION, EXIT_CODE_RESUME_TO_DISAMBIGUATE, DistributedSignalHandler,
    HeartbeatMonitor, QuickStats, RerunDataIterator, RerunDiagnostic, RerunErrorInjector, RerunStateMachine,
    StragglerDetector, maybe_setup_simulated_fault)
from tests.dist_utils import run_distributed


def _too_big(x):
    return bool(x > 100.0)


def _run_step(machine, it, loss_of_batch):
    """One training step in the reference's control-flow shape; returns the list of batches seen by each pass."""
    seen = []
    while machine.should_run_forward_backward(it):
        batch = next(it)
        seen.append(batch)
        machine.validate_result(loss_of_batch(batch), _too_big, "loss", tolerance=0.0)
    return seen


def test_data_iterator_replays_a_step():
    it = RerunDataIterator(iter(range(10)))
    assert [next(it), next(it)] == [0, 1]
    it.rewind()
    assert [next(it), next(it), next(it)] == [0, 1, 2]         # replay, then fresh data
    it.advance()
    assert next(it) == 3
    sd = it.state_dict()
    it2 = RerunDataIterator(iter(range(100, 110)))
    it2.load_state_dict(sd)
    assert next(it2) == 3 and next(it2) == 100


def test_disabled_mode_runs_once():
    m = RerunStateMachine("disabled")
    it = RerunDataIterator(iter(range(5)))
    assert _run_step(m, it, lambda b: 1.0) == [0]
    assert _run_step(m, it, lambda b: 2.0) == [1]
    # nothing is replayed, but a rejected result is still fatal; a non-fatal one passes
    with pytest.raises(RuntimeError, match="validation failed"):
        m.validate_result(1e9, _too_big, "loss")
    m.validate_result(1e9, _too_big, "loss", fatal=False)


def test_spike_detector_needs_history():
    m = RerunStateMachine("disabled")
    for v in range(10):
        assert not m.is_unexpectedly_large(1.0 + 0.01 * v, threshold=10, context="loss", num_samples=10)
    assert not m.is_unexpectedly_large(5.0, threshold=10, context="loss", num_samples=10)
    assert m.is_unexpectedly_large(500.0, threshold=10, context="loss", num_samples=10)
    assert not m.is_unexpectedly_large(500.0, threshold=10, context="other", num_samples=10)   # own history


def test_process_wide_machine():
    from megatron_lm_b200.training.resilience import get_rerun_state_machine, set_rerun_state_machine
    set_rerun_state_machine(None)
    assert get_rerun_state_machine().mode.value == "disabled"
    m = RerunStateMachine("report_stats")
    set_rerun_state_machine(m)
    assert get_rerun_state_machine() is m and m.mode.value == "report_determinism_stats"
    set_rerun_state_machine(None)


def test_clean_step_is_not_replayed():
    m = RerunStateMachine("validate_results")
    it = RerunDataIterator(iter(range(5)))
    assert _run_step(m, it, lambda b: 2.5) == [0]
    assert _run_step(m, it, lambda b: 2.5) == [1]
    assert m.step == 2 and m.diagnostics == [] and m.should_checkpoint_and_exit() == (False, None)


def test_transient_fault_is_replayed_in_place_and_cleared():
    inj = RerunErrorInjector(error_injection_rate=1, error_injection_type="transient_error")
    m = RerunStateMachine("validate_results", error_injector=inj)
    it = RerunDataIterator(iter(range(5)))
    seen = _run_step(m, it, lambda b: 2.5)
    assert seen == [0, 0]                                        # same batch replayed
    assert m.diagnostics == [(0, RerunDiagnostic.TRANSIENT_ERROR, "loss")]
    assert m.should_checkpoint_and_exit() == (False, None)
    assert _run_step(m, it, lambda b: 2.5) == [1]                # training goes on


def test_reproducible_fault_asks_for_replay_elsewhere_and_is_blamed_on_the_device():
    inj = RerunErrorInjector(error_injection_rate=1, error_injection_type="persistent_error")
    m = RerunStateMachine("validate_results", error_injector=inj)
    it = RerunDataIterator(iter(range(5)))
    assert _run_step(m, it, lambda b: 2.5) == [0, 0]
    stop, code = m.should_checkpoint_and_exit()
    assert stop and code == EXIT_CODE_RESUME_TO_DISAMBIGUATE
    sd, it_sd = m.state_dict(), it.state_dict()
    assert sd["state"] == "WILL_RERUN_FROM_CHECKPOINT" and sd["first_result"] > 100
    # "another machine": a fresh state machine without the fault, resumed from the checkpoint
    m2 = RerunStateMachine("validate_results")
    it2 = RerunDataIterator(iter(range(50, 55)))
    m2.load_state_dict(sd)
    it2.load_state_dict(it_sd)
    assert _run_step(m2, it2, lambda b: 2.5) == [0]              # the saved batch, replayed once
    assert m2.diagnostics[-1][1] == RerunDiagnostic.PERSISTENT_ERROR
    assert _run_step(m2, it2, lambda b: 2.5) == [50]


def test_reproducible_result_everywhere_is_a_genuine_failure():
    m = RerunStateMachine("validate_results")
    it = RerunDataIterator(iter(range(5)))
    spike = lambda b: 1e4                                         # the model really produces it
    assert _run_step(m, it, spike) == [0, 0]
    assert m.should_checkpoint_and_exit() == (True, EXIT_CODE_RESUME_TO_DISAMBIGUATE)
    m2 = RerunStateMachine("validate_results")
    it2 = RerunDataIterator(iter(range(5)))
    m2.load_state_dict(m.state_dict())
    it2.load_state_dict(it.state_dict())
    _run_step(m2, it2, spike)
    assert m2.diagnostics[-1][1] == RerunDiagnostic.CORRECT_RESULT
    assert m2.exit_code == EXIT_CODE_FAILED_ON_RESULT_VALIDATION


def test_determinism_report_mode():
    m = RerunStateMachine("report_determinism_stats")
    it = RerunDataIterator(iter(range(5)))
    vals = iter([1.0, 1.0 + 1e-3])
    assert _run_step(m, it, lambda b: next(vals)) == [0, 0]
    mx, mean = m.get_determinism_stats()["loss"]
    assert mx == pytest.approx(1e-3, rel=1e-3) and mean == pytest.approx(1e-3, rel=1e-3)


def test_state_restore_hooks_and_rng_are_rewound():
    saved, restored = [], []
    inj = RerunErrorInjector(1, "transient_error")
    m = RerunStateMachine("validate_results", error_injector=inj, state_save_func=lambda: saved.append(1),
                          state_restore_func=lambda: restored.append(1))
    draws = []
    it = RerunDataIterator(iter(range(3)))
    while m.should_run_forward_backward(it):
        next(it)
        draws.append(torch.rand(1).item())
        m.validate_result(1.0, _too_big, "loss")
    assert len(draws) == 2 and draws[0] == draws[1]
    assert saved == [1] and restored == [1]


def _consensus_rank(rank, world, out):
    inj = RerunErrorInjector(1 if rank == 1 else 0, "transient_error")      # only rank 1 sees the fault
    m = RerunStateMachine("validate_results", error_injector=inj)
    it = RerunDataIterator(iter(range(5)))
    seen = _run_step(m, it, lambda b: 2.0)
    torch.save({"seen": seen, "diag": len(m.diagnostics)}, f"{out}.{rank}")


def test_all_ranks_replay_when_one_rank_rejects(tmp_path):
    out = str(tmp_path / "c")
    run_distributed(_consensus_rank, 2, out)
    r0, r1 = torch.load(f"{out}.0"), torch.load(f"{out}.1")
    assert r0["seen"] == [0, 0] and r1["seen"] == [0, 0]
    assert r0["diag"] == 0 and r1["diag"] == 1


def test_quick_stats():
    q = QuickStats()
    for x in (1.0, 3.0, 2.0):
        q.record(x)
    assert q.max == 3.0 and q.mean() == 2.0


def test_signal_handler_records_and_restores():
    prev = signal.getsignal(signal.SIGUSR1)
    with DistributedSignalHandler(signal.SIGUSR1) as h:
        assert h.signals_received() == [False]
        os.kill(os.getpid(), signal.SIGUSR1)
        time.sleep(0.05)
        assert h.signals_received() == [True]
    assert signal.getsignal(signal.SIGUSR1) == prev


def _signal_rank(rank, world, out):
    with DistributedSignalHandler(signal.SIGUSR1) as h:
        if rank == 1:
            os.kill(os.getpid(), signal.SIGUSR1)
            time.sleep(0.05)
        torch.save(h.signals_received(), f"{out}.{rank}")


def test_signal_seen_by_every_rank(tmp_path):
    out = str(tmp_path / "s")
    run_distributed(_signal_rank, 2, out)
    assert torch.load(f"{out}.0") == [False, True] and torch.load(f"{out}.1") == [False, True]


def _straggler_rank(rank, world, out):
    d = StragglerDetector()
    d._ev = None
    d._t0 = time.perf_counter()
    time.sleep(0.15 if rank == 1 else 0.01)
    if d._ev is not None:
        d._ev = None
    d.times.append(time.perf_counter() - d._t0)
    torch.save(d.report(1, 1e12), f"{out}.{rank}")


def test_straggler_report_names_the_slow_rank(tmp_path):
    out = str(tmp_path / "g")
    run_distributed(_straggler_rank, 2, out)
    rep = torch.load(f"{out}.0")
    assert rep["max"][0] == 1 and rep["min"][0] == 0 and rep["max"][1] > rep["min"][1]


def _toggle_rank(rank, world, out):
    import json
    import urllib.request
    d = StragglerDetector(enabled=False, port=0, minmax_count=2)         # port 0: the system picks a free one
    log = []
    d.start(); d.stop()
    log.append(len(d.times))                                            # disabled: nothing measured
    log.append(d.report(1))                                             # ... and nothing reported
    if rank == 0:
        assert d.port
        reply = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{d.port}/", timeout=5).read())
        assert reply == {"straggler_detector_enabled": True}
    else:
        assert d.port is None
    torch.distributed.barrier()
    log.append(d.enabled)                                               # still off: the flag travels with a report
    d.report(2)
    log.append(d.enabled)                                               # on, on every rank
    d.start(); time.sleep(0.02 * (rank + 1)); d.stop()
    rep = d.report(3)
    log.append((rep["slowest"][0][0], len(rep["slowest"]), rep["enabled"]))
    d.close()
    torch.save(log, f"{out}.{rank}")


def test_straggler_detector_is_toggled_through_its_port(tmp_path):
    out = str(tmp_path / "t")
    run_distributed(_toggle_rank, 2, out)
    for r in range(2):
        assert torch.load(f"{out}.{r}") == [0, None, False, True, (1, 2, True)]


def test_heartbeat_timeout_fires_and_timeouts_persist(tmp_path):
    fired = []
    path = str(tmp_path / "ft_state.json")
    hb = HeartbeatMonitor({"step": 0.15, "setup": 5.0}, on_timeout=lambda s, dt: fired.append((s, dt)), poll_s=0.02,
                          state_path=path)
    try:
        hb.start_section("setup")
        time.sleep(0.1)
        hb.end_section()
        hb.start_section("step")
        for _ in range(3):                       # healthy: beats arrive in time
            time.sleep(0.05)
            hb.heartbeat()
        assert fired == []
        time.sleep(0.4)                          # a hung step: no beats
        assert fired and fired[0][0] == "step" and fired[0][1] > 0.15
        hb.end_section()
        hb.calculate_and_persist_timeouts(safety_factor=2.0)
    finally:
        hb.shutdown()
    hb2 = HeartbeatMonitor(state_path=path, poll_s=0.05)
    try:
        assert hb2.timeouts["step"] >= 1.0 and "setup" in hb2.timeouts
    finally:
        hb2.shutdown()


def test_simulated_fault_picks_one_victim_and_uses_the_kill_hook(monkeypatch):
    monkeypatch.setenv("FT_SIM_FAULT_DESC", "rank_killed,0.05")
    monkeypatch.setenv("FT_SIM_FAULT_SEED", "3")
    calls = []
    done = threading.Event()

    def fake_kill(pid, signum):
        calls.append((pid, signum))
        done.set()
    timers = [maybe_setup_simulated_fault(rank=r, world_size=4, kill_fn=fake_kill) for r in range(4)]
    assert sum(t is not None for t in timers) == 1              # the same victim on every rank
    assert done.wait(2.0)
    assert calls == [(os.getpid(), signal.SIGKILL)]
    monkeypatch.delenv("FT_SIM_FAULT_DESC")
    assert maybe_setup_simulated_fault(rank=0, world_size=4) is None


def test_several_validations_per_step_are_matched_by_position():
    """Three microbatches per step, the second one glitches once: only that call is compared on the replay."""
    m = RerunStateMachine("validate_results")
    it = RerunDataIterator(iter(range(20)))
    passes = []
    glitch = {"armed": True}
    while m.should_run_forward_backward(it):
        vals = []
        for mb in range(3):
            b = next(it)
            v = 1.0 + b
            if mb == 1 and glitch["armed"]:
                v, glitch["armed"] = 1e9, False
            vals.append(v)
            m.validate_result(v, _too_big, "loss")
        passes.append(vals)
    assert len(passes) == 2 and passes[1] == [1.0, 2.0, 3.0]
    assert m.diagnostics == [(0, RerunDiagnostic.TRANSIENT_ERROR, "loss")]
    assert m.should_checkpoint_and_exit() == (False, None)
