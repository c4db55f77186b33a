"""Failure detection and recovery aids, all host-side.

* ``RerunStateMachine`` - numerical-fault triage (reference: megatron/core/rerun_state_machine.py:127):
  a suspicious result (NaN / Inf / spike) makes every rank replay the same step in place; a
  different result on replay is a *transient* fault of this device, an identical one asks for a
  checkpoint-and-restart so the step can be replayed on other hardware (identical again -> the
  result was *correct*, different -> *persistent* fault of the first device).  Consensus runs on
  CPU tensors over a Gloo group when one is available, so triage never depends on the device
  under suspicion.
* ``RerunErrorInjector`` - corrupts a validated scalar with a given probability (:1181).
* ``DistributedSignalHandler`` - catches SIGTERM and lets all ranks agree to save and exit
  (megatron/training/dist_signal_handler.py:51).
* ``StragglerDetector`` - per-rank timing of the step, min/max ranks reported (core/utils.py:1159).
* ``HeartbeatMonitor`` / ``maybe_setup_simulated_fault`` - section heartbeats with timeouts and the
  ``FT_SIM_FAULT_DESC`` fault simulator (megatron/training/ft_integration.py:75-367): a watchdog
  thread flags a rank whose section outlives its timeout; the simulator stops or kills the *host
  process* of a chosen rank after a delay.  No GPU is ever faulted.
"""
from __future__ import annotations

import enum
import json
import math
import os
import random
import signal
import threading
import time
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

EXIT_CODE_RESUME_TO_DISAMBIGUATE = 16
EXIT_CODE_FAILED_ON_RESULT_VALIDATION = 17


class RerunMode(str, enum.Enum):
    DISABLED = "disabled"
    VALIDATE_RESULTS = "validate_results"
    REPORT_DETERMINISM_STATS = "report_determinism_stats"


class RerunState(enum.Enum):
    NOT_RUNNING_YET = 0
    INITIAL_RUN = 1
    RERUNNING_IN_PLACE = 2
    WILL_RERUN_FROM_CHECKPOINT = 3
    RERUNNING_FROM_CHECKPOINT = 4
    RERUNNING_AGAIN_FROM_CHECKPOINT = 5


class RerunDiagnostic(str, enum.Enum):
    CORRECT_RESULT = "correct_result"
    TRANSIENT_ERROR = "transient_error"
    PERSISTENT_ERROR = "persistent_error"


class RerunDataIterator:
    """Wraps an iterator so that a step's batches can be replayed."""

    def __init__(self, it: Iterable):
        self.it = iter(it)
        self.saved: List[Any] = []
        self.replaying = False
        self.pos = 0

    def __next__(self):
        if self.replaying:
            if self.pos < len(self.saved):
                x = self.saved[self.pos]
                self.pos += 1
                return x
            self.replaying = False
        x = next(self.it)
        self.saved.append(x)
        return x

    def __iter__(self):
        return self

    def rewind(self):
        self.replaying, self.pos = True, 0

    def advance(self):
        self.saved, self.replaying, self.pos = [], False, 0

    def state_dict(self):
        return {"saved": self.saved}

    def load_state_dict(self, sd):
        self.saved = sd["saved"]
        self.rewind()


class RerunErrorInjector:
    def __init__(self, error_injection_rate: int = 0, error_injection_type: str = "transient_error"):
        self.rate, self.kind = error_injection_rate, RerunDiagnostic(error_injection_type)
        self.injected_step: Optional[int] = None
        self.rng = random.Random(1234)

    def maybe_inject(self, step: int, is_rerun: bool) -> bool:
        if self.rate <= 0:
            return False
        if self.injected_step is None and not is_rerun and self.rng.randint(0, self.rate - 1) == 0:
            self.injected_step = step
            return True
        if self.injected_step == step and is_rerun:
            # transient: the fault is gone on replay; persistent / "correct": it reproduces
            return self.kind != RerunDiagnostic.TRANSIENT_ERROR
        return False

    def corrupt(self, value: float) -> float:
        return value * 1.0e6 + 1.0


class RerunStateMachine:
    def __init__(self, mode: str = "validate_results", error_injector: Optional[RerunErrorInjector] = None,
                 cpu_group=None, state_save_func: Optional[Callable] = None, state_restore_func: Optional[Callable] = None):
        self.mode = RerunMode({"report_stats": "report_determinism_stats"}.get(mode, mode))
        self.state = RerunState.NOT_RUNNING_YET
        self.injector = error_injector or RerunErrorInjector()
        self.cpu_group = cpu_group
        self.save_fn, self.restore_fn = state_save_func, state_restore_func
        self.step = 0
        self.rerun_requested = False
        self.first_result: Optional[float] = None
        self.suspicious_device: Optional[str] = None
        self.checkpoint_and_exit = False
        self.exit_code: Optional[int] = None
        self.diagnostics: List[tuple] = []
        self.saved_rng = None
        self.stats: Dict[str, List[float]] = {}
        self._resume_pending = False
        self._spike_stats: Dict[str, "QuickStats"] = {}
        # a step validates once per microbatch: calls are told apart by their position within the pass
        self._call_idx = 0
        self._first_results: Dict[int, float] = {}
        self._suspect_idx: Optional[int] = None

    # -- consensus ------------------------------------------------------------
    def _any(self, flag: bool) -> bool:
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return flag
        group = self.cpu_group
        if group is None and dist.get_backend() != "gloo":
            t = torch.tensor([int(flag)], dtype=torch.int32, device="cuda")
        else:
            t = torch.tensor([int(flag)], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return bool(t.item())

    # -- loop control -----------------------------------------------------------
    def should_run_forward_backward(self, data_iterator=None) -> bool:
        """Call in ``while machine.should_run_forward_backward(it): fwd_bwd()``."""
        its = data_iterator if isinstance(data_iterator, (list, tuple)) else [data_iterator]
        its = [i for i in its if isinstance(i, RerunDataIterator)]
        self._call_idx = 0
        if self.mode == RerunMode.DISABLED:
            if self.state == RerunState.NOT_RUNNING_YET:
                self.state = RerunState.INITIAL_RUN
                return True
            self.state = RerunState.NOT_RUNNING_YET
            return False
        if self.state == RerunState.NOT_RUNNING_YET:
            self.state = RerunState.INITIAL_RUN
            self.rerun_requested = False
            self.saved_rng = self._rng_snapshot()
            if self.save_fn:
                self.save_fn()
            for i in its:
                i.advance()
            return True
        if self.state == RerunState.INITIAL_RUN:
            want = self.rerun_requested or self.mode == RerunMode.REPORT_DETERMINISM_STATS
            if self._any(want):
                self.state = RerunState.RERUNNING_IN_PLACE
                self._restore(its)
                return True
            return self._finish(its)
        if self.state == RerunState.RERUNNING_IN_PLACE:
            if self._any(self.checkpoint_and_exit):
                self.state = RerunState.WILL_RERUN_FROM_CHECKPOINT
                self.checkpoint_and_exit = True
                self.exit_code = EXIT_CODE_RESUME_TO_DISAMBIGUATE
            return self._finish(its)
        if self.state in (RerunState.RERUNNING_FROM_CHECKPOINT, RerunState.RERUNNING_AGAIN_FROM_CHECKPOINT):
            if self._resume_pending:
                # first call after a resume: replay the saved step (on possibly different hardware)
                self._resume_pending = False
                if self.saved_rng is not None:
                    self._rng_apply(self.saved_rng)      # the generators as they were when the step first ran
                for i in its:
                    i.rewind()
                return True
            return self._finish(its)
        return self._finish(its)

    @staticmethod
    def _rng_snapshot():
        """Default CPU / CUDA generators and the named model-parallel generators at the start of a step."""
        from ..parallel.random import get_cuda_rng_tracker
        return (torch.get_rng_state(), torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
                get_cuda_rng_tracker().get_states())

    @staticmethod
    def _rng_apply(snap):
        from ..parallel.random import get_cuda_rng_tracker
        torch.set_rng_state(snap[0])
        if snap[1] is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(snap[1])
        if len(snap) > 2 and snap[2]:
            get_cuda_rng_tracker().set_states(snap[2])

    def _restore(self, its):
        self._rng_apply(self.saved_rng)
        if self.restore_fn:
            self.restore_fn()
        for i in its:
            i.rewind()

    def _finish(self, its) -> bool:
        if self.state == RerunState.WILL_RERUN_FROM_CHECKPOINT:
            # the step is not over: the checkpoint written now carries its first result for the replay
            return False
        self.state = RerunState.NOT_RUNNING_YET
        self.step += 1
        self.first_result = None
        return False

    def _track_rejection(self, value: float, message: str, injected: bool) -> None:
        """--result-rejected-tracker-filename: one JSON line per rejected result (iteration, rank, value, reason), so
        that a scheduler can spot the device that keeps producing them (reference: rerun_state_machine.py:700-760)."""
        path = getattr(self, "rejected_tracker_filename", None)
        if not path:
            return
        rec = {"step": self.step, "rank": dist.get_rank() if dist.is_initialized() else 0, "value": value,
               "message": message, "injected": bool(injected), "time": time.time()}
        try:
            with open(path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        except OSError:
            pass

    # -- validation ---------------------------------------------------------------
    def validate_result(self, result, rejection_func: Callable[[Any], bool], message: str = "unexpected result",
                        tolerance: float = 0.0, fatal: bool = True) -> None:
        """Call from the loss function with the value to check (e.g. the loss)."""
        if self.mode == RerunMode.DISABLED:
            # no replay machinery, but a rejected result is still an error (reference: rerun_state_machine.py:470)
            if fatal and rejection_func(result if torch.is_tensor(result) else torch.tensor(float(result))):
                raise RuntimeError(f"result validation failed: {message} (value {float(result)})")
            return
        val = float(result.item()) if torch.is_tensor(result) else float(result)
        idx = self._call_idx
        self._call_idx += 1
        rerun = self.state != RerunState.INITIAL_RUN
        injected = self.injector.maybe_inject(self.step, rerun)
        if injected:
            val = self.injector.corrupt(val)
        if self.state == RerunState.INITIAL_RUN:
            if idx == 0:
                self._first_results, self._suspect_idx = {}, None
            self._first_results[idx] = val
            if not self.rerun_requested:
                self.first_result = val
            # an injected fault counts as rejected whatever the test is: it exercises the replay path
            if (self.mode == RerunMode.VALIDATE_RESULTS and not self.rerun_requested
                    and (injected or rejection_func(torch.tensor(val)))):
                self.rerun_requested = True
                self._suspect_idx = idx
                self.suspicious_device = f"rank {dist.get_rank() if dist.is_initialized() else 0}"
                self._track_rejection(val, message, injected)
        elif self.state == RerunState.RERUNNING_IN_PLACE:
            if self.mode == RerunMode.REPORT_DETERMINISM_STATS:
                first = self._first_results.get(idx, self.first_result)
                rel = abs(val - first) / max(abs(first), 1e-30)
                self.stats.setdefault(message, []).append(rel)
                return
            if self.first_result is None or idx != (self._suspect_idx or 0):
                return
            same = self._same(val, self.first_result, tolerance)
            if not same:
                self.diagnostics.append((self.step, RerunDiagnostic.TRANSIENT_ERROR, message))
            else:
                # reproducible on this device: replay elsewhere to tell a real spike from a bad device
                self.checkpoint_and_exit = True
        elif self.state == RerunState.RERUNNING_FROM_CHECKPOINT:
            if idx != (self._suspect_idx or 0):
                return
            same = self.first_result is None or self._same(val, self.first_result, tolerance)
            self.diagnostics.append((self.step, RerunDiagnostic.CORRECT_RESULT if same
                                     else RerunDiagnostic.PERSISTENT_ERROR, message))
            if same and fatal and rejection_func(torch.tensor(val)):
                self.exit_code = EXIT_CODE_FAILED_ON_RESULT_VALIDATION

    def is_unexpectedly_large(self, result, threshold: float, context: str, num_samples: int = 100) -> bool:
        """Spike test for ``validate_result``: True when ``result`` exceeds ``threshold`` times the largest value seen
        so far in this ``context``, once ``num_samples`` values have been seen (reference:
        rerun_state_machine.py:559).  Values that pass are added to the history."""
        val = float(result.item()) if torch.is_tensor(result) else float(result)
        st = self._spike_stats.setdefault(context, QuickStats())
        if st.n >= num_samples and val > threshold * st.max:
            return True
        if self.state in (RerunState.NOT_RUNNING_YET, RerunState.INITIAL_RUN) or self.mode == RerunMode.DISABLED:
            st.record(val)
        return False

    @staticmethod
    def _same(a: float, b: float, tol: float) -> bool:
        if math.isnan(a) and math.isnan(b):
            return True
        return abs(a - b) <= tol * max(abs(a), abs(b), 1e-30)

    def should_checkpoint_and_exit(self):
        return self.checkpoint_and_exit, self.exit_code

    def get_determinism_stats(self):
        return {k: (max(v) if v else 0.0, sum(v) / max(len(v), 1)) for k, v in self.stats.items()}

    def state_dict(self, data_iterator=None):
        return {"mode": self.mode.value, "state": self.state.name, "step": self.step,
                "first_result": self.first_result, "suspect_idx": self._suspect_idx, "saved_rng": self.saved_rng,
                "suspicious_device": self.suspicious_device,
                "diagnostics": [(s, d.value, m) for s, d, m in self.diagnostics]}

    def load_state_dict(self, sd):
        self.step = sd["step"]
        self.first_result = sd.get("first_result")
        self._suspect_idx = sd.get("suspect_idx")
        self.saved_rng = sd.get("saved_rng")
        self.suspicious_device = sd.get("suspicious_device")
        if sd.get("state") == RerunState.WILL_RERUN_FROM_CHECKPOINT.name:
            self.state = RerunState.RERUNNING_FROM_CHECKPOINT
            # the next fwd/bwd is the replay on (possibly) different hardware
            self._resume_pending = True


class QuickStats:
    """Running max / mean of a stream of numbers (reference: rerun_state_machine.py:1096)."""

    def __init__(self):
        self.n, self.total, self.max = 0, 0.0, 0.0

    def record(self, x: float):
        self.n += 1
        self.total += x
        self.max = max(self.max, x)

    def mean(self):
        return self.total / max(self.n, 1)


# ----------------------------------------------------------------------------- signals
class DistributedSignalHandler:
    def __init__(self, sig=signal.SIGTERM):
        self.sig = sig
        self._received = False
        self._prev = None

    def __enter__(self):
        self._received = False
        try:
            self._prev = signal.getsignal(self.sig)
            signal.signal(self.sig, self._handle)
        except ValueError:
            self._prev = None           # not in the main thread
        return self

    def _handle(self, signum, frame):
        self._received = True

    def signals_received(self) -> List[bool]:
        """Whether each rank has received the signal (one all-gather)."""
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return [self._received]
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        mine = torch.tensor([int(self._received)], dtype=torch.int32, device=dev)
        out = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(out, mine)
        return [bool(t.item()) for t in out]

    def __exit__(self, *a):
        if self._prev is not None:
            signal.signal(self.sig, self._prev)
        return False


# ----------------------------------------------------------------------------- stragglers
class StragglerDetector:
    """Per-rank step times, gathered at report time: the slowest and fastest ``minmax_count`` ranks are printed.

    Measurement can be switched on and off while the job runs: with ``port`` set, rank 0 listens on that TCP port and
    every HTTP GET toggles its flag and answers with the new state; the flag travels to the other ranks with the next
    report's gather, so all ranks switch at the same step (reference: megatron/core/utils.py ``StragglerDetector``
    - ``--straggler-ctrlr-port``, ``--disable-straggler-on-startup``, ``--straggler-minmax-count``)."""

    def __init__(self, enabled: bool = True, port: Optional[int] = None, minmax_count: int = 1):
        self.times: List[float] = []
        self._t0 = None
        self._ev = None
        self.enabled = enabled                 # what start/stop obey (identical on all ranks between reports)
        self._requested = enabled              # rank 0: what the controller last asked for
        self.minmax_count = max(int(minmax_count), 1)
        self.port = None
        self._server = None
        rank0 = not dist.is_initialized() or dist.get_rank() == 0
        if port is not None and rank0:
            self._serve(port)

    # -- controller -----------------------------------------------------------------------------------------------
    def _serve(self, port: int):
        import socket
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            srv.bind(("0.0.0.0", port))
        except OSError as e:
            print(f" straggler controller: cannot listen on port {port} ({e}); the toggle is unavailable", flush=True)
            srv.close()
            return
        srv.listen(4)
        srv.settimeout(0.5)
        self.port = srv.getsockname()[1]
        self._server = srv
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    conn, _ = srv.accept()
                except OSError:
                    continue
                try:
                    conn.settimeout(1.0)
                    conn.recv(1024)
                    self._requested = not self._requested
                    body = json.dumps({"straggler_detector_enabled": self._requested})
                    conn.sendall((f"HTTP/1.0 200 OK\r\nContent-Type: application/json\r\nContent-Length: {len(body)}"
                                  f"\r\n\r\n{body}").encode())
                except OSError:
                    pass
                finally:
                    conn.close()
        threading.Thread(target=loop, daemon=True).start()

    def close(self):
        if self._server is not None:
            self._stop.set()
            self._server.close()
            self._server = None

    # -- measurement ----------------------------------------------------------------------------------------------
    def start(self):
        if not self.enabled:
            return
        if torch.cuda.is_available():
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        else:
            self._t0 = time.perf_counter()

    def stop(self):
        if self._ev is not None:
            self._ev[1].record()
            self._ev[1].synchronize()
            self.times.append(self._ev[0].elapsed_time(self._ev[1]) / 1e3)
            self._ev = None
        elif self._t0 is not None:
            self.times.append(time.perf_counter() - self._t0)
            self._t0 = None

    def report(self, iteration: int, flops_per_step: Optional[float] = None) -> Optional[dict]:
        was_enabled = self.enabled
        mine = sum(self.times) / max(len(self.times), 1) if self.times else 0.0
        self.times = []
        if not dist.is_initialized() or dist.get_world_size() == 1:
            self.enabled = self._requested
            if not was_enabled:
                return None
            print(f" straggler report @ {iteration}: one rank, {mine * 1e3:.1f} ms per step", flush=True)
            return {"min": (0, mine), "max": (0, mine), "fastest": [(0, mine)], "slowest": [(0, mine)],
                    "enabled": self.enabled}
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        t = torch.tensor([mine, 1.0 if self._requested else 0.0], dtype=torch.float32, device=dev)
        allt = [torch.zeros_like(t) for _ in range(dist.get_world_size())]
        dist.all_gather(allt, t)
        self.enabled = self._requested = bool(allt[0][1].item() > 0.5)          # rank 0's controller decides
        if not was_enabled:
            return None
        vals = [float(x[0].item()) for x in allt]
        order = sorted(range(len(vals)), key=vals.__getitem__)
        lo, hi = order[0], order[-1]
        n = min(self.minmax_count, len(vals))
        rep = {"min": (lo, vals[lo]), "max": (hi, vals[hi]), "fastest": [(r, vals[r]) for r in order[:n]],
               "slowest": [(r, vals[r]) for r in order[::-1][:n]], "enabled": self.enabled}
        if dist.get_rank() == 0:
            msg = f" straggler report @ {iteration}: fastest rank {lo} {vals[lo] * 1e3:.1f} ms, slowest rank {hi} {vals[hi] * 1e3:.1f} ms"
            if flops_per_step:
                msg += f" ({flops_per_step / max(vals[hi], 1e-9) / 1e12:.1f} vs {flops_per_step / max(vals[lo], 1e-9) / 1e12:.1f} TFLOP/s)"
            if n > 1:
                msg += " | slowest: " + ", ".join(f"{r}:{v * 1e3:.1f}" for r, v in rep["slowest"]) + \
                       " | fastest: " + ", ".join(f"{r}:{v * 1e3:.1f}" for r, v in rep["fastest"])
            print(msg, flush=True)
        return rep


# ----------------------------------------------------------------------------- heartbeats / simulated faults
class HeartbeatMonitor:
    """Sections (setup / step / checkpointing) with timeouts; a watchdog thread calls ``on_timeout``
    when the open section, or the gap between heartbeats inside it, outlives its limit.  Observed
    durations can be turned into timeouts and persisted (``ft_state.json`` in the reference)."""

    def __init__(self, timeouts: Optional[Dict[str, float]] = None, on_timeout: Optional[Callable[[str, float], None]] = None,
                 poll_s: float = 0.2, state_path: Optional[str] = None):
        self.timeouts = dict(timeouts or {"setup": 600.0, "step": 180.0, "checkpointing": 600.0})
        self.on_timeout = on_timeout or (lambda section, dt: None)
        self.poll_s, self.state_path = poll_s, state_path
        self.section: Optional[str] = None
        self.last_beat = time.monotonic()
        self.observed: Dict[str, float] = {}
        self.timed_out: List[tuple] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._watch, daemon=True)
        self._lock = threading.Lock()
        if state_path and os.path.isfile(state_path):
            with open(state_path) as f:
                self.timeouts.update(json.load(f).get("timeouts", {}))
        self._thread.start()

    def start_section(self, name: str):
        with self._lock:
            self.section, self.last_beat = name, time.monotonic()

    def heartbeat(self):
        with self._lock:
            now = time.monotonic()
            if self.section:
                self.observed[self.section] = max(self.observed.get(self.section, 0.0), now - self.last_beat)
            self.last_beat = now

    def end_section(self):
        self.heartbeat()
        with self._lock:
            self.section = None

    def _watch(self):
        while not self._stop.wait(self.poll_s):
            with self._lock:
                sec, dt = self.section, time.monotonic() - self.last_beat
            if sec is not None and dt > self.timeouts.get(sec, float("inf")):
                self.timed_out.append((sec, dt))
                self.on_timeout(sec, dt)
                with self._lock:
                    self.last_beat = time.monotonic()

    def calculate_and_persist_timeouts(self, safety_factor: float = 5.0):
        for k, v in self.observed.items():
            self.timeouts[k] = max(v * safety_factor, 1.0)
        if self.state_path:
            with open(self.state_path, "w") as f:
                json.dump({"timeouts": self.timeouts}, f)

    def shutdown(self):
        self._stop.set()
        self._thread.join(timeout=2)


def maybe_setup_simulated_fault(rank: Optional[int] = None, world_size: Optional[int] = None,
                                kill_fn: Optional[Callable[[int, int], None]] = None) -> Optional[threading.Timer]:
    """``FT_SIM_FAULT_DESC="rank_hung|rank_killed,<base_delay_s>"``: one rank (chosen from a seed all
    ranks share) stops (SIGSTOP) or kills (SIGKILL) its own host process after a random delay."""
    desc = os.environ.get("FT_SIM_FAULT_DESC")
    if not desc:
        return None
    kind, base = desc.split(",")
    kind, base = kind.strip(), float(base)
    if kind not in ("rank_hung", "rank_killed", "random"):
        raise ValueError(f"unknown simulated fault {kind}")
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
    rng = random.Random(int(os.environ.get("FT_SIM_FAULT_SEED", "0")))
    if kind == "random":
        kind = rng.choice(["rank_hung", "rank_killed"])
    victim = rng.randint(0, world_size - 1)
    delay = base + rng.random() * base * 0.5
    if rank != victim:
        return None
    signum = signal.SIGSTOP if kind == "rank_hung" else signal.SIGKILL
    fn = kill_fn or os.kill
    t = threading.Timer(delay, lambda: fn(os.getpid(), signum))
    t.daemon = True
    t.start()
    return t


# ----------------------------------------------------------------------------- process-wide state machine
_RERUN_MACHINE: Optional[RerunStateMachine] = None


def set_rerun_state_machine(machine: Optional[RerunStateMachine]) -> None:
    global _RERUN_MACHINE
    _RERUN_MACHINE = machine


def get_rerun_state_machine() -> RerunStateMachine:
    """The machine of this process (a disabled one when the program did not configure any), for loss functions
    that validate their result (reference: rerun_state_machine.py:1196 get_rerun_state_machine)."""
    global _RERUN_MACHINE
    if _RERUN_MACHINE is None:
        _RERUN_MACHINE = RerunStateMachine("disabled")
    return _RERUN_MACHINE


SPIKY_LOSS_FACTOR = 10      # a loss this many times the largest seen so far is replayed (reference: pretrain_gpt.py:56)


def validate_loss(loss, args) -> None:
    """NaN / Inf / spike tests of one microbatch's loss through the process-wide machine, under the flags
    ``--check-for-nan-in-loss-and-grad`` and ``--check-for-spiky-loss`` (reference: pretrain_gpt.py:248-278).  Costs
    one host read of the loss."""
    check_nan = getattr(args, "check_for_nan_in_loss_and_grad", False)
    check_spike = getattr(args, "check_for_spiky_loss", False)
    if not (check_nan or check_spike):
        return
    machine = get_rerun_state_machine()
    value = float(loss)
    if check_nan:
        machine.validate_result(value, lambda x: bool(torch.isnan(x)), "found NaN in local forward loss calculation",
                                tolerance=0.0, fatal=True)
        machine.validate_result(value, lambda x: bool(torch.isinf(x)), "found Inf in local forward loss calculation",
                                tolerance=0.0, fatal=True)
    if check_spike:
        def spiky(x):
            return machine.is_unexpectedly_large(x, threshold=SPIKY_LOSS_FACTOR, context="loss")
        machine.validate_result(value, spiky, "Spiky loss", tolerance=0.0, fatal=False)
