"""Number of microbatches per step, constant or ramped up (reference:
megatron/core/num_microbatches_calculator.py: constant :298, ramp-up :360, globals :17-144).
Ramp-up: the global batch grows from ``start`` by ``increment`` every
``ramp_samples / ((global - start) / increment)`` consumed samples until it reaches ``global``."""
from __future__ import annotations

from typing import List, Optional


class NumMicroBatchesCalculator:
    def __init__(self):
        self.num_micro_batches = None
        self.current_global_batch_size = None
        self.micro_batch_size = None
        self.current_running_global_batch_size = None

    def get(self) -> int:
        return self.num_micro_batches

    def get_current_global_batch_size(self) -> int:
        return self.current_global_batch_size

    def get_micro_batch_size(self) -> int:
        return self.micro_batch_size

    def get_current_running_global_batch_size(self) -> int:
        return self.current_running_global_batch_size

    def update(self, consumed_samples: int, consistency_check: bool, verbose: bool = False) -> None:
        pass


class ConstantNumMicroBatchesCalculator(NumMicroBatchesCalculator):
    def __init__(self, global_batch_size: int, micro_batch_size: int, data_parallel_size: int,
                 decrease_batch_size_if_needed: bool = False, rank: int = 0):
        super().__init__()
        per = micro_batch_size * data_parallel_size
        if decrease_batch_size_if_needed:
            running = (global_batch_size // per) * per
            if running <= 0:
                raise ValueError("global batch smaller than micro batch x data parallel size")
            self.num_micro_batches = running // per
        else:
            if global_batch_size % per != 0:
                raise ValueError(f"global batch size ({global_batch_size}) is not divisible by micro batch size "
                                 f"({micro_batch_size}) times data parallel size ({data_parallel_size})")
            running = global_batch_size
            self.num_micro_batches = global_batch_size // per
        if self.num_micro_batches < 1:
            raise ValueError("number of microbatches must be at least 1")
        self.current_global_batch_size = global_batch_size
        self.current_running_global_batch_size = running
        self.micro_batch_size = micro_batch_size


class RampupBatchsizeNumMicroBatchesCalculator(NumMicroBatchesCalculator):
    def __init__(self, global_batch_size: int, micro_batch_size: int, data_parallel_size: int,
                 decrease_batch_size_if_needed: bool, rank: int, start_global_batch_size: int,
                 batch_size_increment: int, ramup_samples: int):
        super().__init__()
        if start_global_batch_size <= 0 or batch_size_increment <= 0 or ramup_samples < 0:
            raise ValueError("bad ramp-up parameters")
        diff = global_batch_size - start_global_batch_size
        if diff < 0 or diff % batch_size_increment != 0:
            raise ValueError("global batch minus start batch must be a non-negative multiple of the increment")
        self.global_batch_size = global_batch_size
        self.micro_batch_size = micro_batch_size
        self.data_parallel_size = data_parallel_size
        self.decrease = decrease_batch_size_if_needed
        self.start = start_global_batch_size
        self.increment = batch_size_increment
        self.ramup_samples = ramup_samples
        self.per = micro_batch_size * data_parallel_size
        n_inc = diff // batch_size_increment
        self.samples_per_increment = ramup_samples / n_inc if n_inc > 0 else 0
        self.update(0, False)

    def update(self, consumed_samples: int, consistency_check: bool, verbose: bool = False) -> None:
        if consumed_samples > self.ramup_samples or self.samples_per_increment == 0:
            cur = self.global_batch_size
        else:
            cur = self.start + int(consumed_samples / self.samples_per_increment) * self.increment
            cur = min(cur, self.global_batch_size)
        self.current_global_batch_size = cur
        if consistency_check and not self.decrease and cur % self.per != 0:
            raise ValueError(f"current global batch size ({cur}) is not divisible by micro-batch-size x "
                             f"data-parallel-size ({self.per})")
        if self.decrease and cur % self.per != 0:
            self.current_running_global_batch_size = (cur // self.per) * self.per
        else:
            self.current_running_global_batch_size = cur
        self.num_micro_batches = max(self.current_running_global_batch_size // self.per, 1)


_CALC: Optional[NumMicroBatchesCalculator] = None


def init_num_microbatches_calculator(rank: int, rampup_batch_size: Optional[List[int]], global_batch_size: int,
                                     micro_batch_size: int, data_parallel_size: int,
                                     decrease_batch_size_if_needed: bool = False) -> None:
    global _CALC
    if rampup_batch_size is None:
        _CALC = ConstantNumMicroBatchesCalculator(global_batch_size, micro_batch_size, data_parallel_size,
                                                  decrease_batch_size_if_needed, rank)
    else:
        if len(rampup_batch_size) != 3:
            raise ValueError("--rampup-batch-size takes <start> <increment> <ramp-up samples>")
        s, i, r = (int(x) for x in rampup_batch_size)
        _CALC = RampupBatchsizeNumMicroBatchesCalculator(global_batch_size, micro_batch_size, data_parallel_size,
                                                         decrease_batch_size_if_needed, rank, s, i, r)


def get_num_microbatches() -> int:
    return _CALC.get()


def get_current_global_batch_size() -> int:
    return _CALC.get_current_global_batch_size()


def get_micro_batch_size() -> int:
    return _CALC.get_micro_batch_size()


def get_current_running_global_batch_size() -> int:
    return _CALC.get_current_running_global_batch_size()


def update_num_microbatches(consumed_samples: int, consistency_check: bool = True, verbose: bool = False) -> None:
    _CALC.update(consumed_samples, consistency_check, verbose)


def destroy_num_microbatches_calculator() -> None:
    global _CALC
    _CALC = None
