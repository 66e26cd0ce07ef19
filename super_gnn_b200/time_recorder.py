"""``TimeRecorder`` with the reference's interface (super_gnn/time_recorder.py:8-56):
``TimeRecorder.ctx.time_block(name)`` context managers around the phases of the
hot path, ``set_mode`` / ``set_epoch``, ``report``.

GPU work is asynchronous, so a wall clock around a launch measures nothing.
Blocks are therefore timed with CUDA events on the current stream, resolved
lazily in ``report()`` / ``get_records()``; recording is off unless
``enabled=True`` (two event records per block are not free), and the reference's
per-block ``print`` is off unless ``verbose=True``.
"""
from __future__ import annotations

import time
from collections import defaultdict

import torch


class _NullBlock:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NULL = _NullBlock()


class TimeRecorder(object):
    ctx = None

    def __init__(self, num_layer=0, num_epoch=0, enabled: bool = False, verbose: bool = False) -> None:
        self.mode = None
        self.current_epoch = None
        self.enabled = enabled
        self.verbose = verbose
        self.records = defaultdict(lambda: defaultdict(list))
        self._pending = []  # (module_name, epoch, start_event, end_event)
        TimeRecorder.ctx = self

    def set_mode(self, mode):
        self.mode = mode

    def set_epoch(self, epoch):
        self.current_epoch = epoch

    def time_block(self, module_name, is_record=True):
        if not self.enabled or self.mode != "training":
            return _NULL
        outer = self

        class TimerContext:
            def __enter__(self_inner):
                if torch.cuda.is_available():
                    self_inner.start = torch.cuda.Event(enable_timing=True)
                    self_inner.start.record()
                else:
                    self_inner.start = time.perf_counter()
                return self_inner

            def __exit__(self_inner, exc_type, exc_val, exc_tb):
                if torch.cuda.is_available():
                    end = torch.cuda.Event(enable_timing=True)
                    end.record()
                    if is_record:
                        outer._pending.append((module_name, outer.current_epoch, self_inner.start, end))
                else:
                    ms = (time.perf_counter() - self_inner.start) * 1000.0
                    if is_record:
                        outer.records[module_name][outer.current_epoch].append(ms)
                    if outer.verbose:
                        print(f"Module: {module_name}, Time: {ms:.6f} ms")
                return False

        return TimerContext()

    def _resolve(self):
        if self._pending:
            torch.cuda.synchronize()
            for name, epoch, start, end in self._pending:
                ms = start.elapsed_time(end)
                self.records[name][epoch].append(ms)
                if self.verbose:
                    print(f"Module: {name}, Time: {ms:.6f} ms")
            self._pending = []

    def get_records(self):
        self._resolve()
        return self.records

    def report(self):
        self._resolve()
        for module_name, epochs in self.records.items():
            print(f"Module: {module_name}")
            for epoch, times in epochs.items():
                print(f"  epoch: {epoch}")
                print(f"    Count: {len(times)}")
                print(f"    Avg Time: {sum(times) / len(times):.6f} ms")
                print(f"    Max Time: {max(times):.6f} ms")
                print(f"    Min Time: {min(times):.6f} ms")
            print()


# a disabled recorder exists from import time so that the hot path never has to test for one
TimeRecorder(0, 0)
