"""Wall-clock timer around ``torch.cuda.synchronize()``.

Same interface as TorchEx's ``TorchTimer`` (torchex/operator_py/timer.py:4-41):
``timer.timing(name)`` is a context manager and the running mean is printed
every ``print_freq`` uses; ``print_freq == -1`` switches a timer off.  The
benchmark in this repository times with CUDA events instead; this class exists
so scripts written against TorchEx keep running.
"""
import time

import torch


class _Section:
    def __init__(self, label, every):
        self.label = label
        self.every = every
        self.total_s = 0.0
        self.uses = 0
        self._t0 = 0.0
        self.last_mean_ms = None

    def _sync(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def __enter__(self):
        if self.every > 0:
            self._sync()
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.every <= 0:
            return False
        self._sync()
        self.total_s += time.perf_counter() - self._t0
        self.uses += 1
        if self.uses % self.every == 0:
            self.last_mean_ms = 1e3 * self.total_s / self.uses
            print("Average time cost of {}: {:.4}ms".format(self.label, self.last_mean_ms))
            self.total_s, self.uses = 0.0, 0
        return False


class TorchTimer:
    def __init__(self, print_freq=10):
        self.print_freq = print_freq
        self.timer_dict = {}

    def timing(self, name, freq=None):
        if name not in self.timer_dict:
            self.timer_dict[name] = _Section(name, self.print_freq if freq is None else freq)
        return self.timer_dict[name]
