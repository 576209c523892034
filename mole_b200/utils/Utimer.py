"""CUDA-event timers for the forward / backward expert pipeline (interface of
MOLE/utils/Utimer.py: ``UATimer`` with ``start_fwd/stop_fwd/start_bwd/stop_bwd``)."""
import torch


class UTimer:
    def __init__(self):
        self.pairs = []
        self._start = None

    def start(self):
        self._start = torch.cuda.Event(enable_timing=True)
        self._start.record()

    def stop(self):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        self.pairs.append((self._start, end))

    def elapsed_ms(self):
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in self.pairs]

    def reset(self):
        self.pairs = []


class UATimer:
    def __init__(self):
        self.fwd, self.bwd = UTimer(), UTimer()

    def start_fwd(self):
        self.fwd.start()

    def stop_fwd(self):
        self.fwd.stop()

    def start_bwd(self):
        self.bwd.start()

    def stop_bwd(self):
        self.bwd.stop()
