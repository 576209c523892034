"""Timers of the expert pipeline (interface of MOLE/utils/Utimer.py).

``UTimer`` keeps the reference's three mutually exclusive modes -- device-synchronised wall
clock, plain wall clock, CUDA events (Utimer.py:5-70) -- and ``UATimer`` its pair of forward /
backward timers, class-level as in the reference (Utimer.py:73-110): the scheduler reads the
gaps between consecutive MoE layers from it to size the prefetches.  Instances additionally offer
``start_fwd/stop_fwd/start_bwd/stop_bwd`` around one layer's expert pipeline (``time_it=True``).
"""
import time

import torch


class UTimer:
    def __init__(self):
        self.gap = []
        self.type = None
        self.lst = None

    def _mode(self, mode):
        if self.type is None:
            self.type = mode
        elif self.type != mode:
            raise AssertionError(f"timer already used in {self.type!r} mode, not {mode!r}")

    def syncstep_start(self):
        self._mode("sync")
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.lst = time.time()

    def syncstep_end(self):
        self._mode("sync")
        if self.lst is None:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.gap.append(time.time() - self.lst)
        self.lst = None

    def cpustep_start(self):
        self._mode("cpu")
        self.lst = time.time()

    def cpustep_end(self):
        self._mode("cpu")
        if self.lst is None:
            return
        self.gap.append(time.time() - self.lst)
        self.lst = None

    def eventstep_start(self):
        self._mode("event")
        self.lst = torch.cuda.Event(enable_timing=True)
        self.lst.record()

    def eventstep_end(self):
        self._mode("event")
        if self.lst is None:
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        end.synchronize()
        self.gap.append(self.lst.elapsed_time(end) * 1e-3)      # seconds, like the other modes
        self.lst = None

    def stats(self):
        return self.gap

    def clear(self):
        self.gap = []
        self.lst = None


class UATimer:
    fwd_timer = UTimer()
    bwd_timer = UTimer()

    def __init__(self):
        self.fwd, self.bwd = UTimer(), UTimer()

    # ---- one layer's expert pipeline (time_it=True) ----------------------------------------
    def start_fwd(self):
        self.fwd.eventstep_start()

    def stop_fwd(self):
        self.fwd.eventstep_end()

    def start_bwd(self):
        self.bwd.eventstep_start()

    def stop_bwd(self):
        self.bwd.eventstep_end()

    # ---- gaps between MoE layers, class-level as in the reference ---------------------------
    @staticmethod
    def track_fwd_start():
        UATimer.fwd_timer.syncstep_start()

    @staticmethod
    def track_fwd_end():
        UATimer.fwd_timer.syncstep_end()

    @staticmethod
    def track_bwd_start():
        UATimer.bwd_timer.syncstep_start()

    @staticmethod
    def track_bwd_end():
        UATimer.bwd_timer.syncstep_end()

    @staticmethod
    def stats():
        return UATimer.fwd_timer.stats(), UATimer.bwd_timer.stats()

    @staticmethod
    def clear():
        UATimer.fwd_timer.clear()
        UATimer.bwd_timer.clear()
