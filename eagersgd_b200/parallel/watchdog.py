"""Host watchdog for the partial allreduce.

Device-side waits are bounded and leave a status word instead of hanging; this thread polls the
status of an eager optimizer's channels at a fixed period and, when a wait has run out (a rank is
missing or dead), calls ``on_failure`` — by default it records the error so that the training
loop's next ``raise_if_failed()`` aborts cleanly.  The reference has no failure detection: a dead
rank hangs the others at the next synchronous round.
"""
from __future__ import annotations

import threading
from typing import Callable, Optional

from ._native import ChannelError


class Watchdog:
    def __init__(self, optimizer, period_s: float = 5.0, on_failure: Optional[Callable[[ChannelError], None]] = None):
        self.opt, self.period = optimizer, period_s
        self.on_failure = on_failure
        self.error: Optional[ChannelError] = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def start(self) -> "Watchdog":
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.period):
            try:
                self.opt.check()
            except ChannelError as e:
                self.error = e
                if self.on_failure is not None:
                    self.on_failure(e)
                return
            except Exception:
                return

    def raise_if_failed(self):
        if self.error is not None:
            raise self.error

    def stop(self):
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=self.period + 1)
