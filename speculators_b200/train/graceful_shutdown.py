"""SIGINT / SIGTERM handling for training runs.

A signal raises ``TrainingInterrupted`` in the main thread at the next bytecode
boundary; the decorator catches it, asks the trainer for an ``interrupted/``
checkpoint and re-raises as a clean exit.  A watchdog thread started at the same
time hard-exits the process if that save has not finished within the timeout
(120 s by default), so a wedged collective cannot keep a preempted job alive.
Behaviour parity: src/speculators/train/graceful_shutdown.py:40-151.
"""

from __future__ import annotations

import functools
import logging
import os
import signal
import threading

log = logging.getLogger("speculators")

__all__ = ["DEFAULT_SHUTDOWN_TIMEOUT", "TrainingInterruptedError", "GracefulShutdownHandler", "TrainingInterrupted", "with_graceful_shutdown"]

DEFAULT_TIMEOUT_S = 120.0
DEFAULT_SHUTDOWN_TIMEOUT = int(DEFAULT_TIMEOUT_S)  # the reference's name for the same budget


class TrainingInterrupted(BaseException):
    def __init__(self, signum: int):
        super().__init__(f"received signal {signum}")
        self.signum = signum


TrainingInterruptedError = TrainingInterrupted  # the reference's name


class GracefulShutdownHandler:
    """Context manager that converts the first SIGINT/SIGTERM into an exception and
    ignores repeats while the shutdown path runs."""

    def __init__(self, signals=(signal.SIGINT, signal.SIGTERM)):
        self.signals = tuple(signals)
        self._previous: dict[int, object] = {}
        self.triggered: int | None = None

    def _handle(self, signum, _frame):  # noqa: ANN001
        if self.triggered is not None:
            log.warning("Signal %d ignored: shutdown already in progress.", signum)
            return
        self.triggered = signum
        raise TrainingInterrupted(signum)

    def __enter__(self) -> "GracefulShutdownHandler":
        if threading.current_thread() is threading.main_thread():
            for sig in self.signals:
                self._previous[sig] = signal.signal(sig, self._handle)
        return self

    def __exit__(self, *exc) -> None:  # noqa: ANN002
        for sig, prev in self._previous.items():
            signal.signal(sig, prev)
        self._previous.clear()


def _start_watchdog(timeout_s: float) -> threading.Timer:
    def _expire() -> None:
        log.error("Graceful shutdown exceeded %.0f s; exiting hard.", timeout_s)
        os._exit(1)

    timer = threading.Timer(timeout_s, _expire)
    timer.daemon = True
    timer.start()
    return timer


def with_graceful_shutdown(timeout_s: float = DEFAULT_TIMEOUT_S, save_method: str = "maybe_save_checkpoint"):
    """Decorate a trainer method (``run_training``).  On a signal the trainer's
    ``save_method("interrupted")`` runs under the watchdog, then ``SystemExit(128+sig)``."""

    def decorate(fn):
        @functools.wraps(fn)
        def wrapper(self, *args, **kwargs):
            with GracefulShutdownHandler() as handler:
                try:
                    return fn(self, *args, **kwargs)
                except TrainingInterrupted as stop:
                    log.warning("Signal %d received: saving an 'interrupted' checkpoint.", stop.signum)
                    watchdog = _start_watchdog(timeout_s)
                    try:
                        saver = getattr(self, save_method, None)
                        if saver is not None:
                            saver("interrupted")
                    finally:
                        watchdog.cancel()
                    del handler
                    raise SystemExit(128 + stop.signum) from None

        return wrapper

    return decorate
