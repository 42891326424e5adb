"""Keeping the ranks of a measurement (or any multi-step procedure) in step when one of them fails.

Every rank runs the same program, and a failure - a bounded device-side wait that ran out and set the error word, a
launch that was refused - may show on some ranks only.  A rank that raised where it noticed would leave the others in
collectives that nobody answers.  With ``Lockstep`` no rank raises where it notices: ``attempt`` notes the failure and
skips that rank's work up to the next ``sync_point``; there all ranks learn of it together (one all-reduce that every
rank reaches, failed or not) and raise together, so their collectives never get out of step."""
from __future__ import annotations

from typing import Any, Callable, Optional


class Lockstep:
    def __init__(self, dist=None, device=None, check: Optional[Callable[[], None]] = None, sync: Optional[Callable[[], None]] = None):
        """``dist``: ``torch.distributed`` (initialised) or None for one rank; ``check``: raises when this rank's device
        reports an error (e.g. ``DeviceModel.check_error``); ``sync``: waits for this rank's device work."""
        self.dist, self.device, self.check, self.sync = dist, device, check, sync
        self.msg = ""

    def attempt(self, fn: Callable[[], Any], default: Any = None) -> Any:
        if self.msg:
            return default
        try:
            return fn()
        except Exception as ex:          # noqa: BLE001 - carried to the next sync point
            self.msg = f"{type(ex).__name__}: {str(ex)[:200]}"
            return default

    def sync_point(self) -> None:
        """A barrier that also spreads failure: raises on every rank when any rank has noted one."""
        if self.sync:
            self.sync()
        if not self.msg and self.check:
            try:
                self.check()
            except RuntimeError as ex:
                self.msg = str(ex)[:200]
        bad = 1.0 if self.msg else 0.0
        if self.dist is not None:
            import torch
            t = torch.tensor([bad], device=self.device)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            bad = float(t)
        if self.sync:
            self.sync()
        if bad > 0:
            raise RuntimeError(self.msg or "failed on another rank")
