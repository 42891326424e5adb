"""A worker rank of a multi-GPU engine (``parallel/rank_group.py``): connects to rank 0, builds its shard of the engine
from the options it is sent, and replays rank 0's calls.

    python -m qwb200.parallel.worker --address 127.0.0.1:PORT --authkey HEX --rank R --world N [--fake | --builder MOD:FUNC]

``--fake`` builds a recorder instead of an engine (no GPU): the host-side protocol's tests use it, also to inject
failures - a call that raises, a call that never returns, a process that exits.  ``--builder MOD:FUNC`` builds the rank's
object with ``FUNC(open_message, world)`` from module ``MOD`` instead of the engine (tests that run real sessions over
a stand-in engine on every rank).
"""
import argparse
import os
import sys
import time


class FakeOps:
    """Records every call; ``fail_on`` / ``hang_on`` / ``exit_on`` (method names in the open message) inject failures."""

    def __init__(self, o: dict):
        self.o = o
        self.log = []

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)

        def method(*args):
            self.log.append((name, args))
            if name == self.o.get("exit_on") and self.o.get("rank") == self.o.get("victim", 1):
                os._exit(7)
            if name == self.o.get("hang_on") and self.o.get("rank") == self.o.get("victim", 1):
                time.sleep(3600)
            if name == self.o.get("fail_on") and self.o.get("rank") == self.o.get("victim", 1):
                raise RuntimeError(f"injected failure in {name}")
            if name == "dump" and args:
                with open(args[0] + f".rank{self.o.get('rank')}", "w") as f:
                    f.write(repr(self.log))
            return 0
        return method


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--address", required=True)
    ap.add_argument("--authkey", required=True)
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--fake", action="store_true")
    ap.add_argument("--builder", default=None)
    a = ap.parse_args()
    from .rank_group import connect, serve
    conn = connect(a.address, a.authkey, a.rank)
    if a.fake:
        return serve(conn, lambda o: FakeOps(o))
    if a.builder:
        import importlib
        mod, _, fn = a.builder.partition(":")
        make = getattr(importlib.import_module(mod), fn)
        return serve(conn, lambda o: make(o, a.world))

    def build(o: dict):
        from ..capi_impl import build_ops
        return build_ops(o["options"], rank=o["rank"], world=a.world, master_port=o["master_port"])
    return serve(conn, build)


if __name__ == "__main__":
    sys.exit(main())
