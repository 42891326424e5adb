"""One engine over several GPUs behind a single caller: rank 0 lives in the caller's process, ranks 1..N-1 are worker
processes, and every call that touches the engine is replayed on all ranks in the same order.

The engine is single-program: each rank holds its shard of the weights and of every slot's state, and the kernels of a
step exchange data among themselves (``ops/csrc/fuse.cuh``, ``tp.cuh``).  What the ranks need from the host is only to
be told the same thing at the same time.  ``RankGroup.call(name, *args)`` sends ``(name, args)`` (plain Python values)
to every worker over a local socket, runs the call on rank 0's own object, then collects one acknowledgement per
worker.  Everything above the kernels - slot choice, prefix cache, sampling with seeded generators on the gathered
logits - is deterministic, so the ranks stay in step without exchanging results.

Failure detection: a worker that raises answers with the error text; one that died closes its socket; one that hangs
lets the acknowledgement time out.  Each of these makes ``failure()`` return a description naming the rank, after which
every call is refused - the engine is then unusable until restart, as in the reference, whose rank threads set a sticky
error that ``qw_engine_failure`` reports (src/engine/engine.hip:327-414, src/capi/capi.cpp:49-84).
"""
from __future__ import annotations

import os
import secrets
import subprocess
import sys
import threading
import time
from multiprocessing.connection import Client, Listener
from typing import Any, Callable, List, Optional, Sequence


class RankFailure(RuntimeError):
    pass


class RankGroup:
    def __init__(self, local: Any, conns: Sequence[Any], procs: Sequence[subprocess.Popen], ack_timeout: float = 120.0):
        self.local, self.conns, self.procs = local, list(conns), list(procs)
        self.ack_timeout = ack_timeout
        self._failure = ""
        self._lock = threading.Lock()

    # ---- start-up
    @staticmethod
    def spawn(world: int, worker_args: Sequence[str], open_msg: Any, build_local: Callable[[], Any], ready_timeout: float = 1800.0,
              ack_timeout: float = 120.0, env: Optional[dict] = None) -> "RankGroup":
        """Start ranks 1..world-1 as ``python -m qwb200.parallel.worker`` processes, hand each the ``open_msg`` (with its
        rank added), build rank 0's object with ``build_local()`` meanwhile, and wait until every worker reports ready."""
        authkey = secrets.token_bytes(16)
        listener = Listener(("127.0.0.1", 0), authkey=authkey)
        host, port = listener.address
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        penv = dict(os.environ if env is None else env)
        penv["PYTHONPATH"] = root + os.pathsep + penv.get("PYTHONPATH", "")
        exe = sys.executable if sys.executable and "python" in os.path.basename(sys.executable) else "python3"
        procs = []
        for r in range(1, world):
            procs.append(subprocess.Popen([exe, "-m", "qwb200.parallel.worker", "--address", f"{host}:{port}", "--authkey", authkey.hex(),
                                           "--rank", str(r), "--world", str(world)] + list(worker_args), env=penv))
        conns: List[Any] = [None] * (world - 1)
        try:
            def accept_all():
                for _ in range(world - 1):
                    c = listener.accept()
                    conns[c.recv() - 1] = c        # the worker introduces itself with its rank
            th = threading.Thread(target=accept_all, daemon=True)
            th.start()
            t0 = time.time()
            while th.is_alive():
                th.join(0.2)
                dead = [r for r, p in enumerate(procs, start=1) if p.poll() is not None]
                if dead:
                    raise RankFailure(f"rank {dead[0]} exited during start-up")
                if time.time() - t0 > ready_timeout:
                    raise RankFailure("the worker ranks did not connect in time")
            for r, c in enumerate(conns, start=1):
                c.send(("open", dict(open_msg, rank=r)))
            local = build_local()
            for r, c in enumerate(conns, start=1):
                if not c.poll(ready_timeout):
                    raise RankFailure(f"rank {r} did not finish start-up within {ready_timeout:.0f} s")
                st, msg = c.recv()
                if st != "ready":
                    raise RankFailure(f"rank {r} failed to start: {msg}")
        except BaseException:
            for p in procs:
                p.kill()
            raise
        finally:
            listener.close()
        return RankGroup(local, conns, procs, ack_timeout)

    # ---- calls
    def failure(self) -> str:
        if not self._failure:
            for r, p in enumerate(self.procs, start=1):
                if p.poll() is not None:
                    self._failure = f"rank {r} is gone (worker exited with code {p.returncode})"
                    break
        return self._failure

    def call(self, name: str, *args):
        """Run ``name(*args)`` on every rank; returns rank 0's result.  Raises ``RankFailure`` once any rank has failed."""
        with self._lock:
            if self.failure():
                raise RankFailure(self._failure)
            sent = []
            for r, c in enumerate(self.conns, start=1):
                try:
                    c.send((name, args))
                    sent.append((r, c))
                except (OSError, EOFError, BrokenPipeError) as ex:
                    self._failure = f"rank {r} is gone ({type(ex).__name__} on send)"
            err: Optional[BaseException] = None
            res = None
            try:
                res = getattr(self.local, name)(*args)
            except BaseException as ex:          # the workers have run the call too: collect their answers before raising
                err = ex
            deadline = time.time() + self.ack_timeout
            for r, c in sent:
                try:
                    if not c.poll(max(0.0, deadline - time.time())):
                        self._failure = self._failure or f"rank {r} did not answer '{name}' within {self.ack_timeout:.0f} s"
                        continue
                    st, msg = c.recv()
                    if st != "ok" and err is None:
                        # a refusal that rank 0 raised too is the caller's error, not a failure of the group; a rank that fails
                        # alone has left the ranks out of step
                        self._failure = self._failure or f"rank {r} failed in '{name}': {msg}"
                except (OSError, EOFError) as ex:
                    self._failure = self._failure or f"rank {r} is gone ({type(ex).__name__} while waiting for '{name}')"
            if err is not None:
                raise err
            if self._failure:
                raise RankFailure(self._failure)
            return res

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *args: self.call(name, *args)

    def shutdown(self, timeout: float = 10.0) -> None:
        for c in self.conns:
            try:
                c.send(None)
            except (OSError, EOFError, BrokenPipeError):
                pass
        t0 = time.time()
        for p in self.procs:
            try:
                p.wait(max(0.1, timeout - (time.time() - t0)))
            except subprocess.TimeoutExpired:
                p.kill()
        for c in self.conns:
            try:
                c.close()
            except OSError:
                pass


def connect(address: str, authkey_hex: str, rank: int):
    """Worker side: connect to rank 0 and say who we are."""
    host, port = address.rsplit(":", 1)
    c = Client((host, int(port)), authkey=bytes.fromhex(authkey_hex))
    c.send(rank)
    return c


def serve(conn, build: Callable[[dict], Any]) -> int:
    """Worker side: build the rank's object from the open message, then run calls until the connection closes."""
    msg = conn.recv()
    if not msg or msg[0] != "open":
        return 2
    try:
        obj = build(msg[1])
    except BaseException as ex:
        conn.send(("error", f"{type(ex).__name__}: {ex}"))
        return 3
    conn.send(("ready", ""))
    while True:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            return 0            # rank 0 went away: nothing left to serve
        if msg is None:
            return 0
        name, args = msg
        try:
            getattr(obj, name)(*args)
            conn.send(("ok", ""))
        except BaseException as ex:
            conn.send(("error", f"{type(ex).__name__}: {ex}"))
