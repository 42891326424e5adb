"""Wait until a running server has been idle for a while: nothing waiting, prefilling or running and no request
completed for ``--idle`` seconds (a long request in flight is not idle, whatever a proxy's request log says).

    python -m qwserve.idle [--url http://127.0.0.1:8000] [--idle 60] [--every 5] [--give-up 3600]

Exit code 0 once idle (``ctl.sh idle-stop`` then stops the server and frees its GPUs), 1 if it never was within
``--give-up`` seconds or the server cannot be reached.  (Role of the reference's scripts/prod-idle-unload.sh.)"""
import argparse
import json
import sys
import time
import urllib.request


def busy_and_done(url: str, timeout: float = 5.0):
    with urllib.request.urlopen(url.rstrip("/") + "/health", timeout=timeout) as r:
        d = json.load(r).get("decode", {})
    return int(d.get("waiting", 0)) + int(d.get("prefilling", 0)) + int(d.get("running", 0)), int(d.get("completed", 0)) + int(d.get("failed", 0))


def wait_idle(url: str, idle_s: float, every_s: float, give_up_s: float, probe=busy_and_done, clock=time.monotonic, sleep=time.sleep) -> bool:
    start = clock()
    quiet_since, last_done = None, None
    while clock() - start <= give_up_s:
        try:
            busy, done = probe(url)
        except Exception:          # noqa: BLE001 - not reachable (yet, or any more): not idle
            busy, done = 1, last_done
        now = clock()
        if busy or (last_done is not None and done != last_done):
            quiet_since = None
        elif quiet_since is None:
            quiet_since = now
        last_done = done
        if quiet_since is not None and now - quiet_since >= idle_s:
            return True
        sleep(every_s)
    return False


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--idle", type=float, default=60.0)
    ap.add_argument("--every", type=float, default=5.0)
    ap.add_argument("--give-up", type=float, default=3600.0)
    a = ap.parse_args()
    ok = wait_idle(a.url, a.idle, a.every, a.give_up)
    print(json.dumps({"idle": ok}), flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
