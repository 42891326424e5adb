"""The staged measurement suite: every bench of this package run in a fixed order, each as its own process, with its last
JSON line collected into one report.

    python -m qwb200.tools.run_suite [--gpus 1] [--out suite.json] [--stages kernels,decode,prefill,serving,comm] [--quick]

Stages: ``kernels`` (gemm_bench, gemv_bench, launch_bench), ``decode`` (bench.py: decode, prefill, long prefill, the
speculative sweep; rows_bench), ``prefill`` (prefill_bench with the split by step), ``serving`` (long_context_bench,
cold_prefill_bench, pin_bench, spill_locality), ``comm`` (comm_bench, p2p_bench; only with --gpus > 1).  A stage that fails is recorded
with its exit code and the end of its output; the suite goes on.  For an A/B comparison run the suite in two
checkouts and compare the reports.  (The reference's bench/run_suite.sh is the same harness as a shell script.)"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def stages(gpus: int, quick: bool):
    py = [sys.executable]
    tr = py + ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(gpus), "--master-addr", "127.0.0.1"]
    multi = gpus > 1
    mod = lambda name, *args, dist=False, port=29540: ((tr + ["--master-port", str(port), "-m"] if dist else py + ["-m"]) + [f"qwb200.tools.{name}", *args])
    bench = (tr + ["--master-port", "29541"] if multi else py) + [os.path.join(ROOT, "bench.py"), "--gpus", str(gpus), "--steps", "32" if quick else "64", "--warmup", "4"]
    s = {
        "kernels": [("gemm_bench", mod("gemm_bench")), ("gemv_bench", mod("gemv_bench")), ("launch_bench", mod("launch_bench"))],
        "decode": [("bench", bench), ("rows_bench", mod("rows_bench"))],
        "prefill": [("prefill_bench", mod("prefill_bench", "--by-step", dist=multi, port=29542))],
        "serving": [("long_context_bench", mod("long_context_bench", *(["--tokens", "32768", "--resident", "8192", "--slots", "4"] if quick else []))),
                    ("cold_prefill_bench", mod("cold_prefill_bench", *(["--tokens", "16384", "--reps", "1"] if quick else []))),
                    ("pin_bench", mod("pin_bench", "--decode-steps", "200")),
                    ("spill_locality", mod("spill_locality", *(["--tokens", "16384", "--resident", "4096", "--steps", "64"] if quick else [])))],
        "comm": [("comm_bench", mod("comm_bench", "--prefill-rows", "4096", dist=True, port=29543)), ("p2p_bench", mod("p2p_bench", dist=True, port=29544))] if multi else [],
    }
    return s


def last_json(text: str):
    for ln in reversed(text.splitlines()):
        ln = ln.strip()
        if ln.startswith("{") and ln.endswith("}"):
            try:
                return json.loads(ln)
            except ValueError:
                continue
    return None


def run_suite(gpus: int, names, quick: bool, timeout: int, runner=subprocess.run):
    report = {"gpus": gpus, "started": time.strftime("%Y-%m-%d %H:%M:%S"), "results": {}}
    plan = stages(gpus, quick)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    for st in names:
        for name, cmd in plan.get(st, []):
            t0 = time.time()
            try:
                r = runner(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
                rc, out = r.returncode, (r.stdout or "") + (r.stderr or "")
            except subprocess.TimeoutExpired as e:
                rc, out = -9, str(e)
            rec = {"stage": st, "rc": rc, "seconds": round(time.time() - t0, 1), "json": last_json(out)}
            if rc != 0 or rec["json"] is None:
                rec["tail"] = out[-1500:]
            report["results"][name] = rec
            print(f"[suite] {st}/{name}: rc={rc} in {rec['seconds']} s", flush=True)
    return report


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--out", default="suite.json")
    ap.add_argument("--stages", default="kernels,decode,prefill,serving,comm")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--timeout", type=int, default=1200)
    a = ap.parse_args()
    rep = run_suite(a.gpus, a.stages.split(","), a.quick, a.timeout)
    with open(a.out, "w") as f:
        json.dump(rep, f, indent=1)
    print(json.dumps({"out": a.out, "failed": [k for k, v in rep["results"].items() if v["rc"] != 0]}))


if __name__ == "__main__":
    main()
