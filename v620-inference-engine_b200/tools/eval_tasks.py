"""Answer-accuracy benchmark through the OpenAI-compatible API, and the paired comparison of two runs.

``run``: asks every question of one or more JSONL task files (one object per line: ``task``, ``id``, ``prompt``,
``gold`` and ``kind`` = ``number`` | ``letter``; optional ``max_tokens``) greedily with thinking off, and writes
``{"<task>:<id>": true|false}``.  Question files are local: this machine has no network, so exporting GSM8K / MMLU /
ARC into that form happens wherever the datasets are (``--export-help`` prints the prompt conventions).
``compare``: accuracy per task for two result files over the questions both contain, and McNemar's exact two-sided
test on the discordant pairs - the test that says whether a kernel or quantisation change moved the quality.
(Roles of the reference's tools/bench_tasks.py:1-90 and tools/bench_compare.py:1-13.)

  python -m qwb200.tools.eval_tasks run out.json tasks/*.jsonl --url http://127.0.0.1:8000 --workers 4
  python -m qwb200.tools.eval_tasks compare a.json b.json --names base new
"""
from __future__ import annotations

import argparse
import json
import re
import threading
import time
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from math import comb
from typing import Callable, Dict, Iterable, List, Optional

EXPORT_HELP = """Prompt conventions (the ones the published accuracy figures of the reference were taken with):
  number  : "<question>\\n\\nSolve step by step, then give the final answer on the last line as: #### <number>"
            gold = the text after '####' of the dataset's answer; max_tokens 768
  letter  : "<question>\\n\\nA. ...\\nB. ...\\n\\nAnswer with only the letter of the correct option."
            gold = the option's letter; max_tokens 8
"""

_NUM = re.compile(r"-?\d+(?:\.\d+)?")


def last_number(text: str) -> Optional[str]:
    """The last number of ``text`` (after '####' when the marker is present), thousands separators and '$' dropped."""
    if "####" in text:
        text = text.split("####")[-1]
    m = _NUM.findall(text.replace(",", "").replace("$", ""))
    return m[-1] if m else None


def same_number(a: Optional[str], b: Optional[str]) -> bool:
    try:
        return a is not None and b is not None and abs(float(a) - float(b)) < 1e-6
    except ValueError:
        return False


def first_letter(text: str) -> Optional[str]:
    """The first stand-alone option letter A..J in the first 40 characters of the answer."""
    m = re.search(r"\b([A-J])\b", text.strip().upper()[:40])
    return m.group(1) if m else None


def is_correct(kind: str, answer: str, gold: str) -> bool:
    if kind == "number":
        return same_number(last_number(answer), last_number(str(gold)))
    if kind == "letter":
        return first_letter(answer) == str(gold).strip().upper()
    raise ValueError(f"unknown kind {kind!r}")


def load_items(paths: Iterable[str], limit: int = 0) -> List[dict]:
    items: List[dict] = []
    per_task: Dict[str, int] = {}
    for p in paths:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                it = json.loads(line)
                n = per_task.get(it["task"], 0)
                if limit and n >= limit:
                    continue
                per_task[it["task"]] = n + 1
                items.append(it)
    return items


def make_asker(url: str, model: str, retries: int = 5, timeout: float = 900.0) -> Callable[[str, int], str]:
    endpoint = url.rstrip("/") + "/v1/chat/completions"

    def ask(prompt: str, max_tokens: int) -> str:
        body = {"model": model, "temperature": 0, "max_tokens": max_tokens, "messages": [{"role": "user", "content": prompt}],
                "chat_template_kwargs": {"enable_thinking": False}}
        for attempt in range(retries):
            try:
                req = urllib.request.Request(endpoint, json.dumps(body).encode(), {"content-type": "application/json"})
                with urllib.request.urlopen(req, timeout=timeout) as r:
                    return json.load(r)["choices"][0]["message"]["content"] or ""
            except Exception:            # noqa: BLE001 - a server restart in the middle of a long run is retried
                time.sleep(5 * (attempt + 1))
        return ""

    return ask


def run_items(items: List[dict], ask: Callable[[str, int], str], workers: int = 4, progress: int = 200) -> Dict[str, bool]:
    res: Dict[str, bool] = {}
    lock = threading.Lock()
    t0 = time.time()

    def one(it: dict) -> None:
        default = 768 if it["kind"] == "number" else 8
        ok = is_correct(it["kind"], ask(it["prompt"], int(it.get("max_tokens", default))), it["gold"])
        with lock:
            res[f"{it['task']}:{it['id']}"] = ok
            if progress and len(res) % progress == 0:
                print(f"{len(res)}/{len(items)} done, {time.time() - t0:.0f} s", flush=True)

    with ThreadPoolExecutor(max(1, workers)) as ex:
        list(ex.map(one, items))
    return res


def accuracy_by_task(res: Dict[str, bool]) -> Dict[str, tuple]:
    out: Dict[str, list] = {}
    for k, ok in res.items():
        c = out.setdefault(k.split(":", 1)[0], [0, 0])
        c[0] += bool(ok)
        c[1] += 1
    return {t: (c[0], c[1]) for t, c in sorted(out.items())}


def mcnemar_exact(only_a: int, only_b: int) -> float:
    """Two-sided exact (binomial, p = 1/2) McNemar p-value for the discordant counts."""
    n = only_a + only_b
    if n == 0:
        return 1.0
    return min(1.0, 2.0 * sum(comb(n, i) for i in range(min(only_a, only_b) + 1)) / 2.0 ** n)


def compare(a: Dict[str, bool], b: Dict[str, bool]) -> List[dict]:
    """One row per task plus 'all': n common questions, both accuracies, discordant counts and the p-value."""
    tasks = sorted({k.split(":", 1)[0] for k in a if k in b})
    rows = []
    for t in tasks + ["all"]:
        keys = [k for k in a if k in b and (t == "all" or k.split(":", 1)[0] == t)]
        if not keys:
            continue
        oa = sum(bool(a[k]) and not b[k] for k in keys)
        ob = sum(bool(b[k]) and not a[k] for k in keys)
        rows.append({"task": t, "n": len(keys), "acc_a": sum(bool(a[k]) for k in keys) / len(keys),
                     "acc_b": sum(bool(b[k]) for k in keys) / len(keys), "only_a": oa, "only_b": ob, "p": mcnemar_exact(oa, ob)})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--export-help", action="store_true")
    sub = ap.add_subparsers(dest="cmd")
    r = sub.add_parser("run")
    r.add_argument("out")
    r.add_argument("tasks", nargs="+")
    r.add_argument("--url", default="http://127.0.0.1:8000")
    r.add_argument("--model", default="x")
    r.add_argument("--limit", type=int, default=0, help="at most this many questions per task")
    r.add_argument("--workers", type=int, default=4)
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    c.add_argument("--names", nargs=2, default=["A", "B"])
    a = ap.parse_args(argv)
    if a.export_help or a.cmd is None:
        print(EXPORT_HELP)
        return 0
    if a.cmd == "run":
        items = load_items(a.tasks, a.limit)
        print(f"{len(items)} questions", flush=True)
        res = run_items(items, make_asker(a.url, a.model), a.workers)
        with open(a.out, "w") as f:
            json.dump(res, f)
        for t, (ok, n) in accuracy_by_task(res).items():
            print(f"{t}: {ok}/{n} = {100.0 * ok / max(1, n):.1f}%", flush=True)
        return 0
    with open(a.a) as f:
        ra = json.load(f)
    with open(a.b) as f:
        rb = json.load(f)
    na, nb = a.names
    for row in compare(ra, rb):
        print(f"{row['task']:8s} n={row['n']:5d}  {na} {100 * row['acc_a']:5.1f}%  {nb} {100 * row['acc_b']:5.1f}%  "
              f"({na} only {row['only_a']}, {nb} only {row['only_b']}; McNemar p={row['p']:.3f})")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
