"""Accuracy benchmark helpers: answer checkers, the run loop with an injected model, McNemar's exact test."""
import json

from qwb200.tools import eval_tasks as et


def test_answer_checkers():
    assert et.last_number("so 1,234 apples\n#### $1,250.50") == "1250.50"
    assert et.last_number("no digits") is None
    assert et.is_correct("number", "steps... the answer is 42.", "#### 42")
    assert not et.is_correct("number", "41", "42")
    assert et.first_letter("  b. because") == "B"
    assert et.first_letter("the answer is C") == "C" and et.first_letter("zzz") is None
    assert et.is_correct("letter", "B", "b") and not et.is_correct("letter", "A", "B")


def test_mcnemar_values():
    assert et.mcnemar_exact(0, 0) == 1.0
    assert abs(et.mcnemar_exact(1, 5) - 2 * (1 + 6) / 64) < 1e-12
    assert et.mcnemar_exact(5, 5) == 1.0
    assert et.mcnemar_exact(0, 10) < 0.01


def test_run_and_compare(tmp_path):
    p = tmp_path / "t.jsonl"
    rows = [{"task": "gsm", "id": i, "prompt": f"q{i}", "gold": str(i), "kind": "number"} for i in range(6)]
    rows += [{"task": "arc", "id": i, "prompt": f"l{i}", "gold": "A", "kind": "letter", "max_tokens": 4} for i in range(4)]
    p.write_text("\n".join(json.dumps(r) for r in rows) + "\n\n")
    items = et.load_items([str(p)])
    assert len(items) == 10 and len(et.load_items([str(p)], limit=2)) == 4
    seen = []

    def model_a(prompt, max_tokens):
        seen.append((prompt, max_tokens))
        return f"#### {prompt[1:]}" if prompt[0] == "q" else "A"

    def model_b(prompt, max_tokens):
        return "#### 0" if prompt[0] == "q" else "A"

    ra = et.run_items(items, model_a, workers=3, progress=0)
    rb = et.run_items(items, model_b, workers=1, progress=0)
    assert ("q0", 768) in seen and ("l0", 4) in seen
    assert et.accuracy_by_task(ra) == {"arc": (4, 4), "gsm": (6, 6)}
    assert et.accuracy_by_task(rb)["gsm"] == (1, 6)
    cmp = {r["task"]: r for r in et.compare(ra, rb)}
    assert cmp["gsm"]["only_a"] == 5 and cmp["gsm"]["only_b"] == 0 and abs(cmp["gsm"]["p"] - 2 / 32) < 1e-12
    assert cmp["arc"]["p"] == 1.0 and cmp["all"]["n"] == 10
    (tmp_path / "a.json").write_text(json.dumps(ra))
    (tmp_path / "b.json").write_text(json.dumps(rb))
    assert et.main(["compare", str(tmp_path / "a.json"), str(tmp_path / "b.json"), "--names", "x", "y"]) == 0
