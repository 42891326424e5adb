"""CPU-side pieces of the small tools: logits dump records / comparison, token id files."""
import json

import torch

from qwb200.tools import logits_dump as ld
from qwb200.tools import text_tokens as tt


def test_logits_dump_compare(tmp_path):
    g = torch.Generator().manual_seed(0)
    rows = [torch.randn(64, generator=g) for _ in range(4)]
    run = {"model": "tiny", "prompt_len": 8, "new": 3, "seed": 0, "graphs": True}
    a = {"run": run, "rows": [ld.row_record(r) for r in rows], "first_row": rows[0].tolist(), "last_row": rows[-1].tolist()}
    assert ld.compare(a, json.loads(json.dumps(a)))["identical"]
    rows2 = [r.clone() for r in rows]
    rows2[2][5] += 1e-3
    rows2[3][int(rows2[3].argmax())] -= 100.0
    b = {"run": run, "rows": [ld.row_record(r) for r in rows2], "first_row": rows2[0].tolist(), "last_row": rows2[-1].tolist()}
    r = ld.compare(a, b)
    assert not r["identical"] and r["first_diff"] == 2 and r["n_diff"] == 2 and r["argmax_diffs"] == 1 and r["kept_max_abs"] > 99
    (tmp_path / "a.json").write_text(json.dumps(a))
    (tmp_path / "b.json").write_text(json.dumps(b))
    assert ld.main(["compare", str(tmp_path / "a.json"), str(tmp_path / "a.json")]) == 0
    assert ld.main(["compare", str(tmp_path / "a.json"), str(tmp_path / "b.json")]) == 1
    c = dict(b, run=dict(run, seed=1))
    assert "error" in ld.compare(a, c)


def test_text_tokens_round_trip(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    tok = Tokenizer(models.WordLevel({"a": 0, "b": 1, "[UNK]": 2}, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(tmp_path / "tok.json"))
    (tmp_path / "x.txt").write_text("a b b")
    (tmp_path / "y.txt").write_text("b zzz a")
    assert tt.main([str(tmp_path / "tok.json"), str(tmp_path / "ids"), str(tmp_path / "x.txt"), str(tmp_path / "y.txt")]) == 0
    assert tt.read_ids(str(tmp_path / "ids")) == [0, 1, 1, 1, 2, 0]
    assert tt.main([]) == 2


def test_prefill_bench_reads_a_token_file(tmp_path):
    from qwb200.tools.prefill_bench import read_token_file
    f = tmp_path / "ids.txt"
    f.write_text("1, 2,3\n4 5\t6,\n")
    assert read_token_file(str(f), 10) == [1, 2, 3, 4, 5, 6]
    import pytest
    with pytest.raises(ValueError, match="outside the vocabulary"):
        read_token_file(str(f), 6)
