"""Token ids of real text for the benchmarks and runners that take ``--prompt`` / ``--tokens-file``.

    python -m qwb200.tools.text_tokens TOKENIZER_JSON OUT FILE...

Encodes every file with the HF ``tokenizers`` tokenizer and writes all ids, in file order, as one comma-separated line
(role of the reference's tools/text_tokens.py:1-12)."""
from __future__ import annotations

import sys
from typing import List, Sequence


def encode_files(tokenizer_json: str, paths: Sequence[str]) -> List[int]:
    from tokenizers import Tokenizer
    tok = Tokenizer.from_file(tokenizer_json)
    ids: List[int] = []
    for p in paths:
        with open(p, errors="replace") as f:
            ids += tok.encode(f.read()).ids
    return ids


def read_ids(path: str) -> List[int]:
    """The inverse: ids of a file written by this tool (commas and / or white space between them)."""
    with open(path) as f:
        return [int(t) for t in f.read().replace(",", " ").split()]


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else list(argv)
    if len(argv) < 3:
        print(__doc__)
        return 2
    ids = encode_files(argv[0], argv[2:])
    with open(argv[1], "w") as f:
        f.write(",".join(map(str, ids)))
    print(f"{len(ids)} token ids from {len(argv) - 2} files -> {argv[1]}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
