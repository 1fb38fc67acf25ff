"""Prompt set of the prefix-cache benchmark: prompts that share a long preamble, and the number of leading tokens
all of them have in common (the part a prefix cache can serve from memory).

Role of the reference's benchmarks/prefix_cache_reader.py:6-80 (CSV with a description row and a header row, column
``raw_input``, prompts wrapped in a chat template, the list cycled to a fixed count, longest common token prefix
measured with the model's tokenizer). Differences: any Hugging Face tokenizer (``AutoTokenizer``) or any object with
``encode``; no hard-wired rows to skip; the template and the count are arguments.

  python benchmarks/prefix_cache_reader.py --input_csv benchmarks/prefix_cache_input.csv --tokenizer_dir /path/to/model
"""
from __future__ import annotations

import argparse
import csv
import itertools
import os
from typing import List, Optional, Sequence, Tuple


def common_prefix_len(token_lists: Sequence[Sequence[int]]) -> int:
    """Number of leading positions at which all lists hold the same token."""
    n = 0
    for column in zip(*token_lists):
        if any(t != column[0] for t in column):
            break
        n += 1
    return n if token_lists else 0


def load_prompts(input_csv: str = "prefix_cache_input.csv", tokenizer_dir: Optional[str] = None, count: int = 220,
                 template: str = "[INST]%s[/INST]", tokenizer=None) -> Tuple[int, List[str]]:
    """(tokens shared by every prompt, ``count`` prompts). Row 0 of the file describes it, row 1 names the columns;
    prompts come from ``raw_input``. Without a tokenizer the shared length is reported as 0."""
    with open(input_csv, "r", encoding="utf-8", newline="") as f:
        rows = list(csv.reader(f))
    if len(rows) < 3:
        raise ValueError(f"{input_csv}: expected a description row, a header row and at least one prompt")
    try:
        col = rows[1].index("raw_input")
    except ValueError:
        raise ValueError(f"{input_csv}: no raw_input column in {rows[1]}") from None
    prompts = [template % r[col].strip() for r in rows[2:] if len(r) > col and r[col].strip()]
    if tokenizer is None and tokenizer_dir:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(tokenizer_dir, trust_remote_code=True)
    shared = 0
    if tokenizer is not None:
        shared = common_prefix_len([list(tokenizer.encode(p, add_special_tokens=True)) for p in prompts])
    final = list(itertools.islice(itertools.cycle(prompts), count)) if count else prompts
    return shared, final


def main():
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--input_csv", default=os.path.join(here, "prefix_cache_input.csv"))
    ap.add_argument("--tokenizer_dir", default=None)
    ap.add_argument("--count", type=int, default=220)
    args = ap.parse_args()
    shared, prompts = load_prompts(args.input_csv, args.tokenizer_dir, args.count)
    print(f"{len(prompts)} prompts, {shared} shared prefix tokens")


if __name__ == "__main__":
    main()
