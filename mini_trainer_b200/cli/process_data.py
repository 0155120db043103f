"""``process_data`` command line (reference process_data.py:140-199): messages JSONL -> tokenised
JSONL with ``input_ids, labels, len, num_loss_counted_tokens`` (other columns are kept)."""
from __future__ import annotations

import json
import random
from concurrent.futures import ProcessPoolExecutor

import typer

from ..data import tokenize as T

app = typer.Typer()

_TOK = None
_DELIMS = None


def _init(model_name_or_path):
    global _TOK, _DELIMS
    from transformers import AutoTokenizer
    _TOK = AutoTokenizer.from_pretrained(model_name_or_path)
    _DELIMS = T.infer_special_token_sequences(_TOK)


def _work(line: str):
    s = T.make_input_ids_from_messages(json.loads(line), _TOK)
    if s["error"]:
        return None
    return s


def process_samples(lines, tokenizer, max_sample_num_tokens: int = 2147483647):
    """Single-process core, reusable from tests with any tokenizer-like object."""
    a_ids, u_ids = T.infer_special_token_sequences(tokenizer)
    out, n_err, n_long = [], 0, 0
    for line in lines:
        s = T.make_input_ids_from_messages(json.loads(line) if isinstance(line, str) else line, tokenizer)
        if s["error"]:
            n_err += 1
            continue
        if s["len"] > max_sample_num_tokens:
            n_long += 1
            continue
        s = T.make_num_loss_tokens_from_labels(T.make_labels_from_input_ids(s, a_ids, u_ids))
        out.append(s)
    return out, n_err, n_long


@app.command()
def process_data(
    input_jsonl: str = typer.Option(..., "--input-file", help="path to the input jsonl file"),
    output_jsonl: str = typer.Option(..., "--output-file", help="path to the output tokenized jsonl file"),
    model_name_or_path: str = typer.Option(..., "--model-name-or-path"),
    max_sample_num_tokens: int = typer.Option(2147483647, help="samples longer than this are removed"),
    string_for_printing_masks: str = typer.Option("<|mAsK|>", "--string-for-printing-masks",
                                                  help="masked label tokens are shown as this string in the preview"),
    num_proc: int = typer.Option(8, help="tokenisation worker processes"),
):
    from transformers import AutoTokenizer
    tokenizer = AutoTokenizer.from_pretrained(model_name_or_path)
    a_ids, u_ids = T.infer_special_token_sequences(tokenizer)
    with open(input_jsonl) as f:
        lines = [l for l in f if l.strip()]
    if num_proc > 1 and len(lines) > 256:
        with ProcessPoolExecutor(num_proc, initializer=_init, initargs=(model_name_or_path,)) as ex:
            toks = list(ex.map(_work, lines, chunksize=64))
    else:
        _init(model_name_or_path)
        toks = [_work(l) for l in lines]
    ok = [s for s in toks if s is not None]
    print("\033[38;5;196m" + f"Total number of filtered samples after removing samples with errors: {len(lines) - len(ok)}" + "\033[0m")
    kept = [s for s in ok if s["len"] <= max_sample_num_tokens]
    print("\033[38;5;196m" + f"Total number of filtered samples after removing samples longer than {max_sample_num_tokens} tokens: {len(lines) - len(kept)}" + "\033[0m")
    kept = [T.make_num_loss_tokens_from_labels(T.make_labels_from_input_ids(s, a_ids, u_ids)) for s in kept]

    tokenizer.add_special_tokens({"additional_special_tokens": [string_for_printing_masks]})
    mask_tk = tokenizer.encode(string_for_printing_masks, add_special_tokens=False)[0]
    for s in random.sample(kept, min(2, len(kept))):
        print("original messages:")
        print("\033[38;5;10m" + str(s["messages"]) + "\033[0m")
        print("input_ids:")
        print("\033[38;5;51m" + tokenizer.decode(s["input_ids"]) + "\033[0m")
        print("labels:")
        print("\033[38;5;208m" + tokenizer.decode([l if l != T.IGNORE else mask_tk for l in s["labels"]]) + "\033[0m")
        print("-" * 100)
    with open(output_jsonl, "w") as f:
        for s in kept:
            f.write(json.dumps(s) + "\n")


if __name__ == "__main__":
    app()
