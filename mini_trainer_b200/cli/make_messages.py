"""Converts question/solution records into the ``messages`` format ``process_data`` reads
(reference make_messages.py:1-36, which does this for the GAIR/LIMO dataset).

    python -m mini_trainer_b200.cli.make_messages --input-file limo.jsonl --output-file limo_messages.jsonl

Input: JSONL (or an HF dataset name when ``datasets`` can reach it) with a question-like and an
answer-like column; output: one ``{"messages": [user, assistant]}`` object per line.
"""
from __future__ import annotations

import json

import typer

app = typer.Typer()


def to_messages(record: dict, question_key: str = "question", answer_key: str = "solution") -> dict:
    return {"messages": [{"role": "user", "content": record[question_key]},
                         {"role": "assistant", "content": record[answer_key]}]}


@app.command()
def make_messages(
    input_file: str = typer.Option("GAIR/LIMO", "--input-file", help="JSONL path or HF dataset name"),
    output_file: str = typer.Option("limo_messages.jsonl", "--output-file"),
    question_key: str = typer.Option("question"),
    answer_key: str = typer.Option("solution"),
):
    if input_file.endswith(".jsonl") or input_file.endswith(".json"):
        with open(input_file) as f:
            records = [json.loads(l) for l in f if l.strip()]
    else:
        from datasets import load_dataset
        records = load_dataset(input_file, split="train")
    with open(output_file, "w") as f:
        for r in records:
            f.write(json.dumps(to_messages(r, question_key, answer_key)) + "\n")
    print(f"wrote {len(records)} samples to {output_file}")


if __name__ == "__main__":
    app()
