"""Offline tokenisation and label masking of chat / pretraining samples.

Rules (reference process_data.py:10-138):

* a sample is ``{"messages": [{"role", "content"}, ...]}``;
* a single message with role ``pretrain`` is encoded as ``content + eos`` without special tokens
  and is fully unmasked (labels = input_ids);
* anything else goes through the tokenizer's chat template; a sample with an empty assistant
  message, or one that raises, is dropped; so is one longer than ``max_sample_num_tokens``;
* the token runs the template puts in front of a user turn and of an assistant turn are inferred
  by templating ``user "1", assistant "1"`` and the reversed order and taking the longest common
  subsequence of the two sightings of each run;
* labels: walking the tokens, an assistant run switches unmasking on (the run itself stays
  masked), a user run switches it off; a token is its own label while unmasking is on and
  ``-100`` otherwise — so every assistant turn of a multi-turn sample is trained on.
"""
from __future__ import annotations

from typing import Sequence

IGNORE = -100


def longest_common_subsequence(a: Sequence[int], b: Sequence[int]) -> list:
    m, n = len(a), len(b)
    dp = [[0] * (n + 1) for _ in range(m + 1)]
    for i in range(m - 1, -1, -1):
        for j in range(n - 1, -1, -1):
            dp[i][j] = dp[i + 1][j + 1] + 1 if a[i] == b[j] else max(dp[i + 1][j], dp[i][j + 1])
    out, i, j = [], 0, 0
    while i < m and j < n:
        if a[i] == b[j]:
            out.append(a[i]); i += 1; j += 1
        elif dp[i + 1][j] >= dp[i][j + 1]:
            i += 1
        else:
            j += 1
    return out


def _template_ids(tokenizer, messages) -> list:
    ids = tokenizer.apply_chat_template(messages, tokenize=True)
    if isinstance(ids, dict) or hasattr(ids, "input_ids"):  # newer tokenizers return a BatchEncoding
        ids = ids["input_ids"]
    return list(ids)


def infer_special_token_sequences(tokenizer):
    """Returns ``(assistant_run, user_run)`` token-id lists."""
    one = tokenizer.encode("1", add_special_tokens=False)
    if len(one) != 1:
        raise ValueError('"1" must encode to a single token to infer the turn delimiters')
    one = one[0]

    def split(messages):
        ids = _template_ids(tokenizer, messages)
        where = [i for i, t in enumerate(ids) if t == one]
        if len(where) != 2:
            raise ValueError("the probe token must appear exactly twice in the templated probe")
        return ids[: where[0]], ids[where[0] + 1: where[1]]

    user_1, assistant_1 = split([{"role": "user", "content": "1"}, {"role": "assistant", "content": "1"}])
    assistant_2, user_2 = split([{"role": "assistant", "content": "1"}, {"role": "user", "content": "1"}])
    return longest_common_subsequence(assistant_1, assistant_2), longest_common_subsequence(user_1, user_2)


def make_input_ids_from_messages(sample: dict, tokenizer) -> dict:
    sample = dict(sample)
    sample.update(pretrain=False, error=False, input_ids=None, len=None)
    try:
        roles = [m["role"] for m in sample["messages"]]
        if "pretrain" in roles:
            if len(roles) != 1:
                raise ValueError("a pretrain message must be the only message")
            sample["input_ids"] = tokenizer.encode(sample["messages"][0]["content"] + tokenizer.eos_token,
                                                   add_special_tokens=False)
            sample["pretrain"] = True
        else:
            sample["input_ids"] = _template_ids(tokenizer, sample["messages"])
            if any(m["role"] == "assistant" and not m["content"] for m in sample["messages"]):
                sample["error"] = True
        sample["len"] = len(sample["input_ids"])
    except Exception:
        sample["error"] = True
    return sample


def make_labels_from_input_ids(sample: dict, assistant_tk_ids: list, user_tk_ids: list) -> dict:
    sample = dict(sample)
    ids = list(sample["input_ids"])
    if sample.get("pretrain"):
        sample["labels"] = ids
        return sample
    labels, unmasking, i = [], False, 0
    na, nu = len(assistant_tk_ids), len(user_tk_ids)
    while i < len(ids):
        if na and ids[i: i + na] == assistant_tk_ids:
            unmasking = True
            labels.extend([IGNORE] * na)
            i += na
            continue
        if nu and ids[i: i + nu] == user_tk_ids:
            unmasking = False
        labels.append(ids[i] if unmasking else IGNORE)
        i += 1
    sample["labels"] = labels
    return sample


def make_num_loss_tokens_from_labels(sample: dict) -> dict:
    sample = dict(sample)
    sample["num_loss_counted_tokens"] = sum(1 for l in sample["labels"] if l != IGNORE)
    return sample
