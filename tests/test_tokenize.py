"""Offline tokenisation / label masking (reference process_data.py:10-138) on a fake chat tokenizer,
the ``process_data`` and ``make_messages`` command lines on a real ``tokenizers`` word-level tokenizer
with a ChatML-style template, and the sequence-length sweep tool on the tiny CPU model."""
import json
import os
import subprocess
import sys

import pytest

from mini_trainer_b200.cli.make_messages import to_messages
from mini_trainer_b200.cli.process_data import process_samples
from mini_trainer_b200.data import tokenize as T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class FakeChatTokenizer:
    """Whitespace tokenizer with a ChatML-like template:
    ``<s> [ <|user|> | <|assistant|> ] \\n  words... <|end|>`` per message."""
    eos_token = "</s>"

    def __init__(self):
        self.vocab = {"<s>": 0, "</s>": 1, "<|user|>": 2, "<|assistant|>": 3, "<|system|>": 4, "<|end|>": 5, "\\n": 6, "1": 7}

    def _id(self, w):
        return self.vocab.setdefault(w, len(self.vocab))

    def encode(self, text, add_special_tokens=False):
        text = text.replace("</s>", " </s> ")
        return [self._id(w) for w in text.split()]

    def apply_chat_template(self, messages, tokenize=True):
        ids = [self._id("<s>")]
        for m in messages:
            if m["role"] not in ("user", "assistant", "system"):
                raise ValueError(f"unknown role {m['role']}")
            ids += [self._id(f"<|{m['role']}|>"), self._id("\\n")] + self.encode(m["content"]) + [self._id("<|end|>")]
        return ids


def test_lcs():
    assert T.longest_common_subsequence([1, 2, 3, 4], [2, 9, 4]) == [2, 4]
    assert T.longest_common_subsequence([], [1]) == []


def test_delimiters_are_inferred_from_the_template():
    tok = FakeChatTokenizer()
    a, u = T.infer_special_token_sequences(tok)
    # <s> and <|end|> only precede a turn in one of the two orderings, so the common subsequence drops them
    assert a == [tok.vocab["<|assistant|>"], tok.vocab["\\n"]]
    assert u == [tok.vocab["<|user|>"], tok.vocab["\\n"]]


def test_multi_turn_masks_everything_but_assistant_content():
    tok = FakeChatTokenizer()
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi there"},
            {"role": "assistant", "content": "hello you"}, {"role": "user", "content": "again"},
            {"role": "assistant", "content": "sure thing friend"}]
    out, n_err, n_long = process_samples([{"messages": msgs}], tok)
    assert (n_err, n_long) == (0, 0) and len(out) == 1
    s = out[0]
    assert len(s["labels"]) == len(s["input_ids"]) == s["len"]
    inv = {v: k for k, v in tok.vocab.items()}
    trained = [inv[t] for t, l in zip(s["input_ids"], s["labels"]) if l != T.IGNORE]
    # both assistant turns (with their end-of-turn token) are trained on; nothing from system / user turns is
    assert trained == ["hello", "you", "<|end|>", "sure", "thing", "friend", "<|end|>"]
    assert all(l == t for t, l in zip(s["input_ids"], s["labels"]) if l != T.IGNORE)
    assert s["num_loss_counted_tokens"] == 7


def test_pretrain_sample_is_fully_unmasked_and_gets_eos():
    tok = FakeChatTokenizer()
    out, _, _ = process_samples([{"messages": [{"role": "pretrain", "content": "plain text to model"}]}], tok)
    s = out[0]
    assert s["pretrain"] and s["labels"] == s["input_ids"] and s["input_ids"][-1] == tok.vocab["</s>"]
    assert s["num_loss_counted_tokens"] == s["len"] == 5


def test_errors_and_overlong_samples_are_filtered():
    tok = FakeChatTokenizer()
    good = {"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}]}
    empty = {"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": ""}]}
    two_pretrain = {"messages": [{"role": "pretrain", "content": "x"}, {"role": "user", "content": "y"}]}
    bad_role = {"messages": [{"role": "robot", "content": "x"}]}
    long = {"messages": [{"role": "user", "content": "w " * 50}, {"role": "assistant", "content": "a"}]}
    out, n_err, n_long = process_samples([json.dumps(x) for x in (good, empty, two_pretrain, bad_role, long)], tok,
                                         max_sample_num_tokens=20)
    assert len(out) == 1 and n_err == 3 and n_long == 1
    assert out[0]["messages"] == good["messages"]   # other columns are kept


def test_to_messages():
    assert to_messages({"question": "q?", "solution": "s."}) == {"messages": [{"role": "user", "content": "q?"},
                                                                                {"role": "assistant", "content": "s."}]}
    assert to_messages({"a": "x", "b": "y"}, "a", "b")["messages"][1]["content"] == "y"


CHATML = ("{% for m in messages %}{{ '<|im_start|>' + m['role'] + '\n' + m['content'] + '<|im_end|>' + '\n' }}{% endfor %}")


def _real_tokenizer_dir(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from transformers import PreTrainedTokenizerFast
    words = ["<pad>", "<s>", "</s>", "<unk>", "<|im_start|>", "<|im_end|>", "user", "assistant", "1", "what", "is", "two",
             "plus", "four", "it", "six", "some", "raw", "text", "\n"]
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Sequence([
        tokenizers.pre_tokenizers.Split(tokenizers.Regex(r"<\|im_start\|>|<\|im_end\|>|\n"), "isolated"),
        tokenizers.pre_tokenizers.WhitespaceSplit()])
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", pad_token="<pad>", unk_token="<unk>")
    fast.chat_template = CHATML
    path = str(tmp_path / "tok")
    fast.save_pretrained(path)
    return path


def test_process_data_and_make_messages_command_lines(tmp_path):
    tok_dir = _real_tokenizer_dir(tmp_path)
    raw = tmp_path / "qa.jsonl"
    raw.write_text(json.dumps({"question": "what is two plus four", "solution": "it is six"}) + "\n")
    msgs = tmp_path / "messages.jsonl"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", TOKENIZERS_PARALLELISM="false")
    p = subprocess.run([sys.executable, "-m", "mini_trainer_b200.cli.make_messages", "--input-file", str(raw),
                        "--output-file", str(msgs)], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    with open(msgs, "a") as f:
        f.write(json.dumps({"messages": [{"role": "pretrain", "content": "some raw text"}]}) + "\n")
        f.write(json.dumps({"messages": [{"role": "user", "content": "what"}, {"role": "assistant", "content": ""}]}) + "\n")
    out = tmp_path / "tokens.jsonl"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "process_data.py"), "--input-file", str(msgs), "--output-file", str(out),
                        "--model-name-or-path", tok_dir, "--max-sample-num-tokens", "64", "--num-proc", "1"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    rows = [json.loads(l) for l in open(out)]
    assert len(rows) == 2                                   # the empty-assistant sample was dropped
    chat, pre = rows
    assert set(chat) >= {"input_ids", "labels", "len", "num_loss_counted_tokens", "messages"}
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(tok_dir)
    trained = tok.convert_ids_to_tokens([t for t, l in zip(chat["input_ids"], chat["labels"]) if l != -100])
    assert trained[:3] == ["it", "is", "six"] and "what" not in trained and chat["num_loss_counted_tokens"] == len(trained)
    assert pre["labels"] == pre["input_ids"] and pre["input_ids"][-1] == tok.eos_token_id
    assert "<|mAsK|>" in p.stdout                           # the preview shows masked label positions
    # the output feeds the training loader as is
    from mini_trainer_b200.data.sampler import JsonlDataset
    ds = JsonlDataset(str(out))
    assert len(ds) == 2 and int(ds.lengths[0]) == chat["len"]


def test_sequence_length_sweep_tool_on_cpu(tmp_path):
    from mini_trainer_b200.cli.seq_sweep import create_uniform_batch, sweep_configs
    assert sweep_configs(4096, 1024) == [(4, 1024), (2, 2048), (1, 4096)]
    assert sweep_configs(3000, 1024) == [(2, 1024), (1, 2048)]
    b = create_uniform_batch(3, 5, vocab_size=11)
    assert b["input_ids"].shape == (1, 15) and b["position_ids"][0].tolist() == [0, 1, 2, 3, 4] * 3
    assert b["cu_seqlens"].tolist() == [0, 5, 10, 15] and b["num_samples"] == 3
    out = tmp_path / "sweep.json"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT="29661")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    p = subprocess.run([sys.executable, "-m", "mini_trainer_b200.cli.seq_sweep", "--model-name-or-path", "random:tiny-qwen2",
                        "--start-tokens", "256", "--budget-increase", "256", "--max-tokens", "512", "--min-seq-len", "128",
                        "--num-iterations", "1", "--output-file", str(out)], cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    res = json.load(open(out))
    assert [(r["token_budget"], r["num_sequences"], r["sequence_length"]) for r in res] == \
        [(256, 2, 128), (256, 1, 256), (512, 4, 128), (512, 2, 256), (512, 1, 512)]
    assert all(r["status"] == "ok" and r["tokens_per_second"] > 0 for r in res)
    assert "tok/s" in p.stdout


def test_property_only_assistant_turns_are_trained_on():
    """Any conversation (optional system turn, any number of user / assistant turns in any order, any words): the
    unmasked tokens are exactly the assistant turns' words with their end-of-turn token, in order, labels equal the
    inputs where unmasked, and the counts add up."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    words = st.lists(st.sampled_from(["alpha", "beta", "gamma", "delta", "x1", "y2", "zed"]), min_size=1, max_size=6)
    turns = st.lists(st.tuples(st.sampled_from(["user", "assistant"]), words), min_size=1, max_size=8)

    @settings(max_examples=80, deadline=None)
    @given(system=st.one_of(st.none(), words), turns=turns)
    def run(system, turns):
        tok = FakeChatTokenizer()
        msgs = ([{"role": "system", "content": " ".join(system)}] if system else []) + \
               [{"role": r, "content": " ".join(w)} for r, w in turns]
        out, n_err, n_long = process_samples([{"messages": msgs}], tok)
        if not any(r == "assistant" for r, _ in turns):   # nothing to learn from: the sample is dropped or fully masked
            assert n_err == 1 or all(l == T.IGNORE for l in out[0]["labels"])
            return
        assert (n_err, n_long) == (0, 0)
        s = out[0]
        inv = {v: k for k, v in tok.vocab.items()}
        trained = [inv[t] for t, l in zip(s["input_ids"], s["labels"]) if l != T.IGNORE]
        want = [w for r, ws in turns if r == "assistant" for w in ws + ["<|end|>"]]
        assert trained == want
        assert all(l == t for t, l in zip(s["input_ids"], s["labels"]) if l != T.IGNORE)
        assert s["num_loss_counted_tokens"] == len(want) and s["len"] == len(s["input_ids"])

    run()
