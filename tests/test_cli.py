"""The ``train.py`` entry point end to end on CPU: reference flag names, files it must leave behind."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def test_train_cli_runs_and_writes_reference_layout(tmp_path):
    out = str(tmp_path / "run")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT=str(_free_port()))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--model-name-or-path", "random:tiny-qwen2",
           "--data-path", "synthetic:tiny-qwen2:48", "--batch-size", "8", "--max-tokens-per-gpu", "2048",
           "--output-dir", out, "--min-samples-per-checkpoint", "16", "--max-steps", "2", "--learning-rate", "1e-4",
           "--num-warmup-steps", "2", "--lr-scheduler", "constant_with_warmup", "--seed", "893", "--use-liger-kernels",
           "--logging-level", "WARNING"]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    params = json.load(open(os.path.join(out, "training_params.json")))
    assert params["batch_size"] == 8 and params["max_tokens_per_gpu"] == 2048 and params["WORLD_SIZE"] == 1
    assert set(params) >= {"model_name_or_path", "data_path", "learning_rate", "num_warmup_steps", "lr_scheduler", "seed",
                           "use_liger_kernels", "output_dir", "logging_level", "min_samples_per_checkpoint", "RANK"}
    rows = [json.loads(l) for l in open(os.path.join(out, "training_metrics_0.jsonl"))]
    assert [r["step"] for r in rows] == [1, 2]
    assert rows[0]["lr"] == 1e-4 and rows[0]["num_samples"] == 8
    ckpt = os.path.join(out, "hf_format", "samples_16.0")
    assert os.path.exists(os.path.join(ckpt, "model.safetensors")) and os.path.exists(os.path.join(ckpt, "config.json"))


def test_bench_reference_arm_reports_unavailable_without_a_gpu():
    """Without CUDA the reference arm cannot run; the contract is one JSON line and exit code 0."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT=str(_free_port()))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                          env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rec = json.loads(proc.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec


def test_train_cli_synthetic_spec_caps_sample_length(tmp_path):
    out = str(tmp_path / "run")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT=str(_free_port()))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--model-name-or-path", "random:tiny-qwen2",
           "--data-path", "synthetic:tiny-qwen2:32:100", "--batch-size", "8", "--max-tokens-per-gpu", "128",
           "--output-dir", out, "--min-samples-per-checkpoint", "100000", "--max-steps", "1", "--adam-beta2", "0.99",
           "--max-shard-gb", "0.001", "--logging-level", "WARNING"]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "exceed max tokens per gpu" not in proc.stdout   # every sample is at most 100 tokens long
    rows = [json.loads(l) for l in open(os.path.join(out, "training_metrics_0.jsonl"))]
    assert rows[0]["num_samples"] == 8


def test_smoke_run_two_gloo_ranks():
    """The sharding smoke script (plain-collectives backend) on two CPU ranks."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "mini_trainer_b200.cli.smoke_run", "--num-steps", "2", "--sequence-length", "32"]
    proc = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "smoke run ok" in proc.stdout
    recs = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert [r["step"] for r in recs] == [1, 2] and recs[1]["loss"] < recs[0]["loss"]


def _train_cli(out, extra, port=None):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT=str(_free_port()))   # a fresh port per launch
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--model-name-or-path", "random:nano-llama",
           "--data-path", "synthetic:tiny-qwen2:40:200", "--batch-size", "8", "--max-tokens-per-gpu", "1024",
           "--output-dir", out, "--learning-rate", "1e-3", "--num-warmup-steps", "3", "--seed", "893",
           "--logging-level", "WARNING", "--save-train-state"] + extra
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]


def test_resume_continues_weights_optimizer_schedule_and_data(tmp_path):
    """4 steps in one go == 2 steps, stop, resume from the written training state, 2 more steps:
    the same batches are drawn (the 40-sample dataset wraps into its second epoch at step 6, not
    reached here, but step 3-4 must not replay step 1-2), the same learning rates are applied, the sample
    counters and checkpoint names continue, and the final weights agree."""
    import torch
    from mini_trainer_b200.ckpt import safetensors_io as st
    a, b = str(tmp_path / "straight"), str(tmp_path / "resumed")
    _train_cli(a, ["--max-steps", "4", "--min-samples-per-checkpoint", "16"], 29651)
    _train_cli(b, ["--max-steps", "2", "--min-samples-per-checkpoint", "16"], 29652)
    state = os.path.join(b, "train_state", "samples_16.0")
    meta = json.load(open(os.path.join(state, "state.json")))
    assert meta["train_step"] == 2 and meta["batches_consumed"] == 2 and meta["total_samples_accumulated"] == 16.0
    _train_cli(b, ["--max-steps", "4", "--min-samples-per-checkpoint", "16", "--resume-from", state], 29653)
    rows_a = [json.loads(l) for l in open(os.path.join(a, "training_metrics_0.jsonl"))]
    rows_b = [json.loads(l) for l in open(os.path.join(b, "training_metrics_0.jsonl"))]
    assert [r["step"] for r in rows_b] == [1, 2, 3, 4]
    for ra, rb in zip(rows_a, rows_b):
        assert ra["lr"] == rb["lr"] and ra["num_total_tokens"] == rb["num_total_tokens"]
        assert abs(ra["loss"] - rb["loss"]) < 1e-5 and abs(ra["grad_norm"] - rb["grad_norm"]) < 1e-4
        assert ra["total_samples_accumulated"] == rb["total_samples_accumulated"]
    wa = st.load_file(os.path.join(a, "hf_format", "samples_32.0", "model.safetensors"))
    wb = st.load_file(os.path.join(b, "hf_format", "samples_32.0", "model.safetensors"))
    assert set(wa) == set(wb) and all(torch.equal(wa[k], wb[k]) for k in wa)


def _train_cli_ranks(out, extra, port=None, world=2):
    port = _free_port()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "train.py"), "--model-name-or-path", "random:nano-llama",
           "--data-path", "synthetic:tiny-qwen2:40:200", "--batch-size", "8", "--max-tokens-per-gpu", "1024",
           "--output-dir", out, "--learning-rate", "1e-3", "--num-warmup-steps", "3", "--seed", "893",
           "--logging-level", "WARNING", "--save-train-state"] + extra
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]


def test_resume_two_ranks_with_osft(tmp_path):
    """The same stop-and-resume on two gloo ranks with OSFT on: every rank writes and reads its own shard of the
    training state, including the trainable factors (and their moments) of the matrices it owns."""
    import torch
    from mini_trainer_b200.ckpt import safetensors_io as st
    a, b = str(tmp_path / "straight"), str(tmp_path / "resumed")
    common = ["--min-samples-per-checkpoint", "16", "--osft", "--osft-rank-ratio", "0.5"]
    _train_cli_ranks(a, ["--max-steps", "4"] + common, 29661)
    _train_cli_ranks(b, ["--max-steps", "2"] + common, 29662)
    state = os.path.join(b, "train_state", "samples_16.0")
    assert sorted(f for f in os.listdir(state) if f.endswith(".safetensors")) == ["rank0-of-2.safetensors", "rank1-of-2.safetensors"]
    shard1 = st.load_file(os.path.join(state, "rank1-of-2.safetensors"))
    assert any(k.startswith("osft.") for k in shard1), sorted(shard1)[:8]
    _train_cli_ranks(b, ["--max-steps", "4", "--resume-from", state] + common, 29663)
    rows_a = [json.loads(l) for l in open(os.path.join(a, "training_metrics_0.jsonl"))]
    rows_b = [json.loads(l) for l in open(os.path.join(b, "training_metrics_0.jsonl"))]
    assert [r["step"] for r in rows_b] == [1, 2, 3, 4]
    for ra, rb in zip(rows_a, rows_b):
        assert ra["lr"] == rb["lr"] and ra["num_total_tokens"] == rb["num_total_tokens"]
        assert abs(ra["loss"] - rb["loss"]) < 1e-5 and abs(ra["grad_norm"] - rb["grad_norm"]) < 1e-4
    wa = st.load_file(os.path.join(a, "hf_format", "samples_32.0", "model.safetensors"))
    wb = st.load_file(os.path.join(b, "hf_format", "samples_32.0", "model.safetensors"))
    assert set(wa) == set(wb) and all(torch.equal(wa[k], wb[k]) for k in wa)


import pytest  # noqa: E402


@pytest.mark.parametrize("osft,new_world", [(False, 1), (True, 3)])
def test_resume_on_another_number_of_ranks(tmp_path, osft, new_world):
    """A training state written by two ranks continues on one rank (plain training) and on three (OSFT): every group's
    flat buffer is re-sliced on load, OSFT factors follow their matrices to the new owners, the data stream and the
    schedule go on where they stopped, and the run matches an uninterrupted one to the precision the different reduction
    orders allow."""
    import torch
    from mini_trainer_b200.ckpt import safetensors_io as st
    a, b = str(tmp_path / "straight"), str(tmp_path / "resharded")
    common = ["--min-samples-per-checkpoint", "16"] + (["--osft"] if osft else [])
    _train_cli(a, ["--max-steps", "4"] + common)
    _train_cli_ranks(b, ["--max-steps", "2"] + common, world=2)
    state = os.path.join(b, "train_state", "samples_16.0")
    if new_world == 1:
        _train_cli(b, ["--max-steps", "4", "--resume-from", state] + common)
    else:
        _train_cli_ranks(b, ["--max-steps", "4", "--resume-from", state] + common, world=new_world)
    rows_a = [json.loads(l) for l in open(os.path.join(a, "training_metrics_0.jsonl"))]
    rows = [json.loads(l) for l in open(os.path.join(b, "training_metrics_0.jsonl"))]
    assert [r["step"] for r in rows] == [1, 2, 3, 4]
    for ra, rb in zip(rows_a, rows):
        assert ra["lr"] == rb["lr"] and ra["num_loss_counted_tokens"] == rb["num_loss_counted_tokens"]
        assert abs(ra["loss"] - rb["loss"]) < 2e-4 * abs(ra["loss"]) and abs(ra["grad_norm"] - rb["grad_norm"]) < 2e-3 * ra["grad_norm"]
    wa = st.load_file(os.path.join(a, "hf_format", "samples_32.0", "model.safetensors"))
    w = st.load_file(os.path.join(b, "hf_format", "samples_32.0", "model.safetensors"))
    assert set(w) == set(wa)
    for k in wa:
        assert torch.allclose(w[k].float(), wa[k].float(), atol=1e-2, rtol=2e-2), k
