"""The benchmark harness itself, on CPU: the step plan both arms share, the wall-clock guard and the
result line's contract (one JSON line, the keys the driver parses, identical ``config`` in both arms)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_plan_steps_honours_requests_that_fit_and_cuts_those_that_do_not():
    # one GPU: 25 steps of the reference arm (32 s each) do not fit ten minutes -> 3 warm-ups + what fits
    steps, warm = bench.plan_steps("llama-3.1-8b", 1, 20, 5, 600.0)
    assert warm == 3 and 1 <= steps < 20
    assert (steps + warm) * 32.0 + bench.SETUP_SECONDS <= 600.0
    # two or more GPUs: the full request runs
    for n in (2, 4, 8):
        assert bench.plan_steps("llama-3.1-8b", n, 20, 5, 600.0) == (20, 5)
    # a small request is never changed
    assert bench.plan_steps("llama-3.1-8b", 1, 3, 3, 600.0) == (3, 3)
    # the plan depends only on its arguments (both arms call it with the same ones)
    assert bench.plan_steps("llama-3.1-8b", 1, 20, 5, 600.0) == bench.plan_steps("llama-3.1-8b", 1, 20, 5, 600.0)
    # a hopeless budget still times one step
    assert bench.plan_steps("llama-3.1-70b", 1, 20, 5, 100.0)[0] == 1


def test_dataset_size_is_shared_and_stable():
    assert bench.dataset_size(128, 6) == bench.dataset_size(128, 25) == 128 * 32
    assert bench.dataset_size(128, 40) == 128 * 40


def test_guard_cuts_steps_when_warmup_was_slow():
    assert bench.guard_steps(20, warmup_wall_s=3.0, warmup=3, budget_s=1e9) == 20
    assert bench.guard_steps(20, warmup_wall_s=300.0, warmup=3, budget_s=bench.time.time() - bench.T_START + 570.0) == 5
    assert bench.guard_steps(20, warmup_wall_s=300.0, warmup=3, budget_s=0.0) == 1


def _run(nproc, extra, port=None):
    import socket
    sk = socket.socket(); sk.bind(("127.0.0.1", 0)); port = sk.getsockname()[1]; sk.close()   # a fresh port per launch
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT=str(port), MASTER_ADDR="127.0.0.1")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    cmd = [sys.executable]
    if nproc > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
                "--master-port", str(port)]
    cmd += [os.path.join(ROOT, "bench.py"), "--gpus", str(nproc), "--model", "tiny-qwen2"] + extra
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, lines   # exactly one JSON line, from rank 0
    return json.loads(lines[0])


def test_native_arm_result_line_on_two_cpu_ranks():
    rec = _run(2, ["--steps", "2", "--warmup", "3", "--batch-size", "8", "--max-tokens-per-gpu", "2048"], 29671)
    assert rec["impl"] == "native" and rec["n_gpus"] == 2 and rec["steps"] == 2 and rec["warmup"] == 3
    assert rec["steps_requested"] == 2 and rec["warmup_requested"] == 3
    assert rec["value"] > 0 and rec["higher_is_better"] is True and rec["scaling"] == "strong"
    assert rec["e2e"]["value"] > 0 and rec["e2e"]["h2d_bytes_per_step"] > 0 and rec["e2e"]["d2h_bytes_per_step"] == 8
    assert rec["config"] == bench.common_config("tiny-qwen2", 8, 2048, 2)
    assert abs(rec["ms_per_step"] * rec["steps"] / 1e3 * rec["value"] - rec["detail"]["tokens_per_step"] * rec["steps"]) < 1.0


def test_time_budget_cuts_the_request_and_reports_both_counts():
    rec = _run(1, ["--steps", "500", "--warmup", "3", "--time-budget-s", "91.5", "--resident", "off", "--batch-size", "8",
                   "--max-tokens-per-gpu", "2048"], 29672)
    # tiny-qwen2 is sized at 0.2 s per step: (91.5 - 90) / 0.2 = 7 steps in all
    assert rec["warmup"] == 3 and rec["steps"] <= 4 and rec["steps_requested"] == 500
    assert "resident" not in rec
