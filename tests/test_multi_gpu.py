"""Sharded engine on 2 GPUs (NCCL and the symmetric-memory backend) against the 1-GPU engine.

Runs as child processes, one per GPU, with NVLS disabled; skipped when fewer than two GPUs are
visible. Ranks only stop between steps, with no kernel or collective in flight.
"""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, os.environ["MTB200_REPO"])
import torch.distributed as dist
from mini_trainer_b200.utils.dist import init_distributed_environment
from mini_trainer_b200.models.config import get_preset
from mini_trainer_b200.ops import get_ops
from mini_trainer_b200.parallel.comm import make_comm
from mini_trainer_b200.parallel.engine import OptimConfig, ShardedEngine
from mini_trainer_b200.data.sampler import get_data_loader
from mini_trainer_b200.data.synthetic import LengthSpec, synthetic_dataset

device = init_distributed_environment(timeout_minutes=3)
rank, world = dist.get_rank(), dist.get_world_size()
cfg = get_preset(os.environ.get("MTB200_PRESET", "smoke-llama"))
comm = make_comm(os.environ.get("MTB200_COMM", "auto"), device)
budget = os.environ.get("MTB200_TEST_BUDGET", "0")
eng = ShardedEngine(cfg, device, get_ops(device), comm=comm, optim=OptimConfig(),
                    activation_budget_bytes=None if budget == "auto" else int(budget))
eng.init_random(seed=5, std=0.05)
if os.environ.get("MTB200_OSFT") == "1":
    from mini_trainer_b200.parallel.osft import enable_osft
    ctl = enable_osft(eng, rank_ratio=0.5)
    if world > 1 and os.environ.get("MTB200_COMM") == "symmetric":
        assert ctl.owner_reduce and ctl.kernels      # ownership by matrix inside the reduction, products on tcgen05
        assert ctl.fused == (os.environ.get("MTB200_OSFT_FUSED", "1") != "0")   # ... and the reduction inside the GEMM itself
init = [g.master.clone() for g in eng.groups]
ds = synthetic_dataset(64, LengthSpec(5.0, 0.7, 8, 700), cfg.vocab_size, seed=1)
loader = iter(get_data_loader(dataset=ds, batch_size=16, max_tokens_per_gpu=1500, seed=3, rank=rank, world_size=world, prefetch=0))
out = []
for step in range(3):
    res = eng.train_step(next(loader), lr=1e-3)
    loss = res["loss_sum"].clone()
    dist.all_reduce(loss)
    out.append({"loss": loss.item(), "grad_norm": res["grad_norm"].item()})
torch.cuda.synchronize()
if hasattr(eng.ops, "check_status"):
    eng.ops.check_status()
if hasattr(comm, "check_status"):
    comm.check_status()
# the UPDATE of every master weight (what three optimizer steps did), gathered with NCCL for the comparison only
deltas = []
for g, m0 in zip(eng.groups, init):
    full = torch.empty(g.layout.padded_numel, dtype=torch.float32, device=device)
    if world == 1:
        full.copy_(g.master - m0)
    else:
        dist.all_gather_into_tensor(full, (g.master - m0).contiguous())
    deltas.append(full[: g.layout.numel].cpu())
if rank == 0:
    if os.environ.get("MTB200_OUT"):
        torch.save(deltas, os.environ["MTB200_OUT"])
    print("RESULT " + json.dumps(out), flush=True)
dist.barrier()
dist.destroy_process_group()
'''


def _run(world: int, comm: str, budget: str = "0", out: str = "", osft: bool = False, extra_env=None):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    # MTB200_POISON: gather targets and gradient buffers are NaN-filled before use, so anything consumed before it
    # arrived (or never written) turns the loss / gradient norm into NaN
    env = dict(os.environ, MTB200_REPO=REPO, MTB200_COMM=comm, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1",
               MASTER_PORT=str(port), MTB200_TEST_BUDGET=budget, MTB200_OUT=out, MTB200_POISON="1",
               MTB200_OSFT="1" if osft else "0", **(extra_env or {}))
    if world == 1:
        cmd = [sys.executable, "-c", WORKER]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), "--no-python", sys.executable, "-c", WORKER]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    for line in proc.stdout.splitlines():
        if line.startswith("RESULT "):
            return json.loads(line[7:])
    raise AssertionError(f"worker failed (rc={proc.returncode}):\n{proc.stdout[-3000:]}\n{proc.stderr[-3000:]}")


def _compare(one, many, f_one, f_many):
    for a, b in zip(one, many):
        assert abs(a["loss"] - b["loss"]) < 2e-2 * abs(a["loss"]), (one, many)
        assert abs(a["grad_norm"] - b["grad_norm"]) < 5e-2 * a["grad_norm"], (one, many)
    # the updated master weights themselves: per group, the update of the sharded run against the 1-GPU run.
    # AdamW's first steps move every element by about lr * sign(g), so elements whose tiny gradient changes sign
    # with the reduction order differ by 2 lr; a wrong shard mapping or a missed reduction gives an error near 1.4.
    d1, dn = torch.load(f_one), torch.load(f_many)
    assert len(d1) == len(dn)
    for x, y in zip(d1, dn):
        assert x.shape == y.shape and torch.isfinite(y).all()
        assert ((x - y).norm() / (x.norm() + 1e-12)).item() < 0.2


@pytest.mark.parametrize("comm,budget", [("torchdist", "0"), ("symmetric", "0"), ("symmetric", "auto")])
def test_two_gpus_match_one_gpu(comm, budget, tmp_path):
    """budget 0: every block recomputed (parameters gathered inside the recompute GEMMs);
    budget auto: activations kept (parameters prefetched by the stand-alone pull in backward)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    f1, f2 = str(tmp_path / "one.pt"), str(tmp_path / "two.pt")
    one = _run(1, "auto", out=f1)
    two = _run(2, comm, budget, out=f2)
    _compare(one, two, f1, f2)


@pytest.mark.parametrize("switch", ["MTB200_REGION_OVERLAP=0", "MTB200_GEMM2=1", "MTB200_FUSED_GATHER=0"])
def test_two_gpus_symmetric_with_switches(switch, tmp_path):
    """The documented switches of the symmetric backend: one reduction per block instead of one per tensor region,
    the CTA-pair GEMM (and its fused all-gather form) for large problems, stand-alone all-gathers instead of fused ones."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    f1, f2 = str(tmp_path / "one.pt"), str(tmp_path / "two.pt")
    one = _run(1, "auto", out=f1)
    k, v = switch.split("=")
    two = _run(2, "symmetric", "0", out=f2, extra_env={k: v})
    _compare(one, two, f1, f2)


@pytest.mark.parametrize("comm,fused", [("symmetric", "1"), ("symmetric", "0"), ("torchdist", "1")])
def test_osft_two_gpus_match_one_gpu(comm, fused, tmp_path):
    """OSFT on 2 GPUs against OSFT on 1 GPU. Symmetric backend: each projection's gradient is pulled from all
    ranks, summed and multiplied by V_lo^T in ONE tcgen05 GEMM kernel on the owning rank (fused = 1), or reduced to
    the owner by the reduce-scatter kernel first (fused = 0); the other factor products run on the tcgen05 GEMM, the
    recomposed weights are pulled over NVLink, and no NCCL call is made in the step. NCCL backend: gather /
    broadcast form of the same update."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    f1, f2 = str(tmp_path / "one.pt"), str(tmp_path / "two.pt")
    one = _run(1, "auto", out=f1, osft=True)
    two = _run(2, comm, "0", out=f2, osft=True, extra_env={"MTB200_OSFT_FUSED": fused})
    _compare(one, two, f1, f2)


def test_two_gpus_mixture_of_experts_match_one_gpu(tmp_path):
    """A small Mixtral over the symmetric backend: the block (router and experts included) arrives by the stand-alone
    peer-load all-gather one block ahead and its gradient buffer is reduced in one piece."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    f1, f2 = str(tmp_path / "one.pt"), str(tmp_path / "two.pt")
    env = {"MTB200_PRESET": "tiny-mixtral"}
    one = _run(1, "auto", out=f1, extra_env=env)
    two = _run(2, "symmetric", "0", out=f2, extra_env=env)
    _compare(one, two, f1, f2)


@pytest.mark.parametrize("world", [4, 8])
def test_more_gpus_symmetric_match_one_gpu(world, tmp_path):
    """World sizes 4 and 8 (their own reduce-scatter instantiations and shard padding) over the symmetric backend."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    f1, fn = str(tmp_path / "one.pt"), str(tmp_path / "many.pt")
    one = _run(1, "auto", out=f1)
    many = _run(world, "symmetric", "0", out=fn)
    _compare(one, many, f1, fn)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_comm_kernels_against_torch_collectives(world):
    """The fused all-gather + GEMM (one Llama-3.1-8B block: 16 chunks of 128 KB under every weight tile, both
    launches, on CTA pairs and on single CTAs), the stand-alone peer-load all-gather and the flag-synchronised reduce-scatter against
    ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` + a plain GEMM, on every GPU count available."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), MTB200_BENCH_TOKENS="4096")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(REPO, "bench_comm.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    recs = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    fused = [r for r in recs if r["op"].startswith("allgather+gemm")]
    assert len(fused) == 4 and all(r["gathered_correct"] and r["rel_err"] < 1e-2 for r in fused), recs
    rs = [r for r in recs if r["op"].startswith("reduce-scatter")]
    assert len(rs) == 1 and rs[0]["rel_err_vs_nccl"] < 1e-2, recs
    ag = [r for r in recs if r["op"].startswith("allgather block")]
    assert len(ag) == 1 and ag[0]["gathered_correct"], recs
