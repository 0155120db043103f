"""Headline benchmark: training tokens/s of Llama-3.1-8B-architecture full SFT (random init,
synthetic data), device-timed, max over ranks.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3
    python bench.py --impl reference ...        # the unmodified reference stack, same config

One "step" is one optimizer step over a global batch of 128 synthetic samples (lengths
lognormal(7.5, 1.0) clipped to [64, 65536], -100 on a uniform 10-60 % prefix), LPT-packed to at
most 64 000 tokens per GPU per minibatch, with gradient accumulation over this rank's minibatches,
global-norm clipping and AdamW — nothing is skipped. The global batch is fixed, so the sweep over
GPU counts is strong scaling.

There is ONE timed pass. Every step goes through the public training-step API
(``ShardedEngine.train_step``): each minibatch is copied from pinned host memory inside the timed
region and the step's loss and gradient norm are read back to the host every step. The pass is
bracketed by barrier + synchronize on both sides and measured twice:

* ``value``      — CUDA events on the compute stream around the ``steps`` timed steps (max over ranks);
* ``e2e.value``  — host wall clock from before the first step's first copy is issued to after the
  closing synchronize and the last read-back (max over ranks).

``resident`` (only when the time budget allows) re-runs a few of the same steps with the batches
already on the device: the kernel-only figure that explains the two above.

Time budget. One 8B step takes about 22 s here and 31 s in the reference arm on one GPU, so the
25 steps a caller may ask for do not fit a ten-minute window there. Both arms therefore pass the
request through ``plan_steps`` (a rule that depends only on the GPU count, so both arms run the
same steps on the same batches) and a wall-clock guard measured on the warm-up steps. The line
printed reports ``steps`` / ``warmup`` as actually run and ``steps_requested`` /
``warmup_requested`` as asked.

Inputs (activations of 64 000 tokens x 4096 features per layer) are far larger than the 126 MB
L2, so no explicit L2 flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
BASELINE_TOKENS_PER_S = None  # the reference publishes no throughput number

MODEL = "llama-3.1-8b"
MODEL_LABEL = {"llama-3.1-8b": "Llama-3.1-8B", "llama-3.1-70b": "Llama-3.1-70B", "qwen2.5-1.5b": "Qwen2.5-1.5B",
               "qwen2.5-7b": "Qwen2.5-7B", "tiny-qwen2": "tiny-Qwen2"}
DEFAULT_BUDGET_S = 600.0
T_START = time.time()

# Seconds per optimizer step of the SLOWER arm (the reference stack) on one B200, per model, as
# measured on this pool; the step count both arms run is sized on it. Other GPU counts scale it by
# 1.15 / N (the global batch is fixed).
REF_STEP_SECONDS_1GPU = {"llama-3.1-8b": 32.0, "qwen2.5-1.5b": 5.0, "qwen2.5-7b": 30.0, "llama-3.1-70b": 160.0,
                         "tiny-qwen2": 0.2}
SETUP_SECONDS = 90.0   # model build + data generation of the slower arm


def plan_steps(model: str, n_gpus: int, steps: int, warmup: int, budget_s: float) -> tuple[int, int]:
    """(steps, warmup) both arms run for a request of ``steps`` / ``warmup``.

    The request is honoured whenever ``(steps + warmup)`` steps of the slower arm fit in
    ``budget_s`` after set-up; otherwise warm-up drops to 3 and the timed steps to what fits
    (at least 1). Depends on nothing but its arguments, so both arms agree."""
    est = REF_STEP_SECONDS_1GPU.get(model, 32.0) * (1.0 if n_gpus == 1 else 1.15 / n_gpus)
    fit = int(max(0.0, budget_s - SETUP_SECONDS) / est)
    if steps + warmup <= fit:
        return steps, warmup
    w = min(warmup, 3)
    return max(1, min(steps, fit - w)), w


def dataset_size(batch_size: int, total_steps: int) -> int:
    """Samples in the synthetic dataset: the same in both arms (the sampler's permutation depends
    on it), independent of the step count up to 32 steps so the reference arm can cache its file."""
    return batch_size * max(32, total_steps)


def common_config(model: str, batch_size: int, max_tokens: int, world: int) -> dict:
    """The ``config`` object of the result line, identical in both arms."""
    return {"model": model, "global_batch": batch_size, "seq_len": f"packed, max_tokens_per_gpu={max_tokens}",
            "parallelism": f"dp{world} fully sharded (ZeRO-3 style)",
            "l2": "inputs larger than L2 (activations of tens of thousands of tokens per layer); no explicit flush"}


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx = float(r[2])
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def physical_gpu_index(local_index: int) -> int:
    """nvidia-smi index of the CUDA device ``local_index`` (they differ under CUDA_VISIBLE_DEVICES)."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p.strip() for p in vis.split(",") if p.strip()]
        if local_index < len(parts) and parts[local_index].isdigit():
            return int(parts[local_index])
    return local_index


def guard_steps(steps: int, warmup_wall_s: float, warmup: int, budget_s: float, reserve_s: float = 20.0) -> int:
    """Wall-clock guard: timed steps that still fit in the budget given what warm-up cost."""
    per_step = warmup_wall_s / max(1, warmup)
    left = budget_s - (time.time() - T_START) - reserve_s
    return max(1, min(steps, int(left / max(per_step, 1e-3))))


# ------------------------------------------------------------------------------------------
# our implementation
# ------------------------------------------------------------------------------------------
def run_native(args) -> dict:
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REPO)
    from mini_trainer_b200.data.sampler import InfiniteSampler, MaxTokensPerRankCollator
    from mini_trainer_b200.data.synthetic import CONFIG_DATA, synthetic_dataset
    from mini_trainer_b200.models import decoder as D
    from mini_trainer_b200.models.config import get_preset
    from mini_trainer_b200.ops import get_ops
    from mini_trainer_b200.parallel.comm import make_comm
    from mini_trainer_b200.parallel.engine import OptimConfig, ShardedEngine, plan_state_dtype
    from mini_trainer_b200.utils.dist import init_distributed_environment
    from mini_trainer_b200.utils.lr import LRSchedule

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N>1")
    device = init_distributed_environment()
    rank = dist.get_rank()
    cfg = get_preset(args.model)
    spec, vocab, max_tokens, batch_size = CONFIG_DATA[args.model]
    max_tokens = args.max_tokens_per_gpu or max_tokens
    batch_size = args.batch_size or batch_size
    steps, warmup = plan_steps(args.model, world, args.steps, args.warmup, args.time_budget_s)

    comm = make_comm(args.comm, device)
    on_gpu = device.type == "cuda"   # a CPU run (gloo) exercises the same harness in the tests; it is not a benchmark
    hbm = torch.cuda.get_device_properties(device).total_memory if on_gpu else 1e15
    sdt = {"auto": plan_state_dtype(cfg, world, hbm, max(max_tokens, spec.hi)), "fp32": torch.float32,
           "bf16": torch.bfloat16}[args.state_dtype]
    ops = get_ops(device)
    eng = ShardedEngine(cfg, device, ops, comm=comm, state_dtype=sdt, optim=OptimConfig(lr=1e-5))
    eng.init_random(seed=893, on_device=on_gpu)
    eng.reserve_host_offload(max(max_tokens, spec.hi))   # pinned buffers for the longest sample, if its inputs will not fit (70B)
    if args.osft:
        from mini_trainer_b200.parallel.osft import enable_osft
        enable_osft(eng, rank_ratio=0.5)
    sched = LRSchedule(1e-5, "constant_with_warmup", 10)

    # identical batches on every rank; each rank packs its own share. Same dataset size, sampler and
    # seed as the reference arm, so both arms draw the same samples in the same order.
    ds = synthetic_dataset(dataset_size(batch_size, steps + warmup), spec, cfg.vocab_size, seed=893)
    sampler = iter(InfiniteSampler(len(ds), seed=893))
    cost_len = cfg.attention_cost_length() if args.balance == "cost" else None
    coll = MaxTokensPerRankCollator(max_tokens, rank=rank, world_size=world, cost_len=cost_len)
    batches = []
    for _ in range(steps + warmup):
        idx = [next(sampler) for _ in range(batch_size)]
        mbs = coll.collate_indices(ds, idx)
        for mb in mbs:
            for k, v in list(mb.items()):
                if isinstance(v, torch.Tensor) and on_gpu:
                    mb[k] = v.pin_memory()
        batches.append((mbs, int(ds.lengths[idx].sum())))

    def sync():
        dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()

    class _HostTimer:   # stands in for a CUDA event on CPU
        def record(self):
            self.t = time.perf_counter()

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

    new_event = (lambda: torch.cuda.Event(enable_timing=True)) if on_gpu else _HostTimer

    h2d = d2h = 0
    last_host = None

    def step_e2e(mbs):
        nonlocal h2d, d2h, last_host
        out = eng.train_step(mbs, sched.current())
        sched.step()
        last_host = torch.stack([out["loss_sum"], out["grad_norm"].reshape(())]).cpu()   # device -> host read of the result
        d2h = last_host.numel() * last_host.element_size()
        h2d = out["h2d_bytes"]   # counted where the copies are issued (models/decoder.py make_packed_batch)

    resident = {}

    def step_resident(mbs):
        key = id(mbs)
        if key not in resident:
            resident[key] = [(D.make_packed_batch(mb, device), 1.0 / max(1, mb["batch_num_loss_counted_tokens"])) for mb in mbs]
        for k, (pb, scale) in enumerate(resident[key]):
            eng.forward_backward(pb, scale, last=k == len(resident[key]) - 1)
        eng.optimizer_step(sched.current())
        sched.step()

    def timed(step_fn, first, n):
        clocks = ClockSampler(physical_gpu_index(torch.cuda.current_device())) if rank == 0 and on_gpu else None
        if clocks:
            clocks.start()
        eng.measure_exposed_comm(world > 1 and on_gpu)
        l0 = getattr(ops, "launches", 0) + getattr(comm, "launches", 0)
        e0, e1 = new_event(), new_event()
        t0 = time.perf_counter()
        e0.record()
        toks = 0
        for i in range(n):
            mbs, ntok = batches[first + i]
            step_fn(mbs)
            toks += ntok
        e1.record()
        sync()
        wall = time.perf_counter() - t0
        exposed = eng.exposed_comm_ms()
        ms = torch.tensor([e0.elapsed_time(e1), exposed["stream_ms"], exposed["in_kernel_ms"], wall * 1e3], device=device)
        eng.measure_exposed_comm(False)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return {"ms": ms[0].item(), "exposed_stream_ms": ms[1].item(), "exposed_kernel_ms": ms[2].item(),
                "wall_ms": ms[3].item(), "tokens": toks, "clocks": clocks.stop() if clocks else None,
                "launches": getattr(ops, "launches", 0) + getattr(comm, "launches", 0) - l0}

    # warm-up through the same public API, then the wall-clock guard on what it cost
    sync()
    tw = time.perf_counter()
    for i in range(warmup):
        step_e2e(batches[i][0])
    sync()
    tw = torch.tensor([time.perf_counter() - tw], device=device)
    dist.all_reduce(tw, op=dist.ReduceOp.MAX)
    agreed = torch.tensor([guard_steps(steps, tw.item(), warmup, args.time_budget_s)], device=device)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN)   # every rank must run the same number of steps
    steps = int(agreed.item())

    r = timed(step_e2e, warmup, steps)
    if hasattr(ops, "check_status"):
        ops.check_status()
    if hasattr(comm, "check_status"):
        comm.check_status()
    loss_last = float(last_host[0]) if last_host is not None else None

    # kernel-only figure on a few of the same batches, if the budget still has room for it
    r_res = None
    n_res = min(steps, 3)
    per_step_s = r["wall_ms"] / 1e3 / steps
    room = torch.tensor([args.time_budget_s - (time.time() - T_START) - (n_res + 1) * per_step_s - 15.0], device=device)
    dist.all_reduce(room, op=dist.ReduceOp.MIN)
    if args.resident != "off" and room.item() > 0:
        for i in range(n_res):   # stage these batches on the device outside the timed region
            mbs = batches[warmup + i][0]
            resident[id(mbs)] = [(D.make_packed_batch(mb, device), 1.0 / max(1, mb["batch_num_loss_counted_tokens"])) for mb in mbs]
        sync()
        r_res = timed(step_resident, warmup, n_res)
        resident.clear()
    if getattr(ops, "profile", None) is not None and rank == 0:
        print("per-op device ms (all phases):", json.dumps({k: round(v, 1) for k, v in ops.profile_summary().items()}), file=sys.stderr)

    tps = r["tokens"] / (r["ms"] / 1e3)
    tps_e2e = r["tokens"] / (r["wall_ms"] / 1e3)
    peak_gb = torch.cuda.max_memory_allocated(device) / 1e9 if on_gpu else 0.0
    exposed_pct = 100.0 * (r["exposed_stream_ms"] + r["exposed_kernel_ms"]) / r["ms"]
    result = {
        "metric": f"train tokens/sec, {MODEL_LABEL.get(args.model, args.model)}-architecture full SFT (device-timed, max over ranks)",
        "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": r["ms"] / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": (tps / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
        "dtype": "bf16" if on_gpu else "fp32 (CPU harness check, not a benchmark)", "data": f"synthetic (random-init weights, lognormal({spec.mu},{spec.sigma}) lengths clipped to [{spec.lo},{spec.hi}], uniform token ids, -100 prefix masks)",
        "impl": "native",
        "config": common_config(args.model, batch_size, max_tokens, world),
        "detail": {"comm": comm.name, "packer_balance": args.balance, "osft": bool(args.osft),
                   "activation_checkpointing": "per block, level chosen from free memory",
                   "optimizer": "AdamW fp32 master, moments " + str(sdt).split(".")[-1],
                   "attention": getattr(ops, "attention_impl", "torch"),
                   "tokens_per_step": r["tokens"] / steps, "peak_mem_gb": round(peak_gb, 1), "loss_last_step_sum": loss_last,
                   "exposed_comm_pct": round(exposed_pct, 2),
                   "exposed_comm_stream_ms_per_step": round(r["exposed_stream_ms"] / steps, 2),
                   "exposed_comm_in_kernel_ms_per_step": round(r["exposed_kernel_ms"] / steps, 2),
                   "exposed_comm_note": "compute-stream time spent waiting on gathers, reductions, peer flags and the "
                                        "post-step barrier (CUDA events) plus the time the fused all-gather GEMMs' TMA "
                                        "producers waited for weight chunks (globaltimer, mean over CTAs); max over ranks",
                   "time_budget_s": args.time_budget_s, "wall_s_total": round(time.time() - T_START, 1)},
        "clocks": r["clocks"],
        "e2e": {"value": tps_e2e, "unit": "tokens/s", "ms_per_step": r["wall_ms"] / steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": "host wall clock around the same steps: pinned-host -> device copies of every minibatch and the "
                       "loss / grad-norm read-back of every step inside the region, closing synchronize included"},
        "gpu_launches": r["launches"],
    }
    if r_res is not None:
        result["resident"] = {"value": r_res["tokens"] / (r_res["ms"] / 1e3), "unit": "tokens/s", "steps": n_res,
                              "ms_per_step": r_res["ms"] / n_res, "note": "batches staged on the device before the region"}
    if rank == 0:
        print(json.dumps(result), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return result


# ------------------------------------------------------------------------------------------
# the unmodified reference (baseline/_ref): FSDP2 + flash-attn 2 + Liger through its own API
# ------------------------------------------------------------------------------------------
def run_reference(args) -> None:
    from baseline.run_reference import main as ref_main
    ref_main(args, sys.modules[__name__])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--comm", default="auto")
    ap.add_argument("--state-dtype", default="auto", choices=["auto", "fp32", "bf16"])
    ap.add_argument("--balance", default="cost", choices=["cost", "tokens"],
                    help="what the LPT packer balances across ranks: estimated compute cost (GEMM + causal attention) "
                         "or tokens (the reference's criterion); the global batch is identical either way")
    ap.add_argument("--batch-size", type=int, default=0)
    ap.add_argument("--max-tokens-per-gpu", type=int, default=0)
    ap.add_argument("--osft", action="store_true", help="orthogonal-subspace fine-tuning of every attention / MLP linear")
    ap.add_argument("--resident", default="auto", choices=["auto", "off"],
                    help="also time a few steps with device-resident batches when the time budget allows")
    ap.add_argument("--time-budget-s", type=float, default=float(os.environ.get("MTB200_BENCH_BUDGET_S", DEFAULT_BUDGET_S)),
                    help="wall-clock budget of one arm, set-up included; the step count is cut to fit (both arms alike)")
    args = ap.parse_args()
    if args.warmup < 3:
        print("note: fewer than 3 warm-up steps requested; results are not a valid measurement", file=sys.stderr)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
