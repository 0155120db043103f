"""Roofline check of the fused compute + collective kernels on N GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29580 bench_comm.py

For one Llama-3.1-8B decoder block (218 M parameters, sharded over the N ranks) it times, with CUDA
events after warm-up and as the max over ranks:

* fused all-gather + GEMM (QKV projection gathering ln1|wqkv|wo|ln2, gate/up projection gathering
  wgu|wd) against the same GEMM on already-gathered weights and against NCCL all-gather + GEMM;
* the stand-alone peer-load all-gather and the flag-synchronised reduce-scatter with fused fp32
  accumulation and sum of squares, against NCCL all_gather_into_tensor / reduce_scatter_tensor.

Roofline of a fused kernel = the slower of (FLOPs / measured cuBLAS bf16 peak) and (bytes that
must cross NVLink into this GPU / 770 GB/s measured peer-copy bandwidth); the script prints
achieved / roofline. Rank 0 prints one JSON line per measurement.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from mini_trainer_b200.models import layout as L  # noqa: E402
from mini_trainer_b200.models.config import get_preset  # noqa: E402
from mini_trainer_b200.ops.native import NativeOps  # noqa: E402
from mini_trainer_b200.parallel.symmetric import SymmetricComm  # noqa: E402
from mini_trainer_b200.utils.dist import init_distributed_environment  # noqa: E402

NVLINK_GBS = 770.0


def peak_tflops():
    p = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    return (json.load(open(p))["bf16_tflops"], "of measured") if os.path.exists(p) else (1590.0, "of fallback")


def main():
    tokens = int(os.environ.get("MTB200_BENCH_TOKENS", "16384"))
    device = init_distributed_environment(timeout_minutes=5)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = get_preset("llama-3.1-8b")
    lay = L.GroupLayout("block", L.block_entries(cfg), world)
    ops = NativeOps(device)
    comm = SymmetricComm(device)
    comm.setup((lay.shard_numel + lay.padded_numel) * 2 + (1 << 20))
    shard = comm.alloc(lay.shard_numel, torch.bfloat16)
    gbuf = comm.alloc(lay.padded_numel, torch.bfloat16)
    shard.copy_((torch.randn(lay.shard_numel, device=device) * 0.02).bfloat16())
    gbuf.copy_((torch.randn(lay.padded_numel, device=device) * 0.01).bfloat16())
    full = torch.zeros(lay.padded_numel, dtype=torch.bfloat16, device=device)
    ref_full = torch.zeros_like(full)
    dist.all_gather_into_tensor(ref_full, shard)
    x = (torch.randn(tokens, cfg.hidden_size, device=device)).bfloat16()
    acc = torch.zeros(lay.shard_numel, dtype=torch.float32, device=device)
    sq = torch.zeros(1, dtype=torch.float32, device=device)
    tf_peak, tag = peak_tflops()
    torch.cuda.synchronize(); dist.barrier()

    def timeit(fn, iters=5, warmup=2):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def emit(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    views = lay.views(full)
    remote = (world - 1) / world
    for two_cta in (True, False):   # CTA pairs (cta_group::2, the default for large problems) and the one-CTA kernel
        ops.use_gemm2 = two_cta
        kern = "2-CTA 256x256" if two_cta else "1-CTA 128x256"
        for stage, wname, desc in ((0, "wqkv", "qkv (gathers ln1|wqkv|wo|ln2)"), (1, "wgu", "gate_up (gathers wgu|wd)")):
            w = views[wname]
            N, K = w.shape

            def fused():
                plan = comm.gather_plan(shard, full, lay, split_before="wgu", small_until="wqkv")
                if stage == 1:   # stage 1 expects the chunks of stage 0 to carry the epoch already
                    plan.flags[: plan.split] = plan.epoch
                return ops.linear(x, w, None, None, gather=(plan, stage))

            probe = comm.gather_plan(shard, full, lay, split_before="wgu", small_until="wqkv")
            if stage == 0:
                full.zero_()
            else:
                full[probe.split * 65536:].zero_()   # keep what stage 0 gathered (it owns the chunk that straddles the boundary)
            out = fused()
            torch.cuda.synchronize()
            plan = comm.gather_plan(shard, full, lay, split_before="wgu", small_until="wqkv")
            lo, hi = (0, plan.split) if stage == 0 else (plan.split, plan.n_chunks)
            lo_e, hi_e = lo * 65536, min(hi * 65536, lay.padded_numel)
            ok_gather = torch.equal(full[lo_e:hi_e], ref_full[lo_e:hi_e])
            ref = x.float() @ ref_full[lay.specs[wname].offset: lay.specs[wname].offset + N * K].view(N, K).float().t()
            err = ((out.float() - ref).norm() / ref.norm()).item()
            t_fused = timeit(fused)
            t_gemm = timeit(lambda: ops.linear(x, w))

            def nccl():
                dist.all_gather_into_tensor(full, shard)
                return ops.linear(x, w)
            t_nccl = timeit(nccl)
            flops = 2.0 * tokens * N * K
            bytes_in = (hi_e - lo_e) * 2 * remote
            roof = max(flops / (tf_peak * 1e9), bytes_in / (NVLINK_GBS * 1e6))
            emit(op=f"allgather+gemm {desc}", kernel=kern, world=world, tokens=tokens, ms_fused=round(t_fused, 3), ms_gemm_only=round(t_gemm, 3),
                 ms_nccl_allgather_whole_block_plus_gemm=round(t_nccl, 3), gathered_correct=bool(ok_gather), rel_err=round(err, 5),
                 nvlink_mb_in=round(bytes_in / 1e6, 1), roofline_ms=round(roof, 3), frac_of_roofline=f"{roof / t_fused:.3f} {tag}",
                 exposed_comm_ms=round(max(0.0, t_fused - t_gemm), 3))


    ops.use_gemm2 = True
    # stand-alone collectives
    full.zero_()
    comm.all_gather(shard, full)
    torch.cuda.synchronize()
    ag_ok = torch.tensor([int(torch.equal(full, ref_full))], device=device)
    dist.all_reduce(ag_ok, op=dist.ReduceOp.MIN)
    t_ag = timeit(lambda: comm.all_gather(shard, full))
    t_ag_nccl = timeit(lambda: dist.all_gather_into_tensor(full, shard))
    nbytes = lay.padded_numel * 2 * remote
    emit(op="allgather block (peer loads)", world=world, ms=round(t_ag, 3), gbs_in=round(nbytes / t_ag / 1e6, 1),
         frac_of_nvlink=round(nbytes / t_ag / 1e6 / NVLINK_GBS, 3), ms_nccl=round(t_ag_nccl, 3), gathered_correct=bool(ag_ok.item()))

    def rs():
        comm.grad_ready(gbuf)
        comm.reduce_scatter_accumulate(gbuf, acc, True, sumsq=sq)
    t_rs = timeit(rs)
    tmp = torch.empty(lay.shard_numel, dtype=torch.bfloat16, device=device)

    def rs_nccl():
        dist.reduce_scatter_tensor(tmp, gbuf)
        acc.add_(tmp)
        sq.add_(acc.pow(2).sum())
    t_rs_nccl = timeit(rs_nccl)
    # correctness of one reduction
    acc.zero_(); rs(); torch.cuda.synchronize(); dist.barrier()
    dist.reduce_scatter_tensor(tmp, gbuf)
    rs_err = ((acc - tmp.float()).norm() / tmp.float().norm()).item()
    emit(op="reduce-scatter block + fp32 accumulate + sumsq " + ("(multimem.ld_reduce in NVSwitch, flags)" if comm.nvls else "(peer loads, flags)"), world=world, ms=round(t_rs, 3),
         gbs_in=round(nbytes / t_rs / 1e6, 1), frac_of_nvlink=round(nbytes / t_rs / 1e6 / NVLINK_GBS, 3),
         ms_nccl_reduce_scatter_plus_torch_ops=round(t_rs_nccl, 3), rel_err_vs_nccl=round(rs_err, 5))
    ops.check_status(); comm.check_status()
    dist.barrier(); dist.destroy_process_group()


if __name__ == "__main__":
    main()
