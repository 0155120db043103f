"""Reference arm of the benchmark: the UNMODIFIED reference modules installed under
``baseline/_ref`` (byte-identical copies of the reference's ``*.py`` files) driven through their
own public functions — ``init_distributed_environment``, ``setup_model`` (FSDP2 + flash-attn 2 +
Liger fused linear-CE), ``setup_training_components``, ``get_data_loader``, ``BatchMetrics`` and
``take_gradient_step`` — on the same architecture, synthetic data, batch size and token budget as
``bench.py``'s native arm.

The reference cannot do a random-init, fixed-step run by itself (``train()`` loops forever and
``setup_model`` only knows ``from_pretrained``), so this harness
  1. writes a random-init HF checkpoint directory (config, bf16 safetensors, a stub tokenizer),
  2. writes the synthetic tokenised JSONL the reference's loader reads,
  3. repeats the body of the reference's ``train()`` loop (train.py:85-122) for a fixed number of
     steps, bracketed by CUDA events.
None of this repository's kernels, models or engine run inside the timed region.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)


def _prepare_model_dir(path: str, model: str, device) -> None:
    """Random-init checkpoint + stub tokenizer (rank 0 only)."""
    import torch
    sys.path.insert(0, os.path.dirname(HERE))
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    from mini_trainer_b200.models.config import get_preset
    from mini_trainer_b200.ops.torch_ref import TorchOps
    from mini_trainer_b200.parallel.engine import ShardedEngine

    if os.path.exists(os.path.join(path, "READY")):
        return
    os.makedirs(path, exist_ok=True)
    cfg = get_preset(model)
    cfg.bos_token_id, cfg.eos_token_id, cfg.pad_token_id = 1, 2, 0
    eng = ShardedEngine(cfg, device, TorchOps(), param_dtype=torch.bfloat16, state_dtype=torch.bfloat16)
    for grp in eng.groups:   # the export only needs weights: drop optimizer-side buffers right away
        grp.m = grp.v = grp.gacc = None
    eng.init_random(seed=893, on_device=True)
    save_hf_checkpoint(eng, path)
    del eng
    torch.cuda.empty_cache()
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {"<pad>": 0, "<s>": 1, "</s>": 2, "<unk>": 3}
    vocab.update({f"w{i}": i + 4 for i in range(252)})
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", pad_token="<pad>",
                            unk_token="<unk>").save_pretrained(path)
    open(os.path.join(path, "READY"), "w").write("ok")


def _run(args, bench) -> None:
    if not os.path.exists(os.path.join(REF, "train.py")):
        return _unavailable("baseline/_ref is empty: the reference was not installed on this machine")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    sys.path.insert(0, REF)
    import torch
    import torch.distributed as dist
    from utils import init_distributed_environment            # reference
    init_distributed_environment()
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device())

    sys.path.insert(0, os.path.dirname(HERE))
    if bench is None:
        import bench
    from mini_trainer_b200.data.synthetic import CONFIG_DATA, write_synthetic_jsonl
    spec, vocab, max_tokens, batch_size = CONFIG_DATA[args.model]
    max_tokens = args.max_tokens_per_gpu or max_tokens
    batch_size = args.batch_size or batch_size
    budget = getattr(args, "time_budget_s", bench.DEFAULT_BUDGET_S)
    steps, warmup = bench.plan_steps(args.model, world, args.steps, args.warmup, budget)   # the rule the native arm uses
    work = os.environ.get("MTB200_REF_WORKDIR", "/tmp/mtb200_ref")
    model_dir = os.path.join(work, args.model)
    n_samples = bench.dataset_size(batch_size, steps + warmup)   # same dataset as the native arm
    data_path = os.path.join(work, f"{args.model}_{n_samples}.jsonl")
    if rank == 0:
        _prepare_model_dir(model_dir, args.model, device)
        if not os.path.exists(data_path):
            from mini_trainer_b200.models.config import get_preset
            write_synthetic_jsonl(data_path + ".tmp", n_samples, spec, get_preset(args.model).vocab_size, seed=893)
            os.replace(data_path + ".tmp", data_path)
    dist.barrier()

    from batch_metrics import BatchMetrics                      # reference
    from sampler import get_data_loader                         # reference
    from setup_model_for_training import setup_model, setup_training_components   # reference
    import importlib.util
    spec_ = importlib.util.spec_from_file_location("reference_train", os.path.join(REF, "train.py"))
    ref_train = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(ref_train)                         # reference train.py (the repo root has its own train.py)
    take_gradient_step = ref_train.take_gradient_step

    model = setup_model(model_name_or_path=model_dir, use_liger_kernels=True)
    model, optimizer, lr_scheduler = setup_training_components(model, learning_rate=1e-5, num_warmup_steps=10,
                                                               lr_scheduler="constant_with_warmup")
    loader = iter(get_data_loader(data_path=data_path, batch_size=batch_size, max_tokens_per_gpu=max_tokens, seed=893))
    model.train()
    batch_totals = BatchMetrics()

    h2d = d2h = 0

    def one_step(batch):
        # body of the reference's train() loop, train.py:85-122
        nonlocal h2d, d2h
        batch_totals.reset_batch()
        ntok = h2d = d2h = 0
        for grad_accum, mb in enumerate(batch):
            mb_start = time.time()
            n_loss = mb.pop("num_loss_counted_tokens")
            n_samples = mb.pop("num_samples")
            bn = mb.pop("batch_num_loss_counted_tokens")
            h2d += sum(v.numel() * v.element_size() for v in mb.values())
            mb = {k: v.to(device) for k, v in mb.items()}
            output = model(**mb)
            loss = output.loss.float().sum()
            loss_metrics = loss.detach().item()
            loss = loss * world / bn
            loss.backward()
            torch.cuda.empty_cache()
            ntok += mb["input_ids"].shape[1]
            batch_totals.accumulate_minibatch_metrics(num_loss_counted_tokens=n_loss, num_total_tokens=mb["input_ids"].shape[1],
                                                      num_samples=n_samples, loss=loss_metrics,
                                                      loss_backward=loss.detach().item() / world,
                                                      time_per_minibatch=time.time() - mb_start)
            d2h += 8   # the two fp32 .item() reads above
        batch_totals.reduce_batch_metrics(device)
        grad_norm = take_gradient_step(model, optimizer, lr_scheduler)
        d2h += 4 * len(batch_totals.totals) + 4   # the reduced metrics vector and the gradient norm
        return batch_totals.totals["num_total_tokens"], float(grad_norm)

    dist.barrier(); torch.cuda.synchronize()
    tw = time.perf_counter()
    for _ in range(warmup):
        one_step(next(loader))
    dist.barrier(); torch.cuda.synchronize()
    tw = torch.tensor([time.perf_counter() - tw], device=device)
    dist.all_reduce(tw, op=dist.ReduceOp.MAX)
    agreed = torch.tensor([bench.guard_steps(steps, tw.item(), warmup, budget)], device=device)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
    steps = int(agreed.item())
    clocks = bench.ClockSampler(bench.physical_gpu_index(torch.cuda.current_device())) if rank == 0 else None
    if clocks:
        clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    toks = 0.0
    for _ in range(steps):
        t, _ = one_step(next(loader))
        toks += t
    e1.record()
    dist.barrier(); torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    ms = torch.tensor([e0.elapsed_time(e1), wall_ms], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tps = toks / (ms[0].item() / 1e3)
    if rank == 0:
        print(json.dumps({
            "impl": "reference",
            "metric": f"train tokens/sec, {bench.MODEL_LABEL.get(args.model, args.model)}-architecture full SFT (device-timed, max over ranks)",
            "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "steps_requested": args.steps, "warmup_requested": args.warmup,
            "ms_per_step": ms[0].item() / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (same generator, dataset size, sampler and seed as the native arm; includes dummy-sample tokens)",
            "config": bench.common_config(args.model, batch_size, max_tokens, world),
            "detail": {"stack": "torch FSDP2 + flash-attn 2 + Liger fused linear-CE",
                       "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 1),
                       "wall_s_total": round(time.time() - bench.T_START, 1)},
            "clocks": clocks.stop() if clocks else None,
            "e2e": {"value": toks / (ms[1].item() / 1e3), "unit": "tokens/s", "ms_per_step": ms[1].item() / steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "host wall clock around the same steps; the reference loop copies every minibatch from host "
                           "memory and reads the loss back twice per minibatch"},
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main(args, bench=None) -> None:
    """``bench`` is the already imported ``bench.py`` module (its start time and step plan are shared)."""
    try:
        _run(args, bench)
    except BaseException as e:  # the contract is one JSON line and exit code 0
        if isinstance(e, KeyboardInterrupt):
            raise
        import traceback
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"{type(e).__name__}: {e}")
