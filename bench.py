"""Headline benchmark: LLaMA-3-8B SFT training throughput (tokens/s over all GPUs).

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # unmodified fairseq2 from baseline/_ref
    python bench.py --config {llama3_70b_tp4_fsdp2,moe_ep8,wav2vec2_large_ddp} ...   # the other configurations

Without ``--config`` the headline configuration below runs; the others are described in their modules under
``benchmarks/`` (ours) and ``baseline/`` (reference arms).

Model/config: LLaMA-3-8B architecture (32 layers, dim 4096, 32/8 heads, FFN
14336, vocab 128256), random init, packed sequences of 8192 tokens per GPU made
of documents of 128-4096 tokens with per-document block-causal attention and a
masked prompt prefix; bf16 compute with fp32 master weights and fp32 AdamW
state, FSDP over N ranks, activation checkpointing off. Synthetic data.

Two numbers are measured, each over exactly K steps after W warm-up steps:
``value`` is timed on the device with CUDA events around steps whose inputs are
already resident; ``e2e`` runs the same public training step but every step
copies its inputs from pinned host memory and reads the loss back to the host.
Each rank's inputs differ per step and exceed no cache assumptions: the working
set of a step (weights + activations) is far larger than the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


from benchmarks.harness import clock_sampler as _clock_sampler  # noqa: E402
from benchmarks.harness import summarize_clocks as _summarize_clocks  # noqa: E402


def _trace_steps(args: argparse.Namespace, step_fn, batches, rank: int, record: bool) -> None:  # type: ignore[no-untyped-def]
    from benchmarks.harness import trace_steps

    trace_steps(args.trace, lambda i: step_fn([batches[i]], 10_000 + i), len(batches), rank, record)


def run_ours(args: argparse.Namespace) -> None:
    import numpy as np
    import torch

    from fairseq2_b200.datasets.synthetic import make_packed_sft_example
    from fairseq2_b200.gang import (FakeGang, ProcessGroupGang, ReduceOperation, create_fsdp_gangs,
                                    create_parallel_gangs)
    from fairseq2_b200.models.llama import create_llama_model, get_llama_config
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}; launch with torch.distributed.run.")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    ext = require_ext()

    root = FakeGang(device) if world == 1 else ProcessGroupGang.create_default_process_group(device)
    gangs = create_fsdp_gangs(create_parallel_gangs(root, tp_size=1))

    cfg = get_llama_config(args.model)
    if args.layers is not None:          # debugging aid only; the JSON line marks such a run
        cfg.num_layers = args.layers
    seq_len = args.seq_len
    torch.manual_seed(2)
    with torch.device("meta"):
        model = create_llama_model(cfg, gangs)
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16, fp32_reduce=True,
                reshard_after_forward=bool(args.reshard_after_forward), wait_limit_s=30.0)
    facade = DataParallelFacade(fsdp)
    optimizer = AdamW(fsdp.parameters(), lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1)

    class SFTUnit(TrainUnit):
        """Loss-masked next-token cross entropy over a packed batch (``lm.sft`` semantics)."""

        @property
        def model(self) -> DataParallelFacade:
            return facade

        def process_batch(self, batch, metric_bag=None):  # type: ignore[no-untyped-def]
            tokens, mask, layout, num_targets = batch
            loss = fsdp(tokens[:-1], layout, targets=tokens[1:], target_mask=mask, reduction="sum")
            return loss, num_targets

    step_fn = TrainStep(SFTUnit(), optimizer, gangs, max_grad_norm=1.0)

    rng = np.random.default_rng(1234 + rank)
    total = args.warmup + 2 * args.steps
    examples = [make_packed_sft_example(rng, seq_len, cfg.vocab_size) for _ in range(total)]

    def stage(ex):  # type: ignore[no-untyped-def]
        tokens = ex.tokens.to(device, non_blocking=True)
        mask = ex.target_mask.to(device, non_blocking=True)
        layout = BatchLayout((seq_len,), ex.seq_lens, packed=True, device=device)
        return tokens, mask, layout, ex.num_targets

    def barrier() -> None:
        if world > 1:
            root.barrier()
        torch.cuda.synchronize(device)

    # ---- warm-up
    for i in range(args.warmup):
        loss, _ = step_fn([stage(examples[i])], i)
    barrier()

    # ---- device-timed region: inputs resident before the clock starts
    staged = [stage(examples[args.warmup + i]) for i in range(args.steps)]
    samples: list[dict] = []
    stop = threading.Event()
    sampler = threading.Thread(target=_clock_sampler, args=(stop, samples, local_rank), daemon=True)
    if rank == 0:
        sampler.start()
    barrier()
    ext.reset_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        loss, gnorm = step_fn([staged[i]], args.warmup + i)
    ev1.record()
    barrier()
    launches = int(ext.launch_count())
    dev_ms = ev0.elapsed_time(ev1)
    del staged

    # ---- end-to-end region: H2D of every step's inputs + D2H of its loss
    barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    h2d = d2h = 0
    last_loss = 0.0
    for i in range(args.steps):
        ex = examples[args.warmup + args.steps + i]
        batch = stage(ex)
        h2d = ex.tokens.numel() * 8 + ex.target_mask.numel() * 4 + (2 * len(ex.seq_lens) + 1 + seq_len) * 4
        loss, gnorm = step_fn([batch], args.warmup + args.steps + i)
        last_loss = float(loss.item())
        d2h = 4
    e1.record()
    barrier()
    e2e_ms = max((time.perf_counter() - t0) * 1e3, e0.elapsed_time(e1))
    stop.set()
    ext.check_status()

    # kernel timeline of two more steps, outside every timed region: the source of the exposed-communication figure
    overlap = None
    if not args.no_trace:
        import tempfile

        own_prefix = args.trace is None
        if own_prefix:
            args.trace = os.path.join(tempfile.mkdtemp(prefix="fs2_trace_"), "t")
        _trace_steps(args, step_fn, [stage(examples[args.warmup + i]) for i in range(2)], rank,
                     record=rank == 0 or args.trace_all_ranks)
        barrier()
        try:
            with open(f"{args.trace}.rank0.overlap.json") as fp:
                overlap = json.load(fp) if rank == 0 else None
        except OSError:
            overlap = None
        if own_prefix and rank == 0:
            import shutil

            shutil.rmtree(os.path.dirname(args.trace), ignore_errors=True)

    times = torch.tensor([dev_ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        root.all_reduce(times, ReduceOperation.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    tokens_per_step = seq_len * world
    value = tokens_per_step * args.steps / (dev_ms * 1e-3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms * 1e-3)

    if rank == 0:
        # model FLOPs of a step: 6 x (parameters that are GEMM operands: everything but the embedding table)
        # per token, plus causal attention (forward 2 GEMMs over half the score matrix, backward twice that)
        gemm_params = sum(s.d0 * s.row for u in fsdp.all_units for s in u.specs
                          if len(s.shape) == 2 and "embed" not in s.fqn)
        attn_flops = sum(6.0 * n * n * cfg.num_attn_heads * (cfg.model_dim // cfg.num_attn_heads)
                         for ex in examples[args.warmup: args.warmup + args.steps] for n in ex.seq_lens)
        attn_flops = attn_flops * cfg.num_layers / max(args.steps, 1)
        flops_per_step = 6.0 * gemm_params * seq_len + attn_flops
        out = {
            "metric": "llama3_8b_fsdp_sft_tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "fairseq2_b200",
            "config": {"model": args.model if args.layers is None else f"{args.model}[layers={args.layers}]",
                       "global_batch": world, "seq_len": seq_len, "parallelism": f"fsdp{world}",
                       "packing": "documents 128-4096 tokens, block-causal, prompt-masked loss",
                       "optimizer": "AdamW lr 1e-5 fp32 state, fp32 master weights, grad clip 1.0",
                       "activation_checkpointing": False, "reshard_after_forward": bool(args.reshard_after_forward),
                       "l2": "per-step working set (weights+activations) >> 126 MB L2; inputs differ every step"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "clocks": _summarize_clocks(samples),
            "final_loss": last_loss,
            "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 2**30,
        }
        out["model_tflops_per_gpu"] = flops_per_step / (dev_ms / args.steps * 1e-3) / 1e12
        if overlap:
            # exposed communication of the step: idle time of the compute stream (kernel timeline of two extra steps
            # recorded after the timed regions); GEMM time is listed so that runs at different N can be compared
            out["exposed_comm_ms"] = round(overlap["compute_stream_idle_ms_per_step"], 3)
            out["gemm_ms_per_step"] = round(overlap["gemm_ms_per_step"], 3)
            out["comm_stream_kernel_ms_per_step"] = round(overlap["other_streams_kernel_ms_per_step"], 3)
        print(json.dumps(out), flush=True)
    if world > 1:
        root.close()


def run_reference(args: argparse.Namespace) -> None:
    from baseline.reference_arm import run_reference_arm

    run_reference_arm(args)


CONFIGS = ("llama3_8b_fsdp", "llama3_70b_tp4_fsdp2", "moe_ep8", "wav2vec2_large_ddp")


def run_config(args: argparse.Namespace) -> None:
    """The configurations other than the headline one live in ``benchmarks/``."""
    if args.config == "wav2vec2_large_ddp":
        from benchmarks.wav2vec2_ddp import run_ours as fn
    elif args.config == "llama3_70b_tp4_fsdp2":
        from benchmarks.llama70b_tp_fsdp import run_ours as fn
    elif args.config == "moe_ep8":
        from benchmarks.moe_ep import run_ours as fn
    else:
        raise SystemExit(f"unknown --config {args.config}")
    fn(args)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llama3_8b_fsdp", choices=list(CONFIGS),
                    help="benchmark configuration; the default is the headline LLaMA-3-8B FSDP SFT step")
    ap.add_argument("--tp", type=int, default=None, help="tensor-parallel size (llama3_70b_tp4_fsdp2: default 4)")
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--reshard-after-forward", type=int, default=1, choices=[0, 1],
                    help="0 keeps the gathered bf16 weights between forward and backward (one all-gather per step)")
    ap.add_argument("--trace", default=None, metavar="PREFIX",
                    help="after the timed regions, write a kernel timeline of two steps to PREFIX.rankN.json")
    ap.add_argument("--trace-all-ranks", action="store_true")
    ap.add_argument("--no-trace", action="store_true",
                    help="skip the two traced steps after the timed regions (no `exposed_comm_ms` in the result)")
    ap.add_argument("--layers", type=int, default=None, help="debugging only: truncates the model (result is not a valid benchmark)")
    args = ap.parse_args()
    if args.warmup < 3 and args.layers is None:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
        return
    from benchmarks.harness import abort_peers, watch_for_abort

    watch_for_abort()
    try:
        if args.config != "llama3_8b_fsdp":
            run_config(args)
        else:
            run_ours(args)
    except BaseException as ex:
        abort_peers(f"{type(ex).__name__}: {ex}")
        raise


if __name__ == "__main__":
    main()
