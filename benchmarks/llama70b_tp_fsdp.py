"""LLaMA-3-70B SFT step under hybrid tensor parallelism x FSDP (``bench.py --config llama3_70b_tp4_fsdp2``): 80
layers, model dim 8192, 64 query / 8 key-value heads, head dim 128, SwiGLU FFN 28672, vocabulary 128256 with a
vocabulary-sharded embedding and output projection; q/k/v/gate/up column-sharded and o/down row-sharded over TP=4
with sequence-parallel activations (all-gather and reduce-scatter fused into the tcgen05 GEMMs), FSDP over the 2
data-parallel ranks; activation checkpointing per layer; packed sequences of 4096 tokens per data-parallel rank made
of documents of 128-2048 tokens with per-document block-causal attention; bf16 compute, fp32 master weights and
AdamW state; the optimizer step of each FSDP unit runs inside its gradient reduce-scatter kernel (no gradient
clipping in this configuration). Random init, synthetic data."""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np


def run_ours(args: argparse.Namespace) -> None:
    import torch

    from benchmarks.harness import env_ranks, result_line, timed_run
    from fairseq2_b200.datasets.synthetic import make_packed_sft_example
    from fairseq2_b200.gang import (FakeGang, ProcessGroupGang, ReduceOperation, create_fsdp_gangs,
                                    create_parallel_gangs)
    from fairseq2_b200.models.llama import create_llama_model, get_llama_config
    from fairseq2_b200.models.utils_ac import apply_layerwise_ac
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.parallel.tp import sequence_parallel
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    rank, world, local_rank = env_ranks()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}; launch with torch.distributed.run.")
    tp = args.tp if args.tp is not None else min(4, world)
    if world % tp:
        raise SystemExit(f"--tp {tp} does not divide the number of GPUs ({world}).")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    ext = require_ext()
    # NCCL only carries control traffic here (barriers, a few scalars; the data moves through the peer-memory
    # kernels), so its communicators go without NVLS buffers, and they are brought up now, while the device is
    # empty: the model state below fills most of the device, and a communicator that initialises lazily at the
    # first barrier after that finds no room (that is how the first 8-GPU attempt of this configuration ended).
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    # Nothing in this configuration uses `multimem` (no replicated gradient buffers), so the arenas (49 GiB for the
    # flat units) need no NVSwitch multicast binding either; torch's symmetric-memory rendezvous skips it when told.
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    root = FakeGang(device) if world == 1 else ProcessGroupGang.create_default_process_group(device)
    gangs = create_fsdp_gangs(create_parallel_gangs(root, tp_size=tp))
    dp = gangs.dp
    if world > 1:
        warmed: set[int] = set()
        for g in (root, gangs.dp, gangs.tp, gangs.sdp, gangs.rdp):
            if g.size > 1 and id(g) not in warmed:
                warmed.add(id(g))
                g.barrier()

    cfg = get_llama_config("llama3_70b")
    seq_len = args.seq_len if args.seq_len != 8192 else 4096
    cfg.max_seq_len = max(seq_len, 4096)
    if args.layers is not None:
        cfg.num_layers = args.layers
    torch.manual_seed(2)                                     # the same full initialisation on every rank
    with torch.device("meta"), sequence_parallel(tp > 1):
        model = create_llama_model(cfg, gangs)
    apply_layerwise_ac(model, 1)
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16, fp32_reduce=True, reshard_after_forward=True,
                wait_limit_s=60.0)
    if tp > 1:
        from fairseq2_b200.parallel.tp import get_tp_context

        get_tp_context(gangs.tp).prepare()                   # the tensor-parallel arena, before the optimizer state
    facade = DataParallelFacade(fsdp)
    optimizer = AdamW(fsdp.parameters(), lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1)

    class SFTUnit(TrainUnit):
        @property
        def model(self) -> DataParallelFacade:
            return facade

        def count_targets(self, batch):  # type: ignore[no-untyped-def]
            return batch[3]

        def process_batch(self, batch, metric_bag=None):  # type: ignore[no-untyped-def]
            tokens, mask, layout, num_targets = batch
            loss = fsdp(tokens[:-1], layout, targets=tokens[1:], target_mask=mask, reduction="sum")
            return loss, num_targets

    step_fn = TrainStep(SFTUnit(), optimizer, gangs, max_grad_norm=None)
    torch.cuda.empty_cache()
    if rank == 0:
        free, total = torch.cuda.mem_get_info(device)
        print(f"model state in place: {torch.cuda.memory_allocated(device) / 2**30:.1f} GiB in tensors, "
              f"{(total - free) / 2**30:.1f} of {total / 2**30:.1f} GiB of the device in use", file=sys.stderr, flush=True)

    rng = np.random.default_rng(1234 + dp.rank)              # tensor-parallel peers read the same sequence
    examples = [make_packed_sft_example(rng, seq_len, cfg.vocab_size, doc_len_range=(128, 2048))
                for _ in range(args.warmup + 2 * args.steps)]

    def stage(ex):  # type: ignore[no-untyped-def]
        tokens = ex.tokens.to(device, non_blocking=True)
        mask = ex.target_mask.to(device, non_blocking=True)
        return tokens, mask, BatchLayout((seq_len,), ex.seq_lens, packed=True, device=device), ex.num_targets

    def step(batch, i):  # type: ignore[no-untyped-def]
        loss, _ = step_fn([batch], i)
        return loss

    def barrier() -> None:
        if world > 1:
            root.barrier()
        torch.cuda.synchronize(device)

    run = timed_run(steps=args.steps, warmup=args.warmup, rank=rank, world=world, local_rank=local_rank,
                    device=device, barrier=barrier,
                    all_reduce_max=lambda t: root.all_reduce(t, ReduceOperation.MAX), stage=stage, step=step,
                    examples=examples,
                    h2d_bytes=lambda ex: ex.tokens.numel() * 8 + ex.target_mask.numel() * 4
                    + (2 * len(ex.seq_lens) + 1 + seq_len) * 4,
                    launch_counter=ext.launch_count, reset_launch_counter=ext.reset_launch_count, trace=args)
    ext.check_status()
    if rank == 0:
        fused_tp = bool(tp > 1 and __import__("fairseq2_b200.parallel.tp", fromlist=["x"]).get_tp_context(gangs.tp).arena)
        print(result_line(
            metric="llama3_70b_tp_fsdp_sft_tokens_per_second", unit="tokens/s", impl="fairseq2_b200",
            units_per_step=float(seq_len * dp.size), world=world, steps=args.steps, warmup=args.warmup, run=run,
            config={"model": "llama3_70b" if args.layers is None else f"llama3_70b[layers={args.layers}]",
                    "global_batch": dp.size, "seq_len": seq_len, "parallelism": f"tp{tp} x fsdp{dp.size}",
                    "sequence_parallel": tp > 1, "tp_collectives": "fused into tcgen05 GEMMs" if fused_tp else "gang",
                    "packing": "documents 128-2048 tokens, block-causal, prompt-masked loss",
                    "optimizer": "AdamW lr 1e-5 fp32 state, fp32 master weights, no clipping; step fused into "
                                 "the gradient reduce-scatter" if fsdp.supports_fused_optimizer else
                                 "AdamW lr 1e-5 fp32 state, fp32 master weights, no clipping",
                    "activation_checkpointing": "per layer",
                    "l2": "per-step working set (weights + activations) >> 126 MB L2; inputs differ every step"}),
              flush=True)
    if world > 1:
        root.close()
