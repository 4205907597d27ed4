"""Mixture-of-experts decoder training step with expert parallelism (``bench.py --config moe_ep8``): 48 layers, model
dim 2048, 32 query / 4 key-value heads of dim 128, vocabulary 151936; every layer is a mixture of 128 SwiGLU experts
of inner dim 768 with top-8 softmax routing and a load-balancing auxiliary loss (coefficient 1e-3); router weights
initialised N(0, 0.02). Experts are expert-parallel over all ranks (each rank owns 128 / W experts; tokens travel to
the owning rank inside the dispatch kernel and come back inside the combine kernel; the experts of a rank run as
three single-launch grouped tcgen05 GEMMs over a tile-aligned inbox whose layout never leaves the device), the dense
parts (attention, embeddings, norms, routers) are fully sharded (FSDP). Two sequences of 4096 uniform random tokens
per GPU; bf16 compute, fp32 master weights and AdamW state; random init; synthetic data."""
from __future__ import annotations

import argparse

import numpy as np


def run_ours(args: argparse.Namespace) -> None:
    import torch

    from benchmarks.harness import env_ranks, result_line, timed_run
    from fairseq2_b200.gang import (FakeGang, ProcessGroupGang, ReduceOperation, create_fsdp_gangs,
                                    create_parallel_gangs)
    from fairseq2_b200.models.moe_lm import create_moe_lm_model
    from fairseq2_b200.models.moe_lm.config import qwen3_moe_30b_a3b
    from fairseq2_b200.models.transformer.experts import GroupedExpertNetwork
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.ops.moe_ep import ExpertParallelExchange
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.parallel.symm import SymmetricArena
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    rank, world, local_rank = env_ranks()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}; launch with torch.distributed.run.")
    if world < 2:
        raise SystemExit("moe_ep8 needs at least 2 GPUs (expert parallelism over peer memory).")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    ext = require_ext()
    root = ProcessGroupGang.create_default_process_group(device)
    gangs = create_fsdp_gangs(create_parallel_gangs(root, tp_size=1))

    cfg = qwen3_moe_30b_a3b()
    if args.layers is not None:
        cfg.num_layers = args.layers
    seq_len, seqs_per_gpu = 4096, 2
    tokens_per_gpu = seq_len * seqs_per_gpu
    rows = tokens_per_gpu * cfg.top_k
    cap = int(cfg.ep_capacity_factor * rows)
    arena = SymmetricArena(root, 2 * (cap + 128 * (cfg.num_experts // world + 2)) * cfg.model_dim * 2 + (8 << 20),
                           wait_limit_s=60.0)
    ep = ExpertParallelExchange(arena, cfg.num_experts, cfg.model_dim, max_tokens=tokens_per_gpu, top_k=cfg.top_k,
                                capacity=cap)
    torch.manual_seed(2 + rank)          # every rank owns different experts; the sharded parts keep their own slices
    with torch.device("meta"):
        model = create_moe_lm_model(cfg, gangs, ep=ep)
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16, fp32_reduce=True, wait_limit_s=60.0,
                local_module_filter=lambda m: isinstance(m, GroupedExpertNetwork))
    facade = DataParallelFacade(fsdp)
    optimizer = AdamW(fsdp.parameters(), lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1)

    class LMUnit(TrainUnit):
        @property
        def model(self) -> DataParallelFacade:
            return facade

        def count_targets(self, batch):  # type: ignore[no-untyped-def]
            return batch.shape[0] * (batch.shape[1] - 1)

        def process_batch(self, batch, metric_bag=None):  # type: ignore[no-untyped-def]
            inp, tgt = batch[:, :-1], batch[:, 1:]
            layout = BatchLayout(tuple(inp.shape), [inp.shape[1]] * inp.shape[0], device=device)
            loss = fsdp(inp, layout, targets=tgt, reduction="sum")
            return loss, tgt.numel()

    step_fn = TrainStep(LMUnit(), optimizer, gangs, max_grad_norm=None)

    rng = np.random.default_rng(1234 + rank)

    def make():  # type: ignore[no-untyped-def]
        t = torch.from_numpy(rng.integers(0, cfg.vocab_size, size=(seqs_per_gpu, seq_len + 1), dtype=np.int64))
        return t.pin_memory()

    examples = [make() for _ in range(args.warmup + 2 * args.steps)]

    def step(batch, i):  # type: ignore[no-untyped-def]
        loss, _ = step_fn([batch], i)
        return loss

    def barrier() -> None:
        root.barrier()
        torch.cuda.synchronize(device)

    run = timed_run(steps=args.steps, warmup=args.warmup, rank=rank, world=world, local_rank=local_rank,
                    device=device, barrier=barrier,
                    all_reduce_max=lambda t: root.all_reduce(t, ReduceOperation.MAX),
                    stage=lambda ex: ex.to(device, non_blocking=True), step=step, examples=examples,
                    h2d_bytes=lambda ex: ex.numel() * 8,
                    launch_counter=ext.launch_count, reset_launch_counter=ext.reset_launch_count, trace=args)
    ext.check_status()
    dropped = ep.dropped.clone()
    root.all_reduce(dropped, ReduceOperation.SUM)
    if rank == 0:
        print(result_line(
            metric="moe_128e_top8_ep_tokens_per_second", unit="tokens/s", impl="fairseq2_b200",
            units_per_step=float(tokens_per_gpu * world), world=world, steps=args.steps, warmup=args.warmup, run=run,
            config={"model": "moe_48l_2048d_128e_top8" if args.layers is None else f"moe[layers={args.layers}]",
                    "global_batch": seqs_per_gpu * world, "seq_len": seq_len,
                    "parallelism": f"ep{world} (experts) + fsdp{world} (dense parts)",
                    "routing": "softmax top-8, aux loss 1e-3, router init N(0, 0.02)",
                    "ep_capacity_factor": cfg.ep_capacity_factor, "dropped_rows_total": int(dropped),
                    "optimizer": "AdamW lr 1e-5 fp32 state, fp32 master weights, no clipping",
                    "activation_checkpointing": False,
                    "l2": "per-step working set >> 126 MB L2; inputs differ every step"}), flush=True)
    root.close()
