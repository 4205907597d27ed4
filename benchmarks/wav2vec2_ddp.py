"""wav2vec 2.0 "large" self-supervised pre-training step under replicated data parallelism (``bench.py --config
wav2vec2_large_ddp``): 7-layer convolutional feature extractor with layer norms, 24-layer encoder (1024 / 16 heads /
FFN 4096, convolutional position encoding k=128 g=16), Gumbel quantizer 2 x 320 with 768-dimensional code words,
span masking (p = 0.65, span 10), contrastive loss over 100 distractors plus diversity loss; raw 16 kHz waveforms
drawn from N(0, 0.1^2) with lengths uniform in [32000, 250000], length-bucketed to at most 1.4 M samples per GPU
batch, with padding masks; bf16 compute, fp32 master weights and AdamW state; random init; synthetic data."""
from __future__ import annotations

import argparse
from typing import Any

import numpy as np

MAX_SAMPLES = 1_400_000


def make_waveform_batch(rng: np.random.Generator, max_samples: int = MAX_SAMPLES, lo: int = 32_000,
                        hi: int = 250_000) -> tuple[Any, list[int]]:
    """One length bucket: the longest utterance sets the width, the others are at most 15 % shorter, and as many
    utterances as fit into ``max_samples`` padded samples. Returns the pinned ``[N, L]`` fp32 batch and lengths."""
    import torch

    longest = int(rng.integers(lo, hi + 1))
    n = max(1, max_samples // longest)
    lens = [longest] + sorted((int(x) for x in rng.integers(max(lo, int(0.85 * longest)), longest + 1, size=n - 1)),
                              reverse=True)
    wave = rng.normal(0.0, 0.1, size=(n, longest)).astype(np.float32)
    for i, m in enumerate(lens):
        wave[i, m:] = 0.0
    t = torch.from_numpy(wave)
    if torch.cuda.is_available():
        t = t.pin_memory()
    return t, lens


def wav2vec2_large_config(layers: int | None = None):  # type: ignore[no-untyped-def]
    from fairseq2_b200.models.wav2vec2.config import large

    c = large()
    e = c.encoder_config
    e.feature_extractor_layer_norm_convs = True
    e.feature_extractor_bias = True
    e.max_seq_len = 4096
    c.max_temporal_mask_prob = 0.65
    c.temporal_mask_span_len = 10
    if layers is not None:
        e.num_encoder_layers = layers
    return c


def run_ours(args: argparse.Namespace) -> None:
    import torch

    from benchmarks.harness import env_ranks, result_line, timed_run
    from fairseq2_b200.gang import FakeGang, ProcessGroupGang, ReduceOperation, create_parallel_gangs
    from fairseq2_b200.models.wav2vec2 import create_wav2vec2_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    rank, world, local_rank = env_ranks()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}; launch with torch.distributed.run.")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    ext = require_ext()
    root = FakeGang(device) if world == 1 else ProcessGroupGang.create_default_process_group(device)
    gangs = create_parallel_gangs(root, tp_size=1)            # rdp = dp: replicated data parallelism

    cfg = wav2vec2_large_config(args.layers)
    torch.manual_seed(2)
    with torch.device("meta"):
        model = create_wav2vec2_model(cfg)
    # flat parameter units, replicated: bf16 compute copies, fp32 master weights, gradients averaged over the
    # replicas by the in-place all-reduce kernel as each unit's backward pass finishes
    ddp = FSDP(model, gangs, param_dtype=torch.bfloat16, wait_limit_s=30.0)
    facade = DataParallelFacade(ddp)
    optimizer = AdamW(ddp.parameters(), lr=5e-4, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.01)

    class SslUnit(TrainUnit):
        @property
        def model(self) -> DataParallelFacade:
            return facade

        def process_batch(self, batch, metric_bag=None):  # type: ignore[no-untyped-def]
            wave, layout = batch
            loss, out = ddp(wave, layout)
            return loss.aggregate, out.num_targets

    step_fn = TrainStep(SslUnit(), optimizer, gangs, max_grad_norm=None)

    rng = np.random.default_rng(1234 + rank)
    examples = [make_waveform_batch(rng) for _ in range(args.warmup + 2 * args.steps)]
    samples_per_step = float(np.mean([sum(l) for _, l in examples[args.warmup:]]))

    def stage(ex):  # type: ignore[no-untyped-def]
        wave, lens = ex
        w = wave.to(device, non_blocking=True).to(torch.bfloat16)
        return w, BatchLayout(tuple(w.shape), lens, device=device)

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
                    examples=examples, h2d_bytes=lambda ex: ex[0].numel() * 4 + (len(ex[1]) + 1) * 4,
                    launch_counter=ext.launch_count, reset_launch_counter=ext.reset_launch_count, trace=args)
    ext.check_status()
    tot = torch.tensor([samples_per_step], device=device, dtype=torch.float64)
    if world > 1:
        root.all_reduce(tot, ReduceOperation.SUM)
    if rank == 0:
        e = cfg.encoder_config
        print(result_line(
            metric="wav2vec2_large_ssl_audio_samples_per_second", unit="audio samples/s", impl="fairseq2_b200",
            units_per_step=float(tot[0]), world=world, steps=args.steps, warmup=args.warmup, run=run,
            config={"model": "wav2vec2_large" if args.layers is None else f"wav2vec2_large[layers={args.layers}]",
                    "global_batch": f"<= {MAX_SAMPLES} padded samples per GPU x {world}", "seq_len": "32000-250000",
                    "parallelism": f"ddp{world}", "encoder_layers": e.num_encoder_layers,
                    "optimizer": "AdamW lr 5e-4 fp32 state, fp32 master weights", "layer_drop_p": e.layer_drop_p,
                    "l2": "per-step working set (activations of 1.4 M samples) >> 126 MB L2; inputs differ every step"}),
              flush=True)
    if world > 1:
        root.close()
