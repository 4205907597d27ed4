"""Reference arm for ``bench.py --config wav2vec2_large_ddp --impl reference``: the unmodified fairseq2 package in
``baseline/_ref`` builds wav2vec 2.0 "large" with its own ``Wav2Vec2Factory``, wraps it with its own ``to_ddp``
(torch DDP over NCCL), and runs the step of its ``Trainer`` for this recipe: autocast(bf16) forward, backward,
``normalize_grads``, torch fused AdamW. Nothing of the framework under test is imported."""
from __future__ import annotations

import json
import os
from argparse import Namespace

MAX_SAMPLES = 1_400_000


def _make_batch(rng, max_samples=MAX_SAMPLES, lo=32_000, hi=250_000):  # type: ignore[no-untyped-def]
    import numpy as np
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


def run(args: Namespace) -> None:
    import time

    import numpy as np
    import torch

    import fairseq2
    from fairseq2.data_type import set_dtype
    from fairseq2.gang import ProcessGroupGang, ReduceOperation, create_fake_gangs, create_parallel_gangs, set_gangs
    from fairseq2.models.wav2vec2.config import Wav2Vec2Config, Wav2Vec2EncoderConfig
    from fairseq2.models.wav2vec2.factory import Wav2Vec2Factory
    from fairseq2.nn import BatchLayout
    from fairseq2.nn.ddp import to_ddp
    from fairseq2.nn.utils.grad import normalize_grads

    fairseq2.init_fairseq2()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local_rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        root = ProcessGroupGang.create_default_process_group(device)
        gangs = create_parallel_gangs(root)
    else:
        gangs = create_fake_gangs(device)

    enc = Wav2Vec2EncoderConfig(model_dim=1024, num_encoder_layers=24 if args.layers is None else args.layers,
                                num_encoder_attn_heads=16, ffn_inner_dim=4096, dropout_p=0.0, layer_drop_p=0.2,
                                feature_extractor_layer_norm_convs=True, feature_extractor_bias=True)
    cfg = Wav2Vec2Config(encoder_config=enc, quantized_dim=768, final_dim=768, max_temporal_mask_prob=0.65,
                         temporal_mask_span_len=10)
    torch.manual_seed(2)
    with device, set_gangs(gangs), set_dtype(torch.float32):
        model = Wav2Vec2Factory(cfg).create_model()
    model.train()
    dp_model = to_ddp(model, gangs, find_unused_parameters=False, static_graph=False) if world > 1 else model
    optimizer = torch.optim.AdamW(dp_model.parameters(), lr=5e-4, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.01,
                                  fused=cuda)

    def stage(ex):  # type: ignore[no-untyped-def]
        wave, lens = ex
        w = wave.to(device, non_blocking=True)
        return w, BatchLayout(tuple(w.shape), lens, device=device)

    def step(batch, i):  # type: ignore[no-untyped-def]
        wave, layout = batch
        with torch.autocast(device_type=device.type, dtype=torch.bfloat16, enabled=cuda):
            loss, out = dp_model(wave, layout)
        n = out.logits.shape[0] * out.logits.shape[1]
        loss.aggregate.backward()
        normalize_grads(dp_model, gangs.dp, n)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss.aggregate.detach()

    def barrier() -> None:
        if world > 1:
            gangs.root.barrier()
        if cuda:
            torch.cuda.synchronize(device)

    rng = np.random.default_rng(1234 + rank)
    examples = [_make_batch(rng) for _ in range(args.warmup + 2 * args.steps)]
    samples_per_step = float(np.mean([sum(l) for _, l in examples[args.warmup:]]))
    for i in range(args.warmup):
        step(stage(examples[i]), i)
    barrier()
    staged = [stage(examples[args.warmup + i]) for i in range(args.steps)]
    barrier()
    if cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(staged[i], i)
    if cuda:
        ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1) if cuda else (time.perf_counter() - t0) * 1e3
    del staged
    barrier()
    t0 = time.perf_counter()
    h2d, last = 0, 0.0
    losses: list[float] = []
    for i in range(args.steps):
        ex = examples[args.warmup + args.steps + i]
        h2d = ex[0].numel() * 4 + (len(ex[1]) + 1) * 4
        last = float(step(stage(ex), i).item())
        losses.append(last)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([dev_ms, e2e_ms, 0.0], device=device, dtype=torch.float64)
    s = torch.tensor([samples_per_step], device=device, dtype=torch.float64)
    if world > 1:
        gangs.root.all_reduce(t, ReduceOperation.MAX)
        gangs.root.all_reduce(s, ReduceOperation.SUM)
    dev_ms, e2e_ms, units = float(t[0]), float(t[1]), float(s[0])
    if rank == 0:
        out = {"metric": "wav2vec2_large_ssl_audio_samples_per_second", "impl": "reference",
               "value": units * args.steps / (dev_ms * 1e-3), "unit": "audio samples/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "config": {"model": "wav2vec2_large" if args.layers is None else f"wav2vec2_large[layers={args.layers}]",
                          "global_batch": f"<= {MAX_SAMPLES} padded samples per GPU x {world}",
                          "seq_len": "32000-250000",
                          "parallelism": f"ddp{world} (torch DDP, fp32 parameters under autocast bf16)"},
               "e2e": {"value": units * args.steps / (e2e_ms * 1e-3), "unit": "audio samples/s",
                       "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
               "final_loss": last, "losses": losses}
        if cuda:
            out["peak_mem_gb"] = torch.cuda.max_memory_allocated(device) / 2**30
        print(json.dumps(out), flush=True)
    if world > 1:
        gangs.root.close()
