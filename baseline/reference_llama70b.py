"""Reference arm for ``bench.py --config llama3_70b_tp4_fsdp2 --impl reference``: the unmodified fairseq2 package in
``baseline/_ref`` builds LLaMA-3-70B with its own ``LLaMAFactory`` under ``create_parallel_gangs(tp_size=4)`` (so
the factory shards q/k/v/gate/up by columns, o/down by rows, the embedding and output projection by vocabulary),
applies its layer-wise activation checkpointing, wraps the result with its ``to_fsdp2`` over the data-parallel gang
(recipe defaults) and runs the step of its ``Trainer``: forward with fused loss, backward, ``normalize_grads``,
torch fused AdamW. Nothing of the framework under test is imported."""
from __future__ import annotations

import json
import os
import time
from argparse import Namespace


def _make_example(rng, seq_len: int, vocab: int):  # type: ignore[no-untyped-def]
    import numpy as np
    import torch

    lens: list[int] = []
    total = 0
    while total < seq_len:
        n = min(int(rng.integers(128, 2049)), seq_len - total)
        lens.append(n)
        total += n
    tokens = rng.integers(0, vocab, size=seq_len + 1, dtype=np.int64)
    mask = np.ones(seq_len, dtype=bool)
    off = 0
    for n in lens:
        p = int(n * rng.uniform(0.1, 0.5))
        mask[off: off + max(p - 1, 0)] = False
        mask[off + n - 1] = False
        off += n
    t, m = torch.from_numpy(tokens), torch.from_numpy(mask)
    if torch.cuda.is_available():
        t, m = t.pin_memory(), m.pin_memory()
    return t, m, lens, int(mask.sum())


def run(args: Namespace) -> None:
    import numpy as np
    import torch

    import fairseq2
    from fairseq2.data_type import set_dtype
    from fairseq2.gang import (ProcessGroupGang, ReduceOperation, create_fake_gangs, create_fsdp_gangs,
                               create_parallel_gangs, set_gangs)
    from fairseq2.models.llama.config import LLaMAConfig
    from fairseq2.models.llama.factory import LLaMAFactory
    from fairseq2.models.transformer.sdpa.default import set_default_sdpa_factory
    from fairseq2.models.transformer.sdpa.flash2 import Flash2SDPA
    from fairseq2.models.transformer_lm.ac import apply_ac_to_transformer_lm
    from fairseq2.models.transformer_lm.fsdp import apply_fsdp_to_transformer_lm
    from fairseq2.nn import BatchLayout
    from fairseq2.nn.fsdp import to_fsdp2
    from fairseq2.nn.utils.grad import normalize_grads

    fairseq2.init_fairseq2()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    set_default_sdpa_factory(Flash2SDPA)
    tp = args.tp if getattr(args, "tp", None) is not None else min(4, world)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        root = ProcessGroupGang.create_default_process_group(device)
        gangs = create_fsdp_gangs(create_parallel_gangs(root, tp_size=tp))
    else:
        gangs = create_fake_gangs(device)
    dp = gangs.dp
    seq_len = args.seq_len if args.seq_len != 8192 else 4096
    cfg = LLaMAConfig(model_dim=8192, max_seq_len=max(seq_len, 4096), vocab_size=128_256, pad_idx=128_004,
                      num_layers=80 if args.layers is None else args.layers, num_attn_heads=64,
                      num_key_value_heads=8, ffn_inner_dim=int(8192 * 4 * 1.3), ffn_inner_dim_multiple_of=4096,
                      rope_theta=500_000.0, shard_embed_dim=False)
    torch.manual_seed(2)
    # as in the reference's own `ModelFamily._do_create_model`: the gangs must also be registered for the meta device,
    # otherwise the layers built there see single-rank gangs and come out unsharded
    with torch.device("meta"), set_gangs(gangs, meta=True), set_dtype(torch.float32):
        model = LLaMAFactory(cfg).create_model()
    if tp > 1:
        from fairseq2.nn import ColumnShardedLinear

        q = model.decoder.layers[0].self_attn.q_proj
        if not (isinstance(q, ColumnShardedLinear) and q.weight.shape[0] == cfg.model_dim // tp):
            raise RuntimeError(f"the reference model is not tensor-parallel: q_proj weight {tuple(q.weight.shape)}")
    apply_ac_to_transformer_lm(model, every_nth_layer=1)

    def applier(m, wrapper):  # type: ignore[no-untyped-def]
        return apply_fsdp_to_transformer_lm(m, "layer", wrapper)

    dp_model = to_fsdp2(model, gangs, applier, mixed_precision_dtype=torch.bfloat16, fp32_reduce=True,
                        broadcast_state=False, skip_init=False, reshard_after_forward=True)
    optimizer = torch.optim.AdamW(dp_model.parameters(), lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    def stage(ex):  # type: ignore[no-untyped-def]
        tokens, mask, lens, n = ex
        return (tokens.to(device, non_blocking=True), mask.to(device, non_blocking=True),
                BatchLayout((seq_len,), lens, packed=True, device=device), n)

    def step(batch):  # type: ignore[no-untyped-def]
        tokens, mask, layout, n = batch
        loss = dp_model(tokens[:-1], layout, targets=tokens[1:], target_mask=mask, reduction="sum")
        loss.backward()
        normalize_grads(dp_model, gangs.dp, n)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss.detach()

    def barrier() -> None:
        if world > 1:
            gangs.root.barrier()
        torch.cuda.synchronize(device)

    rng = np.random.default_rng(1234 + dp.rank)
    examples = [_make_example(rng, seq_len, cfg.vocab_size) for _ in range(args.warmup + 2 * args.steps)]
    for i in range(args.warmup):
        step(stage(examples[i]))
    barrier()
    staged = [stage(examples[args.warmup + i]) for i in range(args.steps)]
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        step(staged[i])
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    del staged
    barrier()
    t0 = time.perf_counter()
    h2d, last = 0, 0.0
    for i in range(args.steps):
        ex = examples[args.warmup + args.steps + i]
        h2d = ex[0].numel() * 8 + ex[1].numel() + (2 * len(ex[2]) + 1 + seq_len) * 4
        last = float(step(stage(ex)).item())
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([dev_ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        gangs.root.all_reduce(t, ReduceOperation.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    units = float(seq_len * dp.size)
    if rank == 0:
        out = {"metric": "llama3_70b_tp_fsdp_sft_tokens_per_second", "impl": "reference",
               "value": units * args.steps / (dev_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "config": {"model": "llama3_70b" if args.layers is None else f"llama3_70b[layers={args.layers}]",
                          "global_batch": dp.size, "seq_len": seq_len, "parallelism": f"tp{tp} x fsdp{dp.size}",
                          "sdpa": "flash2 varlen", "activation_checkpointing": "per layer"},
               "e2e": {"value": units * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                       "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
               "final_loss": last, "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 2**30}
        print(json.dumps(out), flush=True)
    if world > 1:
        gangs.root.close()
