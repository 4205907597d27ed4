"""Reference arm of ``bench.py``: the UNMODIFIED fairseq2 package installed in
``baseline/_ref`` runs the headline configuration through its own public API
and stock code path -- its LLaMA factory, ``TransformerLM`` forward with fused
loss, ``to_fsdp2`` with the recipe defaults (layer granularity, static bf16
mixed precision, ``fp32_reduce=True``, reshard after forward),
``normalize_grads``, ``clip_grad_norm`` and torch's fused AdamW -- in the order
of its ``Trainer._do_run_step``. With one rank the reference recipe does not
wrap the model and falls back to autocast (``recipe/internal/trainer.py:84-89``),
which is what this arm does too.

Import stand-ins for packages that cannot be installed offline (the native
``fairseq2n`` in documentation mode, ``torcheval``, ``ruamel.yaml``, ...) live in
``baseline/ref_shims``; none of them is on the timed path.

None of this framework's models, kernels or engine is imported here.
"""
from __future__ import annotations

import json
import os
import sys
import threading
import time
from argparse import Namespace
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _abort_marker() -> Path:
    """One file per launch: all workers of a ``torch.distributed.run`` share their parent process."""
    return Path("/tmp") / f"fs2_ref_abort_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}"


def _watch_for_abort() -> None:
    """A rank that fails (say, out of memory) leaves its peers inside collectives that never complete. It writes the
    reason to the marker file; this thread, running on every rank, sees the file, lets rank 0 print the
    ``unavailable`` line, and ends the process with exit code 0 so that the launcher returns at once."""
    marker = _abort_marker()

    def loop() -> None:
        while True:
            time.sleep(0.5)
            try:
                why = marker.read_text()
            except OSError:
                continue
            if not why.endswith("\n"):
                continue                                    # still being written
            _unavailable(why.strip())
            sys.stdout.flush()
            os._exit(0)

    threading.Thread(target=loop, daemon=True).start()


def run_reference_arm(args: Namespace) -> None:
    ref_dir = HERE / "_ref"
    if not (ref_dir / "fairseq2").exists():
        _unavailable("baseline/_ref is not installed (pip install --no-index --no-deps --target baseline/_ref)")
        return
    sys.path.insert(0, str(HERE / "ref_shims"))
    sys.path.insert(0, str(ref_dir))
    multi = int(os.environ.get("WORLD_SIZE", "1")) > 1
    if multi:
        try:
            _abort_marker().unlink()
        except OSError:
            pass
        _watch_for_abort()
    try:
        config = getattr(args, "config", "llama3_8b_fsdp")
        if config == "wav2vec2_large_ddp":
            from baseline.reference_wav2vec2 import run as run_w2v

            run_w2v(args)
        elif config == "llama3_70b_tp4_fsdp2":
            from baseline.reference_llama70b import run as run_70b

            run_70b(args)
        elif config == "moe_ep8":
            from baseline.reference_moe import run as run_moe

            run_moe(args)
        else:
            _run(args)
    except Exception as ex:  # noqa: BLE001 - the arm must always print a line and exit 0
        import traceback

        traceback.print_exc()
        why = f"{type(ex).__name__}: {str(ex).splitlines()[0][:300] if str(ex) else ''}"
        if multi:
            # the peers are stuck in collectives: tell them (and rank 0, which prints the line) and leave
            tmp = _abort_marker().with_suffix(f".{os.getpid()}")
            tmp.write_text(why + "\n")
            try:
                os.replace(tmp, _abort_marker())
            except OSError:
                pass
            time.sleep(3.0)                                 # the watcher thread of this rank ends the process
        _unavailable(why)


def _make_example(rng, seq_len: int, vocab: int):  # type: ignore[no-untyped-def]
    """Same synthetic data recipe as the other arm (kept separate on purpose so
    that this file imports nothing from the framework under test)."""
    import numpy as np
    import torch

    lens: list[int] = []
    total = 0
    while total < seq_len:
        n = min(int(rng.integers(128, 4097)), seq_len - total)
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


def _run(args: Namespace) -> None:
    import numpy as np
    import torch

    import fairseq2
    from fairseq2.data_type import set_dtype
    from fairseq2.gang import (ProcessGroupGang, create_fake_gangs, create_fsdp_gangs, create_parallel_gangs,
                               set_gangs)
    from fairseq2.models.llama.config import LLaMAConfig
    from fairseq2.models.llama.factory import LLaMAFactory
    from fairseq2.models.transformer.sdpa.default import set_default_sdpa_factory
    from fairseq2.models.transformer.sdpa.flash2 import Flash2SDPA
    from fairseq2.models.transformer_lm.fsdp import apply_fsdp_to_transformer_lm
    from fairseq2.nn import BatchLayout
    from fairseq2.nn.fsdp import to_fsdp2
    from fairseq2.nn.utils.grad import clip_grad_norm, normalize_grads

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
        set_default_sdpa_factory(Flash2SDPA)

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        root = ProcessGroupGang.create_default_process_group(device)
        gangs = create_fsdp_gangs(create_parallel_gangs(root))
    else:
        gangs = create_fake_gangs(device)

    if args.model == "llama3_8b":
        cfg = LLaMAConfig(model_dim=4096, max_seq_len=8192, vocab_size=128_256, pad_idx=128_004, num_layers=32,
                          num_attn_heads=32, num_key_value_heads=8, ffn_inner_dim=4096 * 4,
                          ffn_inner_dim_multiplier=1.3, ffn_inner_dim_multiple_of=1024, rope_theta=500_000.0,
                          shard_embed_dim=False)
    else:  # tiny plumbing configuration used to check this arm on CPU
        cfg = LLaMAConfig(model_dim=256, max_seq_len=8192, vocab_size=8192, num_layers=2, num_attn_heads=4,
                          num_key_value_heads=2, ffn_inner_dim=688, ffn_inner_dim_scale=1.0,
                          ffn_inner_dim_multiple_of=1, shard_embed_dim=False)
    if args.layers is not None:
        cfg.num_layers = args.layers
    seq_len = args.seq_len

    torch.manual_seed(2)
    if world > 1:
        # tensor parallel size 1 here: the factory needs no gangs on the meta device (the 70B arm registers them)
        with torch.device("meta"), set_gangs(gangs), set_dtype(torch.float32):
            model = LLaMAFactory(cfg).create_model()

        def applier(m, wrapper):  # type: ignore[no-untyped-def]
            return apply_fsdp_to_transformer_lm(m, "layer", wrapper)

        dp_model = to_fsdp2(model, gangs, applier, mixed_precision_dtype=torch.bfloat16, fp32_reduce=True,
                            broadcast_state=False, skip_init=False, reshard_after_forward=True)
        amp = False
    else:
        with device, set_gangs(gangs), set_dtype(torch.float32):
            model = LLaMAFactory(cfg).create_model()
        dp_model = model
        amp = cuda
    optimizer = torch.optim.AdamW(dp_model.parameters(), lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1,
                                  fused=cuda)

    def stage(ex):  # type: ignore[no-untyped-def]
        tokens, mask, lens, num_targets = ex
        tokens = tokens.to(device, non_blocking=True)
        mask = mask.to(device, non_blocking=True)
        layout = BatchLayout((seq_len,), lens, packed=True, device=device)
        return tokens, mask, layout, num_targets

    def step(batch):  # type: ignore[no-untyped-def]
        tokens, mask, layout, num_targets = batch
        with torch.autocast(device_type=device.type, dtype=torch.bfloat16, enabled=amp):
            loss = dp_model(tokens[:-1], layout, targets=tokens[1:], target_mask=mask, reduction="sum")
        loss.backward()
        normalize_grads(dp_model, gangs.dp, num_targets)
        clip_grad_norm(dp_model, max_norm=1.0)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss.detach()

    def barrier() -> None:
        if world > 1:
            gangs.root.barrier()
        if cuda:
            torch.cuda.synchronize(device)

    rng = np.random.default_rng(1234 + rank)
    total = args.warmup + 2 * args.steps
    examples = [_make_example(rng, seq_len, cfg.vocab_size) for _ in range(total)]

    for i in range(args.warmup):
        step(stage(examples[i]))
    barrier()

    staged = [stage(examples[args.warmup + i]) for i in range(args.steps)]
    barrier()
    if cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(staged[i])
    if cuda:
        ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1) if cuda else (time.perf_counter() - t0) * 1e3
    del staged

    barrier()
    t0 = time.perf_counter()
    h2d = 0
    last = 0.0
    for i in range(args.steps):
        ex = examples[args.warmup + args.steps + i]
        batch = stage(ex)
        h2d = ex[0].numel() * 8 + ex[1].numel() * 1 + (2 * len(ex[2]) + 1 + seq_len) * 4
        last = float(step(batch).item())
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    times = torch.tensor([dev_ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        from fairseq2.gang import ReduceOperation

        gangs.root.all_reduce(times, ReduceOperation.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    tokens_per_step = seq_len * world
    if rank == 0:
        out = {
            "metric": "llama3_8b_fsdp_sft_tokens_per_second", "impl": "reference",
            "value": tokens_per_step * args.steps / (dev_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": args.model if args.layers is None else f"{args.model}[layers={args.layers}]",
                       "global_batch": world, "seq_len": seq_len,
                       "parallelism": f"fsdp{world}" if world > 1 else "single-rank (autocast, as the reference recipe does)",
                       "sdpa": "flash2 varlen" if cuda else "torch"},
            "e2e": {"value": tokens_per_step * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "final_loss": last,
        }
        if cuda:
            out["peak_mem_gb"] = torch.cuda.max_memory_allocated(device) / 2**30
        print(json.dumps(out), flush=True)
    if world > 1:
        gangs.root.close()
