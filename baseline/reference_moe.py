"""Reference arm for ``bench.py --config moe_ep8 --impl reference`` -- the "NCCL-only" formulation.

The reference has no expert parallelism, no top-k softmax gate and no auxiliary loss (its only mixture-of-experts
layer, ``models/llama4/moe.py:109-157``, feeds every token to every expert). This arm therefore is the reference's
own building blocks from ``baseline/_ref`` -- ``TransformerLM``, ``StandardTransformerLMDecoderLayer``,
``StandardMultiheadAttention`` with ``Flash2SDPA``, ``RMSNorm``, ``RotaryEncoder``, ``GroupedExpertNetwork`` (its
batched ``torch.bmm`` expert math), ``fully_shard`` on the dense parts as ``to_fsdp2`` applies it -- around a
feed-forward module that expresses the same expert-parallel layer with library calls only: ``torch.topk`` +
softmax gate + load-balancing loss, ``torch.distributed.all_to_all_single`` for dispatch and combine, the
reference's ``torch.bmm`` experts over the received rows. Nothing of the framework under test is imported."""
from __future__ import annotations

import json
import os
import time
from argparse import Namespace


def run(args: Namespace) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist
    from torch import Tensor
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from torch.nn import Module, Parameter

    import fairseq2
    from fairseq2.data_type import set_dtype
    from fairseq2.gang import ProcessGroupGang, ReduceOperation, create_fsdp_gangs, create_parallel_gangs, set_gangs
    from fairseq2.models.transformer import (CausalAttentionBias, FeedForwardNetwork, StandardMultiheadAttention,
                                             TransformerEmbeddingFrontend, TransformerNormOrder)
    from fairseq2.models.transformer.experts import GroupedExpertNetwork
    from fairseq2.models.transformer.sdpa.flash2 import Flash2SDPA
    from fairseq2.models.transformer_lm import (StandardTransformerLMDecoder, StandardTransformerLMDecoderLayer,
                                                TransformerLM)
    from fairseq2.nn import BatchLayout, Linear, RMSNorm, RotaryEncoder, StandardEmbedding
    from fairseq2.nn.utils.grad import normalize_grads

    fairseq2.init_fairseq2()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise RuntimeError("the expert-parallel configuration needs at least 2 ranks")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    torch.backends.cuda.matmul.allow_tf32 = True
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    root = ProcessGroupGang.create_default_process_group(device)
    gangs = create_fsdp_gangs(create_parallel_gangs(root))
    pg = root.as_process_group()

    D, H, HKV, HD, V, E, F, K = 2048, 32, 4, 128, 151_936, 128, 768, 8
    L = 48 if args.layers is None else args.layers
    El = E // world
    AUX = 1e-3
    aux_terms: list[Tensor] = []

    class _A2A(torch.autograd.Function):
        """``all_to_all_single`` with variable splits; the backward is the reverse exchange."""

        @staticmethod
        def forward(ctx, x: Tensor, out_splits: list[int], in_splits: list[int]) -> Tensor:  # type: ignore[override]
            ctx.splits = (out_splits, in_splits)
            out = x.new_empty((sum(out_splits), x.shape[1]))
            dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=pg)
            return out

        @staticmethod
        def backward(ctx, g: Tensor):  # type: ignore[override]
            out_splits, in_splits = ctx.splits
            gi = g.new_empty((sum(in_splits), g.shape[1]))
            dist.all_to_all_single(gi, g.contiguous(), in_splits, out_splits, group=pg)
            return gi, None, None

    class ExpertParallelMoE(FeedForwardNetwork):
        def __init__(self) -> None:
            super().__init__()
            self.router = Parameter(torch.empty((D, E)))
            self.experts = GroupedExpertNetwork(El, D, F)          # the reference's bmm experts, this rank's share
            torch.nn.init.normal_(self.router, std=0.02)
            for p in self.experts.parameters():                    # (the reference leaves them to the checkpoint)
                torch.nn.init.trunc_normal_(p, std=0.02, a=-0.06, b=0.06)

        def forward(self, seqs: Tensor) -> Tensor:
            x = seqs.reshape(-1, D)
            T = x.shape[0]
            logits = (x @ self.router).float()
            top, ids = torch.topk(logits, K, dim=1)
            gates = torch.softmax(top, dim=1)
            if self.training:
                probs = torch.softmax(logits, dim=-1).mean(dim=0)
                frac = torch.bincount(ids.reshape(-1), minlength=E).float() / (T * K)
                aux_terms.append(E * (frac * probs).sum())
            flat = ids.reshape(-1)
            order = torch.argsort(flat, stable=True)               # rows grouped by expert, hence by owner rank
            tok = order // K
            rows = x.index_select(0, tok) * gates.reshape(-1)[order].to(x.dtype).unsqueeze(1)
            per_expert = torch.bincount(flat, minlength=E)
            recv_per_expert = torch.empty_like(per_expert)
            dist.all_to_all_single(recv_per_expert, per_expert, group=pg)          # [W, El] counts I will receive
            send = per_expert.view(world, El).sum(1).tolist()
            recv_mat = recv_per_expert.view(world, El)
            recv = recv_mat.sum(1).tolist()
            got = _A2A.apply(rows, recv, send)                     # grouped by source rank, then by local expert
            # regroup by local expert and pad every expert to the largest group: the reference's experts are a bmm
            src_expert = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(world),
                                                 recv_mat.reshape(-1))
            eorder = torch.argsort(src_expert, stable=True)
            n_e = recv_mat.sum(0)
            cap = int(n_e.max())
            slot_in_e = torch.arange(eorder.numel(), device=x.device) - torch.repeat_interleave(
                torch.cumsum(n_e, 0) - n_e, n_e)
            padded = got.new_zeros((El, max(cap, 1), D))
            e_sorted = src_expert[eorder]
            padded[e_sorted, slot_in_e] = got[eorder]
            out_p = self.experts(padded)                            # [El, cap, D]
            back = torch.empty_like(got)
            back[eorder] = out_p[e_sorted, slot_in_e]
            ret = _A2A.apply(back, send, recv)                      # my rows again, in `order`
            out = torch.zeros_like(x).index_add(0, tok, ret)
            return out.view(seqs.shape)

    def init(p):  # type: ignore[no-untyped-def]
        torch.nn.init.trunc_normal_(p.weight, std=0.02, a=-0.06, b=0.06)

    torch.manual_seed(2 + rank)
    with device, set_gangs(gangs), set_dtype(torch.float32):
        embed = StandardEmbedding(V, D)
        frontend = TransformerEmbeddingFrontend(D, embed, pos_encoder=None, no_scale=True, dropout_p=0.0)
        pe = RotaryEncoder(HD, 4096, theta=1_000_000.0)
        layers = []
        for _ in range(L):
            attn = StandardMultiheadAttention(D, H, Flash2SDPA(CausalAttentionBias()), head_dim=HD,
                                              num_key_value_heads=HKV, qkv_proj_init_fn=init, pos_encoder=pe,
                                              output_proj_init_fn=init, bias=False)
            layers.append(StandardTransformerLMDecoderLayer(attn, RMSNorm(D, bias=False), ExpertParallelMoE(),
                                                            RMSNorm(D, bias=False),
                                                            norm_order=TransformerNormOrder.PRE))
        decoder = StandardTransformerLMDecoder(layers, RMSNorm(D, bias=False))
        model = TransformerLM(D, frontend, decoder, Linear(D, V, bias=False, init_fn=init), pad_idx=None,
                              max_seq_len=4096)
    model.train()
    # Without activation checkpointing the full-size model does not fit this formulation (48 layers of padded
    # per-expert batches and their fp32 autocast copies: out of memory at 177 GiB on a B200), so from 32 layers on
    # every layer is checkpointed the way the reference recipes do it; the result line says so.
    use_ac = L >= 32 or os.environ.get("FS2_BENCH_REF_AC") == "1"
    if use_ac:
        from fairseq2.models.transformer_lm.ac import apply_ac_to_transformer_lm

        apply_ac_to_transformer_lm(model, every_nth_layer=1)
        layers = list(model.decoder.layers)
    # FSDP2 on the dense parts, the way the reference's `to_fsdp2` applies `fully_shard` (bf16 parameters, fp32
    # reduction, one unit per layer, the root last); the expert weights differ from rank to rank and stay local
    mesh = torch.distributed.device_mesh.DeviceMesh.from_group(pg, "cuda")
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    expert_params = {p for layer in layers for p in layer.ffn.experts.parameters()}
    for layer in layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp, reshard_after_forward=True,
                    ignored_params={p for p in layer.ffn.experts.parameters()})
    fully_shard(model, mesh=mesh, mp_policy=mp, reshard_after_forward=False, ignored_params=expert_params)
    hp = dict(lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    dense = [p for p in model.parameters() if p not in expert_params]
    optimizers = [torch.optim.AdamW(dense, **hp), torch.optim.AdamW(list(expert_params), **hp)]

    seq_len, seqs_per_gpu = 4096, 2

    def step(batch: Tensor) -> Tensor:
        inp, tgt = batch[:, :-1], batch[:, 1:]
        layout = BatchLayout(tuple(inp.shape), [inp.shape[1]] * inp.shape[0], device=device)
        aux_terms.clear()
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):      # the local experts compute in bf16 too
            loss = model(inp, layout, targets=tgt, reduction="sum")
        if aux_terms:
            loss = loss + AUX * torch.stack(aux_terms).mean() * tgt.numel()
        loss.backward()
        for p in expert_params:                                   # local gradients cover all ranks' tokens already
            if p.grad is not None:
                p.grad.div_(world)
        normalize_grads(model, gangs.dp, tgt.numel())
        for opt in optimizers:
            opt.step()
            opt.zero_grad(set_to_none=True)
        return loss.detach()

    def barrier() -> None:
        root.barrier()
        torch.cuda.synchronize(device)

    rng = np.random.default_rng(1234 + rank)
    examples = [torch.from_numpy(rng.integers(0, V, size=(seqs_per_gpu, seq_len + 1), dtype=np.int64)).pin_memory()
                for _ in range(args.warmup + 2 * args.steps)]
    for i in range(args.warmup):
        step(examples[i].to(device, non_blocking=True))
    barrier()
    staged = [examples[args.warmup + i].to(device, non_blocking=True) for i in range(args.steps)]
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
    last = 0.0
    for i in range(args.steps):
        ex = examples[args.warmup + args.steps + i]
        last = float(step(ex.to(device, non_blocking=True)).item())
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([dev_ms, e2e_ms], device=device, dtype=torch.float64)
    root.all_reduce(t, ReduceOperation.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    units = float(seq_len * seqs_per_gpu * world)
    if rank == 0:
        out = {"metric": "moe_128e_top8_ep_tokens_per_second", "impl": "reference",
               "value": units * args.steps / (dev_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "config": {"model": "moe_48l_2048d_128e_top8" if args.layers is None else f"moe[layers={L}]",
                          "global_batch": seqs_per_gpu * world, "seq_len": seq_len,
                          "parallelism": f"ep{world} (NCCL all_to_all_single + torch.bmm experts) + fsdp2 (dense parts)",
                          "activation_checkpointing": "per layer (does not fit without)" if use_ac else False,
                          "note": "NCCL-only formulation: the reference has no expert parallelism of its own"},
               "e2e": {"value": units * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                       "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": examples[0].numel() * 8,
                       "d2h_bytes_per_step": 4},
               "final_loss": last, "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 2**30}
        print(json.dumps(out), flush=True)
    root.close()
