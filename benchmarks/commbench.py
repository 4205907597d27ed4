"""Device-timed microbenchmarks of the peer-memory collectives and the fused compute+collective kernels.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m benchmarks.commbench [--cases all] [--iters 10]

Every case is timed with CUDA events on the launching stream after warm-up, a barrier on both sides, and reported as
the MAX over ranks. Rank 0 prints one JSON line per case with the achieved rate and its fraction of the roofline

    target = max(FLOPs / measured GEMM peak, bytes that must cross NVLink per GPU / link bandwidth)

(and local HBM bytes / measured copy bandwidth where that is the larger term), where the link bandwidth defaults to the measured peer-copy figure of 770 GB/s per direction per GPU. For each case
the NCCL (or NCCL + separate kernel) formulation of the same work is timed next to it.

The shapes are the ones a LLaMA-3-8B layer produces: an FSDP unit of 218 M bf16 parameters; the row-parallel
``[8192, 14336/W] x [4096, 14336/W]`` and column-parallel ``[8192, 4096] x [14336/W, 4096]`` feed-forward GEMMs.
"""

from __future__ import annotations

import argparse
import json
import os
from collections.abc import Callable

import torch
import torch.distributed as dist


def _time(fn: Callable[[], None], barrier: Callable[[], None], iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(ms, dist.ReduceOp.MAX)
    return float(ms)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="all")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--unit-params", type=int, default=218_112_000, help="parameters of one FSDP unit")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--gemm-tflops", type=float, default=None, help="defaults to MEASURED_PEAKS.json or 1590")
    args = ap.parse_args()

    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.ops.fused_collective import FusedAllGatherGemm, FusedGemmReduceScatter
    from fairseq2_b200.ops.gemm import gemm as gemm_nt
    from fairseq2_b200.ops.optim import multi_tensor_adamw
    from fairseq2_b200.parallel.symm import SymmetricArena

    rank, W = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    pg = base.as_process_group()
    peak = args.gemm_tflops
    if peak is None:
        try:
            with open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")) as fp:
                peak = float(json.load(fp)["bf16_tflops"])
        except (OSError, KeyError, ValueError):
            peak = 1590.0
    link = args.link_gbs * 1e9
    hbm = 6.5e12
    try:
        with open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")) as fp:
            hbm = float(json.load(fp)["hbm_gbs"]) * 1e9
    except (OSError, KeyError, ValueError):
        pass
    cases = args.cases.split(",")
    want = lambda c: "all" in cases or c in cases  # noqa: E731

    want_tp = "all" in cases or "tp_mlp" in cases
    n = (args.unit_params // W + 2047) // 2048 * 2048            # shard elements
    T = args.tokens
    arena_bytes = ((W + 1) * n * 2 + (128 << 20) + 2 * (T // W) * 4096 * 4 + 2 * T * 4096 * 2 + 3 * (T + 64) * 4096 * 2
                   + 3 * (14336 + 64) * 4096 * 2 + (64 << 20)
                   + ((3 * T + 2 * (T // W)) * 8192 * 2 + (64 << 20) if want_tp else 0))
    arena = SymmetricArena(base, arena_bytes)
    ext = arena.ext
    epoch = {"v": 0}

    def barrier() -> None:
        arena.barrier_next(0)
        torch.cuda.synchronize()

    def emit(case: str, ms: float, *, nvlink_bytes: float = 0.0, flops: float = 0.0, hbm_bytes: float = 0.0,
             baseline_ms: float | None = None, **extra: object) -> None:
        if rank != 0:
            return
        target_ms = max(flops / (peak * 1e12), nvlink_bytes / link, hbm_bytes / hbm) * 1e3
        row = {"case": case, "world": W, "ms": round(ms, 4), "target_ms": round(target_ms, 4),
               "frac_of_roofline": round(target_ms / ms, 3) if ms > 0 else None}
        if nvlink_bytes:
            row["nvlink_gbs_per_gpu"] = round(nvlink_bytes / ms / 1e6, 1)
        if flops:
            row["tflops"] = round(flops / ms / 1e9, 1)
        if baseline_ms is not None:
            row["nccl_formulation_ms"] = round(baseline_ms, 4)
        row.update(extra)
        print(json.dumps(row), flush=True)

    segs_off, segs_n = [0], [n]
    shard_off, shard = arena.alloc_tensor(n, torch.bfloat16)
    grad_off, grad_full = arena.alloc_tensor(W * n, torch.bfloat16)
    shard.normal_()
    grad_full.normal_(std=0.01)
    full = torch.empty(W * n, device=dev, dtype=torch.bfloat16)
    peer_bytes = (W - 1) * n * 2                                  # received (AG) or read (RS) over NVLink per GPU

    if want("allgather"):
        for blocks in (max(32 // W, 4), 16):
            def ag() -> None:
                epoch["v"] += 1
                ext.comm_allgather_segments(arena.peer_ptrs, rank, segs_off, segs_n, shard_off, full, 1, 0, blocks,
                                            arena.wait_limit_s)
            ms = _time(ag, barrier, args.iters)
            nccl = _time(lambda: dist.all_gather_into_tensor(full, shard, group=pg), barrier, args.iters)
            emit("fsdp_unit_allgather", ms, nvlink_bytes=peer_bytes, baseline_ms=nccl, blocks_per_peer=blocks,
                 mbytes=round(W * n * 2 / 1e6, 1))

    if want("reducescatter"):
        gshard = torch.empty(n, device=dev, dtype=torch.float32)
        rs_epoch = {"v": 0}

        def rs() -> None:
            rs_epoch["v"] += 1
            ext.comm_reducescatter_segments(arena.peer_ptrs, rank, segs_off, segs_n, grad_off, gshard, 1.0 / W, False, 3,
                                            rs_epoch["v"], 48, arena.wait_limit_s)
        ms = _time(rs, barrier, args.iters)
        out16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
        nccl = _time(lambda: dist.reduce_scatter_tensor(out16, grad_full, op=dist.ReduceOp.AVG, group=pg), barrier,
                     args.iters)
        emit("fsdp_unit_reducescatter_fp32acc", ms, nvlink_bytes=peer_bytes, baseline_ms=nccl)

        master, m, v = torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        low = torch.empty(n, device=dev, dtype=torch.bfloat16)
        hp = dict(lr=1e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
        fe = {"v": 0}

        def rs_adamw() -> None:
            fe["v"] += 1
            ext.comm_reducescatter_adamw(arena.peer_ptrs, rank, segs_off, segs_n, grad_off, master, m, v, low, 1.0 / W,
                                         hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["weight_decay"], fe["v"], 4,
                                         fe["v"], 96, arena.wait_limit_s)

        def rs_then_adamw() -> None:
            rs()
            multi_tensor_adamw([master], [gshard], [m], [v], [low], step=max(rs_epoch["v"], 1), **hp)

        ms_f = _time(rs_adamw, barrier, args.iters)
        ms_u = _time(rs_then_adamw, barrier, args.iters)
        # local HBM traffic of the optimizer half: p, m, v read + written (fp32) and the bf16 copy written
        emit("fsdp_unit_reducescatter_adamw_fused", ms_f, nvlink_bytes=peer_bytes, hbm_bytes=n * (24 + 2 + 2),
             baseline_ms=ms_u, note="baseline = our reduce-scatter kernel + our AdamW kernel")

    if want("allreduce"):
        numel = 64 * 1024 * 1024                                  # 128 MB of bf16, a DDP-scale bucket
        off, bucket = arena.alloc_tensor(numel, torch.bfloat16)
        coff, counter = arena.alloc(64, align=64)
        counter.zero_()
        bucket.normal_(std=0.01)
        ae = {"v": 0}

        def ar() -> None:
            ae["v"] += 1
            ext.comm_allreduce_inplace(arena.peer_ptrs, rank, off, numel, False, 1.0 / W, 5, 6, ae["v"], coff,
                                       arena.device_index, 64, arena.wait_limit_s)
        ms = _time(ar, barrier, args.iters)
        ref = torch.empty(numel, device=dev, dtype=torch.bfloat16).normal_(std=0.01)
        nccl = _time(lambda: dist.all_reduce(ref, op=dist.ReduceOp.AVG, group=pg), barrier, args.iters)
        emit("ddp_bucket_allreduce_inplace_128MB", ms, nvlink_bytes=2 * (W - 1) / W * numel * 2, baseline_ms=nccl)
        if arena.multicast_ptr:
            me = {"v": 0}

            def ar_mm() -> None:
                me["v"] += 1
                ext.comm_allreduce_multimem(arena.peer_ptrs, rank, arena.multicast_ptr, off, numel, False, 1.0 / W, 7, 8,
                                            me["v"], coff, arena.device_index, 64, arena.wait_limit_s)
            ms = _time(ar_mm, barrier, args.iters)
            # through the switch every GPU sends and receives the whole buffer once (1/W reduced in, 1/W broadcast
            # out, and serves the other ranks' reads of its copy)
            emit("ddp_bucket_allreduce_multimem_128MB", ms, nvlink_bytes=numel * 2, baseline_ms=nccl)

    K_ffn, D = 14336, 4096
    if want("gemm_rs") and K_ffn % W == 0 and T % (W * 128) == 0:
        kl = K_ffn // W
        x = torch.randn(T, kl, device=dev, dtype=torch.bfloat16)
        w = torch.randn(D, kl, device=dev, dtype=torch.bfloat16) * 0.02
        op = FusedGemmReduceScatter(arena, T // W, D, mode="red")
        ms = _time(lambda: op(x, w), barrier, args.iters)
        op_s = FusedGemmReduceScatter(arena, T // W, D, mode="scatter")
        ms_s = _time(lambda: op_s(x, w), barrier, args.iters)
        out = torch.empty(T // W, D, device=dev, dtype=torch.bfloat16)

        def unfused() -> None:
            y = gemm_nt(x, w)
            dist.reduce_scatter_tensor(out, y, group=pg)
        nccl = _time(unfused, barrier, args.iters)
        gemm_only = _time(lambda: gemm_nt(x, w), barrier, args.iters)
        emit("tp_row_gemm_reducescatter_fused_red_f32", ms, flops=2.0 * T * kl * D, nvlink_bytes=(W - 1) / W * T * D * 4,
             baseline_ms=nccl, gemm_alone_ms=round(gemm_only, 4),
             note="fp32 red.global.add (4 B/element on the wire); baseline = our GEMM + NCCL bf16 reduce-scatter")
        emit("tp_row_gemm_reducescatter_fused_scatter_bf16", ms_s, flops=2.0 * T * kl * D,
             nvlink_bytes=(W - 1) / W * T * D * 2, baseline_ms=nccl, gemm_alone_ms=round(gemm_only, 4),
             note="bf16 tiles stored into the owner's slices + local sum; baseline = our GEMM + NCCL bf16 reduce-scatter")

    if want("ag_gemm") and K_ffn % W == 0 and (T // W) % 128 == 0:
        nl = K_ffn // W
        w = torch.randn(nl, D, device=dev, dtype=torch.bfloat16) * 0.02
        best = None
        for ncopy in (4, 8, 16):
            op_a = FusedAllGatherGemm(arena, T // W, D, gather="a", num_copy_ctas=ncopy)
            op_a.shard.normal_()
            t = _time(lambda: op_a(w), barrier, args.iters)
            if best is None or t < best[0]:
                best = (t, ncopy)
        ms, ncopy_a = best
        xs = op_a.shard.clone()
        xg = torch.empty(T, D, device=dev, dtype=torch.bfloat16)

        def unfused_a() -> None:
            dist.all_gather_into_tensor(xg, xs, group=pg)
            gemm_nt(xg, w)
        nccl = _time(unfused_a, barrier, args.iters)
        gemm_only = _time(lambda: gemm_nt(xg, w), barrier, args.iters)
        emit("tp_column_allgather_gemm_fused", ms, flops=2.0 * T * D * nl, nvlink_bytes=(W - 1) / W * T * D * 2,
             baseline_ms=nccl, gemm_alone_ms=round(gemm_only, 4), copier_ctas=ncopy_a)

    if want("ag_gemm") and (K_ffn // W) % 256 == 0:
        rows = K_ffn // W                                          # FSDP unshard of the [14336, 4096] up-projection
        x = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
        best = None
        for ncopy in (4, 8, 16):
            op_b = FusedAllGatherGemm(arena, rows, D, gather="b", num_copy_ctas=ncopy)
            op_b.shard.normal_(std=0.02)
            t = _time(lambda: op_b(x), barrier, args.iters)
            if best is None or t < best[0]:
                best = (t, ncopy)
        ms, ncopy_b = best
        ws = op_b.shard.clone()
        wg = torch.empty(K_ffn, D, device=dev, dtype=torch.bfloat16)

        def unfused_b() -> None:
            dist.all_gather_into_tensor(wg, ws, group=pg)
            gemm_nt(x, wg)
        nccl = _time(unfused_b, barrier, args.iters)
        gemm_only = _time(lambda: gemm_nt(x, wg), barrier, args.iters)
        emit("fsdp_unshard_allgather_gemm_fused", ms, flops=2.0 * T * D * K_ffn, nvlink_bytes=(W - 1) / W * K_ffn * D * 2,
             baseline_ms=nccl, gemm_alone_ms=round(gemm_only, 4), copier_ctas=ncopy_b)

    if want("tp_mlp") and T % (W * 128) == 0:
        # LLaMA-3-70B feed-forward block under tensor parallelism: D = 8192, F = 28672 / W per rank, T tokens.
        # ours: token-sharded activations, all-gather inside the column GEMM, reduce-scatter inside the row GEMM,
        # same kernels with swapped roles in the backward pass. baseline: the Megatron formulation the reference
        # uses (replicated activations, GEMMs + one NCCL all-reduce forward and one backward), our GEMM kernel.
        from fairseq2_b200.ops.fused_collective import SequenceParallelLinears

        D2, F2 = 8192, 28672
        if F2 % W == 0 and (F2 // W) % 8 == 0:
            Fl, Tl = F2 // W, T // W
            sp = SequenceParallelLinears(arena, Tl, D2)
            w1 = (torch.randn(Fl, D2, device=dev) * D2 ** -0.5).to(torch.bfloat16).requires_grad_(True)
            w2 = (torch.randn(D2, Fl, device=dev) * F2 ** -0.5).to(torch.bfloat16).requires_grad_(True)
            xs = torch.randn(Tl, D2, device=dev, dtype=torch.bfloat16, requires_grad=True)
            gs = torch.randn(Tl, D2, device=dev, dtype=torch.bfloat16)

            def ours() -> None:
                xs.grad = w1.grad = w2.grad = None
                y = sp.row(torch.nn.functional.gelu(sp.column(xs, w1)), w2)
                y.backward(gs)

            xf = torch.randn(T, D2, device=dev, dtype=torch.bfloat16, requires_grad=True)
            gf = torch.randn(T, D2, device=dev, dtype=torch.bfloat16)

            class _AllReduceBwd(torch.autograd.Function):          # identity forward, all-reduce backward
                @staticmethod
                def forward(ctx, t):  # type: ignore[no-untyped-def]
                    return t

                @staticmethod
                def backward(ctx, g):  # type: ignore[no-untyped-def]
                    g = g.contiguous()
                    dist.all_reduce(g, group=pg)
                    return g

            from fairseq2_b200.ops.gemm import linear as k_linear

            def megatron() -> None:
                xf.grad = w1.grad = w2.grad = None
                h = torch.nn.functional.gelu(k_linear(_AllReduceBwd.apply(xf), w1))
                y = k_linear(h, w2)
                dist.all_reduce(y, group=pg)
                y.backward(gf)

            ms = _time(ours, barrier, args.iters)
            base_ms = _time(megatron, barrier, args.iters)
            flops = 3 * 2 * 2.0 * T * D2 * Fl                     # two GEMMs, forward + dgrad + wgrad
            emit("tp_mlp_70b_fwd_bwd_sequence_parallel_fused", ms, flops=flops,
                 nvlink_bytes=4 * (W - 1) / W * T * D2 * 2, baseline_ms=base_ms, tokens=T, model_dim=D2, inner_dim=F2,
                 note="baseline = replicated activations, same GEMM kernel, NCCL all-reduce forward and backward")

    if want("moe_ep"):
        # Expert-parallel dispatch and combine of one MoE layer of the 128-expert top-8 model: 8192 tokens per GPU,
        # model dim 2048, near-uniform routing. ours: counts exchange + layout + rows stored straight into the
        # owners' tile-aligned inboxes (dispatch), outputs loaded from the owners' outboxes and gate-weighted
        # (combine). baseline: sort by expert + two NCCL all_to_all_single (counts, rows) and the inverse.
        from fairseq2_b200.ops.moe import moe_route
        from fairseq2_b200.ops.moe_ep import ExpertParallelExchange
        from fairseq2_b200.parallel.symm import SymmetricArena as _Arena

        E, k, Dm, Tm = 128, 8, 2048, 8192
        if E % W == 0:
            rows_total = Tm * k
            cap = 2 * rows_total
            ep_arena = _Arena(base, 2 * (cap + 128 * (E // W + 2)) * Dm * 2 + (8 << 20))
            ep = ExpertParallelExchange(ep_arena, E, Dm, max_tokens=Tm, top_k=k, capacity=cap)
            xm = torch.randn(Tm, Dm, device=dev, dtype=torch.bfloat16)
            logits = torch.randn(Tm, E, device=dev) * 0.02
            ids, gates, counts = moe_route(logits, k, softmax_gate=True)
            state: dict[str, object] = {}

            def disp() -> None:
                state["out"] = ep.dispatch_padded(xm, ids, counts)

            def comb() -> None:
                rows, dest = state["out"][0], state["out"][1]     # type: ignore[index]
                ep.combine(rows, dest, Tm, gates)

            disp()
            ms_d = _time(disp, barrier, args.iters)
            ms_c = _time(comb, barrier, args.iters)
            # NCCL formulation
            El = E // W
            flat = ids.reshape(-1).long()
            def nccl_disp() -> None:
                order = torch.argsort(flat, stable=True)
                rows = xm.index_select(0, order // k)
                per = torch.bincount(flat, minlength=E)
                recv_per = torch.empty_like(per)
                dist.all_to_all_single(recv_per, per, group=pg)
                send = per.view(W, El).sum(1).tolist()
                recv = recv_per.view(W, El).sum(1).tolist()
                got = rows.new_empty((sum(recv), Dm))
                dist.all_to_all_single(got, rows, recv, send, group=pg)
                state["nccl"] = (got, order, send, recv)

            def nccl_comb() -> None:
                got, order, send, recv = state["nccl"]            # type: ignore[misc]
                back = got.new_empty((sum(send), Dm))
                dist.all_to_all_single(back, got, send, recv, group=pg)
                w = gates.reshape(-1)[order].unsqueeze(1).to(back.dtype)
                torch.zeros_like(xm).index_add_(0, order // k, back * w)

            nccl_disp()
            nd = _time(nccl_disp, barrier, args.iters)
            nc = _time(nccl_comb, barrier, args.iters)
            link_bytes = (W - 1) / W * rows_total * Dm * 2
            emit("moe_ep_dispatch_128e_top8", ms_d, nvlink_bytes=link_bytes, hbm_bytes=2.0 * rows_total * Dm * 2,
                 baseline_ms=nd, rows=rows_total, model_dim=Dm)
            emit("moe_ep_combine_128e_top8", ms_c, nvlink_bytes=link_bytes, hbm_bytes=2.0 * rows_total * Dm * 2,
                 baseline_ms=nc, rows=rows_total, model_dim=Dm)

    barrier()
    ext.check_status()
    base.close()


if __name__ == "__main__":
    main()
