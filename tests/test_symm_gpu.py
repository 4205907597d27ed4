"""Symmetric-memory collectives and the zero-copy FSDP path on 2+ GPUs,
checked against closed-form expectations and against the NCCL path."""
from __future__ import annotations

import os
import sys

import pytest
import torch

from tests.dist_utils import run_distributed

pytestmark = pytest.mark.gpu


WORLDS = [2, 4, 8]     # every multi-rank test runs at each of these that the box can host


def _need_gpus(n: int) -> None:
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _collectives_worker(rank: int, world: int):
    from datetime import timedelta

    from fairseq2_b200.gang import ProcessGroupGang, ReduceOperation, create_parallel_gangs, setup_root_gang
    from fairseq2_b200.parallel.symm import SymmGang, symmetric_memory_available

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    g = setup_root_gang(dev, timeout=timedelta(seconds=30), collectives="symm")   # the factory the recipes use
    assert isinstance(g, SymmGang) and isinstance(g.base_gang(), ProcessGroupGang)
    assert symmetric_memory_available(g) and g.arena.wait_limit_s == 30.0
    assert create_parallel_gangs(g).dp is g                       # tp = 1: the data-parallel gang is the root gang
    out = {}
    # exact in 64-bit integers (goes to the wrapped gang: fp32 staging would round)
    big = torch.tensor([2**40 + rank + 1], device=dev)
    g.all_reduce(big, ReduceOperation.SUM)
    out["int_sum"] = int(big[0])
    t = torch.full((1000,), float(rank + 1), device=dev)
    g.all_reduce(t, ReduceOperation.SUM)
    out["sum"] = float(t[0]), float(t[-1])
    t = torch.full((7,), float(rank + 1), device=dev, dtype=torch.bfloat16)
    g.all_reduce(t, ReduceOperation.MAX)
    out["max"] = float(t[0])
    inp = torch.arange(10, device=dev, dtype=torch.int64) + 100 * rank
    ag = torch.empty((world, 10), device=dev, dtype=torch.int64)
    g.all_gather(ag, inp)
    out["ag"] = ag.cpu().tolist()
    b = torch.full((33,), float(rank), device=dev)
    g.broadcast(b, source_rank=world - 1)
    out["bcast"] = float(b[0])
    rs_in = torch.stack([torch.full((16,), float(rank * 10 + j), device=dev) for j in range(world)])
    rs_out = torch.empty(16, device=dev)
    g.reduce_scatter(rs_out, rs_in, ReduceOperation.SUM)
    out["rs"] = float(rs_out[0])
    # variable all-to-all: rank r sends (r + j + 1) rows to rank j
    isz = [rank + j + 1 for j in range(world)]
    osz = [j + rank + 1 for j in range(world)]
    send = torch.cat([torch.full((n, 4), float(rank * 100 + j), device=dev) for j, n in enumerate(isz)])
    recv = torch.empty((sum(osz), 4), device=dev)
    g.all_to_all(recv, send, osz, isz)
    out["a2a"] = [float(x[0, 0]) for x in recv.split(osz)]
    g.barrier()
    torch.cuda.synchronize()
    g.arena.ext.check_status()
    g.close()
    return out


@pytest.mark.parametrize("world", WORLDS)
def test_symm_gang_collectives(world: int) -> None:
    _need_gpus(world)
    res = run_distributed(_collectives_worker, world)
    for rank, r in enumerate(res):
        assert r["sum"] == (world * (world + 1) / 2,) * 2
        assert r["int_sum"] == world * 2**40 + world * (world + 1) // 2
        assert r["max"] == float(world)
        assert r["ag"] == [[i + 100 * q for i in range(10)] for q in range(world)]
        assert r["bcast"] == float(world - 1)
        assert r["rs"] == sum(q * 10 + rank for q in range(world))
        assert r["a2a"] == [float(q * 100 + rank) for q in range(world)]


def _fsdp_worker(rank: int, world: int, comm: str):
    import numpy as np

    from fairseq2_b200.datasets.synthetic import make_packed_sft_example
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.llama import LLaMAConfig, create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_fsdp_gangs(create_parallel_gangs(root))
    cfg = LLaMAConfig(model_dim=512, max_seq_len=2048, vocab_size=4096, num_layers=3, num_attn_heads=4,
                      num_key_value_heads=2, ffn_inner_dim=1408, ffn_inner_dim_scale=1.0,
                      ffn_inner_dim_multiple_of=1, rope_theta=500000.0, shard_embed_dim=False)
    torch.manual_seed(0)
    with torch.device("meta"):
        model = create_llama_model(cfg, gangs)
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16, comm=comm, fp32_reduce=True)
    assert (fsdp.arena is not None) == (comm == "symm")
    opt = AdamW(fsdp.parameters(), lr=1e-3)
    rng = np.random.default_rng(5 + rank)
    losses = []
    for _ in range(3):
        ex = make_packed_sft_example(rng, 1024, cfg.vocab_size, doc_len_range=(64, 512))
        tokens, mask = ex.tokens.to(dev), ex.target_mask.to(dev)
        layout = BatchLayout((1024,), ex.seq_lens, packed=True, device=dev)
        fsdp.zero_grad()
        loss = fsdp(tokens[:-1], layout, targets=tokens[1:], target_mask=mask)
        loss.backward()
        fsdp.finish_backward()
        fsdp.scale_grads(1.0 / 1024)
        gn = fsdp.clip_grad_norm(1.0)
        opt.step(grad_scale=fsdp.grad_scale)
        fsdp.after_optimizer_step()
        losses.append((float(loss), float(gn)))
    torch.cuda.synchronize()
    require_ext().check_status()
    root.close()
    return losses


@pytest.mark.parametrize("world", WORLDS)
def test_fsdp_symm_matches_nccl(world: int) -> None:
    _need_gpus(world)
    a = run_distributed(_fsdp_worker, world, "symm")
    b = run_distributed(_fsdp_worker, world, "nccl")
    for ra, rb in zip(a, b):
        for (la, ga), (lb, gb) in zip(ra, rb):
            assert abs(la - lb) / abs(lb) < 2e-2
            assert abs(ga - gb) / abs(gb) < 5e-2


def _gemm_rs_worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.ops.fused_collective import FusedGemmReduceScatter, gemm_reduce_scatter_reference
    from fairseq2_b200.parallel.symm import SymmetricArena

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    M, N, Kl = 1024, 768, 512
    arena = SymmetricArena(base, 8 * M * N * 4 + (1 << 20))
    errs = []
    for mode in ("red", "scatter"):
        op = FusedGemmReduceScatter(arena, M // world, N, mode=mode)
        for it in range(3):                                   # three calls exercise both buffer slots
            gen = torch.Generator(device="cpu").manual_seed(100 + it)
            xs = [torch.randn(M, Kl, generator=gen).to(torch.bfloat16) for _ in range(world)]
            ws = [(torch.randn(N, Kl, generator=gen) * 0.05).to(torch.bfloat16) for _ in range(world)]
            out = op(xs[rank].to(dev), ws[rank].to(dev))
            ref = gemm_reduce_scatter_reference(xs, ws, rank).to(dev)
            errs.append(float((out.float() - ref).norm() / ref.norm()))
    torch.cuda.synchronize()
    arena.ext.check_status()
    base.close()
    return errs


@pytest.mark.parametrize("world", WORLDS)
def test_fused_gemm_reduce_scatter(world: int) -> None:
    _need_gpus(world)
    for errs in run_distributed(_gemm_rs_worker, world):
        assert all(e < 1e-2 for e in errs), errs


def _ddp_symm_worker(rank: int, world: int, allreduce: str = "p2p"):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.parallel.ddp import DDP

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_parallel_gangs(base)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 257), torch.nn.ReLU(), torch.nn.Linear(257, 33)).to(dev)
    ddp = DDP(model, gangs, bucket_bytes=32 * 1024, comm="symm", average=True, allreduce=allreduce)
    assert ddp.arena is not None and len(ddp.buckets) >= 2
    if allreduce == "multimem" and ddp.arena.multicast_ptr == 0:
        base.close()
        return None                            # no NVSwitch multicast mapping on this box: nothing ran
    out = []
    for step in range(3):
        gen = torch.Generator().manual_seed(1000 * step + rank)
        x = torch.randn(16, 64, generator=gen).to(dev)
        ddp.zero_grad()
        ddp(x).square().sum().backward()
        ddp.finish_backward()
        torch.cuda.synchronize()
        # oracle: average of the per-rank gradients computed locally from every rank's input
        ref = [torch.zeros_like(p) for p in model.parameters()]
        for r in range(world):
            g2 = torch.Generator().manual_seed(1000 * step + r)
            xr = torch.randn(16, 64, generator=g2).to(dev)
            grads = torch.autograd.grad(model(xr).square().sum(), list(model.parameters()))
            for a, g in zip(ref, grads):
                a += g / world
        out.append(max(float((p.grad - a).abs().max() / a.abs().max().clamp(min=1e-6))
                       for p, a in zip(model.parameters(), ref)))
    ddp.arena.ext.check_status()
    base.close()
    return out


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("allreduce", ["p2p", "multimem"])
def test_ddp_symmetric_allreduce(allreduce: str, world: int) -> None:
    _need_gpus(world)
    results = run_distributed(_ddp_symm_worker, world, allreduce)
    if any(r is None for r in results):
        pytest.skip("the symmetric arena has no NVSwitch multicast mapping here: the multimem kernel did not run")
    for errs in results:
        assert len(errs) == 3 and all(e < 1e-5 for e in errs), errs


def _rs_adamw_worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.ops.optim import multi_tensor_adamw
    from fairseq2_b200.parallel.symm import SymmetricArena

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    n = 8 * 1024 + 64                       # shard elements (two segments)
    segs_off, segs_n = [0, 8 * 1024], [8 * 1024, 64]
    arena = SymmetricArena(base, 2 * world * n + (1 << 16))
    goff, full = arena.alloc_tensor(world * n, torch.bfloat16)
    gen = torch.Generator().manual_seed(7 + rank)
    full.copy_((torch.randn(world * n, generator=gen) * 0.1).to(torch.bfloat16))
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    torch.manual_seed(3)
    master0 = torch.randn(n, device=dev)
    errs = []
    # unfused: reduce-scatter into an fp32 shard, then the AdamW kernel
    m1, mm1, vv1 = master0.clone(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    low1 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    gshard = torch.empty(n, device=dev)
    arena.ext.comm_reducescatter_segments(arena.peer_ptrs, rank, segs_off, segs_n, goff, gshard, 1.0 / world, False,
                                          10, 1, 8, 5.0)
    multi_tensor_adamw([m1], [gshard], [mm1], [vv1], [low1], step=1, **hp)
    # fused
    m2, mm2, vv2 = master0.clone(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    low2 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    arena.ext.comm_reducescatter_adamw(arena.peer_ptrs, rank, segs_off, segs_n, goff, m2, mm2, vv2, low2, 1.0 / world,
                                       hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["weight_decay"], 1, 11, 1, 8,
                                       5.0)
    torch.cuda.synchronize()
    for a, b in ((m1, m2), (mm1, mm2), (vv1, vv2), (low1.float(), low2.float())):
        errs.append(float((a - b).abs().max()))
    arena.barrier(12, 1)
    torch.cuda.synchronize()
    arena.ext.check_status()
    base.close()
    return errs


@pytest.mark.parametrize("world", WORLDS)
def test_fused_reduce_scatter_adamw_matches_two_kernels(world: int) -> None:
    _need_gpus(world)
    for errs in run_distributed(_rs_adamw_worker, world):
        assert all(e < 1e-6 for e in errs), errs


def _ag_gemm_worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.ops.fused_collective import FusedAllGatherGemm
    from fairseq2_b200.parallel.symm import SymmetricArena

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    arena = SymmetricArena(base, (16 * world + 32) << 20)
    errs = []
    for gather, rows, other_rows, K in (("a", 512, 768, 1024), ("b", 512, 640, 1024)):
        op = FusedAllGatherGemm(arena, rows, K, gather=gather, num_copy_ctas=4)
        for it in range(2):
            gen = torch.Generator().manual_seed(50 + it)
            shards = [(torch.randn(rows, K, generator=gen) * 0.5).to(torch.bfloat16) for _ in range(world)]
            other = (torch.randn(other_rows, K, generator=gen) * 0.1).to(torch.bfloat16)
            op.shard.copy_(shards[rank])
            out = op(other.to(dev))
            full = torch.cat(shards).float().to(dev)
            ref = other.float().to(dev) @ full.t() if gather == "b" else full @ other.float().to(dev).t()
            errs.append(float((out.float() - ref).norm() / ref.norm()))
    arena.barrier(13, 1)
    torch.cuda.synchronize()
    arena.ext.check_status()
    base.close()
    return errs


@pytest.mark.parametrize("world", WORLDS)
def test_fused_allgather_gemm(world: int) -> None:
    _need_gpus(world)
    for errs in run_distributed(_ag_gemm_worker, world):
        assert all(e < 1e-2 for e in errs), errs


def _missing_peer_worker(rank: int, world: int):
    """Rank 1 withholds its signal for one barrier: rank 0's wait runs out after 0.3 s, the kernel records a status
    and returns, the host raises, and the context stays usable for a later barrier that everyone joins."""
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.parallel.symm import SymmetricArena

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    arena = SymmetricArena(base, 1 << 20, wait_limit_s=0.3)
    print(f"[missing-peer rank {rank}] arena ready", file=sys.stderr, flush=True)
    arena.barrier(20, 1)                       # everyone joins: passes
    torch.cuda.synchronize()
    arena.ext.check_status()
    print(f"[missing-peer rank {rank}] first barrier passed", file=sys.stderr, flush=True)
    detected = ""
    if rank == 0:
        arena.barrier(21, 1)                   # nobody else signals slot 21
        torch.cuda.synchronize()
        try:
            arena.ext.check_status()
        except Exception as ex:  # noqa: BLE001
            detected = str(ex)
    print(f"[missing-peer rank {rank}] after the withheld barrier", file=sys.stderr, flush=True)
    arena.wait_limit_s = 20.0                  # rank 1 gets here 0.3 s before rank 0
    arena.barrier(22, 1)                       # the GPU context still works on both ranks
    probe = torch.ones(4, device=dev).sum().item()
    torch.cuda.synchronize()
    arena.ext.check_status()
    print(f"[missing-peer rank {rank}] closing", file=sys.stderr, flush=True)
    base.close()
    print(f"[missing-peer rank {rank}] closed", file=sys.stderr, flush=True)
    return detected, probe


def test_bounded_wait_reports_missing_peer() -> None:
    _need_gpus(2)
    results = run_distributed(_missing_peer_worker, 2, timeout=60.0)
    assert "bounded wait" in results[0][0] and results[0][1] == 4.0 and results[1] == ("", 4.0)


def _moe_ep_worker(rank: int, world: int):
    """Expert-parallel MoE layer on 2 ranks against a single-rank layer that holds all experts: outputs for this
    rank's tokens, input gradients, and the gradients of this rank's experts and of the (replicated) router."""
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.models.transformer.experts import MoE
    from fairseq2_b200.ops.moe_ep import ExpertParallelExchange
    from fairseq2_b200.parallel.symm import SymmetricArena

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    D, F, E, K, T = 256, 512, 8, 2, 192
    arena = SymmetricArena(base, (4 * world + 8) << 20)
    ep = ExpertParallelExchange(arena, E, D, max_tokens=T, top_k=K)
    torch.manual_seed(0)
    full = MoE(D, F, True, E, 1.0, K, inner_dim_scale=1.0).to(dev, torch.bfloat16)
    torch.manual_seed(1)
    local = MoE(D, F, True, E, 1.0, K, inner_dim_scale=1.0, ep=ep).to(dev, torch.bfloat16)
    El = E // world
    with torch.no_grad():
        local.router.copy_(full.router)
        for name in ("gate_proj", "inner_proj", "output_proj"):
            getattr(local.experts, name).copy_(getattr(full.experts, name)[rank * El:(rank + 1) * El])
        local.shared_expert.load_state_dict(full.shared_expert.state_dict())
    errs = []
    for step in range(2):                                   # two rounds reuse inbox and outbox
        xs = [torch.randn(T, D, generator=torch.Generator().manual_seed(50 + 10 * step + r)).to(dev, torch.bfloat16)
              for r in range(world)]
        x_all = torch.cat(xs).requires_grad_(True)
        y_all = full(x_all)
        w_out = torch.randn(world * T, D, generator=torch.Generator().manual_seed(7 + step)).to(dev, torch.bfloat16)
        full.zero_grad()
        (y_all.float() * w_out.float()).sum().backward()
        x = xs[rank].clone().requires_grad_(True)
        y = local(x)
        local.zero_grad()
        (y.float() * w_out[rank * T:(rank + 1) * T].float()).sum().backward()
        sl = slice(rank * T, (rank + 1) * T)

        def rel(a, b):
            return float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-6))

        errs.append(rel(y, y_all[sl]))
        errs.append(rel(x.grad, x_all.grad[sl]))
        errs.append(rel(local.experts.output_proj.grad, full.experts.output_proj.grad[rank * El:(rank + 1) * El]))
        errs.append(rel(local.experts.gate_proj.grad, full.experts.gate_proj.grad[rank * El:(rank + 1) * El]))
    torch.cuda.synchronize()
    arena.ext.check_status()
    base.close()
    return errs


@pytest.mark.parametrize("world", WORLDS)
def test_moe_expert_parallel_matches_single_rank(world: int) -> None:
    _need_gpus(world)
    for errs in run_distributed(_moe_ep_worker, world):
        assert all(e < 3e-2 for e in errs), errs


def _sp_mlp_worker(rank: int, world: int):
    """Sequence-parallel tensor-parallel MLP (column -> GELU -> row) built from the fused kernels vs the same MLP on
    one rank: outputs for this rank's tokens, input gradient, both weight-gradient shards."""
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.ops.fused_collective import SequenceParallelLinears
    from fairseq2_b200.parallel.symm import SymmetricArena

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    Tl, D, F = 256, 256, 1024
    arena = SymmetricArena(base, (8 * world + 16) << 20)
    sp = SequenceParallelLinears(arena, Tl, D)
    gen = torch.Generator().manual_seed(3)
    w1 = (torch.randn(F, D, generator=gen) * D ** -0.5).to(dev, torch.bfloat16)
    w2 = (torch.randn(D, F, generator=gen) * F ** -0.5).to(dev, torch.bfloat16)
    Fl = F // world
    w1_l = w1[rank * Fl:(rank + 1) * Fl].clone().requires_grad_(True)          # column shard [F / W, D]
    w2_l = w2[:, rank * Fl:(rank + 1) * Fl].clone().contiguous().requires_grad_(True)   # row shard [D, F / W]
    errs = []
    for step in range(2):
        x = torch.randn(world * Tl, D, generator=torch.Generator().manual_seed(10 + step)).to(dev, torch.bfloat16)
        g = torch.randn(world * Tl, D, generator=torch.Generator().manual_seed(20 + step)).to(dev, torch.bfloat16)
        xs = x[rank * Tl:(rank + 1) * Tl].clone().requires_grad_(True)
        w1_l.grad = w2_l.grad = None
        y = sp.row(torch.nn.functional.gelu(sp.column(xs, w1_l)), w2_l)
        y.backward(g[rank * Tl:(rank + 1) * Tl])
        xr = x.float().requires_grad_(True)
        w1r, w2r = w1.float().requires_grad_(True), w2.float().requires_grad_(True)
        yr = torch.nn.functional.gelu(xr @ w1r.t()) @ w2r.t()
        yr.backward(g.float())

        def rel(a, b):
            return float((a.float() - b).norm() / b.norm().clamp(min=1e-6))

        sl = slice(rank * Tl, (rank + 1) * Tl)
        errs += [rel(y, yr[sl].detach()), rel(xs.grad, xr.grad[sl]), rel(w1_l.grad, w1r.grad[rank * Fl:(rank + 1) * Fl]),
                 rel(w2_l.grad, w2r.grad[:, rank * Fl:(rank + 1) * Fl])]
    torch.cuda.synchronize()
    arena.ext.check_status()
    base.close()
    return errs


@pytest.mark.parametrize("world", WORLDS)
def test_sequence_parallel_mlp_from_fused_kernels(world: int) -> None:
    _need_gpus(world)
    for errs in run_distributed(_sp_mlp_worker, world):
        assert all(e < 3e-2 for e in errs), errs


def _embed_push_worker(rank: int, world: int):
    """Vocabulary-parallel embedding whose rows are pushed to the token owners, against the plain lookup in fp32:
    this rank's tokens of the output and this rank's rows of the table gradient, over two calls (buffer turns)."""
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.ops.embedding import embed_vocab_parallel_scatter
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.parallel.tp import get_tp_context

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["FAIRSEQ2_B200_TP_ARENA_MB"] = "64"
    os.environ["FAIRSEQ2_B200_WAIT_LIMIT_S"] = "20"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    V, D, Tl = 1024, 256, 96
    rows = V // world
    gen = torch.Generator().manual_seed(5)
    table = torch.randn(V, D, generator=gen).to(dev, torch.bfloat16)
    shard = table[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    errs = []
    for call in range(3):
        g = torch.Generator().manual_seed(30 + call)
        ids = torch.randint(0, V, (world * Tl,), generator=g).to(dev)
        ids[::7] = ids[0]                                            # repeated tokens: the backward accumulates
        dout = torch.randn(world * Tl, D, generator=g).to(dev, torch.bfloat16)
        shard.grad = None
        y = embed_vocab_parallel_scatter(ids, shard, rank * rows, base)
        sl = slice(rank * Tl, (rank + 1) * Tl)
        y.backward(dout[sl])
        tr = table.float().requires_grad_(True)
        yr = torch.nn.functional.embedding(ids, tr)
        yr.backward(dout.float())
        errs.append(float((y.float() - yr[sl]).abs().max()))
        want = tr.grad[rank * rows:(rank + 1) * rows]
        errs.append(float((shard.grad.float() - want).norm() / want.norm()))
    used = get_tp_context(base).arena is not None
    torch.cuda.synchronize()
    require_ext().check_status()
    base.close()
    return errs, used


@pytest.mark.parametrize("world", WORLDS)
def test_vocab_parallel_embedding_push_matches_lookup(world: int) -> None:
    _need_gpus(world)
    for errs, used in run_distributed(_embed_push_worker, world):
        assert used
        assert all(e < 1e-2 for e in errs), errs


def _skipping_units_worker(rank: int, world: int, sharded: bool):
    """Ranks run DIFFERENT subsets of the layers in a step (LayerDrop with per-rank random numbers): the per-unit
    reductions must still pair up across ranks. Gradients after the reduction against the mean of the per-rank
    gradients of a plain copy of the model."""
    import torch.distributed as dist

    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.parallel.fsdp import FSDP

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["FAIRSEQ2_B200_DDP_ALLREDUCE"] = "p2p"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_parallel_gangs(root)
    if sharded:
        gangs = create_fsdp_gangs(gangs)

    class Net(torch.nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.inp = torch.nn.Linear(256, 256)
            self.layers = torch.nn.ModuleList(torch.nn.Linear(256, 256) for _ in range(6))
            self.skip: set[int] = set()

        def forward(self, x):  # type: ignore[no-untyped-def]
            x = self.inp(x)
            for i, layer in enumerate(self.layers):
                if i not in self.skip:
                    x = x + torch.tanh(layer(x))
            return x

    torch.manual_seed(0)
    plain = Net().to(dev)
    model = Net().to(dev)
    model.load_state_dict(plain.state_dict())
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16, wait_limit_s=20.0)
    errs = []
    # step 0: rank 0 drops {1, 4}, rank 1 drops {0, 4, 5}, others nothing; step 1: rank-dependent single drops
    plans = [{0: {1, 4}, 1: {0, 4, 5}}, {r: {(r + 2) % 6} for r in range(world)}]
    for step, plan in enumerate(plans):
        skip = plan.get(rank, set())
        model.skip = plain.skip = skip
        x = torch.randn(64, 256, generator=torch.Generator().manual_seed(10 * step + rank)).to(dev)
        fsdp.zero_grad()
        plain.zero_grad()
        fsdp(x.to(torch.bfloat16)).float().pow(2).mean().backward()
        fsdp.finish_backward()
        plain.to(torch.bfloat16)(x.to(torch.bfloat16)).float().pow(2).mean().backward()
        plain.float()
        want = {}
        for n, p in plain.named_parameters():
            g = (p.grad if p.grad is not None else torch.zeros_like(p)).float()
            dist.all_reduce(g)
            want[n] = g / world
        for u in fsdp.all_units:
            for sp in u.specs:
                if sp.rows_local == 0:
                    continue
                full = want[sp.fqn].reshape(sp.d0, sp.row)[u.rank * sp.chunk: u.rank * sp.chunk + sp.rows_local]
                got = u.grad_shard[sp.shard_off: sp.shard_off + sp.rows_local * sp.row].float().view(full.shape)
                if float(full.norm()) > 0:
                    errs.append(_rel(got, full))
                else:
                    errs.append(float(got.abs().max()))
    torch.cuda.synchronize()
    require_ext().check_status()
    root.close()
    return max(errs)


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("sharded", [False, True])
def test_ranks_running_different_units_reduce_in_one_order(world: int, sharded: bool) -> None:
    _need_gpus(world)
    for worst in run_distributed(_skipping_units_worker, world, sharded):
        assert worst < 2e-2, worst


# ------------------------------------------------------------------ whole-model checks against an fp32 oracle
def _small_llama_cfg():
    from fairseq2_b200.models.llama import LLaMAConfig

    return LLaMAConfig(model_dim=512, max_seq_len=4096, vocab_size=4096, num_layers=2, num_attn_heads=8,
                       num_key_value_heads=4, ffn_inner_dim=1536, ffn_inner_dim_scale=1.0,
                       ffn_inner_dim_multiple_of=1, rope_theta=500000.0, shard_embed_dim=False)


def _oracle_grads(cfg, batches, dev):
    """fp32 single-process gradients of the SUM of the per-batch losses (no TF32, no bf16, PyTorch formulations)."""
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.ops import _ext

    torch.backends.cuda.matmul.allow_tf32 = False
    torch.manual_seed(0)
    model = create_llama_model(cfg).to(dev)
    total = 0.0
    with _ext.kernels_enabled(False):
        for tokens, mask, lens in batches:
            layout = BatchLayout((tokens.numel() - 1,), lens, packed=True, device=dev)
            loss = model(tokens[:-1].to(dev), layout, targets=tokens[1:].to(dev), target_mask=mask.to(dev))
            loss.backward()
            total += float(loss)
    return total, {n: p.grad.detach() for n, p in model.named_parameters()}


def _make_batches(n: int, tokens_per_batch: int, vocab: int):
    import numpy as np

    from fairseq2_b200.datasets.synthetic import make_packed_sft_example

    out = []
    for r in range(n):
        ex = make_packed_sft_example(np.random.default_rng(77 + r), tokens_per_batch, vocab, doc_len_range=(64, 300),
                                     pin=False)
        out.append((ex.tokens, ex.target_mask, ex.seq_lens))
    return out


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12))


def _fsdp_grads_worker(rank: int, world: int, rs_engine: str):
    """Every rank's reduced gradient shard (bf16 model, symmetric-memory collectives) against the matching rows of
    the fp32 single-process gradient of the mean over the ranks' batches; also the fused norm partial."""
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.parallel.fsdp import FSDP

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["FAIRSEQ2_B200_FSDP_REDUCESCATTER"] = rs_engine
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_fsdp_gangs(create_parallel_gangs(root))
    cfg = _small_llama_cfg()
    batches = _make_batches(world, 1024, cfg.vocab_size)
    ref_loss, ref = _oracle_grads(cfg, batches, dev)
    torch.manual_seed(0)
    model = create_llama_model(cfg, gangs).to(dev)        # same construction order as the oracle: same weights
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16, comm="symm", wait_limit_s=20.0)
    tokens, mask, lens = batches[rank]
    layout = BatchLayout((1024,), lens, packed=True, device=dev)
    fsdp.zero_grad()
    loss = fsdp(tokens[:-1].to(dev), layout, targets=tokens[1:].to(dev), target_mask=mask.to(dev))
    loss.backward()
    fsdp.finish_backward()
    errs = {}
    norm_sq = torch.zeros((), device=dev)
    for u in fsdp.all_units:
        assert u.norm_fused, "the reduce-scatter pass did not emit the unit's norm"
        norm_sq += u.local_grad_norm_sq().float()
        for s in u.specs:
            if s.rows_local == 0:
                continue
            got = u.grad_shard[s.shard_off: s.shard_off + s.rows_local * s.row].view(s.rows_local, *s.shape[1:])
            want = ref[s.fqn].reshape(s.shape)[rank * s.chunk: rank * s.chunk + s.rows_local] / world
            errs[s.fqn] = _rel(got, want)
    want_sq = sum(float((g.reshape(-1) / world).pow(2).sum()) for g in ref.values())
    total_sq = norm_sq.clone()
    root.all_reduce(total_sq, __import__("fairseq2_b200.gang", fromlist=["x"]).ReduceOperation.SUM)
    torch.cuda.synchronize()
    require_ext().check_status()
    out = (max(errs.values()), max(errs, key=errs.get), abs(float(total_sq) - want_sq) / want_sq,
           float(loss), ref_loss)
    root.close()
    return out


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("rs_engine", ["kernel", "copy"])
def test_fsdp_full_gradients_match_fp32_single_rank(world: int, rs_engine: str) -> None:
    _need_gpus(world)
    for worst, name, norm_err, loss, _ in run_distributed(_fsdp_grads_worker, world, rs_engine):
        assert worst < 4e-2, (name, worst)
        assert norm_err < 2e-2, norm_err


def _fused_opt_worker(rank: int, world: int, fuse: bool):
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_fsdp_gangs(create_parallel_gangs(root))
    cfg = _small_llama_cfg()
    torch.manual_seed(0)
    with torch.device("meta"):
        model = create_llama_model(cfg, gangs)
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16, comm="symm", wait_limit_s=20.0)
    facade = DataParallelFacade(fsdp)
    opt = AdamW(fsdp.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)

    class Unit(TrainUnit):
        @property
        def model(self):
            return facade

        def count_targets(self, batch):
            return int(batch[1].sum())

        def process_batch(self, batch, metric_bag=None):
            tokens, mask, lens = batch
            layout = BatchLayout((1024,), lens, packed=True, device=dev)
            return fsdp(tokens[:-1].to(dev), layout, targets=tokens[1:].to(dev), target_mask=mask.to(dev)), \
                int(mask.sum())

    step = TrainStep(Unit(), opt, gangs, max_grad_norm=None, fuse_optimizer=fuse)
    losses = []
    for i in range(3):
        b = _make_batches(world * 3, 1024, cfg.vocab_size)[i * world + rank]
        loss, _ = step([b], i)
        losses.append(float(loss))
    armed = any(u.fused_step is not None or u.fused_done for u in fsdp.all_units)
    masters = torch.cat([u.master for u in fsdp.all_units]).cpu()
    steps = int(opt.state[fsdp.all_units[0].shard_params[0]]["step"])
    torch.cuda.synchronize()
    require_ext().check_status()
    root.close()
    return losses, masters.numpy(), steps, armed


@pytest.mark.parametrize("world", WORLDS)
def test_fsdp_fused_optimizer_matches_unfused(world: int) -> None:
    """The optimizer step inside the reduce-scatter kernel must leave the same weights as reduce-scatter followed
    by the AdamW kernel (same math in a different place; fp32 rounding of the gradient shard is the only gap)."""
    _need_gpus(world)
    fused = run_distributed(_fused_opt_worker, world, True)
    plain = run_distributed(_fused_opt_worker, world, False)
    for (lf, mf, sf, _), (lp, mp, sp, _) in zip(fused, plain):
        assert sf == sp == 3
        mf, mp = torch.from_numpy(mf), torch.from_numpy(mp)
        info = f"losses fused {lf} plain {lp}; max |dw| {float((mf - mp).abs().max()):.3e}, rel {_rel(mf, mp):.3e}"
        assert lf[0] == lp[0], info                      # identical weights and data before the first update
        # Adam turns a sign flip of a near-zero gradient into a full +-lr step, so single weights may differ by a
        # few lr after three steps; the bulk must agree
        assert float((mf - mp).abs().max()) < 8e-3 and _rel(mf, mp) < 2e-3, info
        for a, b in zip(lf, lp):
            assert abs(a - b) / abs(b) < 1e-2, info


def _ddp_accum_worker(rank: int, world: int, no_sync: bool, comm: str):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.parallel.ddp import DDP

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_parallel_gangs(base)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 257), torch.nn.ReLU(), torch.nn.Linear(257, 33)).to(dev)
    ddp = DDP(model, gangs, bucket_bytes=32 * 1024, comm=comm, average=True, allreduce="p2p")
    out = []
    for step in range(2):
        ddp.zero_grad()
        for mb in range(2):
            x = torch.randn(16, 64, generator=torch.Generator().manual_seed(100 * step + 10 * mb + rank)).to(dev)
            if no_sync and mb == 0:
                with ddp.no_sync():
                    ddp(x).square().sum().backward()
            else:
                ddp(x).square().sum().backward()
        ddp.finish_backward()
        torch.cuda.synchronize()
        out.append(torch.cat([p.grad.reshape(-1) for p in model.parameters()]).cpu().numpy())
    if ddp.arena is not None:
        ddp.arena.ext.check_status()
    base.close()
    return out


@pytest.mark.parametrize("no_sync", [False, True])
def test_ddp_symmetric_gradient_accumulation_matches_nccl(no_sync: bool) -> None:
    """Two micro-batches per step, with and without ``no_sync``: every reduction of a bucket has its own epoch, so
    the symmetric in-place all-reduce gives what NCCL gives."""
    _need_gpus(2)
    a = run_distributed(_ddp_accum_worker, 2, no_sync, "symm")
    b = run_distributed(_ddp_accum_worker, 2, no_sync, "nccl")
    for ra, rb in zip(a, b):
        for ga, gb in zip(ra, rb):
            assert _rel(torch.from_numpy(ga), torch.from_numpy(gb)) < 1e-5
    assert _rel(torch.from_numpy(a[0][1]), torch.from_numpy(a[1][1])) < 1e-6     # replicas agree


def _flat_ddp_worker(rank: int, world: int, comm: str):
    """Replicated data parallelism on flat units (the bf16 DDP of this framework): two optimizer steps."""
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["FAIRSEQ2_B200_DDP_ALLREDUCE"] = "p2p"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_parallel_gangs(root)                      # rdp = dp, nothing sharded
    cfg = _small_llama_cfg()
    torch.manual_seed(0)
    with torch.device("meta"):
        model = create_llama_model(cfg, gangs)
    ddp = FSDP(model, gangs, param_dtype=torch.bfloat16, comm=comm, wait_limit_s=20.0)
    assert (ddp.replica_arena is not None) == (comm == "symm")
    facade = DataParallelFacade(ddp)
    opt = AdamW(ddp.parameters(), lr=1e-3)

    class Unit(TrainUnit):
        @property
        def model(self):
            return facade

        def process_batch(self, batch, metric_bag=None):
            tokens, mask, lens = batch
            layout = BatchLayout((1024,), lens, packed=True, device=dev)
            return ddp(tokens[:-1].to(dev), layout, targets=tokens[1:].to(dev), target_mask=mask.to(dev)), \
                int(mask.sum())

    step = TrainStep(Unit(), opt, gangs, max_grad_norm=1.0)
    res = []
    for i in range(2):
        loss, gn = step([_make_batches(world * 2, 1024, cfg.vocab_size)[i * world + rank]], i)
        res.append((float(loss), float(gn)))
    masters = torch.cat([u.master for u in ddp.all_units]).cpu().numpy()
    torch.cuda.synchronize()
    require_ext().check_status()
    root.close()
    return res, masters


@pytest.mark.parametrize("world", WORLDS)
def test_flat_unit_ddp_symmetric_allreduce_matches_nccl(world: int) -> None:
    _need_gpus(world)
    a = run_distributed(_flat_ddp_worker, world, "symm")
    b = run_distributed(_flat_ddp_worker, world, "nccl")
    for (ra, ma), (rb, mb) in zip(a, b):
        for (la, ga), (lb, gb) in zip(ra, rb):
            assert abs(la - lb) / abs(lb) < 1e-3 and abs(ga - gb) / abs(gb) < 2e-2
        # the in-place kernel sums in fp32 and rounds once to bf16, NCCL reduces in bf16: single weights may end a
        # step on the other side of an Adam sign decision
        assert _rel(torch.from_numpy(ma), torch.from_numpy(mb)) < 2e-3
    assert _rel(torch.from_numpy(a[0][1]), torch.from_numpy(a[-1][1])) == 0.0     # replicas stay identical


def _tp_model_worker(rank: int, world: int, fused: bool):
    """A LLaMA model under tensor parallelism with sequence-parallel activations (column/row linears on the fused
    all-gather / reduce-scatter GEMMs): loss and every gradient against the fp32 single-process model."""
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.sharded import get_shard_dims
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.parallel.tp import get_tp_context, sequence_parallel

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["FAIRSEQ2_B200_TP_FUSED"] = "1" if fused else "0"
    os.environ["FAIRSEQ2_B200_TP_ARENA_MB"] = "256"
    os.environ["FAIRSEQ2_B200_WAIT_LIMIT_S"] = "20"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_fsdp_gangs(create_parallel_gangs(root, tp_size=world))
    cfg = _small_llama_cfg()
    T = 256 * world
    batches = _make_batches(1, T, cfg.vocab_size)
    ref_loss, ref = _oracle_grads(cfg, batches, dev)
    torch.manual_seed(0)
    with sequence_parallel():
        model = create_llama_model(cfg, gangs).to(dev)    # shards of the oracle's initialisation
    dims = get_shard_dims(model)
    fsdp = FSDP(model, gangs, param_dtype=torch.bfloat16)
    tokens, mask, lens = batches[0]
    layout = BatchLayout((T,), lens, packed=True, device=dev)
    fsdp.zero_grad()
    loss = fsdp(tokens[:-1].to(dev), layout, targets=tokens[1:].to(dev), target_mask=mask.to(dev))
    loss.backward()
    fsdp.finish_backward()
    used_fused = get_tp_context(gangs.tp).arena is not None
    errs = {}
    for u in fsdp.all_units:
        for s in u.specs:
            got = u.grad_shard[s.shard_off: s.shard_off + s.d0 * s.row].view(s.shape)
            want = ref[s.fqn]
            if s.fqn in dims:
                want = want.chunk(world, dim=dims[s.fqn])[rank]
            errs[s.fqn] = _rel(got, want)
    torch.cuda.synchronize()
    require_ext().check_status()
    out = (float(loss), ref_loss, max(errs.values()), max(errs, key=errs.get), used_fused)
    root.close()
    return out


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("fused", [True, False])
def test_tensor_parallel_llama_matches_fp32_single_rank(world: int, fused: bool) -> None:
    _need_gpus(world)
    for loss, ref_loss, worst, name, used_fused in run_distributed(_tp_model_worker, world, fused):
        assert used_fused == fused
        assert abs(loss - ref_loss) / abs(ref_loss) < 5e-3
        assert worst < 5e-2, (name, worst)


def _moe_ep_overflow_worker(rank: int, world: int):
    """An inbox that is too small: the layout cuts the expert ranges, the push kernel drops what does not fit and
    counts it -- nothing is written out of range, the status word stays clear, the step still runs both ways."""
    from fairseq2_b200.gang import ProcessGroupGang, ReduceOperation
    from fairseq2_b200.models.transformer.experts import MoE
    from fairseq2_b200.ops.moe_ep import ExpertParallelExchange
    from fairseq2_b200.parallel.symm import SymmetricArena

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    base = ProcessGroupGang.create_default_process_group(dev)
    D, F, E, K, T = 256, 512, 8, 2, 640
    El = E // world
    arena = SymmetricArena(base, (4 * world + 8) << 20, wait_limit_s=20.0)
    ep = ExpertParallelExchange(arena, E, D, max_tokens=T, top_k=K, capacity=0)      # one 128-row tile per expert
    assert ep.capacity == 128 * El
    torch.manual_seed(1)
    moe = MoE(D, F, False, E, 1.0, K, inner_dim_scale=1.0, ep=ep, softmax_gate=True, aux_loss=True,
              router_init_std=0.02).to(dev, torch.bfloat16)
    with torch.no_grad():                                       # every rank routes with the same router
        moe.router.copy_(torch.randn(D, E, generator=torch.Generator().manual_seed(5)).mul_(0.02))
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(50 + rank)).to(dev, torch.bfloat16)
    x.requires_grad_(True)
    moe.train()
    y = moe(x)
    (y.float().pow(2).sum() + moe.last_aux_loss).backward()
    # expected number of dropped rows, from the global routing counts
    logits = (x.detach().float() @ moe.router.detach().float())
    ids = torch.topk(logits, K, dim=1).indices.reshape(-1)
    counts = torch.bincount(ids, minlength=E).float()
    base.all_reduce(counts, ReduceOperation.SUM)
    expected = int(sum(max(int(c) - 128, 0) for c in counts.tolist()))
    dropped = ep.dropped.clone().float()
    base.all_reduce(dropped, ReduceOperation.SUM)
    torch.cuda.synchronize()
    arena.ext.check_status()
    out = (int(dropped), expected, bool(torch.isfinite(y).all()), bool(torch.isfinite(x.grad).all()),
           float(moe.last_aux_loss))
    base.close()
    return out


@pytest.mark.parametrize("world", WORLDS)
def test_moe_expert_parallel_overflow_is_dropped_and_counted(world: int) -> None:
    _need_gpus(world)
    for dropped, expected, y_ok, dx_ok, aux in run_distributed(_moe_ep_overflow_worker, world):
        assert expected > 0 and abs(dropped - expected) <= 4      # bf16 router logits may flip a near-tie
        assert y_ok and dx_ok and 0.9 < aux < 2.0
