"""Multi-rank (gloo, CPU) numerics of the FSDP and DDP engines against
single-process training of the same model on the concatenated batch."""
from __future__ import annotations

import copy

import pytest
import torch

from tests.dist_utils import run_distributed


def _build(num_layers: int = 2):
    from fairseq2_b200.models.llama import create_llama_model, get_llama_config

    cfg = get_llama_config("tiny")
    cfg.num_layers = num_layers
    torch.manual_seed(7)
    return cfg, create_llama_model(cfg)


def _data(world: int, steps: int):
    g = torch.Generator().manual_seed(11)
    return [[torch.randint(0, 8192, (2, 24), generator=g) for _ in range(world)] for _ in range(steps)]


def _single_rank_reference(world: int, steps: int):
    from fairseq2_b200.nn import BatchLayout

    _, model = _build()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    losses = []
    for batch_per_rank in _data(world, steps):
        opt.zero_grad()
        total = 0.0
        ntgt = sum(b.numel() for b in batch_per_rank)
        for b in batch_per_rank:
            loss = model(b, BatchLayout.of(b), targets=b)
            (loss / ntgt).backward()
            total += float(loss)
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        losses.append(total)
    return losses, {k: v.detach().clone() for k, v in model.state_dict().items()}


def _fsdp_worker(rank: int, world: int, steps: int, kind: str):
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.ddp import DDP
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    dev = torch.device("cpu")
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_parallel_gangs(root)
    _, model = _build()
    if kind == "fsdp":
        gangs = create_fsdp_gangs(gangs)
        wrapped = FSDP(model, gangs, param_dtype=torch.float32)
        opt = AdamW(wrapped.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    else:
        wrapped = DDP(model, gangs)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    facade = DataParallelFacade(wrapped)

    class Unit(TrainUnit):
        @property
        def model(self):
            return facade

        def process_batch(self, batch, metric_bag=None):
            return wrapped(batch, BatchLayout.of(batch), targets=batch), batch.numel()

    step = TrainStep(Unit(), opt, gangs, max_grad_norm=1.0)
    losses = []
    for i, per_rank in enumerate(_data(world, steps)):
        loss, _ = step([per_rank[rank]], i)
        t = loss.clone()
        root.all_reduce(t, __import__("fairseq2_b200.gang", fromlist=["ReduceOperation"]).ReduceOperation.SUM)
        losses.append(float(t))
    if kind == "fsdp":
        full = wrapped.full_state_dict()
        local = {k: v.clone() for k, v in wrapped.state_dict().items()}
    else:
        full = {k: v.detach().clone() for k, v in model.state_dict().items()}
        local = full
    root.close()
    # numpy arrays pickle by value (tensors would be passed as shared-memory handles that die with the child)
    return losses, {k: v.numpy() for k, v in full.items()}, {k: tuple(v.shape) for k, v in local.items()}


@pytest.mark.parametrize("kind", ["fsdp", "ddp"])
def test_two_rank_training_matches_single_rank(kind: str) -> None:
    world, steps = 2, 3
    ref_losses, ref_sd = _single_rank_reference(world, steps)
    results = run_distributed(_fsdp_worker, world, steps, kind)
    for losses, full, shapes in results:
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) / abs(b) < 1e-4
        for k, v in ref_sd.items():
            # Adam normalises the update, so rows with near-zero gradients (rare tokens of the
            # embedding) amplify fp32 summation-order noise up to lr * steps
            atol = 3e-3 if "embed" in k else 1e-4
            assert torch.allclose(torch.from_numpy(full[k]), v, atol=atol, rtol=1e-4), k
    if kind == "fsdp":
        # local state dict = dim-0 shards, as FSDP2's DTensor.to_local() would give
        _, _, shapes = results[0]
        assert shapes["decoder.layers.0.self_attn.q_proj.weight"] == (128, 256)
        assert shapes["decoder_frontend.embed.weight"] == (4096, 256)


def _sync_bn_worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.parallel.ddp import convert_batch_norms

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root)
    with_bn = torch.nn.Sequential(torch.nn.Conv1d(2, 2, 1), torch.nn.BatchNorm1d(2))
    without = torch.nn.Sequential(torch.nn.Linear(2, 2), torch.nn.LayerNorm(2))
    a, b = convert_batch_norms(with_bn, gangs), convert_batch_norms(without, gangs)
    root.barrier()
    return type(a[1]).__name__, b is without


def test_ddp_converts_batch_norms_to_sync_batch_norm() -> None:
    """Buffers are not broadcast during training, so batch norms must reduce their statistics over the gang."""
    for name, untouched in run_distributed(_sync_bn_worker, 2):
        assert name == "SyncBatchNorm" and untouched


def _accum_worker(rank: int, world: int, kind: str, no_sync: bool):
    """Two micro-batches per step: the result must equal one step over the four batches of both ranks."""
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.ddp import DDP
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root)
    _, model = _build()
    if kind == "fsdp":
        gangs = create_fsdp_gangs(gangs)
        wrapped = FSDP(model, gangs, param_dtype=torch.float32)
        opt = AdamW(wrapped.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    else:
        wrapped = DDP(model, gangs)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    facade = DataParallelFacade(wrapped)

    class Unit(TrainUnit):
        @property
        def model(self):
            return facade

        def process_batch(self, batch, metric_bag=None):
            return wrapped(batch, BatchLayout.of(batch), targets=batch), batch.numel()

    step = TrainStep(Unit(), opt, gangs, max_grad_norm=1.0, no_sync=no_sync)
    data = _data(2 * world, 2)
    for i, per_slot in enumerate(data):
        step([per_slot[2 * rank], per_slot[2 * rank + 1]], i)
    full = wrapped.full_state_dict() if kind == "fsdp" else {k: v.detach().clone() for k, v in model.state_dict().items()}
    root.close()
    return {k: v.numpy() for k, v in full.items()}


@pytest.mark.parametrize("kind", ["ddp", "fsdp"])
@pytest.mark.parametrize("no_sync", [False, True])
def test_gradient_accumulation_matches_one_big_step(kind: str, no_sync: bool) -> None:
    world = 2
    _, ref_sd = _single_rank_reference(2 * world, 2)
    for full in run_distributed(_accum_worker, world, kind, no_sync):
        for k, v in ref_sd.items():
            atol = 3e-3 if "embed" in k else 1e-4
            assert torch.allclose(torch.from_numpy(full[k]), v, atol=atol, rtol=1e-4), k


def test_fsdp_frozen_parameter_is_untouched_by_the_optimizer() -> None:
    """A parameter without a gradient gets no weight decay and no moment update (``torch.optim.AdamW`` skips
    parameters whose ``grad`` is None); the flat-unit launch must do the same."""
    from fairseq2_b200.gang import create_fake_gangs
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP

    _, model = _build()
    model.decoder.layers[0].ffn.gate_proj.weight.requires_grad_(False)
    before = model.decoder.layers[0].ffn.gate_proj.weight.detach().clone()
    other = model.decoder.layers[0].ffn.output_proj.weight.detach().clone()
    fsdp = FSDP(model, create_fake_gangs(torch.device("cpu")), param_dtype=torch.float32)
    opt = AdamW(fsdp.parameters(), lr=1e-2, weight_decay=0.5)
    b = _data(1, 1)[0][0]
    for _ in range(2):
        fsdp.zero_grad()
        loss = fsdp(b, BatchLayout.of(b), targets=b)
        loss.backward()
        fsdp.finish_backward()
        opt.step()
        fsdp.after_optimizer_step()
    sd = fsdp.full_state_dict()
    assert torch.equal(sd["decoder.layers.0.ffn.gate_proj.weight"], before)
    assert not torch.equal(sd["decoder.layers.0.ffn.output_proj.weight"], other)


def test_fsdp_replica_only_layout_reduces_over_the_replica_gang() -> None:
    """With one shard rank and several replicas the gradients still have to be averaged over the replicas."""
    from fairseq2_b200.gang import FakeGang, Gangs
    from fairseq2_b200.parallel.fsdp import FSDP

    dev = torch.device("cpu")
    root = FakeGang(dev, rank=0, size=2)
    gangs = Gangs(root=root, dp=root, rdp=root, sdp=FakeGang(dev), tp=FakeGang(dev), pp=FakeGang(dev))
    _, model = _build()
    fsdp = FSDP(model, gangs, param_dtype=torch.float32)
    assert fsdp.replica_gang is root and fsdp.gang.size == 1


def _skipping_units_cpu_worker(rank: int, world: int, sharded: bool):
    """Ranks run different subsets of the layers (LayerDrop with per-rank random numbers): the per-unit gradient
    reductions are blocking collectives, so they only complete if every rank issues them in the same order."""
    import torch.distributed as dist

    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.parallel.fsdp import FSDP

    dev = torch.device("cpu")
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_parallel_gangs(root)
    if sharded:
        gangs = create_fsdp_gangs(gangs)

    class Net(torch.nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.inp = torch.nn.Linear(16, 16)
            self.layers = torch.nn.ModuleList(torch.nn.Linear(16, 16) for _ in range(6))
            self.skip: set[int] = set()

        def forward(self, x):  # type: ignore[no-untyped-def]
            x = self.inp(x)
            for i, layer in enumerate(self.layers):
                if i not in self.skip:
                    x = x + torch.tanh(layer(x))
            return x

    torch.manual_seed(0)
    plain = Net()
    model = Net()
    model.load_state_dict(plain.state_dict())
    fsdp = FSDP(model, gangs, param_dtype=torch.float32)
    worst = 0.0
    plans = [{0: {1, 4}, 1: {0, 4, 5}}, {0: {0, 1, 2, 3, 4, 5}, 1: set()}, {0: {5}, 1: {0}}]
    for step, plan in enumerate(plans):
        model.skip = plain.skip = plan.get(rank, set())
        x = torch.randn(8, 16, generator=torch.Generator().manual_seed(10 * step + rank))
        fsdp.zero_grad()
        plain.zero_grad()
        fsdp(x).pow(2).mean().backward()
        fsdp.finish_backward()
        plain(x).pow(2).mean().backward()
        for u in fsdp.all_units:
            for sp in u.specs:
                if sp.rows_local == 0:
                    continue
                p = dict(plain.named_parameters())[sp.fqn]
                g = (p.grad if p.grad is not None else torch.zeros_like(p)).clone()
                dist.all_reduce(g)
                want = (g / world).reshape(sp.d0, sp.row)[u.rank * sp.chunk: u.rank * sp.chunk + sp.rows_local]
                got = u.grad_shard[sp.shard_off: sp.shard_off + sp.rows_local * sp.row].view(want.shape)
                worst = max(worst, float((got - want).abs().max()))
    root.close()
    return worst


def test_ranks_running_different_units_reduce_in_one_order() -> None:
    """Replicated units only: with sharded units over process-group collectives the forward all-gathers are
    collectives too, and ranks that skip different layers cannot pair them up (as with torch's FSDP); over the
    symmetric arena the all-gathers are one-sided and the sharded case works (GPU test of the same name)."""
    for worst in run_distributed(_skipping_units_cpu_worker, 2, False, timeout=120.0):
        assert worst < 1e-5, worst


def _odd_shapes_worker(rank: int, world: int, intra: int | None = None):
    """Parameters whose rows do not divide evenly, and whose per-rank piece is smaller than the alignment of the
    flat buffers (a bias of 40 over 3 ranks): outputs, reduced gradients and the gathered state must equal a plain
    copy of the model. Some ranks own no row of the small parameters."""
    import torch.distributed as dist

    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP

    dev = torch.device("cpu")
    root = ProcessGroupGang.create_default_process_group(dev)
    gangs = create_fsdp_gangs(create_parallel_gangs(root), intra)      # `intra`: hybrid, shards inside groups of it

    class Net(torch.nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.inp = torch.nn.Linear(24, 40)
            self.layers = torch.nn.ModuleList(torch.nn.Linear(40, 40) for _ in range(2))
            self.scale = torch.nn.Parameter(torch.ones(5, 3, 7))           # 21 elements per row

        def forward(self, x):  # type: ignore[no-untyped-def]
            x = self.inp(x)
            for layer in self.layers:
                x = x + torch.tanh(layer(x))
            return x * self.scale.sum()

    torch.manual_seed(0)
    plain = Net()
    model = Net()
    model.load_state_dict(plain.state_dict())
    fsdp = FSDP(model, gangs, param_dtype=torch.float32)
    layout = {s.fqn: (s.chunk, s.row, s.shard_numel, s.rows_local) for u in fsdp.all_units for s in u.specs}
    opt = AdamW(fsdp.parameters(), lr=1e-2, weight_decay=0.0)
    ref_opt = torch.optim.AdamW(plain.parameters(), lr=1e-2, weight_decay=0.0)
    out = {"layout": layout, "fwd": 0.0, "grad": 0.0, "state": 0.0}
    for step in range(2):
        x = torch.randn(8, 24, generator=torch.Generator().manual_seed(10 * step + rank))
        fsdp.zero_grad()
        plain.zero_grad()
        y, yp = fsdp(x), plain(x)
        out["fwd"] = max(out["fwd"], float((y - yp).abs().max()))
        y.pow(2).mean().backward()
        fsdp.finish_backward()
        yp.pow(2).mean().backward()
        want = {}
        for n, p in plain.named_parameters():
            g = p.grad.clone()
            dist.all_reduce(g)
            p.grad = g / world
            want[n] = p.grad
        for u in fsdp.all_units:
            for sp in u.specs:
                if sp.rows_local == 0:
                    continue
                w = want[sp.fqn].reshape(sp.d0, sp.row)[u.rank * sp.chunk: u.rank * sp.chunk + sp.rows_local]
                got = u.grad_shard[sp.shard_off: sp.shard_off + sp.rows_local * sp.row].view(w.shape)
                out["grad"] = max(out["grad"], float((got - w).abs().max()))
        opt.step()
        fsdp.after_optimizer_step()
        ref_opt.step()
        full = fsdp.full_state_dict()
        for n, p in plain.named_parameters():
            out["state"] = max(out["state"], float((full[n] - p.detach()).abs().max()))
    root.close()
    return out


@pytest.mark.parametrize("world,intra", [(2, None), (3, None), (4, 2)])
def test_shards_smaller_than_the_buffer_alignment(world: int, intra: int | None) -> None:
    outs = run_distributed(_odd_shapes_worker, world, intra, timeout=120.0)
    for out in outs:
        assert out["fwd"] < 1e-4 and out["grad"] < 1e-3 and out["state"] < 1e-5, out   # outputs are O(100)
        for chunk, row, shard_numel, _ in out["layout"].values():
            assert shard_numel == chunk * row and shard_numel % 64 == 0      # no padding inside a gathered region
    # the 40-element bias: 64 rows per rank after rounding, so one rank of every shard group owns all of it
    assert sum(1 for o in outs if o["layout"]["layers.0.bias"][3] > 0) == world // (intra or world)
