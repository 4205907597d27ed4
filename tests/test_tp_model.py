"""Tensor parallelism on a whole LLaMA model over gloo ranks: a TP=2 (and TP=2 x FSDP=2) run with
sequence-parallel activations, and the reference-style TP with replicated activations, must train exactly like a
single process on the concatenated batch -- same losses, same parameters after two optimizer steps."""
from __future__ import annotations

import pytest
import torch

from tests.dist_utils import run_distributed


def _cfg():
    from fairseq2_b200.models.llama import get_llama_config

    cfg = get_llama_config("tiny")
    cfg.num_layers = 2
    cfg.vocab_size = 512
    cfg.shard_embed_dim = False
    return cfg


def _data(dp: int, steps: int):
    g = torch.Generator().manual_seed(21)
    return [[torch.randint(0, 512, (33,), generator=g) for _ in range(dp)] for _ in range(steps)]


def _reference(dp: int, steps: int):
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout

    torch.manual_seed(13)
    model = create_llama_model(_cfg())
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    losses = []
    for per_rank in _data(dp, steps):
        opt.zero_grad()
        n = sum(b.numel() - 1 for b in per_rank)
        tot = 0.0
        for b in per_rank:
            layout = BatchLayout((32,), [18, 14], packed=True)
            loss = model(b[:-1], layout, targets=b[1:])
            (loss / n).backward()
            tot += float(loss.detach())
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        losses.append(tot)
    return losses, {k: v.detach().clone() for k, v in model.state_dict().items()}


def _worker(rank: int, world: int, tp: int, sp: bool, steps: int):
    from fairseq2_b200.gang import ProcessGroupGang, ReduceOperation, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.nn.sharded import get_shard_dims
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP
    from fairseq2_b200.parallel.tp import sequence_parallel
    from fairseq2_b200.trainer import TrainStep, TrainUnit

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_fsdp_gangs(create_parallel_gangs(root, tp_size=tp))
    torch.manual_seed(13)
    with sequence_parallel(sp):
        model = create_llama_model(_cfg(), gangs)
    dims = get_shard_dims(model)
    fsdp = FSDP(model, gangs, param_dtype=torch.float32)
    facade = DataParallelFacade(fsdp)
    opt = AdamW(fsdp.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)

    class Unit(TrainUnit):
        @property
        def model(self):
            return facade

        def process_batch(self, batch, metric_bag=None):
            layout = BatchLayout((32,), [18, 14], packed=True)
            return fsdp(batch[:-1], layout, targets=batch[1:]), batch.numel() - 1

    step = TrainStep(Unit(), opt, gangs, max_grad_norm=1.0)
    losses = []
    for i, per_rank in enumerate(_data(gangs.dp.size, steps)):
        loss, _ = step([per_rank[gangs.dp.rank]], i)
        t = loss.clone()
        gangs.dp.all_reduce(t, ReduceOperation.SUM)
        losses.append(float(t))
    full = fsdp.full_state_dict()
    out = (gangs.tp.rank, gangs.dp.rank, losses, {k: v.numpy() for k, v in full.items()}, dims)
    root.close()
    return out


@pytest.mark.parametrize("world,tp,sp", [(2, 2, True), (2, 2, False), (4, 2, True)])
def test_tensor_parallel_training_matches_single_rank(world: int, tp: int, sp: bool) -> None:
    steps = 2
    dp = world // tp
    ref_losses, ref_sd = _reference(dp, steps)
    results = run_distributed(_worker, world, tp, sp, steps)
    by_tp = {}
    for tp_rank, dp_rank, losses, full, dims in results:
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) / abs(b) < 2e-4, (losses, ref_losses)
        if dp_rank == 0:
            by_tp[tp_rank] = (full, dims)
    dims = by_tp[0][1]
    for k, v in ref_sd.items():
        parts = [torch.from_numpy(by_tp[r][0][k]) for r in range(tp)]
        got = torch.cat(parts, dim=dims[k]) if k in dims else parts[0]
        if k not in dims:
            for p in parts[1:]:
                assert torch.allclose(p, parts[0], atol=1e-6), f"{k}: replicas over the tp gang differ"
        atol = 3e-3 if "embed" in k else 2e-4
        assert torch.allclose(got, v, atol=atol, rtol=1e-3), k


# ------------------------------------------------------------------ Gemma 3n
def _gemma_cfg():
    from dataclasses import replace

    from fairseq2_b200.models.gemma3n.config import gemma3n_tiny

    return replace(gemma3n_tiny(), num_kv_shared_layers=2, num_layers=6)


def _gemma_batches(steps: int):
    g = torch.Generator().manual_seed(5)
    return [torch.randint(1, 320, (2, 18), generator=g) for _ in range(steps)]


def _gemma_reference(steps: int):
    from fairseq2_b200.models.gemma3n import create_gemma3n_model
    from fairseq2_b200.nn import BatchLayout

    torch.manual_seed(17)
    model = create_gemma3n_model(_gemma_cfg())
    with torch.no_grad():                                    # zero-initialised upstream: would hide the AltUp scale
        for n, p in model.named_parameters():
            if "correct_output_scale" in n:
                p.fill_(0.3)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.0)
    losses = []
    for ids in _gemma_batches(steps):
        opt.zero_grad()
        loss = model(ids[:, :-1], BatchLayout.of(ids[:, :-1]), targets=ids[:, 1:], reduction="mean")
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    with torch.no_grad():
        logits = model(_gemma_batches(1)[0][:, :-1], BatchLayout.of(_gemma_batches(1)[0][:, :-1]))
    return losses, logits


def _gemma_worker(rank: int, world: int, steps: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.gemma3n import create_gemma3n_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.sharded import get_shard_dims

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root, tp_size=world)
    torch.manual_seed(17)
    model = create_gemma3n_model(_gemma_cfg(), gangs)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "correct_output_scale" in n:
                p.fill_(0.3)
    dims = get_shard_dims(model)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.0)
    losses = []
    for ids in _gemma_batches(steps):
        opt.zero_grad()
        loss = model(ids[:, :-1], BatchLayout.of(ids[:, :-1]), targets=ids[:, 1:], reduction="mean")
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    with torch.no_grad():
        logits = model(_gemma_batches(1)[0][:, :-1], BatchLayout.of(_gemma_batches(1)[0][:, :-1]))
    heads = (model.layers[0].self_attn.H, model.layers[0].self_attn.Hkv)
    root.close()
    return losses, logits.numpy(), dims, heads


def test_gemma3n_tensor_parallel_training_matches_single_rank() -> None:
    """Heads and the FFN inner dimension split over two ranks (including the layers with activation sparsity, whose
    cut-off needs moments over the whole inner dimension, and the layers that reuse earlier keys / values): losses of
    three optimizer steps and the logits afterwards equal the single-process model's."""
    steps = 3
    want_losses, want_logits = _gemma_reference(steps)
    for losses, logits, dims, heads in run_distributed(_gemma_worker, 2, steps, timeout=180.0):
        assert heads == (2, 1)
        assert losses == pytest.approx(want_losses, rel=2e-4)
        logits = torch.from_numpy(logits)
        assert torch.allclose(logits, want_logits, atol=2e-3), float((logits - want_logits).abs().max())
        assert dims["layers.0.self_attn.q_proj.weight"] == 0 and dims["layers.0.self_attn.o_proj.weight"] == 1
        assert dims["layers.1.mlp.gate_proj.weight"] == 0 and dims["layers.1.mlp.down_proj.weight"] == 1
        assert "layers.0.laurel.linear_left.weight" not in dims
    from fairseq2_b200.gang import FakeGang, Gangs
    from fairseq2_b200.models.gemma3n import create_gemma3n_model

    dev = torch.device("cpu")
    one = FakeGang(dev)
    four = Gangs(root=FakeGang(dev, rank=0, size=4), dp=one, rdp=one, sdp=one, tp=FakeGang(dev, rank=0, size=4), pp=one)
    with pytest.raises(ValueError, match="key-value heads"):
        create_gemma3n_model(_gemma_cfg(), four)


# ------------------------------------------------------------------ per-head q/k norms (Qwen 3) with replicated activations
def _qwen_cfg():  # type: ignore[no-untyped-def]
    from dataclasses import replace

    from fairseq2_b200.models.qwen.config import qwen_tiny

    return replace(qwen_tiny(), tied_embeddings=False)


def _qwen_train(model, steps: int):  # type: ignore[no-untyped-def]
    from fairseq2_b200.nn import BatchLayout

    with torch.no_grad():                                    # norm weights start at one: make their gradients matter
        for n, p in model.named_parameters():
            if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
                p.copy_(torch.linspace(0.5, 1.5, p.numel()))
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(3)
    losses = []
    for _ in range(steps):
        ids = torch.randint(0, 512, (2, 17), generator=g)
        opt.zero_grad()
        loss = model(ids[:, :-1], BatchLayout.of(ids[:, :-1]), targets=ids[:, 1:], reduction="mean")
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    norms = {n: p.detach().clone() for n, p in model.named_parameters() if "_norm.weight" in n and "self_attn" in n}
    return losses, norms


def _qwen_worker(rank: int, world: int, steps: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.qwen.factory import create_qwen_model
    from fairseq2_b200.parallel.tp import sequence_parallel

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root, tp_size=world)
    torch.manual_seed(23)
    with sequence_parallel(False):
        model = create_qwen_model(_qwen_cfg(), gangs)
    losses, norms = _qwen_train(model, steps)
    root.close()
    return losses, {k: v.numpy() for k, v in norms.items()}


def test_per_head_norm_weights_get_the_whole_gradient_under_tensor_parallelism() -> None:
    """Qwen 3 normalises every query / key head with one shared weight vector. With the heads split over two ranks and
    replicated activations each rank computes the gradient of its own heads only; the weight must still move as in
    the single-process model, and identically on both ranks."""
    from fairseq2_b200.models.qwen.factory import create_qwen_model

    torch.manual_seed(23)
    want_losses, want_norms = _qwen_train(create_qwen_model(_qwen_cfg()), 3)
    results = run_distributed(_qwen_worker, 2, 3, timeout=180.0)
    for losses, norms in results:
        assert losses == pytest.approx(want_losses, rel=1e-4)
        for k, v in want_norms.items():
            assert torch.allclose(torch.from_numpy(norms[k]), v, atol=1e-5), k


# ------------------------------------------------------------------ FFN with activation sparsity
def _altup_ffn_worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.transformer.ffn import AltUpFeedForwardNetwork

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root, tp_size=world)
    torch.manual_seed(4)
    ffn = AltUpFeedForwardNetwork(32, 96, bias=True, activation_sparsity=0.7, gangs=gangs)
    x = torch.randn(5, 32, generator=torch.Generator().manual_seed(8), requires_grad=True)
    y = ffn(x)
    y.pow(2).sum().backward()
    out = (y.detach().numpy(), x.grad.numpy(), ffn.output_proj.bias.grad.numpy(), gangs.tp.rank,
           ffn.gate_proj.weight.grad.numpy())
    root.close()
    return out


def test_altup_ffn_activation_sparsity_under_tensor_parallelism() -> None:
    """The cut-off of the Gaussian top-k is a statistic over the whole inner dimension: with the dimension split
    over two ranks, outputs, input gradients and weight gradients equal the unsplit module's."""
    from fairseq2_b200.models.transformer.ffn import AltUpFeedForwardNetwork, gaussian_topk

    torch.manual_seed(4)
    ffn = AltUpFeedForwardNetwork(32, 96, bias=True, activation_sparsity=0.7)
    x = torch.randn(5, 32, generator=torch.Generator().manual_seed(8), requires_grad=True)
    y = ffn(x)
    y.pow(2).sum().backward()
    for got_y, got_dx, got_db, tp_rank, got_dw in run_distributed(_altup_ffn_worker, 2, timeout=120.0):
        assert torch.allclose(torch.from_numpy(got_y), y.detach(), atol=1e-5)
        assert torch.allclose(torch.from_numpy(got_dx), x.grad, atol=1e-4)
        assert torch.allclose(torch.from_numpy(got_db), ffn.output_proj.bias.grad, atol=1e-4)
        assert torch.allclose(torch.from_numpy(got_dw), ffn.gate_proj.weight.grad[tp_rank * 48:(tp_rank + 1) * 48], atol=1e-4)
    g = torch.randn(1000, 512)
    kept = (gaussian_topk(g, 0.9) > 0).float().mean()
    assert 0.08 < float(kept) < 0.12                       # about a tenth of a normal sample survives
    with pytest.raises(ValueError):
        AltUpFeedForwardNetwork(8, 8, False, activation_sparsity=1.0)


# ------------------------------------------------------------------ LLaMA 4 (MoE layers with tensor-parallel experts)
def _llama4_train(model, steps: int):  # type: ignore[no-untyped-def]
    from fairseq2_b200.nn import BatchLayout

    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(6)
    losses = []
    for _ in range(steps):
        ids = torch.randint(1, 500, (2, 41), generator=g)
        layout = BatchLayout((2, 40), [40, 33])
        opt.zero_grad()
        loss = model(ids[:, :-1], layout, targets=ids[:, 1:], reduction="mean")
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses


def _llama4_worker(rank: int, world: int, steps: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.llama4.config import llama4_tiny
    from fairseq2_b200.models.llama4.factory import create_llama4_model
    from fairseq2_b200.parallel.tp import sequence_parallel

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root, tp_size=world)
    from fairseq2_b200.nn.sharded import get_shard_dims

    with sequence_parallel(False):
        model = create_llama4_model(llama4_tiny(), gangs)
    # the same weights as the single-process model: its state, cut along every parameter's tensor-parallel dimension
    torch.manual_seed(29)
    full = create_llama4_model(llama4_tiny()).state_dict()
    dims = get_shard_dims(model)
    own = model.state_dict()
    assert set(own) == set(full)
    with torch.no_grad():
        for k, v in own.items():
            src = full[k]
            if k in dims:
                src = src.chunk(world, dim=dims[k])[gangs.tp.rank]
            assert src.shape == v.shape, (k, tuple(src.shape), tuple(v.shape))
            v.copy_(src)
    losses = _llama4_train(model, steps)
    root.close()
    return losses, sorted(dims)


def test_llama4_tensor_parallel_training_matches_single_rank() -> None:
    """Dense and MoE layers (router, routed experts and the shared expert split over the inner dimension), chunked
    and NoPE attention, q/k norms without weights: three SGD steps on two ranks give the single-process losses."""
    from fairseq2_b200.models.llama4.config import llama4_tiny
    from fairseq2_b200.models.llama4.factory import create_llama4_model

    torch.manual_seed(29)
    want = _llama4_train(create_llama4_model(llama4_tiny()), 3)
    for losses, sharded in run_distributed(_llama4_worker, 2, 3, timeout=180.0):
        assert losses == pytest.approx(want, rel=2e-4)
        assert any("experts" in k for k in sharded) and any("shared_expert" in k for k in sharded)


def test_sequence_parallel_model_is_refused_by_the_bucketed_ddp_wrapper() -> None:
    """Token-sharded activations leave partial gradients on replicated parameters; only the flat-unit engine sums
    them over the tensor-parallel gang, so the bucketed wrapper must not accept such a model silently."""
    from fairseq2_b200.error import NotSupportedError
    from fairseq2_b200.gang import FakeGang, Gangs
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.parallel.ddp import DDP
    from fairseq2_b200.parallel.tp import sequence_parallel

    dev = torch.device("cpu")
    one = FakeGang(dev)
    gangs = Gangs(root=FakeGang(dev, rank=0, size=4), dp=FakeGang(dev, rank=0, size=2), rdp=FakeGang(dev, rank=0, size=2),
                  sdp=one, tp=FakeGang(dev, rank=0, size=2), pp=one)
    with sequence_parallel(True):
        model = create_llama_model(_cfg(), gangs)
    with pytest.raises(NotSupportedError, match="sequence-parallel"):
        DDP(model, gangs, broadcast_parameters=False)
    with sequence_parallel(False):
        plain = create_llama_model(_cfg(), gangs)
    DDP(plain, gangs, broadcast_parameters=False)


def _clip_worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.utils.grad import clip_grad_norm
    from fairseq2_b200.parallel.tp import sequence_parallel

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root, tp_size=world)
    torch.manual_seed(13)
    with sequence_parallel(False):
        model = create_llama_model(_cfg(), gangs)
    b = _data(1, 1)[0][0]
    model(b[:-1], BatchLayout((32,), [18, 14], packed=True), targets=b[1:]).backward()
    total = float(clip_grad_norm(model, 1.0))
    after = float(clip_grad_norm(model, None))
    norm_w = model.decoder.layers[0].self_attn_layer_norm.weight.grad.clone().numpy()
    root.close()
    return total, after, norm_w


def test_gradient_clipping_of_a_tensor_parallel_model_uses_the_whole_model_norm() -> None:
    """Without a data-parallel wrapper: both ranks must arrive at the single-process norm (split parameters summed
    over the gang, replicated ones counted once) and scale by the same factor."""
    from fairseq2_b200.models.llama import create_llama_model
    from fairseq2_b200.nn import BatchLayout

    torch.manual_seed(13)
    model = create_llama_model(_cfg())
    b = _data(1, 1)[0][0]
    model(b[:-1], BatchLayout((32,), [18, 14], packed=True), targets=b[1:]).backward()
    want = float(torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0))
    want_w = model.decoder.layers[0].self_attn_layer_norm.weight.grad
    assert want > 1.0
    for total, after, norm_w in run_distributed(_clip_worker, 2, timeout=120.0):
        assert total == pytest.approx(want, rel=1e-4) and after == pytest.approx(1.0, rel=1e-3)
        assert torch.allclose(torch.from_numpy(norm_w), want_w, rtol=1e-3, atol=1e-7)


# ------------------------------------------------------------------ OLMo 2 (q/k norms that span all heads)
def _olmo_train(model, steps: int):  # type: ignore[no-untyped-def]
    from fairseq2_b200.nn import BatchLayout

    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
                p.copy_(torch.linspace(0.5, 1.5, 128)[: p.numel()] if p.numel() == 128 else
                        torch.linspace(0.5, 1.5, 128).chunk(2)[_olmo_train.rank])
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(11)
    losses = []
    for _ in range(steps):
        ids = torch.randint(1, 512, (2, 25), generator=g)
        opt.zero_grad()
        loss = model(ids[:, :-1], BatchLayout.of(ids[:, :-1]), targets=ids[:, 1:], reduction="mean")
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses


_olmo_train.rank = 0  # type: ignore[attr-defined]


def _olmo_worker(rank: int, world: int, steps: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.olmo.config import olmo_tiny
    from fairseq2_b200.models.olmo.factory import create_olmo_model
    from fairseq2_b200.nn.sharded import get_shard_dims
    from fairseq2_b200.parallel.tp import sequence_parallel

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_parallel_gangs(root, tp_size=world)
    torch.manual_seed(31)
    with sequence_parallel(False):
        model = create_olmo_model(olmo_tiny(), gangs)
    _olmo_train.rank = gangs.tp.rank  # type: ignore[attr-defined]
    dims = get_shard_dims(model)
    q_norm_shape = tuple(model.decoder.layers[0].self_attn.q_norm.weight.shape)
    losses = _olmo_train(model, steps)
    root.close()
    return losses, dims.get("decoder.layers.0.self_attn.q_norm.weight"), q_norm_shape


def test_olmo_norms_over_all_heads_under_tensor_parallelism() -> None:
    """OLMo 2 normalises the whole query / key projection. With the heads split over two ranks every rank holds
    half of the vector and of the norm weight; the mean of squares is taken over both halves."""
    from fairseq2_b200.gang import create_fake_gangs
    from fairseq2_b200.models.olmo.config import olmo_tiny
    from fairseq2_b200.models.olmo.factory import create_olmo_model

    torch.manual_seed(31)
    _olmo_train.rank = 0  # type: ignore[attr-defined]
    want = _olmo_train(create_olmo_model(olmo_tiny(), create_fake_gangs(torch.device("cpu"))), 3)
    for losses, dim, shape in run_distributed(_olmo_worker, 2, 3, timeout=180.0):
        assert dim == 0 and shape == (64,)
        assert losses == pytest.approx(want, rel=2e-4)
