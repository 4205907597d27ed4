"""Mixture-of-experts LM family on CPU: load-balancing loss against its definition, softmax gates, the model's
objective, and training with the experts as rank-local FSDP units."""
from __future__ import annotations

import torch

from fairseq2_b200.models.moe_lm import create_moe_lm_model
from fairseq2_b200.models.moe_lm.config import tiny
from fairseq2_b200.nn import BatchLayout


def test_load_balancing_loss_definition() -> None:
    from fairseq2_b200.ops.moe import load_balancing_loss

    torch.manual_seed(0)
    T, E, k = 64, 8, 2
    logits = torch.randn(T, E, requires_grad=True)
    ids = torch.topk(logits, k, dim=1).indices
    counts = torch.bincount(ids.reshape(-1), minlength=E)
    aux = load_balancing_loss(logits, counts, k)
    f = counts.float() / (T * k)
    p = torch.softmax(logits, -1).mean(0)
    assert torch.allclose(aux, E * (f * p).sum())
    aux.backward()
    assert logits.grad is not None and float(logits.grad.abs().sum()) > 0
    # a uniform router scores exactly 1
    uni = load_balancing_loss(torch.zeros(T, E), torch.full((E,), T * k // E), k)
    assert abs(float(uni) - 1.0) < 1e-6


def test_softmax_gates_sum_to_one_and_model_adds_aux_term() -> None:
    from fairseq2_b200.models.transformer.experts import route_tokens

    logits = torch.randn(10, 8)
    tok, gates, order, sizes = route_tokens(logits, 3, softmax_gate=True)
    per_token = torch.zeros(10).index_add(0, tok, gates)
    assert torch.allclose(per_token, torch.ones(10), atol=1e-6) and sum(sizes) == 30
    torch.manual_seed(0)
    cfg = tiny()
    m = create_moe_lm_model(cfg)
    x = torch.randint(0, cfg.vocab_size, (2, 17))
    inp, tgt = x[:, :-1], x[:, 1:]
    m.train()
    with_aux = float(m(inp, BatchLayout.of(inp), targets=tgt))
    aux = torch.stack([l.ffn.last_aux_loss for l in m.decoder.layers]).mean()
    m.aux_loss_coef = 0.0
    without = float(m(inp, BatchLayout.of(inp), targets=tgt))
    assert abs((with_aux - without) - cfg.aux_loss_coef * float(aux) * tgt.numel()) < 1e-2


def test_training_with_rank_local_expert_units() -> None:
    from fairseq2_b200.gang import create_fake_gangs
    from fairseq2_b200.models.transformer.experts import GroupedExpertNetwork
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP

    torch.manual_seed(0)
    cfg = tiny()
    with torch.device("meta"):
        model = create_moe_lm_model(cfg)
    fsdp = FSDP(model, create_fake_gangs(torch.device("cpu")), param_dtype=torch.float32,
                local_module_filter=lambda m: isinstance(m, GroupedExpertNetwork))
    assert len(fsdp.local_units) == cfg.num_layers and all(u.local_only for u in fsdp.local_units)
    names = dict(fsdp.named_parameters())
    assert "decoder.layers.0.ffn.experts.gate_proj" in names and "decoder.layers.0.ffn.router" in names
    opt = AdamW(fsdp.parameters(), lr=3e-3)
    x = torch.randint(0, cfg.vocab_size, (4, 33))
    inp, tgt = x[:, :-1], x[:, 1:]
    losses = []
    for _ in range(8):
        fsdp.zero_grad()
        loss = fsdp(inp, BatchLayout.of(inp), targets=tgt)
        loss.backward()
        fsdp.finish_backward()
        fsdp.scale_grads(1.0 / tgt.numel())
        fsdp.clip_grad_norm(1.0)
        opt.step(grad_scale=fsdp.grad_scale)
        fsdp.after_optimizer_step()
        losses.append(float(loss))
    assert losses[-1] < 0.8 * losses[0]


def test_expert_parallel_option_without_peers_keeps_replicated_experts() -> None:
    from fairseq2_b200.gang import create_fake_gangs
    from fairseq2_b200.models.moe_lm import create_moe_lm_model
    from fairseq2_b200.models.moe_lm.config import tiny

    cfg = tiny()
    cfg.expert_parallel = True
    model = create_moe_lm_model(cfg, create_fake_gangs(torch.device("cpu")))
    assert not hasattr(model, "fsdp_local_module_filter")          # one rank: nothing to exchange


def _ep_cpu_worker(rank: int, world: int):
    from fairseq2_b200.error import NotSupportedError
    from fairseq2_b200.gang import ProcessGroupGang, create_parallel_gangs
    from fairseq2_b200.models.moe_lm import create_moe_lm_model
    from fairseq2_b200.models.moe_lm.config import tiny

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    cfg = tiny()
    cfg.expert_parallel = True
    try:
        create_moe_lm_model(cfg, create_parallel_gangs(root))
        out = "built"
    except NotSupportedError as ex:
        out = str(ex)
    root.close()
    return out


def test_expert_parallel_option_on_cpu_ranks_is_refused() -> None:
    from tests.dist_utils import run_distributed

    for msg in run_distributed(_ep_cpu_worker, 2):
        assert "peer access" in msg
