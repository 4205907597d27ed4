"""Sparse token-choice MoE against the dense every-token-to-every-expert formulation."""
import torch

from fairseq2_b200.gang import create_fake_gangs
from fairseq2_b200.models.family import get_model_family
from fairseq2_b200.models.transformer.experts import MoE, route_tokens
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.ops.grouped_gemm import grouped_mm, grouped_mm_reference


def _dense_moe(m: MoE, seqs: torch.Tensor) -> torch.Tensor:
    x = seqs.reshape(-1, m.model_dim)
    logits = x @ m.router
    s, ti = torch.topk(logits, m.top_k, dim=1)
    sc = torch.full_like(logits, float("-inf")).scatter_(1, ti, s).transpose(0, 1)
    rin = x.unsqueeze(0) * torch.sigmoid(sc).unsqueeze(-1)
    e = m.experts
    h = torch.nn.functional.silu(torch.bmm(rin, e.gate_proj)) * torch.bmm(rin, e.inner_proj)
    out = torch.bmm(h, e.output_proj).sum(0)
    if m.shared_expert is not None:
        out = out + m.shared_expert(x)
    return out.view(seqs.shape)


def test_moe_matches_dense_formulation() -> None:
    torch.manual_seed(0)
    for top_k, shared in ((1, True), (2, False)):
        m = MoE(64, 256, shared, 4, 1.0, top_k, inner_dim_scale=1.0)
        x = torch.randn(3, 10, 64, requires_grad=True)
        y, yr = m(x), _dense_moe(m, x)
        assert torch.allclose(y, yr, atol=1e-5)
        params = [x, m.router, m.experts.gate_proj, m.experts.output_proj]
        g1 = torch.autograd.grad(y.square().sum(), params, retain_graph=True)
        g2 = torch.autograd.grad(yr.square().sum(), params)
        for a, b in zip(g1, g2):
            assert torch.allclose(a, b, atol=1e-4)


def test_route_tokens_groups_rows_by_expert() -> None:
    logits = torch.tensor([[0.1, 2.0, -1.0], [3.0, 0.0, 1.0], [0.0, 0.5, 0.2], [1.0, -1.0, 4.0]])
    tok, scores, order, sizes = route_tokens(logits, 1)
    assert sizes == [1, 2, 1]
    assert tok.tolist() == [1, 0, 2, 3]
    assert torch.allclose(scores, torch.sigmoid(torch.tensor([3.0, 2.0, 0.5, 4.0])))


def test_grouped_mm_with_empty_group() -> None:
    torch.manual_seed(0)
    x = torch.randn(7, 16, requires_grad=True)
    w = torch.randn(3, 16, 8, requires_grad=True)
    sizes = [4, 0, 3]
    y = grouped_mm(x, w, sizes)
    assert torch.allclose(y, grouped_mm_reference(x, w, sizes), atol=1e-5)
    y.sum().backward()
    assert w.grad is not None and float(w.grad[1].abs().max()) == 0.0


def test_llama4_tiny_trains() -> None:
    torch.manual_seed(0)
    g = create_fake_gangs(torch.device("cpu"))
    fam = get_model_family("llama4")
    cfg = fam.get_arch_config("tiny")
    model = fam.create_new_model(cfg, g)
    kinds = [type(l.ffn).__name__ for l in model.decoder.layers]
    assert kinds == ["GLUFeedForwardNetwork", "MoE", "GLUFeedForwardNetwork", "MoE"]
    assert model.decoder.layers[3].self_attn.pos_encoder is None       # NoPE layer attends globally
    x = torch.randint(1, 500, (2, 70))
    layout = BatchLayout((2, 70), [70, 50])
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    losses = []
    for _ in range(5):
        loss = model(x, layout, targets=x.roll(-1, 1), reduction="mean")
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]


def test_llama4_reference_checkpoint_keys() -> None:
    from fairseq2_b200.models.llama4 import convert_llama4_state_dict

    g = create_fake_gangs(torch.device("cpu"))
    fam = get_model_family("llama4")
    cfg = fam.get_arch_config("tiny")
    model = fam.create_new_model(cfg, g)
    hd = cfg.model_dim // cfg.num_attn_heads
    E = cfg.experts.num_experts
    F = model.decoder.layers[1].ffn.inner_dim
    sd = {
        "layers.1.attention.wqkv.weight": torch.randn((cfg.num_attn_heads + 2 * cfg.num_key_value_heads) * hd, cfg.model_dim),
        "layers.1.feed_forward.experts.moe_w_in_eD_F": torch.randn(E * cfg.model_dim, F),
        "layers.1.feed_forward.router_DE": torch.randn(cfg.model_dim, E),
        "layers.1.feed_forward.w_in_shared_FD.weight": torch.randn(F, cfg.model_dim),
        "tok_embeddings.weight": torch.randn(cfg.vocab_size, cfg.model_dim),
        "rope.freqs": torch.zeros(4),
    }
    out = convert_llama4_state_dict(sd, cfg)
    ref = model.state_dict()
    for k, v in out.items():
        assert k in ref and ref[k].shape == v.shape, k
    assert "decoder.layers.1.self_attn.k_proj.weight" in out and "decoder.layers.1.ffn.router" in out
