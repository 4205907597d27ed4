"""Every registered model family builds its smallest architecture and runs a training step on CPU."""
import pytest
import torch

from fairseq2_b200.gang import create_fake_gangs
from fairseq2_b200.models.family import get_model_families, get_model_family
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag


def _gangs():  # type: ignore[no-untyped-def]
    return create_fake_gangs(torch.device("cpu"))


def test_registered_families() -> None:
    names = set(get_model_families())
    assert {"llama", "llama4", "mistral", "qwen", "olmo", "nllb", "s2t_transformer", "s2t_conformer", "wav2vec2",
            "wav2vec2_asr", "w2vbert"} <= names


@pytest.mark.parametrize("family", ["llama", "llama4", "mistral", "qwen", "olmo"])
def test_causal_lm_families_train_and_decode(family: str) -> None:
    torch.manual_seed(0)
    fam = get_model_family(family)
    cfg = fam.get_arch_config("tiny")
    model = fam.create_new_model(cfg, _gangs())
    x = torch.randint(1, 500, (2, 24))
    layout = BatchLayout((2, 24), [24, 24])
    loss = model(x, layout, targets=x.roll(-1, 1), reduction="mean")
    loss.backward()
    assert torch.isfinite(loss)
    assert all(p.grad is not None for p in model.parameters() if p.requires_grad)
    # incremental decoding reproduces the full forward pass
    model.eval()
    with torch.no_grad():
        full = model(x, layout)
        bag = IncrementalStateBag(64)
        steps = []
        for t in range(x.shape[1]):
            steps.append(model(x[:, t:t + 1], BatchLayout((2, 1), [1, 1]), state_bag=bag))
            bag.increment_step_nr()
    assert torch.allclose(torch.cat(steps, dim=1), full, atol=2e-4), float((torch.cat(steps, 1) - full).abs().max())


def test_nllb_incremental_decoding_matches_full_forward() -> None:
    torch.manual_seed(0)
    fam = get_model_family("nllb")
    model = fam.create_new_model(fam.get_arch_config("tiny"), _gangs())
    src, sl = torch.randint(4, 200, (2, 11)), BatchLayout((2, 11), [11, 7])
    tgt, tl = torch.randint(4, 200, (2, 9)), BatchLayout((2, 9), [9, 9])
    model(src, sl, tgt, tl, targets=tgt.roll(-1, 1)).backward()
    model.eval()
    with torch.no_grad():
        full = model(src, sl, tgt, tl)
        bag = IncrementalStateBag(32)
        outs = []
        for t in range(9):
            outs.append(model(src, sl, tgt[:, t:t + 1], BatchLayout((2, 1), [1, 1]), state_bag=bag))
            bag.increment_step_nr()
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-4)


@pytest.mark.parametrize("family,arch", [("s2t_transformer", "tiny"), ("s2t_conformer", "medium"),
                                         ("s2t_conformer", "medium_rel_pos")])
def test_speech_to_text_families(family: str, arch: str) -> None:
    torch.manual_seed(0)
    fam = get_model_family(family)
    cfg = fam.get_arch_config(arch)
    cfg.num_encoder_layers, cfg.num_decoder_layers = 2, 1
    model = fam.create_new_model(cfg, _gangs())
    x, xl = torch.randn(2, 120, 80), BatchLayout((2, 120), [120, 90])
    t, tl = torch.randint(2, cfg.target_vocab_size, (2, 7)), BatchLayout((2, 7), [7, 5])
    loss = model(x, xl, t, tl, targets=t.roll(-1, 1))
    loss.backward()
    assert torch.isfinite(loss)


def test_wav2vec2_ssl_asr_and_w2vbert() -> None:
    torch.manual_seed(0)
    g = _gangs()
    fam = get_model_family("wav2vec2")
    model = fam.create_new_model(fam.get_arch_config("tiny"), g)
    x, xl = torch.randn(3, 4000), BatchLayout((3, 4000), [4000, 3500, 3000])
    loss, out = model(x, xl)
    loss.aggregate.backward()
    assert out.logits.shape[0] == 3 and out.logits.shape[2] == 11
    assert out.temporal_mask.sum(dim=1).unique().numel() == 1      # same number of masked steps per row
    assert all(p.grad is not None for p in model.parameters())

    fam = get_model_family("wav2vec2_asr")
    asr = fam.create_new_model(fam.get_arch_config("tiny"), g)
    t, tl = torch.randint(1, 16, (3, 12)), BatchLayout((3, 12), [12, 10, 8])
    asr(x, xl, t, tl).backward()
    asr.eval()
    logits, layout = asr(x, xl)
    assert layout.seq_lens == [199, 174, 149] and logits.shape == (3, 199, 16)

    fam = get_model_family("w2vbert")
    wb = fam.create_new_model(fam.get_arch_config("tiny"), g)
    fb, fl = torch.randn(2, 200, 16), BatchLayout((2, 200), [200, 160])
    loss, out = wb(fb, fl)
    loss.aggregate.backward()
    assert out.bert_logits.shape[1:] == (16, 1) and out.bert_targets.shape[0] == out.bert_logits.shape[0]


def test_jepa_and_classifier() -> None:
    torch.manual_seed(0)
    g = _gangs()
    fam = get_model_family("jepa")
    model = fam.create_new_model(fam.get_arch_config("test"), g)
    x, xl = torch.randn(2, 3, 32, 32), BatchLayout((2, 3), [3, 3])
    y, yl = model(x, xl)
    assert y.shape == (2, 16, 64) and yl.seq_lens == [16, 16]
    fam = get_model_family("jepa_classifier")
    clf = fam.create_new_model(fam.get_arch_config("test"), g)
    out = clf(x, xl)
    out.sum().backward()
    assert out.shape == (2, 10)


def test_jepa_checkpoint_conversion_splits_fused_qkv() -> None:
    from fairseq2_b200.models.jepa import JepaConfig, convert_jepa_state_dict

    sd = {"encoder": {"module.backbone.blocks.0.attn.qkv.weight": torch.randn(192, 64),
                      "module.backbone.blocks.0.attn.proj.bias": torch.randn(64),
                      "module.backbone.pos_embed": torch.randn(1, 16, 64),
                      "module.backbone.patch_embed.proj.weight": torch.randn(64, 3, 8, 8)}}
    out = convert_jepa_state_dict(sd, JepaConfig())
    assert set(out) == {"encoder.layers.0.self_attn.q_proj.weight", "encoder.layers.0.self_attn.k_proj.weight",
                        "encoder.layers.0.self_attn.v_proj.weight", "encoder.layers.0.self_attn.output_proj.bias",
                        "encoder_frontend.patch_feature_extractor.conv.weight"}


def test_hg_adapter_wraps_causal_lm() -> None:
    transformers = pytest.importorskip("transformers")
    from fairseq2_b200.models.hg import HgCausalLMAdapter, HuggingFaceModelConfig, create_hg_model

    hc = transformers.GPT2Config(n_layer=2, n_head=2, n_embd=64, vocab_size=300, n_positions=128)
    model = create_hg_model(HuggingFaceModelConfig(hf_name="unused", model_type="causal_lm", random_init=True),
                            hf_config=hc)
    assert isinstance(model, HgCausalLMAdapter) and model.max_seq_len == 128
    x, layout = torch.randint(0, 300, (2, 10)), BatchLayout((2, 10), [10, 6])
    loss = model(x, layout, targets=x.roll(-1, 1))
    loss.backward()
    assert model(x, layout).shape == (2, 10, 300) and hasattr(model, "generate")
