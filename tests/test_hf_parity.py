"""Logit parity of the LM families against Hugging Face ``transformers`` reference
implementations with random weights (CPU, fp32)."""
import pytest
import torch

from fairseq2_b200.gang import create_fake_gangs
from fairseq2_b200.models.family import get_model_family
from fairseq2_b200.nn.batch_layout import BatchLayout

transformers = pytest.importorskip("transformers")


def _ours(family: str, config, hf_model):  # type: ignore[no-untyped-def]
    fam = get_model_family(family)
    g = create_fake_gangs(torch.device("cpu"))
    model = fam.create_new_model(config, g)
    sd = fam.state_dict_converter({k: v.clone() for k, v in hf_model.state_dict().items()}, config)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("final_proj" in k for k in missing), missing
    return model.eval()


def _check(model, hf_model, vocab: int, atol: float = 2e-4) -> None:  # type: ignore[no-untyped-def]
    torch.manual_seed(0)
    x = torch.randint(1, vocab, (2, 48))
    with torch.no_grad():
        ref = hf_model(x).logits
        out = model(x, BatchLayout((2, 48), [48, 48]))
    assert torch.allclose(out, ref, atol=atol, rtol=1e-3), float((out - ref).abs().max())


def test_llama_matches_hf() -> None:
    from fairseq2_b200.models.llama import LLaMAConfig

    hc = transformers.LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                  num_key_value_heads=2, vocab_size=512, max_position_embeddings=256,
                                  rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hc).eval()
    c = LLaMAConfig(model_dim=128, max_seq_len=256, vocab_size=512, num_layers=2, num_attn_heads=4,
                    num_key_value_heads=2, ffn_inner_dim=256, ffn_inner_dim_scale=1.0, ffn_inner_dim_multiple_of=1)
    _check(_ours("llama", c, hf), hf, 512)


def test_mistral_matches_hf() -> None:
    from fairseq2_b200.models.mistral import MistralConfig

    hc = transformers.MistralConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, vocab_size=512,
                                    max_position_embeddings=256, sliding_window=16, rope_theta=10000.0,
                                    rms_norm_eps=1e-5, attn_implementation="eager")
    hf = transformers.MistralForCausalLM(hc).eval()
    c = MistralConfig(model_dim=128, max_seq_len=256, vocab_size=512, attn_window_len=16, num_layers=2,
                      num_attn_heads=4, num_key_value_heads=2, ffn_inner_dim=256)
    _check(_ours("mistral", c, hf), hf, 512)


@pytest.mark.parametrize("v3", [False, True])
def test_qwen_matches_hf(v3: bool) -> None:
    from fairseq2_b200.models.qwen import QwenConfig

    kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=512, max_position_embeddings=256, rope_theta=1e6, rms_norm_eps=1e-6,
              tie_word_embeddings=True)
    if v3:
        hf = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(head_dim=64, **kw)).eval()
    else:
        hf = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**kw)).eval()
    for n, p in hf.named_parameters():   # biases and norm weights are not random by default
        if p.ndim == 1:
            torch.nn.init.normal_(p, mean=1.0 if "norm" in n else 0.0, std=0.1)
    c = QwenConfig(model_dim=128, max_seq_len=256, vocab_size=512, tied_embeddings=True, num_layers=2,
                   num_attn_heads=4, num_key_value_heads=2, head_dim=64 if v3 else None, qkv_proj_bias=not v3,
                   q_norm=v3, k_norm=v3, ffn_inner_dim=256)
    _check(_ours("qwen", c, hf), hf, 512)


def test_olmo2_matches_hf() -> None:
    from fairseq2_b200.models.olmo import OLMOConfig

    hc = transformers.Olmo2Config(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                  num_key_value_heads=2, vocab_size=512, max_position_embeddings=256,
                                  rope_theta=500000.0, rms_norm_eps=1e-6, pad_token_id=0, tie_word_embeddings=False)
    hf = transformers.Olmo2ForCausalLM(hc).eval()
    for n, p in hf.named_parameters():
        if p.ndim == 1:
            torch.nn.init.normal_(p, mean=1.0, std=0.1)
    c = OLMOConfig(model_dim=128, max_seq_len=256, vocab_size=512, pad_idx=0, num_layers=2, num_attn_heads=4,
                   num_key_value_heads=2, ffn_inner_dim=256)
    _check(_ours("olmo", c, hf), hf, 512)


@pytest.mark.parametrize("stable", [False, True])
def test_wav2vec2_asr_matches_hf(stable: bool) -> None:
    from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
    from fairseq2_b200.models.wav2vec2 import Wav2Vec2EncoderConfig
    from fairseq2_b200.models.wav2vec2.asr import Wav2Vec2AsrConfig

    hc = transformers.Wav2Vec2Config(
        vocab_size=16, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
        conv_dim=(32, 32, 32), conv_stride=(5, 2, 2), conv_kernel=(10, 3, 2), conv_bias=stable,
        feat_extract_norm="layer" if stable else "group", do_stable_layer_norm=stable, num_conv_pos_embeddings=16,
        num_conv_pos_embedding_groups=4, hidden_dropout=0.0, attention_dropout=0.0, activation_dropout=0.0,
        feat_proj_dropout=0.0, final_dropout=0.0, layerdrop=0.0, mask_time_prob=0.0)
    hf = transformers.Wav2Vec2ForCTC(hc).eval()
    e = Wav2Vec2EncoderConfig(
        model_dim=64, max_seq_len=512, feature_dim=32, feature_extractor_layer_descs=[(32, 10, 5), (32, 3, 2), (32, 2, 2)],
        feature_extractor_bias=stable, feature_extractor_layer_norm_convs=stable, pos_conv_kernel_size=16,
        num_pos_conv_groups=4, num_encoder_layers=2, num_encoder_attn_heads=4, ffn_inner_dim=128, dropout_p=0.0,
        attn_dropout_p=0.0, layer_drop_p=0.0, norm_order=TransformerNormOrder.PRE if stable else TransformerNormOrder.POST)
    c = Wav2Vec2AsrConfig(encoder_config=e, target_vocab_size=16, use_masking=False)
    model = _ours("wav2vec2_asr", c, hf)
    torch.manual_seed(0)
    x = torch.randn(2, 3000)
    with torch.no_grad():
        ref = hf(x).logits
        out, layout = model(x, BatchLayout((2, 3000), [3000, 3000]))
    assert layout.seq_lens == [ref.shape[1]] * 2
    assert torch.allclose(out, ref, atol=2e-4, rtol=1e-3), float((out - ref).abs().max())


@pytest.mark.parametrize("shared", [0, 2])
def test_gemma3n_text_logits_match_hf(shared: int) -> None:
    """AltUp, LAuReL, per-layer inputs, local/global attention with two RoPE bases, activation sparsity, soft-cap;
    with ``shared`` > 0 the last layers reuse earlier keys/values (Hugging Face does so when its cache is on)."""
    from dataclasses import replace

    from transformers.models.gemma3n import Gemma3nForCausalLM, Gemma3nTextConfig

    from fairseq2_b200.models.gemma3n import convert_gemma3n_state_dict, create_gemma3n_model, export_gemma3n_to_hg
    from fairseq2_b200.models.gemma3n.config import gemma3n_tiny

    torch.manual_seed(0)
    cfg = replace(gemma3n_tiny(), num_kv_shared_layers=shared, num_layers=8 if shared else 6)
    _, hg = export_gemma3n_to_hg({}, cfg)
    for key in ("architectures", "model_type"):
        hg.pop(key)
    hf = Gemma3nForCausalLM(Gemma3nTextConfig(**hg, attn_implementation="eager")).eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if "correct_output_scale" in name:
                p.normal_(std=0.5)                       # zero-initialised upstream: would hide the AltUp scale
            elif "norm" in name and p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    model = create_gemma3n_model(cfg).eval()
    missing, unexpected = model.load_state_dict(convert_gemma3n_state_dict(hf.state_dict(), cfg), strict=False)
    assert not missing and not unexpected
    ids = torch.randint(1, cfg.vocab_size, (2, 20))
    lens = [20, 13]
    mask = torch.zeros(2, 20, dtype=torch.long)
    for i, n in enumerate(lens):
        mask[i, :n] = 1
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask, use_cache=shared > 0).logits
        out = model(ids, BatchLayout((2, 20), lens))
    for i, n in enumerate(lens):
        assert torch.allclose(out[i, :n], ref[i, :n], atol=2e-4), float((out[i, :n] - ref[i, :n]).abs().max())
    # packed batch: the same two sequences back to back
    packed = torch.cat([ids[0, :20], ids[1, :13]])
    with torch.no_grad():
        pk = model(packed, BatchLayout((33,), lens, packed=True))
    assert torch.allclose(pk[:20], out[0, :20], atol=2e-4) and torch.allclose(pk[20:], out[1, :13], atol=2e-4)
    # round trip of the exporter
    sd, _ = export_gemma3n_to_hg(model.state_dict(), cfg)
    assert set(sd) == {k for k in hf.state_dict() if k != "lm_head.weight"}


def test_gemma3n_incremental_decoding_matches_full_forward() -> None:
    """Prefill + single steps through the KV cache (incl. KV-sharing layers and the sliding window) reproduce the
    logits of one full forward; the sampling generator runs on the model."""
    from dataclasses import replace

    from fairseq2_b200.generation import SamplingSequenceGenerator
    from fairseq2_b200.models.gemma3n import create_gemma3n_model
    from fairseq2_b200.models.gemma3n.config import gemma3n_tiny
    from fairseq2_b200.nn.incremental_state import IncrementalStateBag

    torch.manual_seed(0)
    cfg = replace(gemma3n_tiny(), num_kv_shared_layers=2, num_layers=8)
    model = create_gemma3n_model(cfg).eval()
    ids = torch.randint(1, cfg.vocab_size, (2, 20))
    with torch.no_grad():
        full = model(ids, BatchLayout((2, 20), [20, 20]))
        bag = IncrementalStateBag(64)
        outs = [model(ids[:, :11], BatchLayout.of(ids[:, :11]), state_bag=bag)]
        bag.increment_step_nr(11)
        for t in range(11, 20):
            outs.append(model(ids[:, t:t + 1], BatchLayout.of(ids[:, t:t + 1]), state_bag=bag))
            bag.increment_step_nr(1)
    assert torch.allclose(torch.cat(outs, dim=1), full, atol=1e-4)
    gen = SamplingSequenceGenerator(model, eos_idx=2, pad_idx=0, max_gen_len=6)
    out = gen(ids[:, :5], BatchLayout((2, 5), [5, 4]))
    assert len(out.hypotheses) == 2 and all(len(h[0].seq) >= 5 for h in out.hypotheses)


def test_gemma3n_audio_tower_and_multimodal_merge_match_hf() -> None:
    """The conformer audio tower (banded attention formulation) and the multimodal embedder against the Hugging Face
    modules; the merged text + audio forward against the Hugging Face text model fed with the same embeddings."""
    from dataclasses import replace

    from transformers.models.gemma3n import Gemma3nAudioConfig as HFAudioConfig
    from transformers.models.gemma3n import Gemma3nForCausalLM, Gemma3nTextConfig
    from transformers.models.gemma3n.modeling_gemma3n import Gemma3nAudioEncoder as HFEncoder
    from transformers.models.gemma3n.modeling_gemma3n import Gemma3nMultimodalEmbedder as HFEmbedder

    from fairseq2_b200.models.gemma3n import convert_gemma3n_state_dict, create_gemma3n_model, export_gemma3n_to_hg
    from fairseq2_b200.models.gemma3n.config import Gemma3nAudioConfig, gemma3n_tiny

    torch.manual_seed(0)
    akw = dict(input_feat_size=32, hidden_size=48, conf_num_hidden_layers=2, conf_num_attention_heads=4,
               conf_attention_chunk_size=4, conf_attention_context_left=5, conf_attention_context_right=0,
               sscp_conv_channel_size=(16, 8), conf_reduction_factor=2, vocab_size=16, vocab_offset=320)
    cfg = replace(gemma3n_tiny(), vocab_size=336, audio_config=Gemma3nAudioConfig(**akw))
    _, hg = export_gemma3n_to_hg({}, cfg)
    for key in ("architectures", "model_type"):
        hg.pop(key)
    text_cfg = Gemma3nTextConfig(**hg, attn_implementation="eager")
    hf_text = Gemma3nForCausalLM(text_cfg).eval()
    hf_audio = HFEncoder(HFAudioConfig(**akw)).eval()
    hf_embed = HFEmbedder(HFAudioConfig(**akw), text_cfg).eval()
    with torch.no_grad():
        for mod in (hf_text, hf_audio, hf_embed):
            for name, p in mod.named_parameters():
                if "per_dim_scale" in name or "correct_output_scale" in name:
                    p.normal_(std=0.3)
                elif "norm" in name and p.dim() == 1:
                    p.add_(0.1 * torch.randn_like(p))
    sd = {k: v for k, v in hf_text.state_dict().items()}
    sd.update({"model.audio_tower." + k: v for k, v in hf_audio.state_dict().items()})
    sd.update({"model.embed_audio." + k: v for k, v in hf_embed.state_dict().items()})
    model = create_gemma3n_model(cfg).eval()
    missing, unexpected = model.load_state_dict(convert_gemma3n_state_dict(sd, cfg), strict=False)
    assert not missing and not unexpected, (missing, unexpected)

    mel = torch.randn(2, 80, 32)
    invalid = torch.zeros(2, 80, dtype=torch.bool)
    invalid[1, 57:] = True
    with torch.no_grad():
        ref = hf_audio(mel, invalid)
        enc, enc_invalid = model.audio_tower(mel, invalid)
        assert torch.allclose(enc, ref.last_hidden_state, atol=1e-4) and torch.equal(enc_invalid, ref.audio_mel_mask)
        assert torch.allclose(model.embed_audio(inputs_embeds=enc), hf_embed(inputs_embeds=enc), atol=1e-5)
        hard = torch.tensor([[320, 327, 335]])
        assert torch.allclose(model.embed_audio(input_ids=hard), hf_embed(input_ids=hard), atol=1e-5)

        # merged forward: 12 soft tokens per clip (10 from the tower + 2 padding) at the placeholder id 5
        S, placeholder, per_clip = 24, 5, 12
        ids = torch.randint(6, 300, (2, S))
        ids[:, 4:4 + per_clip] = placeholder
        ids[0, 20] = 330                                       # an audio hard token
        out = model(ids, BatchLayout((2, S), [S, S]), audio_features=mel, audio_invalid=invalid,
                    audio_token_idx=placeholder, num_audio_tokens=per_clip)
        embeds = model.embed_inputs(ids.reshape(-1), mel, invalid, placeholder, per_clip).view(2, S, -1)
        in_vocab = ids < cfg.vocab_size_per_layer_input
        per_layer = hf_text.model.get_per_layer_inputs(torch.where(in_vocab, ids, torch.zeros_like(ids)))
        ref_logits = hf_text(inputs_embeds=embeds, per_layer_inputs=per_layer, use_cache=False).logits
    assert torch.allclose(out, ref_logits, atol=2e-4), float((out - ref_logits).abs().max())
