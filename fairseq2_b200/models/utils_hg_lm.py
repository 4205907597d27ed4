"""Shared Hugging Face <-> native conversion for LLaMA-style decoder LMs.

HF checkpoints store q/k projections (and per-head q/k norms) for
half-rotation RoPE. The fused QKV+RoPE attention path here rotates interleaved
pairs, so rows are permuted once at load time and permuted back on export;
attention scores are invariant because q and k are permuted identically."""
from __future__ import annotations

from typing import Any, Mapping

from torch import Tensor

from fairseq2_b200.models.llama.interop import _HG_KEY_MAP, _hf_to_interleaved, _interleaved_to_hf, convert_state_dict

HG_LM_KEY_MAP = dict(_HG_KEY_MAP)
HG_LM_KEY_MAP.update({
    r"^model\.layers\.([0-9]+)\.self_attn\.q_norm\.": r"decoder.layers.\1.self_attn.q_norm.",
    r"^model\.layers\.([0-9]+)\.self_attn\.k_norm\.": r"decoder.layers.\1.self_attn.k_norm.",
})


def _permute_vec(v: Tensor, num_heads: int, to_native: bool) -> Tensor:
    """Permutes a ``[H*D]`` (or ``[D]`` with ``num_heads=1``) vector like the projection rows."""
    m = v.unsqueeze(-1)
    m = _hf_to_interleaved(m, num_heads) if to_native else _interleaved_to_hf(m, num_heads)
    return m.squeeze(-1)


def permute_qk(sd: dict[str, Any], num_heads: int, num_kv_heads: int, *, to_native: bool, prefix: str,
               per_head_norm: bool) -> None:
    """In-place layout change of every q/k projection weight, bias and q/k norm weight under keys
    containing ``prefix`` (``self_attn.`` natively)."""
    fn = _hf_to_interleaved if to_native else _interleaved_to_hf
    for k in list(sd):
        if prefix not in k:
            continue
        for name, h in (("q_proj", num_heads), ("k_proj", num_kv_heads)):
            if k.endswith(f"{name}.weight"):
                sd[k] = fn(sd[k], h)
            elif k.endswith(f"{name}.bias"):
                sd[k] = _permute_vec(sd[k], h, to_native)
        for name, h in (("q_norm", num_heads), ("k_norm", num_kv_heads)):
            if k.endswith(f"{name}.weight"):
                sd[k] = _permute_vec(sd[k], 1 if per_head_norm else h, to_native)


def is_hg_state_dict(sd: Mapping[str, Any]) -> bool:
    return any(k.startswith("model.layers.") or k.startswith("model.embed_tokens") for k in sd)


def convert_hg_lm_state_dict(sd: dict[str, Any], *, num_heads: int, num_kv_heads: int, tied: bool,
                             per_head_norm: bool = True, key_map: Mapping[str, str] | None = None) -> dict[str, Any]:
    if not is_hg_state_dict(sd):
        return dict(sd)
    out = convert_state_dict(sd, key_map or HG_LM_KEY_MAP)
    permute_qk(out, num_heads, num_kv_heads, to_native=True, prefix="self_attn.", per_head_norm=per_head_norm)
    if tied:
        out.pop("final_proj.weight", None)
    return {k: v for k, v in out.items() if not k.endswith("rotary_emb.inv_freq")}


def invert_key_map(key_map: Mapping[str, str]) -> dict[str, str]:
    inv = {}
    for p, r in key_map.items():
        src = r.replace("\\1", "([0-9]+)").replace(".", r"\.")
        dst = p.strip("^").replace("([0-9]+)", r"\1").replace("\\.", ".")
        inv["^" + src] = dst
    return inv


def export_hg_lm_state_dict(sd: Mapping[str, Any], *, num_heads: int, num_kv_heads: int, tied: bool,
                            per_head_norm: bool = True, key_map: Mapping[str, str] | None = None) -> dict[str, Any]:
    out = dict(sd)
    permute_qk(out, num_heads, num_kv_heads, to_native=False, prefix="self_attn.", per_head_norm=per_head_norm)
    out = convert_state_dict(out, invert_key_map(key_map or HG_LM_KEY_MAP))
    if tied and "lm_head.weight" not in out:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    return out
