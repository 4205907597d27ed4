"""Exports a training checkpoint as a Hugging Face model directory (cf. fairseq2
``models/utils/hg_export.py:67-321``).

    python -m fairseq2_b200.models.utils.hg_export --checkpoint-dir DIR checkpoint_step_N OUT_DIR

The sharded checkpoint is consolidated on the CPU (the checkpoint loader re-shards to a world of one),
converted with the family's exporter and written as ``model.safetensors`` (or ``pytorch_model.bin``)
plus ``config.json``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Any

import torch

from fairseq2_b200.assets import AssetStore, get_asset_store, register_checkpoint_models
from fairseq2_b200.gang import create_fake_gangs
from fairseq2_b200.logging import configure_logging, log
from fairseq2_b200.models.family import get_model_family


class HuggingFaceExportError(Exception):
    pass


def export_model_to_hg(model_name: str, output_dir: Path, *, store: AssetStore | None = None,
                       dtype: torch.dtype = torch.bfloat16, safe_serialization: bool = True) -> Path:
    store = store or get_asset_store()
    card = store.retrieve_card(model_name)
    family_name = card.get_field("model_family", str)
    family = get_model_family(family_name)
    if family.hg_exporter is None:
        raise HuggingFaceExportError(f"The '{family_name}' model family does not support Hugging Face export.")
    config = family.get_model_config(card)
    gangs = create_fake_gangs(torch.device("cpu"))
    model = family.create_new_model(config, gangs, torch.float32)
    family.load_into(model, Path(card.get_field("checkpoint", str)), config, gangs, strict=True)
    sd = {k: v.detach().to(dtype) if v.is_floating_point() else v.detach() for k, v in model.state_dict().items()}
    hg_sd, hg_config = family.hg_exporter(sd, config)
    output_dir.mkdir(parents=True, exist_ok=True)
    hg_sd = {k: v.contiguous().clone() for k, v in hg_sd.items()}      # safetensors refuses aliased storage
    if safe_serialization:
        from safetensors.torch import save_file

        save_file(hg_sd, str(output_dir / "model.safetensors"), metadata={"format": "pt"})
    else:
        torch.save(hg_sd, output_dir / "pytorch_model.bin")
    hg_config = dict(hg_config)
    hg_config["torch_dtype"] = str(dtype).removeprefix("torch.")
    with open(output_dir / "config.json", "w", encoding="utf-8") as fp:
        json.dump(hg_config, fp, indent=2)
    return output_dir


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Export a model checkpoint in Hugging Face format.")
    ap.add_argument("--checkpoint-dir", type=Path, default=None,
                    help="checkpoint directory whose steps become `checkpoint_step_N` / `last_checkpoint` models")
    ap.add_argument("--no-safetensors", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("model", help="model (card) name, e.g. checkpoint_step_1000")
    ap.add_argument("output_dir", type=Path)
    args = ap.parse_args(argv)
    configure_logging()
    store = get_asset_store()
    if args.checkpoint_dir is not None:
        register_checkpoint_models(store, args.checkpoint_dir)
    try:
        out = export_model_to_hg(args.model, args.output_dir, store=store, dtype=getattr(torch, args.dtype),
                                 safe_serialization=not args.no_safetensors)
    except Exception as ex:  # noqa: BLE001
        log.error("The export of '{}' failed: {}", args.model, ex)
        return 1
    log.info("Model '{}' exported to {}.", args.model, out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
