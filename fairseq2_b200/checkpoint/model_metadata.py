"""``checkpoints/model.yaml``: which model family/config the checkpoints belong
to (cf. fairseq2 ``checkpoint/model_metadata.py:29-173``). The loader
synthesises asset cards ``checkpoint_step_N``, ``last_checkpoint`` and
``best_checkpoint`` that point at the step directories."""
from __future__ import annotations

from pathlib import Path
from typing import Any

from fairseq2_b200.gang import Gangs
from fairseq2_b200.utils.structured import unstructure
from fairseq2_b200.utils.yaml import dump_yaml, read_yaml


def save_model_metadata(checkpoint_dir: Path, gangs: Gangs, family: str, config: object) -> None:
    if gangs.root.rank == 0:
        checkpoint_dir.mkdir(parents=True, exist_ok=True)
        meta = {"name": "checkpoint", "model_family": family, "model_config": unstructure(config)}
        dump_yaml(meta, checkpoint_dir / "model.yaml")
    gangs.root.barrier()


def load_checkpoint_cards(checkpoint_dir: Path) -> list[dict[str, Any]]:
    """Asset-card dictionaries for every committed step under ``checkpoint_dir``."""
    f = checkpoint_dir / "model.yaml"
    if not f.exists():
        return []
    base = read_yaml(f) or {}
    cards: list[dict[str, Any]] = [base]
    steps = sorted(int(d.name[5:]) for d in checkpoint_dir.glob("step_*")
                   if d.is_dir() and d.suffix != ".tmp" and d.name[5:].isdigit())
    for s in steps:
        cards.append({"name": f"checkpoint_step_{s}", "base": "checkpoint",
                      "checkpoint": str(checkpoint_dir / f"step_{s}" / "model")})
    if steps:
        cards.append({"name": "last_checkpoint", "base": "checkpoint",
                      "checkpoint": str(checkpoint_dir / f"step_{steps[-1]}" / "model")})
    scores = []
    sd = checkpoint_dir / "scores"
    if sd.exists():
        for sf in sd.glob("step_*.txt"):
            try:
                scores.append((float(sf.read_text().strip()), int(sf.stem[5:])))
            except ValueError:
                continue
    scores = [(sc, st) for sc, st in scores if st in steps]
    scores.sort(reverse=True)
    for i, (_, st) in enumerate(scores):
        cards.append({"name": "best_checkpoint" if i == 0 else f"best_checkpoint_{i}", "base": "checkpoint",
                      "checkpoint": str(checkpoint_dir / f"step_{st}" / "model")})
    return cards
