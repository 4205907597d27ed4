"""``python -m fairseq2_b200.assets list|show`` over the cards shipped with the package."""
from __future__ import annotations

import pytest
import yaml

from fairseq2_b200.assets.cli import main


def test_list_shows_every_family(capsys: pytest.CaptureFixture[str]) -> None:
    assert main(["list", "--kind", "model"]) == 0
    lines = capsys.readouterr().out.splitlines()
    names = {line.split()[1] for line in lines}
    assert all(line.startswith("model") for line in lines)
    for expected in ("llama3_8b", "llama3_8b_instruct", "qwen25_7b", "mistral_7b", "wav2vec2_base"):
        assert expected in names, expected
    assert main(["list", "--kind", "dataset"]) == 0
    assert "librispeech" in capsys.readouterr().out


def test_show_resolves_the_base_chain(capsys: pytest.CaptureFixture[str]) -> None:
    assert main(["show", "llama3_8b"]) == 0
    card = yaml.safe_load(capsys.readouterr().out)
    assert card["model_family"] == "llama" and card["model_arch"] == "llama3_8b"
    assert main(["show", "no_such_asset"]) == 1
    assert "no_such_asset" in capsys.readouterr().err
