"""Helpers shared by the language-model recipes (cf. fairseq2 ``recipes/lm/common.py``)."""
from __future__ import annotations

from typing import Any

from fairseq2_b200.recipe.error import RecipeError


class ModelVocabularyMismatchError(RecipeError):
    exit_code = 2


def check_model_vocabulary(model_config: Any, tokenizer: Any) -> None:
    """The tokenizer must not produce indices beyond the model's embedding table."""
    vocab = getattr(model_config, "vocab_size", None)
    if vocab is not None and tokenizer.vocab_info.size > vocab:
        raise ModelVocabularyMismatchError(
            f"The tokenizer has {tokenizer.vocab_info.size} entries, but the model vocabulary has only {vocab}.")
