"""Validation during training: the ``Validator`` interface the trainer calls every ``validate_every_n_steps`` and
its standard implementation over ``EvalUnit``s with score tracking (fairseq2 ``validator.py:69-419``)."""

from fairseq2_b200.evaluator import EvalUnit, StandardValidator
from fairseq2_b200.trainer import NoopValidator, Validator

__all__ = ["EvalUnit", "NoopValidator", "StandardValidator", "Validator"]
