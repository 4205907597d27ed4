"""The generation task: runs ``GeneratorUnit``s over data readers under inference mode and publishes their metrics
(fairseq2 ``generator.py:69-268``)."""

from fairseq2_b200.evaluator import Generator, GeneratorUnit

__all__ = ["Generator", "GeneratorUnit"]
