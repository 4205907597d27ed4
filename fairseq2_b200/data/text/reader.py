"""Line-by-line text reader (cf. fairseq2 ``data/text/reader.py:24-34``)."""
from __future__ import annotations

from enum import Enum
from pathlib import Path

from fairseq2_b200.data.data_pipeline import DataPipelineBuilder, _n


class LineEnding(Enum):
    INFER = "infer"
    LF = "lf"
    CRLF = "crlf"


def read_text(path: Path | str, key: str | None = None, encoding: str | None = None,
              line_ending: LineEnding = LineEnding.INFER, ltrim: bool = False, rtrim: bool = False,
              skip_empty: bool = False, memory_map: bool = False, block_size: int | None = None
              ) -> DataPipelineBuilder:
    le = line_ending.value if isinstance(line_ending, LineEnding) else str(line_ending)
    return _n.read_text(str(path), key, encoding, le, ltrim, rtrim, skip_empty, memory_map, block_size)
