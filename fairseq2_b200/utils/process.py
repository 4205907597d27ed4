"""Runs child processes with captured text output (cf. ``src/fairseq2/utils/process.py``)."""
from __future__ import annotations

import subprocess
from pathlib import Path
from typing import Mapping, Sequence


class ProcessError(Exception):
    pass


class ProcessRunner:
    def run_text(self, args: Sequence[str], *, stdout: Path | None = None, stderr: Path | None = None,
                 env: Mapping[str, str] | None = None, cwd: Path | None = None) -> subprocess.Popen[str]:
        out = stdout.open("w") if stdout is not None else subprocess.DEVNULL
        err = stderr.open("w") if stderr is not None else subprocess.DEVNULL
        try:
            return subprocess.Popen(list(args), stdout=out, stderr=err, env=dict(env) if env else None, cwd=cwd,
                                    text=True)
        except OSError as ex:
            raise ProcessError(f"The process '{args[0]}' cannot be started: {ex}") from ex
