"""Out-of-process Hugging Face export of saved checkpoints (cf. fairseq2 ``checkpoint/hg.py:80-212``).

After a checkpoint is committed, rank 0 spawns ``python -m fairseq2_b200.models.utils.hg_export`` so that
consolidation and conversion never block (or share memory with) the training process. The exporter leaves
``step_N/hg.run`` while it runs and ``hg.stdout`` / ``hg.stderr`` with the child's output."""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path
from typing import IO

from fairseq2_b200.gang import Gangs
from fairseq2_b200.logging import log


class HuggingFaceExporter:
    def export(self, step_nr: int) -> None: ...

    def complete_pending_export_operations(self, *, blocking: bool = True) -> None: ...

    @property
    def is_exporting(self) -> bool:
        return False


class NoopHuggingFaceExporter(HuggingFaceExporter):
    pass


class OutOfProcHuggingFaceExporter(HuggingFaceExporter):
    def __init__(self, checkpoint_dir: Path, gangs: Gangs, *, dtype: str = "bfloat16") -> None:
        self._dir, self._gangs, self._dtype = checkpoint_dir, gangs, dtype
        self._children: list[tuple[int, subprocess.Popen[bytes], Path, IO[bytes], IO[bytes]]] = []

    def export(self, step_nr: int) -> None:
        if self._gangs.root.rank != 0:
            return
        self.complete_pending_export_operations(blocking=False)
        step_dir = self._dir / f"step_{step_nr}"
        out_dir = step_dir / "hg"
        run_file = step_dir / "hg.run"
        run_file.touch()
        so, se = open(step_dir / "hg.stdout", "wb"), open(step_dir / "hg.stderr", "wb")
        cmd = [sys.executable, "-m", "fairseq2_b200.models.utils.hg_export", "--checkpoint-dir", str(self._dir),
               "--dtype", self._dtype, f"checkpoint_step_{step_nr}", str(out_dir)]
        log.info("Exporting the checkpoint of step {} to Hugging Face format in the background.", step_nr)
        child = subprocess.Popen(cmd, stdout=so, stderr=se, stdin=subprocess.DEVNULL,
                                 env=_cpu_only_env())
        self._children.append((step_nr, child, run_file, so, se))

    def complete_pending_export_operations(self, *, blocking: bool = True) -> None:
        rest = []
        for step_nr, child, run_file, so, se in self._children:
            rc = child.wait() if blocking else child.poll()
            if rc is None:
                rest.append((step_nr, child, run_file, so, se))
                continue
            so.close()
            se.close()
            run_file.unlink(missing_ok=True)
            if rc != 0:
                log.warning("The Hugging Face export of step {} failed with exit code {}; see {}.", step_nr, rc,
                            run_file.with_name("hg.stderr"))
            else:
                log.info("The Hugging Face export of step {} finished.", step_nr)
        self._children = rest

    @property
    def is_exporting(self) -> bool:
        return any(c.poll() is None for _, c, _, _, _ in self._children)


def _cpu_only_env() -> dict[str, str]:
    import os

    env = dict(os.environ)
    env["CUDA_VISIBLE_DEVICES"] = ""           # the exporter consolidates on the CPU and must not touch the GPUs
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    return env
