"""Cluster environment handling (cf. fairseq2 ``cluster.py:22-139``): under
Slurm the ``SLURM_*`` variables are translated into the torchrun-style
``RANK/WORLD_SIZE/LOCAL_RANK/MASTER_ADDR/MASTER_PORT`` that the gang layer reads."""
from __future__ import annotations

import os
import subprocess
from typing import MutableMapping


class ClusterError(Exception):
    def __init__(self, cluster: str, message: str) -> None:
        super().__init__(message)
        self.cluster = cluster


class ClusterHandler:
    def set_torch_distributed_variables(self) -> None: ...

    def supports_current_cluster(self) -> bool:
        return False


class SlurmHandler(ClusterHandler):
    def __init__(self, env: MutableMapping[str, str] | None = None) -> None:
        self._env = os.environ if env is None else env

    def supports_current_cluster(self) -> bool:
        return "SLURM_JOB_ID" in self._env

    def set_torch_distributed_variables(self) -> None:
        e = self._env
        if "SLURM_JOB_ID" not in e:
            raise ClusterError("slurm", "Slurm is not detected (`SLURM_JOB_ID` is not set).")
        try:
            e["WORLD_SIZE"] = e["SLURM_NTASKS"]
            e["RANK"] = e["SLURM_PROCID"]
            e["LOCAL_RANK"] = e["SLURM_LOCALID"]
            e["LOCAL_WORLD_SIZE"] = e.get("SLURM_NTASKS_PER_NODE", e["SLURM_NTASKS"]).split("(")[0]
        except KeyError as ex:
            raise ClusterError("slurm", f"The Slurm variable {ex} is not set; launch the job with `srun`.") from None
        if "MASTER_ADDR" not in e:
            nodelist = e.get("SLURM_JOB_NODELIST", "")
            try:
                out = subprocess.run(["scontrol", "show", "hostnames", nodelist], capture_output=True, text=True,
                                     check=True).stdout.split()
                e["MASTER_ADDR"] = out[0]
            except (OSError, subprocess.CalledProcessError, IndexError):
                e["MASTER_ADDR"] = nodelist.split(",")[0].split("[")[0] or "127.0.0.1"
        e.setdefault("MASTER_PORT", str(10000 + int(e["SLURM_JOB_ID"]) % 50000))


def prepare_cluster(name: str = "auto") -> None:
    """``auto``: use Slurm if detected and torchrun variables are absent; ``none``: do nothing."""
    if name == "none":
        return
    h = SlurmHandler()
    if name == "slurm":
        h.set_torch_distributed_variables()
    elif name == "auto":
        if h.supports_current_cluster() and "RANK" not in os.environ:
            h.set_torch_distributed_variables()
    else:
        raise ClusterError(name, f"'{name}' is not a known cluster type (auto, slurm, none).")
