"""Shared measurement code of ``bench.py`` and the per-configuration benchmarks.

Every configuration is measured the same way: W untimed warm-up steps, then exactly K steps timed on the device with
CUDA events between two barriers (inputs resident before the clock starts), then K more steps timed end to end --
each step copies its inputs from pinned host memory and reads its loss back to the host -- and the maximum over ranks
of both times. SM clocks and throttle reasons are sampled with ``nvidia-smi`` (read-only) during the timed regions.
"""
from __future__ import annotations

import json
import os
import subprocess
import threading
import time
from typing import Any, Callable, Sequence


def clock_sampler(stop: threading.Event, out: list[dict], gpu_index: int) -> None:
    q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    try:
        proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200",
                                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
        return
    assert proc.stdout is not None
    try:
        while not stop.is_set():
            line = proc.stdout.readline()
            if not line:
                break
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                try:
                    out.append({"sm": float(parts[0]), "max": float(parts[1]), "power": float(parts[2]),
                                "hw_slowdown": parts[3], "hw_thermal": parts[4], "sw_thermal": parts[5],
                                "sw_power_cap": parts[6]})
                except ValueError:
                    pass
    finally:
        proc.terminate()


def summarize_clocks(samples: list[dict]) -> dict:
    if not samples:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    sm = sorted(s["sm"] for s in samples)
    reasons = []
    for key, name in (("hw_slowdown", "hw_slowdown"), ("hw_thermal", "hw_thermal_slowdown"),
                      ("sw_thermal", "sw_thermal_slowdown"), ("sw_power_cap", "sw_power_cap")):
        if any(s[key].lower().startswith("active") for s in samples):
            reasons.append(name)
    return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": samples[0]["max"], "reasons": reasons,
            "samples": len(samples), "power_w_max": max(s["power"] for s in samples)}


def timed_run(*, steps: int, warmup: int, rank: int, world: int, local_rank: int, device: Any,
              barrier: Callable[[], None], all_reduce_max: Callable[[Any], None],
              stage: Callable[[Any], Any], step: Callable[[Any, int], Any], examples: Sequence[Any],
              h2d_bytes: Callable[[Any], int], launch_counter: Callable[[], int] | None = None,
              reset_launch_counter: Callable[[], None] | None = None) -> dict[str, Any]:
    """``examples`` holds ``warmup + 2 * steps`` host-resident inputs; ``stage(ex)`` copies one to the device,
    ``step(batch, i)`` runs one optimizer step and returns the loss as a device scalar."""
    import torch

    cuda = device.type == "cuda"
    for i in range(warmup):
        step(stage(examples[i]), i)
    barrier()
    staged = [stage(examples[warmup + i]) for i in range(steps)]
    samples: list[dict] = []
    stop = threading.Event()
    sampler = threading.Thread(target=clock_sampler, args=(stop, samples, local_rank), daemon=True)
    if rank == 0 and cuda:
        sampler.start()
    barrier()
    if reset_launch_counter is not None:
        reset_launch_counter()
    if cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.perf_counter()
    for i in range(steps):
        step(staged[i], warmup + i)
    if cuda:
        ev1.record()
    barrier()
    launches = launch_counter() if launch_counter is not None else None
    dev_ms = ev0.elapsed_time(ev1) if cuda else (time.perf_counter() - t0) * 1e3
    del staged

    barrier()
    t0 = time.perf_counter()
    h2d, last = 0, 0.0
    losses: list[float] = []
    for i in range(steps):
        ex = examples[warmup + steps + i]
        h2d = h2d_bytes(ex)
        last = float(step(stage(ex), warmup + steps + i).item())
        losses.append(last)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    stop.set()
    times = torch.tensor([dev_ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        all_reduce_max(times)
    out: dict[str, Any] = {"dev_ms": float(times[0]), "e2e_ms": float(times[1]), "h2d_bytes": h2d, "d2h_bytes": 4,
                           "final_loss": last, "losses": losses, "clocks": summarize_clocks(samples)}
    if launches is not None:
        out["gpu_launches"] = int(launches)
    if cuda:
        out["peak_mem_gb"] = torch.cuda.max_memory_allocated(device) / 2**30
    return out


def result_line(*, metric: str, unit: str, impl: str, units_per_step: float, world: int, steps: int, warmup: int,
                run: dict[str, Any], config: dict[str, Any], extra: dict[str, Any] | None = None) -> str:
    value = units_per_step * steps / (run["dev_ms"] * 1e-3)
    out: dict[str, Any] = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": run["dev_ms"] / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": impl, "config": config,
        "e2e": {"value": units_per_step * steps / (run["e2e_ms"] * 1e-3), "unit": unit,
                "ms_per_step": run["e2e_ms"] / steps, "h2d_bytes_per_step": run["h2d_bytes"],
                "d2h_bytes_per_step": run["d2h_bytes"]},
        "clocks": run["clocks"], "final_loss": run["final_loss"], "losses": run.get("losses"),
    }
    if "gpu_launches" in run:
        out["gpu_launches"] = run["gpu_launches"]
    if "peak_mem_gb" in run:
        out["peak_mem_gb"] = run["peak_mem_gb"]
    if extra:
        out.update(extra)
    return json.dumps(out)


def env_ranks() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))
