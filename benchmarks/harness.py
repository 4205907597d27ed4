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


def trace_steps(prefix: str, run_step: Callable[[int], Any], num_steps: int, rank: int, record: bool) -> None:
    """Kernel timeline of two more steps (outside every timed region): one JSON row per kernel with stream, start
    and duration in microseconds, for overlap analysis of the compute and communication streams."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    if not record:                       # the other ranks only take part in the collectives
        for i in range(num_steps):
            run_step(i)
        torch.cuda.synchronize()
        return
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(num_steps):
            run_step(i)
        torch.cuda.synchronize()
    raw = f"{prefix}.rank{rank}.raw.json"
    os.makedirs(os.path.dirname(os.path.abspath(raw)), exist_ok=True)
    prof.export_chrome_trace(raw)
    with open(raw) as fp:
        events = json.load(fp)["traceEvents"]
    os.remove(raw)
    rows = [{"name": e["name"][:96], "ts": e["ts"], "dur": e["dur"], "stream": e.get("args", {}).get("stream")}
            for e in events if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset")]
    path = f"{prefix}.rank{rank}.json"
    with open(path, "w") as fp:
        json.dump(rows, fp)
    # per-kernel totals, milliseconds per step (the trace covers num_steps steps)
    totals: dict[str, list[float]] = {}
    for r in rows:
        t = totals.setdefault(r["name"], [0.0, 0])
        t[0] += r["dur"] / 1000.0 / num_steps
        t[1] += 1
    # exposed communication: what the compute stream (the one that runs the GEMMs) spends idle between the first and
    # the last kernel of the traced steps -- time in which the step waits for a collective, a copy or the host
    by_stream: dict[object, list[tuple[float, float]]] = {}
    gemm_us: dict[object, float] = {}
    for r in rows:
        by_stream.setdefault(r["stream"], []).append((r["ts"], r["ts"] + r["dur"]))
        if "gemm" in r["name"]:
            gemm_us[r["stream"]] = gemm_us.get(r["stream"], 0.0) + r["dur"]
    stats = {}
    if gemm_us:
        cs = max(gemm_us, key=gemm_us.get)  # type: ignore[arg-type]
        iv = sorted(by_stream[cs])
        busy, cur_s, cur_e = 0.0, iv[0][0], iv[0][1]
        for s_, e_ in iv[1:]:
            if s_ > cur_e:
                busy += cur_e - cur_s
                cur_s, cur_e = s_, e_
            else:
                cur_e = max(cur_e, e_)
        busy += cur_e - cur_s
        span = iv[-1][1] - iv[0][0]
        stats = {"compute_stream_idle_ms_per_step": (span - busy) / 1000.0 / num_steps,
                 "compute_stream_busy_ms_per_step": busy / 1000.0 / num_steps,
                 "gemm_ms_per_step": gemm_us[cs] / 1000.0 / num_steps,
                 "other_streams_kernel_ms_per_step": sum(e_ - s_ for k_, v in by_stream.items() if k_ != cs
                                                         for s_, e_ in v) / 1000.0 / num_steps}
        with open(f"{prefix}.rank{rank}.overlap.json", "w") as fp:
            json.dump(stats, fp)
    with open(f"{prefix}.rank{rank}.kernels.txt", "w") as fp:
        fp.write(f"# kernel time per step (torch.profiler CUDA activity, {num_steps} steps averaged)\n")
        fp.write(f"TOTAL {sum(t[0] for t in totals.values()):.1f} ms/step\n")
        for name, (ms, n) in sorted(totals.items(), key=lambda kv: -kv[1][0])[:40]:
            fp.write(f"{ms:9.2f} ms {n // num_steps:6d}x  {name}\n")




def timed_run(*, steps: int, warmup: int, rank: int, world: int, local_rank: int, device: Any,
              barrier: Callable[[], None], all_reduce_max: Callable[[Any], None],
              stage: Callable[[Any], Any], step: Callable[[Any, int], Any], examples: Sequence[Any],
              h2d_bytes: Callable[[Any], int], launch_counter: Callable[[], int] | None = None,
              reset_launch_counter: Callable[[], None] | None = None, trace: Any | None = None) -> dict[str, Any]:
    """``examples`` holds ``warmup + 2 * steps`` host-resident inputs; ``stage(ex)`` copies one to the device,
    ``step(batch, i)`` runs one optimizer step and returns the loss as a device scalar. ``trace``: the parsed
    command line (``trace``, ``trace_all_ranks``, ``no_trace``); unless switched off, two more steps run under the
    profiler after the timed regions and give the exposed-communication figure."""
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
    overlap = None
    if cuda and trace is not None and not getattr(trace, "no_trace", False):
        import shutil
        import tempfile

        prefix = getattr(trace, "trace", None)
        own = prefix is None
        if own:
            prefix = os.path.join(tempfile.mkdtemp(prefix="fs2_trace_"), "t")
        traced = [stage(examples[warmup + i % max(steps, 1)]) for i in range(2)]
        trace_steps(prefix, lambda i: step(traced[i], 10_000 + i), 2, rank,
                    record=rank == 0 or bool(getattr(trace, "trace_all_ranks", False)))
        barrier()
        if rank == 0:
            try:
                with open(f"{prefix}.rank0.overlap.json") as fp:
                    overlap = json.load(fp)
            except OSError:
                overlap = None
        if own and rank == 0:
            shutil.rmtree(os.path.dirname(prefix), ignore_errors=True)
    times = torch.tensor([dev_ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        all_reduce_max(times)
    out: dict[str, Any] = {"dev_ms": float(times[0]), "e2e_ms": float(times[1]), "h2d_bytes": h2d, "d2h_bytes": 4,
                           "final_loss": last, "losses": losses, "clocks": summarize_clocks(samples)}
    if launches is not None:
        out["gpu_launches"] = int(launches)
    if overlap:
        out["overlap"] = overlap
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
    if run.get("overlap"):
        # idle time of the stream that runs the GEMMs, from a kernel timeline of two extra steps: what the step
        # waits for (collectives, copies, the host) while no kernel of its own runs
        ov = run["overlap"]
        out["exposed_comm_ms"] = round(ov["compute_stream_idle_ms_per_step"], 3)
        out["gemm_ms_per_step"] = round(ov["gemm_ms_per_step"], 3)
        out["comm_stream_kernel_ms_per_step"] = round(ov["other_streams_kernel_ms_per_step"], 3)
    if extra:
        out.update(extra)
    return json.dumps(out)


def _abort_marker() -> str:
    # one file per launch: all workers of a `torch.distributed.run` share their parent process
    return f"/tmp/fs2_bench_abort_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}"


def watch_for_abort() -> None:
    """With several ranks, a rank that raises (say, out of memory) leaves its peers inside collectives until their
    time-outs expire. Every rank polls a marker file from a daemon thread and exits with status 3 when a peer wrote
    it, so that a failed run ends within a second instead of minutes."""
    if int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    marker = _abort_marker()
    try:
        os.unlink(marker)
    except OSError:
        pass

    def loop() -> None:
        while True:
            time.sleep(0.5)
            if os.path.exists(marker):
                try:
                    why = open(marker).read().strip()
                except OSError:
                    why = ""
                print(f"[rank {os.environ.get('RANK', '?')}] a peer rank failed: {why[:300]}", flush=True)
                os._exit(3)

    threading.Thread(target=loop, daemon=True).start()


def abort_peers(why: str) -> None:
    if int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    try:
        with open(_abort_marker(), "w") as fp:
            fp.write(why[:1000] + "\n")
    except OSError:
        pass


def env_ranks() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))
