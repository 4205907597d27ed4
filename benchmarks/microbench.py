"""Per-kernel micro-benchmarks on one GPU.

    python -m benchmarks.microbench gemm --m 8192 --n 6144 --k 4096
    python -m benchmarks.microbench attention --tokens 8192 --seq-len 8192
    python -m benchmarks.microbench all

Every case warms up, flushes L2 (a 256 MiB write) between timed iterations,
times with CUDA events on the launching stream and prints one JSON line with
the median time and the achieved TFLOP/s or GB/s. ``--iters 1 --warmup 0`` makes
a case small enough for a profiler capture of a single launch.
"""
from __future__ import annotations

import argparse
import json
import math
import time
from typing import Any, Callable

import torch

from fairseq2_b200.ops._ext import require_ext

_DEV = "cuda"


def _time(fn: Callable[[], Any], iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=_DEV)
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def _time_sustained(fn: Callable[[], Any], seconds: float) -> float:
    """Average time of `fn` launched back to back for `seconds` (the GPU settles at its power-capped clock)."""
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.perf_counter()
    s.record()
    while True:
        for _ in range(50):
            fn()
        n += 50
        torch.cuda.synchronize()
        if time.perf_counter() - t0 >= seconds:
            break
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / n


def _emit(case: str, ms: float, *, flops: float | None = None, nbytes: float | None = None, **kw: Any) -> None:
    r: dict[str, Any] = {"case": case, "ms": round(ms, 4), **kw}
    if flops is not None:
        r["tflops"] = round(flops / ms / 1e9, 1)
    if nbytes is not None:
        r["gbs"] = round(nbytes / ms / 1e6, 1)
    r["status"] = require_ext().read_status()
    print(json.dumps(r), flush=True)


def bench_gemm(a: argparse.Namespace) -> None:
    ext = require_ext()
    M, N, K = a.m, a.n, a.k
    x = torch.randn((K, M) if a.a_mn else (M, K), device=_DEV, dtype=torch.bfloat16)
    w = torch.randn((K, N) if a.b_mn else (N, K), device=_DEV, dtype=torch.bfloat16)
    out = torch.empty((M, N), device=_DEV, dtype=torch.bfloat16)
    ms = _time(lambda: ext.gemm_bf16(x, w, out, a.a_mn, a.b_mn, False), a.iters, a.warmup)
    r: dict[str, Any] = {}
    if a.compare:
        A, B = (x.t() if a.a_mn else x), (w if a.b_mn else w.t())
        ref = torch.matmul(A, B)
        r["rel_err"] = float((out.float() - ref.float()).norm() / ref.float().norm())
        r["ms_cublas"] = round(_time(lambda: torch.matmul(A, B, out=ref), a.iters, a.warmup), 4)
    if a.sustained > 0:
        # seconds-long loops under the power cap: the figure a kernel reaches inside a long training step
        fl = 2.0 * M * N * K
        r["tflops_sustained"] = round(fl / _time_sustained(lambda: ext.gemm_bf16(x, w, out, a.a_mn, a.b_mn, False),
                                                            a.sustained) / 1e9, 1)
        if a.compare:
            r["tflops_cublas_sustained"] = round(fl / _time_sustained(lambda: torch.matmul(A, B, out=ref),
                                                                      a.sustained) / 1e9, 1)
    _emit("gemm", ms, flops=2.0 * M * N * K, M=M, N=N, K=K, a_mn=a.a_mn, b_mn=a.b_mn, **r)


def _attn_inputs(a: argparse.Namespace):  # type: ignore[no-untyped-def]
    """``--doc-lens LO,HI``: the tokens are packed documents with lengths uniform in [LO, HI] (the SFT benchmark's
    workload: 128,4096) instead of equal sequences of ``--seq-len``."""
    T, S, H, Hkv, D = a.tokens, a.seq_len, a.heads, a.kv_heads, a.head_dim
    qkv = torch.randn(T, H + 2 * Hkv, D, device=_DEV, dtype=torch.bfloat16)
    if a.doc_lens:
        import numpy as np

        lo, hi = (int(v) for v in a.doc_lens.split(","))
        rng, doc, total = np.random.default_rng(0), [], 0
        while total < T:
            n = min(int(rng.integers(lo, hi + 1)), T - total)
            doc.append(n)
            total += n
        lens = torch.tensor(doc, device=_DEV, dtype=torch.int32)
        begins = (torch.cumsum(lens, 0) - lens).to(torch.int32)
        return qkv, begins, lens
    nseq = T // S
    begins = torch.arange(nseq, device=_DEV, dtype=torch.int32) * S
    lens = torch.full((nseq,), S, device=_DEV, dtype=torch.int32)
    return qkv, begins, lens


def bench_attention(a: argparse.Namespace) -> None:
    ext = require_ext()
    T, S, H, Hkv, D = a.tokens, a.seq_len, a.heads, a.kv_heads, a.head_dim
    qkv, begins, lens = _attn_inputs(a)
    q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
    scale = 1.0 / math.sqrt(D)
    S = int(lens.max())
    fl_fwd = 4.0 * H * D * float((lens.double() ** 2).sum()) / 2      # causal: half of the score matrix
    drop, seed = a.dropout, 1234
    tag = {"docs": a.doc_lens or None, "dropout": drop or None}
    out, lse = ext.attn_fwd(q, k, v, begins, lens, begins, lens, S, S, True, scale, 0, drop, seed)
    ms = _time(lambda: ext.attn_fwd(q, k, v, begins, lens, begins, lens, S, S, True, scale, 0, drop, seed), a.iters,
               a.warmup)
    _emit("attention_fwd", ms, flops=fl_fwd, tokens=T, seq_len=S, heads=H, kv_heads=Hkv, head_dim=D, **tag)
    dout = torch.randn_like(out)
    dqkv = torch.empty_like(qkv)

    def bwd() -> None:
        ext.attn_bwd_out(dout, q, k, v, out, lse, begins, lens, begins, lens, S, S, True, scale, dqkv[:, :H],
                         dqkv[:, H:H + Hkv], dqkv[:, H + Hkv:], 0, drop, seed)

    ms = _time(bwd, a.iters, a.warmup)
    _emit("attention_bwd", ms, flops=2.5 * fl_fwd, tokens=T, seq_len=S, heads=H, kv_heads=Hkv, head_dim=D, **tag)


def bench_norm(a: argparse.Namespace) -> None:
    from fairseq2_b200.ops.norm import rms_norm

    T, Dm = a.tokens, a.dim
    x = torch.randn(T, Dm, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(Dm, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    ms = _time(lambda: rms_norm(x.detach(), (Dm,), w.detach(), 1e-5), a.iters, a.warmup)
    _emit("rms_norm_fwd", ms, nbytes=2.0 * T * Dm * 2, tokens=T, dim=Dm)
    y = rms_norm(x, (Dm,), w, 1e-5)
    g = torch.randn_like(y)
    ms = _time(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True), a.iters, a.warmup)
    _emit("rms_norm_bwd", ms, nbytes=3.0 * T * Dm * 2, tokens=T, dim=Dm)


def bench_swiglu(a: argparse.Namespace) -> None:
    from fairseq2_b200.ops.activation import swiglu

    T, F = a.tokens, a.ffn_dim
    gu = torch.randn(T, 2 * F, device=_DEV, dtype=torch.bfloat16)
    ms = _time(lambda: swiglu(gu), a.iters, a.warmup)
    _emit("swiglu_fwd", ms, nbytes=3.0 * T * F * 2, tokens=T, ffn_dim=F)


def bench_adamw(a: argparse.Namespace) -> None:
    from fairseq2_b200.ops.optim import multi_tensor_adamw

    n = a.numel
    p = torch.randn(n, device=_DEV)
    g = torch.randn(n, device=_DEV)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    low = torch.empty(n, device=_DEV, dtype=torch.bfloat16)

    def run() -> None:
        multi_tensor_adamw([p], [g], [m], [v], [low], step=1, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                           weight_decay=0.1)

    ms = _time(run, a.iters, a.warmup)
    _emit("adamw", ms, nbytes=n * (4 * 4 + 3 * 4 + 2.0), numel=n)


def bench_ce(a: argparse.Namespace) -> None:
    from fairseq2_b200.ops.cross_entropy import fused_linear_cross_entropy

    T, Dm, V = a.tokens, a.dim, a.vocab
    h = torch.randn(T, Dm, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, Dm, device=_DEV, dtype=torch.bfloat16) * 0.02).requires_grad_()
    t = torch.randint(0, V, (T,), device=_DEV)

    def run() -> None:
        loss = fused_linear_cross_entropy(h, w, t)
        loss.backward()
        h.grad = w.grad = None

    ms = _time(run, a.iters, a.warmup)
    _emit("fused_linear_ce_fwd_bwd", ms, flops=6.0 * T * Dm * V, tokens=T, dim=Dm, vocab=V)


def bench_conv(a: argparse.Namespace) -> None:
    """One strided feature-encoder convolution (wav2vec 2.0 layers 2-5: 512 -> 512 channels, k=3, s=2) as a GEMM over
    overlapping-row views vs cuDNN ``conv1d`` on the channels-first layout, forward and backward; then the fused
    LayerNorm+GELU kernel vs the two PyTorch ops."""
    import torch.nn.functional as F

    from fairseq2_b200.ops.conv import conv1d_channels_last
    from fairseq2_b200.ops.norm import layer_norm_gelu

    B, L, C, k, s = 32, 8192, 512, 3, 2
    x = torch.randn(B, L, C, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(C, C, k, device=_DEV) * (C * k) ** -0.5).to(torch.bfloat16).requires_grad_(True)
    fl = 2.0 * B * (L // s) * C * C * k
    y = conv1d_channels_last(x, w, None, s)
    g = torch.randn_like(y)
    ms = _time(lambda: conv1d_channels_last(x, w, None, s), a.iters, a.warmup)
    _emit("conv1d_view_gemm_fwd", ms, flops=fl, batch=B, length=L, channels=C, kernel=k, stride=s)

    def ours_fb() -> None:
        x.grad = w.grad = None
        conv1d_channels_last(x, w, None, s).backward(g)

    ms = _time(ours_fb, a.iters, a.warmup)
    _emit("conv1d_view_gemm_fwd_bwd", ms, flops=3 * fl)
    xc = x.detach().transpose(1, 2).contiguous().requires_grad_(True)
    wc = w.detach().clone().requires_grad_(True)
    yc = F.conv1d(xc, wc, stride=s)
    gc = torch.randn_like(yc)
    ms = _time(lambda: F.conv1d(xc, wc, stride=s), a.iters, a.warmup)
    _emit("conv1d_cudnn_fwd", ms, flops=fl)

    def cudnn_fb() -> None:
        xc.grad = wc.grad = None
        F.conv1d(xc, wc, stride=s).backward(gc)

    ms = _time(cudnn_fb, a.iters, a.warmup)
    _emit("conv1d_cudnn_fwd_bwd", ms, flops=3 * fl)
    rows = B * (L // s)
    h = torch.randn(rows, C, device=_DEV, dtype=torch.bfloat16)
    lw, lb = torch.ones(C, device=_DEV, dtype=torch.bfloat16), torch.zeros(C, device=_DEV, dtype=torch.bfloat16)
    ms = _time(lambda: layer_norm_gelu(h, lw, lb, 1e-5), a.iters, a.warmup)
    _emit("layer_norm_gelu_fused_fwd", ms, nbytes=2.0 * rows * C * 2)
    ms = _time(lambda: F.gelu(F.layer_norm(h, (C,), lw, lb, 1e-5)), a.iters, a.warmup)
    _emit("layer_norm_then_gelu_torch_fwd", ms, nbytes=2.0 * rows * C * 2)


def bench_first_conv(a: argparse.Namespace) -> None:
    """First wav2vec 2.0 feature-extractor layer in one kernel: ~1.4 M samples per step in the SSL benchmark."""
    from fairseq2_b200.ops.conv import first_conv_ln_gelu

    B, L, C, k, s = 8, a.samples // 8, 512, 10, 5
    x = (torch.randn(B, L, device=_DEV) * 0.1).to(torch.bfloat16)
    w = (torch.randn(C, 1, k, device=_DEV) * 0.3).to(torch.bfloat16).requires_grad_(True)
    b = torch.zeros(C, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    lw = torch.ones(C, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    lb = torch.zeros(C, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    T = (L - k) // s + 1
    ms = _time(lambda: first_conv_ln_gelu(x, w.detach(), b.detach(), lw.detach(), lb.detach(), s, T), a.iters, a.warmup)
    _emit("wav2vec2_first_conv_ln_gelu_fwd", ms, nbytes=B * T * C * 2.0 + B * L * 2.0, samples=B * L, channels=C)
    y = first_conv_ln_gelu(x, w, b, lw, lb, s, T)
    g = torch.randn_like(y)
    ms = _time(lambda: torch.autograd.grad(y, (w, b, lw, lb), g, retain_graph=True), a.iters, a.warmup)
    _emit("wav2vec2_first_conv_ln_gelu_bwd", ms, nbytes=B * T * C * 2.0 + B * L * 2.0, samples=B * L, channels=C)


def bench_swiglu2(a: argparse.Namespace) -> None:
    """Two-input SwiGLU of the expert path: capacity-sized buffers of which half the rows hold data."""
    from fairseq2_b200.ops.moe import swiglu_gate_up

    rows, F = 131072, 768
    g = torch.randn(rows, F, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    u = torch.randn(rows, F, device=_DEV, dtype=torch.bfloat16, requires_grad=True)
    nt = torch.tensor([rows // 256], device=_DEV, dtype=torch.int32)
    used = rows // 2
    ms = _time(lambda: swiglu_gate_up(g.detach(), u.detach(), nt), a.iters, a.warmup)
    _emit("swiglu_gate_up_bounded_fwd", ms, nbytes=3.0 * used * F * 2, rows_with_data=used, inner_dim=F)
    y = swiglu_gate_up(g, u, nt)
    dy = torch.randn_like(y)
    ms = _time(lambda: torch.autograd.grad(y, (g, u), dy, retain_graph=True), a.iters, a.warmup)
    _emit("swiglu_gate_up_bounded_bwd", ms, nbytes=5.0 * used * F * 2, rows_with_data=used, inner_dim=F)


def bench_add_norm(a: argparse.Namespace) -> None:
    from fairseq2_b200.ops.norm import add_rms_norm

    T, Dm = a.tokens, a.dim
    x = torch.randn(T, Dm, device=_DEV, dtype=torch.bfloat16)
    r = torch.randn(T, Dm, device=_DEV, dtype=torch.bfloat16)
    w = torch.ones(Dm, device=_DEV, dtype=torch.bfloat16)
    ms = _time(lambda: add_rms_norm(x, r, w, 1e-5), a.iters, a.warmup)
    _emit("add_rms_norm_fwd", ms, nbytes=4.0 * T * Dm * 2, tokens=T, dim=Dm)


_CASES = {"first_conv": bench_first_conv, "swiglu2": bench_swiglu2, "add_norm": bench_add_norm, "conv": bench_conv, "gemm": bench_gemm, "attention": bench_attention, "norm": bench_norm, "swiglu": bench_swiglu,
          "adamw": bench_adamw, "ce": bench_ce}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=[*_CASES, "all"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--a-mn", action="store_true", help="A is stored [K, M]")
    ap.add_argument("--b-mn", action="store_true", help="B is stored [K, N]")
    ap.add_argument("--compare", action="store_true", help="also time torch.matmul and report the relative error")
    ap.add_argument("--sustained", type=float, default=0.0,
                    help="gemm: also loop back to back for this many seconds and report the power-capped throughput")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--ffn-dim", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--doc-lens", default="", metavar="LO,HI", help="attention: packed documents of these lengths")
    ap.add_argument("--dropout", type=float, default=0.0, help="attention: dropout probability (mma.sync kernels)")
    ap.add_argument("--samples", type=int, default=1_400_000, help="first_conv: waveform samples per step")
    a = ap.parse_args()
    torch.manual_seed(0)
    for name in (_CASES if a.case == "all" else [a.case]):
        _CASES[name](a)


if __name__ == "__main__":
    main()
