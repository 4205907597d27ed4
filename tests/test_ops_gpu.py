"""Numerics of every sm_100a kernel against a plain PyTorch fp32 formulation of
the same op (the oracle lives next to each op as ``*_reference``)."""
from __future__ import annotations

import math

import pytest
import torch

from fairseq2_b200.ops import require_ext
from fairseq2_b200.ops.activation import swiglu, swiglu_reference
from fairseq2_b200.ops.attention import attention_reference, qkv_rope_attention, varlen_attention
from fairseq2_b200.ops.cross_entropy import cross_entropy_reference, fused_linear_cross_entropy
from fairseq2_b200.ops.gemm import gemm, gemm_reference, linear
from fairseq2_b200.ops.norm import layer_norm, rms_norm, rms_norm_reference
from fairseq2_b200.ops.optim import (adamw_reference, multi_tensor_adamw, multi_tensor_l2_norm_sq,
                                     multi_tensor_scale)
from fairseq2_b200.ops.rope import apply_rope, rope_reference

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp(min=1e-12))


@pytest.fixture(autouse=True)
def _status():
    ext = require_ext()
    ext.reset_status()
    yield
    torch.cuda.synchronize()
    assert ext.read_status() == 0, f"kernel status word = {ext.read_status():#x}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (200, 264, 72), (1024, 1536, 1024), (16, 24, 40)])
def test_gemm_layouts(a_mn: bool, b_mn: bool, shape: tuple[int, int, int]) -> None:
    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    out = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
    require_ext().gemm_bf16(a, b, out, a_mn, b_mn, False)
    assert _rel_err(out, ref) < 5e-3
    out32 = torch.empty((M, N), device=DEV, dtype=torch.float32)
    require_ext().gemm_bf16(a, b, out32, a_mn, b_mn, False)
    assert _rel_err(out32, ref) < 1e-4


def test_gemm_accumulate() -> None:
    torch.manual_seed(1)
    M, N, K = 384, 520, 320
    a = torch.randn((M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((N, K), device=DEV, dtype=torch.bfloat16)
    base = torch.randn((M, N), device=DEV, dtype=torch.float32)
    out = base.clone()
    require_ext().gemm_bf16(a, b, out, False, False, True)
    ref = base + gemm_reference(a, b, out_dtype=torch.float32)
    assert _rel_err(out, ref) < 1e-4
    outb = base.to(torch.bfloat16)
    require_ext().gemm_bf16(a, b, outb, False, False, True)
    assert _rel_err(outb, ref) < 1e-2


@pytest.mark.parametrize("pair", ["0", "1"])
def test_gemm_large_persistent(pair: str, monkeypatch: pytest.MonkeyPatch) -> None:
    """More tiles than SMs: exercises the persistent loop, both accumulators and every stage phase (single-CTA kernel
    and CTA-pair kernel)."""
    monkeypatch.setenv("FAIRSEQ2_B200_GEMM_PAIR", pair)
    torch.manual_seed(2)
    M, N, K = 4096, 4096, 2048
    a = torch.randn((M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((N, K), device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b)
    ref = torch.matmul(a, b.t())
    assert _rel_err(out, ref) < 5e-3


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_cta_pair_kernel(a_mn: bool, b_mn: bool, monkeypatch: pytest.MonkeyPatch) -> None:
    """The `cta_group::2` kernel (two CTAs per 256 x 256 tile): all operand layouts, a ragged M and N, bf16 and fp32
    outputs, accumulation, against an fp32 matmul."""
    monkeypatch.setenv("FAIRSEQ2_B200_GEMM_PAIR", "1")
    torch.manual_seed(12)
    M, N, K = 4096 + 136, 4096 + 72, 576                 # 17 x 17 tiles of 256 x 256, 9 K blocks
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    out = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
    require_ext().gemm_bf16(a, b, out, a_mn, b_mn, False)
    assert require_ext().read_status() == 0
    assert _rel_err(out, ref) < 5e-3
    out32 = torch.randn((M, N), device=DEV, dtype=torch.float32)
    base = out32.clone()
    require_ext().gemm_bf16(a, b, out32, a_mn, b_mn, True)
    assert _rel_err(out32, base + ref) < 1e-4


def test_gemm_cta_pair_tail_split(monkeypatch: pytest.MonkeyPatch) -> None:
    """A partial last wave of 256 x 256 tiles is cut along K and reduce-added: once into a zeroed bf16 output (long K,
    where zeroing pays) and once into an accumulated fp32 output."""
    monkeypatch.setenv("FAIRSEQ2_B200_GEMM_PAIR", "1")
    torch.manual_seed(13)
    M, N = 4096, 4096                                    # 256 tiles: three full waves of 74 pairs and 34 more
    for K, f32 in ((8192, False), (1024, True)):
        a = torch.randn((M, K), device=DEV, dtype=torch.bfloat16)
        b = torch.randn((N, K), device=DEV, dtype=torch.bfloat16)
        ref = gemm_reference(a, b, out_dtype=torch.float32)
        if f32:
            out = torch.randn((M, N), device=DEV, dtype=torch.float32)
            base = out.clone()
            require_ext().gemm_bf16(a, b, out, False, False, True)
            assert _rel_err(out, base + ref) < 1e-4
        else:
            out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
            require_ext().gemm_bf16(a, b, out, False, False, False)
            assert _rel_err(out, ref) < 5e-3
        assert require_ext().read_status() == 0


def test_linear_autograd() -> None:
    torch.manual_seed(3)
    x = torch.randn((4, 96, 256), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn((384, 256), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 5e-3
    assert _rel_err(x.grad, xr.grad) < 5e-3
    assert _rel_err(w.grad, wr.grad) < 5e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,D", [(7, 64), (300, 4096), (33, 1024), (5, 8192)])
def test_rms_norm(dtype: torch.dtype, rows: int, D: int) -> None:
    torch.manual_seed(4)
    x = torch.randn((rows, D), device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(dtype).requires_grad_(True)
    y = rms_norm(x, (D,), w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = rms_norm_reference(xr, wr, 1e-5)
    yr.backward(g.float())
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(y, yr) < tol
    assert _rel_err(x.grad, xr.grad) < tol
    assert _rel_err(w.grad, wr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,D", [(7, 64), (300, 4096), (5, 8192)])
def test_add_rms_norm_fused_residual(dtype: torch.dtype, rows: int, D: int) -> None:
    """Residual add + RMSNorm in one kernel (and the residual gradient added in its backward) against the two
    separate fp32 operations; both outputs, the sum and the normalised sum, carry gradients."""
    from fairseq2_b200.ops.norm import add_rms_norm

    torch.manual_seed(5)
    x = torch.randn((rows, D), device=DEV, dtype=dtype, requires_grad=True)
    r = torch.randn((rows, D), device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(dtype).requires_grad_(True)
    h, y = add_rms_norm(x, r, w, 1e-5)
    gh, gy = torch.randn_like(h), torch.randn_like(y)
    torch.autograd.backward([h, y], [gh, gy])
    xr, rr, wr = (t.detach().double().requires_grad_(True) for t in (x, r, w))
    hr = xr + rr
    hq = hr + (hr.to(dtype).double() - hr).detach()          # the kernel rounds the sum to the activation dtype
    yr = hq * torch.rsqrt(hq.pow(2).mean(dim=-1, keepdim=True) + 1e-5)
    yr = (yr + (yr.to(dtype).double() - yr).detach()) * wr
    torch.autograd.backward([hr, yr], [gh.double(), gy.double()])
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(h, hr) < tol and _rel_err(y, yr) < tol
    assert _rel_err(x.grad, xr.grad) < tol and _rel_err(r.grad, rr.grad) < tol
    assert _rel_err(w.grad, wr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_layer_norm(dtype: torch.dtype) -> None:
    torch.manual_seed(5)
    rows, D = 130, 1024
    x = torch.randn((rows, D), device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(dtype).requires_grad_(True)
    b = (0.1 * torch.randn(D, device=DEV)).to(dtype).requires_grad_(True)
    y = layer_norm(x, (D,), w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (D,), wr, br, 1e-5)
    yr.backward(g.float())
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(y, yr) < tol
    assert _rel_err(x.grad, xr.grad) < tol
    assert _rel_err(w.grad, wr.grad) < tol
    assert _rel_err(b.grad, br.grad) < tol


def test_swiglu() -> None:
    torch.manual_seed(6)
    gu = torch.randn((77, 2 * 1024), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_(True)
    yr = swiglu_reference(gr)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(gu.grad, gr.grad) < 1e-2


def _freqs(L: int, D: int, theta: float = 10000.0) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=DEV, dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(L, device=DEV, dtype=torch.float32), inv)
    return torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()


def test_rope() -> None:
    torch.manual_seed(7)
    T, H, D = 50, 6, 128
    x = torch.randn((T, H, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    pos = torch.arange(T, device=DEV, dtype=torch.int32) % 23
    pos[-3:] = -1
    f = _freqs(64, D)
    y = apply_rope(x, f, pos)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    yr = rope_reference(xr, f, pos)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2


def _seqs(lens: list[int]):
    b = [0]
    for l in lens:
        b.append(b[-1] + l)
    return (torch.tensor(b[:-1], device=DEV, dtype=torch.int32), torch.tensor(lens, device=DEV, dtype=torch.int32))


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D,H,Hkv", [(128, 8, 2), (64, 4, 4)])
@pytest.mark.parametrize("lens", [[5], [64, 128], [1, 37, 200, 130], [300, 77]])
def test_attention_fwd_bwd(causal: bool, D: int, H: int, Hkv: int, lens: list[int]) -> None:
    torch.manual_seed(8)
    T = sum(lens)
    q = torch.randn((T, H, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b, l = _seqs(lens)
    out = varlen_attention(q, k, v, b, l, b, l, max(lens), max(lens), causal=causal)
    g = torch.randn_like(out)
    out.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, b, l, b, l, causal)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    assert _rel_err(q.grad, qr.grad) < 2e-2
    assert _rel_err(k.grad, kr.grad) < 2e-2
    assert _rel_err(v.grad, vr.grad) < 2e-2


def _dropout_keep_mask(seed: int, H: int, q_tok: torch.Tensor, k_tok: torch.Tensor, p: float) -> torch.Tensor:
    """Host restatement of the kernels' stateless dropout hash -> bool [H, Lq, Lk] (True = kept)."""
    import numpy as np

    def mix(a):  # type: ignore[no-untyped-def]
        a = a.astype(np.uint32)
        a ^= a >> np.uint32(16)
        a = (a.astype(np.uint64) * np.uint64(0x85EBCA6B)).astype(np.uint32)
        a ^= a >> np.uint32(13)
        a = (a.astype(np.uint64) * np.uint64(0xC2B2AE35)).astype(np.uint32)
        a ^= a >> np.uint32(16)
        return a

    lo, hi = np.uint32(seed & 0xFFFFFFFF), np.uint32((seed >> 32) & 0xFFFFFFFF)
    q = q_tok.cpu().numpy().astype(np.uint32)[None, :, None]
    k = k_tok.cpu().numpy().astype(np.uint64)[None, None, :]
    h = np.arange(H, dtype=np.uint64)[:, None, None]
    a = mix(q ^ lo).astype(np.uint64)
    a = (a + k * np.uint64(0x9E3779B1) + h * np.uint64(0x7F4A7C15) + np.uint64(hi)).astype(np.uint32)   # mod 2^32
    a = mix(a)
    thr = np.uint32(min(4294967295.0, max(1.0, p * 4294967296.0)))
    return torch.from_numpy(a >= thr)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D,H,Hkv", [(64, 4, 4), (128, 8, 2)])
def test_attention_dropout_matches_masked_reference(causal: bool, D: int, H: int, Hkv: int) -> None:
    """Dropout inside the attention kernels: forward and all gradients against the fp32 formulation that applies
    the same (hash-derived) mask, plus the keep rate."""
    torch.manual_seed(3)
    lens, p_drop, seed = [150, 70, 257], 0.25, 0x1234_5678_9ABC
    T = sum(lens)
    q = torch.randn((T, H, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b, l = _seqs(lens)
    out = varlen_attention(q, k, v, b, l, b, l, max(lens), max(lens), causal=causal, dropout_p=p_drop, seed=seed)
    g = torch.randn_like(out)
    out.backward(g)
    qr, kr, vr = (t.detach().float().cpu().requires_grad_(True) for t in (q, k, v))
    ref = torch.zeros(T, H, D)
    kept = total = 0
    off = 0
    for n in lens:
        tok = torch.arange(off, off + n)
        mask = _dropout_keep_mask(seed, H, tok, tok, p_drop)
        qs = qr[off:off + n].transpose(0, 1)
        ks = kr[off:off + n].transpose(0, 1).repeat_interleave(H // Hkv, 0)
        vs = vr[off:off + n].transpose(0, 1).repeat_interleave(H // Hkv, 0)
        s = qs @ ks.transpose(1, 2) * D ** -0.5
        if causal:
            s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
        pr = torch.softmax(s, -1) * mask / (1 - p_drop)
        ref = ref + torch.nn.functional.pad((pr @ vs).transpose(0, 1), (0, 0, 0, 0, off, T - off - n))
        kept += int(mask.sum())
        total += mask.numel()
        off += n
    ref.backward(g.float().cpu())
    assert abs(kept / total - (1 - p_drop)) < 0.01
    assert _rel_err(out.float().cpu(), ref.detach()) < 1.5e-2
    assert _rel_err(q.grad.float().cpu(), qr.grad) < 2.5e-2
    assert _rel_err(k.grad.float().cpu(), kr.grad) < 2.5e-2
    assert _rel_err(v.grad.float().cpu(), vr.grad) < 2.5e-2
    # another seed gives another mask; p = 0 is the plain kernel
    out2 = varlen_attention(q, k, v, b, l, b, l, max(lens), max(lens), causal=causal, dropout_p=p_drop, seed=seed + 1)
    assert _rel_err(out2.float(), out.float()) > 0.1


@pytest.mark.parametrize("causal", [True, False])
def test_attention_long_sequences(causal: bool) -> None:
    """Many key/value tiles per query tile: exercises the ring phases of the tcgen05 forward kernel."""
    torch.manual_seed(12)
    H, Hkv, D = 4, 2, 128
    lens = [1500, 700, 129, 1]
    T = sum(lens)
    q = torch.randn((T, H, D), device=DEV, dtype=torch.bfloat16)
    k = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16)
    v = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16)
    b, l = _seqs(lens)
    out = varlen_attention(q, k, v, b, l, b, l, max(lens), max(lens), causal=causal)
    ref = attention_reference(q.float(), k.float(), v.float(), b, l, b, l, causal)
    assert _rel_err(out, ref) < 1e-2
    from fairseq2_b200.ops._ext import require_ext

    assert require_ext().read_status() == 0


@pytest.mark.parametrize("window", [1, 50, 128, 300, 5000])
def test_attention_sliding_window(window: int) -> None:
    """Causal attention restricted to the `window` most recent keys (tcgen05 kernels, head_dim 128): key tiles
    before the window are skipped, the tile at its edge is masked; forward and all three gradients."""
    torch.manual_seed(21)
    H, Hkv, D = 4, 2, 128
    lens = [700, 129, 1, 333]
    T = sum(lens)
    q = torch.randn((T, H, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn((T, Hkv, D), device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b, l = _seqs(lens)
    out = varlen_attention(q, k, v, b, l, b, l, max(lens), max(lens), causal=True, window=window)
    g = torch.randn_like(out)
    out.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, b, l, b, l, True, None, window)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    if window > 1:
        assert _rel_err(q.grad, qr.grad) < 2e-2
        assert _rel_err(k.grad, kr.grad) < 2e-2
    else:       # a softmax over one key is constant: dq and dk vanish
        assert float(q.grad.float().abs().max()) < 1e-4 and float(k.grad.float().abs().max()) < 1e-4
    assert _rel_err(v.grad, vr.grad) < 2e-2
    from fairseq2_b200.ops._ext import require_ext

    assert require_ext().read_status() == 0


def test_attention_cross_lengths() -> None:
    """Lk > Lq (prefill against a cache): bottom-right aligned causal mask."""
    torch.manual_seed(9)
    H, Hkv, D = 4, 2, 128
    ql, kl = [3, 70], [40, 133]
    q = torch.randn((sum(ql), H, D), device=DEV, dtype=torch.bfloat16)
    k = torch.randn((sum(kl), Hkv, D), device=DEV, dtype=torch.bfloat16)
    v = torch.randn((sum(kl), Hkv, D), device=DEV, dtype=torch.bfloat16)
    qb, qlt = _seqs(ql)
    kb, klt = _seqs(kl)
    out = varlen_attention(q, k, v, qb, qlt, kb, klt, max(ql), max(kl), causal=True)
    ref = attention_reference(q.float(), k.float(), v.float(), qb, qlt, kb, klt, True)
    assert _rel_err(out, ref) < 1e-2


def test_qkv_rope_attention_fused() -> None:
    torch.manual_seed(10)
    H, Hkv, D = 8, 2, 128
    lens = [100, 28, 129]
    T = sum(lens)
    qkv = torch.randn((T, H + 2 * Hkv, D), device=DEV, dtype=torch.bfloat16)
    b, l = _seqs(lens)
    pos = torch.cat([torch.arange(n, device=DEV, dtype=torch.int32) for n in lens])
    f = _freqs(256, D)
    leaf = qkv.clone().requires_grad_(True)
    out = qkv_rope_attention(leaf * 1.0, f, pos, b, l, max(lens), num_heads=H, num_kv_heads=Hkv, causal=True)
    g = torch.randn_like(out)
    out.backward(g)
    ref_leaf = qkv.detach().float().requires_grad_(True)
    qr = rope_reference(ref_leaf[:, :H], f, pos)
    kr = rope_reference(ref_leaf[:, H:H + Hkv], f, pos)
    ref = attention_reference(qr, kr, ref_leaf[:, H + Hkv:], b, l, b, l, True)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    assert _rel_err(leaf.grad, ref_leaf.grad) < 2e-2


def test_fused_linear_cross_entropy() -> None:
    torch.manual_seed(11)
    T, D, V = 300, 256, 1024
    h = (0.5 * torch.randn((T, D), device=DEV)).to(torch.bfloat16).requires_grad_(True)
    w = (0.05 * torch.randn((V, D), device=DEV)).to(torch.bfloat16).requires_grad_(True)
    t = torch.randint(0, V, (T,), device=DEV)
    t[5] = 7
    mask = (torch.rand(T, device=DEV) > 0.3)
    loss = fused_linear_cross_entropy(h, w, t, target_mask=mask, pad_idx=7, reduction="sum", chunk_size=128)
    (loss * 0.5).backward()
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lr = cross_entropy_reference(torch.nn.functional.linear(hr, wr), t, 7, target_mask=mask, reduction="sum")
    (lr * 0.5).backward()
    assert abs(float(loss) - float(lr)) / abs(float(lr)) < 5e-3
    assert _rel_err(h.grad, hr.grad) < 2e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adamw_and_norm(gdtype: torch.dtype) -> None:
    torch.manual_seed(12)
    n = 100_003 - 3  # multiple of 8 keeps the flat views aligned
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV).to(gdtype)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    low = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    scale = torch.tensor(0.5, device=DEV)
    for step in (1, 2, 3):
        multi_tensor_adamw([p], [g], [m], [v], [low], lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                           step=step, grad_scale=scale)
        adamw_reference(pr, g, mr, vr, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                        grad_scale=0.5)
    assert _rel_err(p, pr) < 1e-5
    assert _rel_err(m, mr) < 1e-5
    assert _rel_err(v, vr) < 1e-5
    assert _rel_err(low, pr) < 5e-3
    nsq = multi_tensor_l2_norm_sq([g, p])
    ref = g.float().pow(2).sum() + p.pow(2).sum()
    assert abs(float(nsq) - float(ref)) / float(ref) < 1e-4
    gc = g.clone()
    multi_tensor_scale([gc], scale)
    assert _rel_err(gc, g.float() * 0.5) < 5e-3


# ------------------------------------------------------------------ generation kernels
@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_ngram_repeat_block_kernel(n: int) -> None:
    from fairseq2_b200.ops.sampling import ngram_repeat_block, ngram_repeat_block_reference

    torch.manual_seed(n)
    seqs = torch.randint(0, 6, (9, 37), device="cuda")
    probs = torch.rand(9, 50, device="cuda")
    ref = probs.clone()
    ngram_repeat_block_reference(seqs, ref, n, 0.0)
    ngram_repeat_block(seqs, probs, n, 0.0)
    assert torch.equal(probs, ref)


@pytest.mark.gpu
@pytest.mark.parametrize("V", [1000, 32000, 128256])
def test_sample_kernel_support_matches_reference(V: int) -> None:
    """Every sampled token must lie in the reference's kept set, and extreme uniforms must hit its ends."""
    from fairseq2_b200.ops.sampling import sample_top_p_top_k

    torch.manual_seed(0)
    N = 16
    probs = torch.softmax(torch.randn(N, V, device="cuda") * 3, dim=-1)
    for p, k in ((0.9, 0), (0.5, 0), (1.0, 10), (1.0, 1), (0.7, 50)):
        sp, si = torch.sort(probs, dim=-1, descending=True)
        keep = torch.ones_like(sp, dtype=torch.bool)
        if p < 1.0:
            keep &= (torch.cumsum(sp, -1) - sp) <= p
        if k > 0:
            keep &= torch.arange(V, device="cuda")[None, :] < k
        kept = torch.zeros_like(keep).scatter(1, si, keep)
        for _ in range(4):
            u = torch.rand(N, device="cuda")
            tok = sample_top_p_top_k(probs, p=p, k=k, uniform=u)
            assert bool(kept.gather(1, tok[:, None]).all()), (p, k)
        # u -> 0 picks the first kept index, u -> 1 the last
        first = kept.float().argmax(dim=1)
        last = V - 1 - kept.flip(1).float().argmax(dim=1)
        assert torch.equal(sample_top_p_top_k(probs, p=p, k=k, uniform=torch.zeros(N, device="cuda")), first)
        assert torch.equal(sample_top_p_top_k(probs, p=p, k=k, uniform=torch.ones(N, device="cuda")), last)


@pytest.mark.gpu
def test_sample_kernel_distribution() -> None:
    from fairseq2_b200.ops.sampling import sample_top_p_top_k

    torch.manual_seed(1)
    V, draws = 64, 40000
    base = torch.softmax(torch.randn(V, device="cuda"), dim=-1)
    probs = base.expand(draws, V).contiguous()
    tok = sample_top_p_top_k(probs, p=0.8, k=0, uniform=torch.rand(draws, device="cuda"))
    sp, si = torch.sort(base, descending=True)
    keep = (torch.cumsum(sp, 0) - sp) <= 0.8
    expect = torch.zeros(V, device="cuda").scatter(0, si, sp * keep)
    expect = expect / expect.sum()
    freq = torch.bincount(tok, minlength=V).float() / draws
    assert float((freq - expect).abs().max()) < 0.01


@pytest.mark.gpu
@pytest.mark.parametrize("beams,V,k", [(1, 1000, 2), (4, 32000, 8), (5, 128256, 10)])
def test_beam_topk_kernel(beams: int, V: int, k: int) -> None:
    from fairseq2_b200.ops.sampling import beam_topk, beam_topk_reference

    torch.manual_seed(0)
    lp = torch.log_softmax(torch.randn(3, beams, V, device="cuda"), dim=-1)
    sc = torch.randn(3, beams, device="cuda")
    s, i = beam_topk(lp, sc, k)
    rs, ri = beam_topk_reference(lp, sc, k)
    assert torch.allclose(s, rs) and torch.equal(i, ri)


# ------------------------------------------------------------------------- MoE kernels
@pytest.mark.gpu
@pytest.mark.parametrize("E,k,softmax", [(16, 1, False), (128, 2, True), (8, 2, False)])
def test_moe_route_kernel(E: int, k: int, softmax: bool) -> None:
    from fairseq2_b200.ops.moe import moe_route, moe_route_reference

    torch.manual_seed(0)
    logits = torch.randn(777, E, device="cuda", dtype=torch.bfloat16)
    ids, gates, counts = moe_route(logits, k, softmax)
    rids, rgates, rcounts = moe_route_reference(logits, k, softmax)
    # bf16 logits tie often; the kernel breaks ties toward the smaller index while torch.topk leaves the order
    # unspecified, so compare the selected values and check the histogram against the kernel's own ids
    lf = logits.float()
    assert torch.equal(lf.gather(1, ids.long()), lf.gather(1, rids))
    assert torch.equal(counts.long(), torch.bincount(ids.long().reshape(-1), minlength=E))
    untied = lf.gather(1, rids)[:, -1:] != torch.topk(lf, k + 1, dim=1).values[:, -1:]
    assert torch.equal(torch.where(untied, ids.long(), rids).sort(dim=1).values, rids.sort(dim=1).values)
    assert torch.allclose(gates, rgates, atol=1e-5)


@pytest.mark.gpu
def test_moe_layer_kernels_match_reference_path() -> None:
    """The fused routing/dispatch/grouped-GEMM/combine path (bf16, CUDA) against the same layer evaluated in fp32
    on the CPU with the index_select/index_add formulation, forward and backward."""
    import copy

    from fairseq2_b200.models.transformer.experts import MoE
    from fairseq2_b200.ops import _ext

    torch.manual_seed(0)
    moe = MoE(256, 512, True, 8, 1.0, 2, inner_dim_scale=1.0).to("cuda", torch.bfloat16)
    oracle = copy.deepcopy(moe).to("cpu", torch.float32)
    x = torch.randn(300, 256, device="cuda", dtype=torch.bfloat16)
    xi = x.clone().requires_grad_(True)
    y = moe(xi)
    (y.float() ** 2).sum().backward()
    xo = x.detach().cpu().float().requires_grad_(True)
    with _ext.kernels_enabled(False):
        yo = oracle(xo)
        (yo ** 2).sum().backward()
    # Routing is discrete: a token whose two best router logits are closer than a bf16 rounding step may be sent
    # to a different expert than in fp32. Per-token results must therefore agree for (almost) all tokens, the
    # parameter gradients (sums over all tokens) within a tolerance that leaves room for those few.
    def row_err(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        a, b = a.detach().float().cpu(), b.detach().float()
        return (a - b).norm(dim=-1) / b.norm(dim=-1).clamp(min=1e-6)

    for name, a, b in (("y", y, yo), ("dx", xi.grad, xo.grad)):
        e = row_err(a, b)
        frac = float((e < 3e-2).float().mean())
        assert frac >= 0.97, f"{name}: only {frac:.3f} of the tokens within 3e-2 (median {float(e.median()):.2e})"
    for name, a, b in (("router.grad", moe.router.grad, oracle.router.grad),
                       ("gate_proj.grad", moe.experts.gate_proj.grad, oracle.experts.gate_proj.grad)):
        err = _rel_err(a.detach().cpu(), b.detach())
        assert err < 8e-2, f"{name}: relative error {err:.3e}"


# ------------------------------------------------------------------- speech feature encoder kernels
@pytest.mark.gpu
@pytest.mark.parametrize("B,L,C,C_out,k,s", [(3, 640, 512, 512, 3, 2), (2, 250, 64, 128, 2, 2), (1, 96, 8, 8, 10, 4)])
def test_conv1d_channels_last_view_gemm(B: int, L: int, C: int, C_out: int, k: int, s: int) -> None:
    from fairseq2_b200.ops.conv import conv1d_channels_last, conv1d_cl_reference, conv1d_cl_supported

    torch.manual_seed(0)
    x = torch.randn(B, L, C, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    w = (torch.randn(C_out, C, k, device="cuda") * (C * k) ** -0.5).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(C_out, device="cuda", dtype=torch.bfloat16)
    assert conv1d_cl_supported(x, w, s)
    T_out = (L - k) // s + 1                                   # rows that are true convolution outputs
    y = conv1d_channels_last(x, w, b, s)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = conv1d_cl_reference(xr, wr, b.float(), s)
    assert y.shape == (B, L // s, C_out)
    assert _rel_err(y[:, :T_out].float(), ref[:, :T_out]) < 1e-2
    g = torch.randn(B, T_out, C_out, device="cuda", dtype=torch.bfloat16)
    y[:, :T_out].backward(g)                                   # the invalid tail rows receive zero gradient
    ref[:, :T_out].backward(g.float())
    assert _rel_err(w.grad.float(), wr.grad) < 1.5e-2
    assert _rel_err(x.grad.float(), xr.grad) < 1.5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,C,stride,with_ln,with_bias", [(3, 4003, 512, 5, True, True), (2, 1500, 256, 5, True, False),
                                                            (2, 977, 768, 4, False, True), (1, 50_000, 512, 5, True, True)])
def test_wav2vec2_first_conv_fused(B: int, L: int, C: int, stride: int, with_ln: bool, with_bias: bool) -> None:
    """conv (1 input channel, width 10) + bias + LayerNorm + GELU in one kernel and its recomputing backward against
    the fp32 formulation on the CPU: output (valid rows and zeroed padding) and all parameter gradients."""
    from fairseq2_b200.ops.conv import first_conv_ln_gelu, first_conv_reference, first_conv_supported

    torch.manual_seed(0)
    k = 10
    x = torch.randn(B, L, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(C, 1, k, device="cuda") * (2.0 / k) ** 0.5).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(C, device="cuda")).to(torch.bfloat16).requires_grad_(True) if with_bias else None
    lw = (1 + 0.1 * torch.randn(C, device="cuda")).to(torch.bfloat16).requires_grad_(True) if with_ln else None
    lb = (0.1 * torch.randn(C, device="cuda")).to(torch.bfloat16).requires_grad_(True) if with_ln else None
    assert first_conv_supported(x, w)
    t_valid = (L - k) // stride + 1
    t_pad = (t_valid + 63) // 64 * 64
    y = first_conv_ln_gelu(x, w, b, lw, lb, stride, t_pad, 1e-5)
    assert y.shape == (B, t_pad, C) and y.dtype == torch.bfloat16
    params = [t for t in (w, b, lw, lb) if t is not None]
    cpu = [t.detach().float().cpu().requires_grad_(True) for t in params]
    it = iter(cpu)
    wr = next(it)
    br = next(it) if with_bias else None
    lwr, lbr = (next(it), next(it)) if with_ln else (None, None)
    ref = first_conv_reference(x.float().cpu(), wr, br, lwr, lbr, stride, t_pad, 1e-5)
    assert _rel_err(y[:, :t_valid].float().cpu(), ref[:, :t_valid].detach()) < 1e-2
    assert float(y[:, t_valid:].abs().max()) == 0.0 if t_pad > t_valid else True
    g = torch.randn(B, t_pad, C, device="cuda", dtype=torch.bfloat16)
    y.backward(g)
    ref[:, :t_valid].backward(g[:, :t_valid].float().cpu())
    for got, want in zip(params, cpu):
        assert _rel_err(got.grad.float().cpu(), want.grad) < 2e-2, (got.shape, _rel_err(got.grad.float().cpu(), want.grad))


@pytest.mark.gpu
def test_layer_norm_gelu_fused() -> None:
    from fairseq2_b200.ops.norm import layer_norm_gelu

    torch.manual_seed(0)
    x = torch.randn(1000, 512, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(512, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(512, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    y = layer_norm_gelu(x, w, b, 1e-5)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    ref = torch.nn.functional.gelu(torch.nn.functional.layer_norm(xr, (512,), wr, br, 1e-5))
    assert _rel_err(y.float(), ref) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float())
    assert _rel_err(x.grad.float(), xr.grad) < 1.5e-2
    assert _rel_err(w.grad.float(), wr.grad) < 1.5e-2 and _rel_err(b.grad.float(), br.grad) < 1.5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_wav2vec2_contrastive_kernel(dtype: torch.dtype) -> None:
    from fairseq2_b200.ops.wav2vec2 import contrastive_logits_and_loss, contrastive_reference

    torch.manual_seed(0)
    P, K, M = 333, 100, 256
    x = torch.randn(P, M, device="cuda").to(dtype).requires_grad_(True)
    t = torch.randn(P, M, device="cuda").to(dtype)
    t[7] = t[3]                                                # a distractor identical to a target must give -inf
    t = t.requires_grad_(True)
    d = torch.randint(0, P, (P, K), device="cuda", dtype=torch.int32)
    d[3, 5] = 7
    logits, loss = contrastive_logits_and_loss(x, t, d, 0.1)
    xr, tr = x.detach().float().requires_grad_(True), t.detach().float().requires_grad_(True)
    rlogits, rloss = contrastive_reference(xr, tr, d, 0.1)
    assert torch.isinf(logits[3, 6]) and torch.isinf(rlogits[3, 6])
    fin = torch.isfinite(rlogits)
    assert torch.equal(fin, torch.isfinite(logits))
    assert torch.allclose(logits[fin], rlogits[fin], atol=2e-3)
    assert abs(float(loss) - float(rloss)) / float(rloss) < 1e-3
    (loss * 0.5).backward()
    (rloss * 0.5).backward()
    assert _rel_err(x.grad.float(), xr.grad) < 1e-2 and _rel_err(t.grad.float(), tr.grad) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("training", [True, False])
def test_wav2vec2_gumbel_quantizer_kernel(training: bool) -> None:
    from fairseq2_b200.ops.wav2vec2 import gumbel_quantize, gumbel_quantize_reference, sample_gumbel_noise

    torch.manual_seed(0)
    frames, G, V, E = 257, 2, 320, 128
    logits = torch.randn(frames * G, V, device="cuda").requires_grad_(True)
    entries = torch.rand(G * V, E, device="cuda").requires_grad_(True)
    noise = sample_gumbel_noise((frames * G, V), logits.device) if training else None
    q, sel, prob_sum, hard = gumbel_quantize(logits, noise, entries, G, 1.7, training)
    lr, er = logits.detach().clone().requires_grad_(True), entries.detach().clone().requires_grad_(True)
    rq, rsel, rprob, rhard = gumbel_quantize_reference(lr, noise, er, G, 1.7, training)
    assert torch.equal(sel.long(), rsel) and torch.allclose(hard, rhard) and torch.allclose(prob_sum, rprob, atol=1e-4)
    rows = torch.arange(frames * G, device="cuda")
    assert torch.equal(q, entries.detach().view(G, V, E)[rows % G, sel.long()])      # an exact code-book lookup
    assert torch.allclose(q, rq, atol=2e-3)                # the dense oracle may run its contraction in TF32
    if training:
        w = torch.randn_like(q)
        (q * w).sum().backward()
        (rq * w).sum().backward()
        assert _rel_err(logits.grad, lr.grad) < 5e-3 and _rel_err(entries.grad, er.grad) < 5e-3


@pytest.mark.gpu
@pytest.mark.parametrize("layer_norm", [True, False])
def test_wav2vec2_feature_extractor_channels_last_path(layer_norm: bool) -> None:
    """The GEMM-on-views path of the feature extractor against the Conv1d path, forward and weight gradients."""
    from fairseq2_b200.models.wav2vec2.feature_extractor import Wav2Vec2FeatureExtractor
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.ops import _ext

    import copy

    torch.manual_seed(0)
    descs = [(64, 10, 5), (64, 3, 2), (64, 3, 2), (64, 2, 2)]
    fe = Wav2Vec2FeatureExtractor(descs, bias=layer_norm, layer_norm=layer_norm).to("cuda", torch.bfloat16)
    oracle = copy.deepcopy(fe).to("cpu", torch.float32)      # fp32 Conv1d path on the CPU: no TF32, no bf16
    wave = torch.randn(3, 4000, device="cuda", dtype=torch.bfloat16)
    layout = BatchLayout((3, 4000), [4000, 3300, 2801], device=wave.device)
    assert fe._channels_last_ok(wave.unsqueeze(1))
    y, y_layout = fe(wave, layout)
    g = torch.randn(y.shape, device="cuda", dtype=torch.bfloat16, generator=torch.Generator("cuda").manual_seed(1))
    (y.float() * g.float()).sum().backward()
    with _ext.kernels_enabled(False):
        yo, _ = oracle(wave.cpu().float(), BatchLayout((3, 4000), [4000, 3300, 2801], device=torch.device("cpu")))
        (yo * g.cpu().float()).sum().backward()
    assert y.shape == yo.shape and list(y_layout.seq_lens) == fe._contract_seq_lens([4000, 3300, 2801])
    assert _rel_err(y.cpu(), yo) < 2e-2
    for p, po in zip(fe.parameters(), oracle.parameters()):
        assert _rel_err(p.grad.cpu(), po.grad) < 5e-2


@pytest.mark.gpu
def test_grouped_gemm_single_launch_padded_layout() -> None:
    """Device-resident routing tables: forward, dgrad and per-expert wgrad of the single-launch grouped GEMM against
    a per-expert fp32 loop; one expert receives no token."""
    from fairseq2_b200.ops.grouped_gemm import grouped_mm_device
    from fairseq2_b200.ops.moe import moe_dispatch_padded

    torch.manual_seed(0)
    T, K, N, E, k = 700, 256, 384, 8, 2
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, E - 1, (T, k), device="cuda", dtype=torch.int32)       # expert E-1 stays empty
    ids[:, 1] = (ids[:, 0] + 1 + ids[:, 1] % (E - 2)) % (E - 1)                   # two distinct experts per token
    gates = torch.rand(T, k, device="cuda")
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E).to(torch.int32)
    w = (torch.randn(E, K, N, device="cuda") * K ** -0.5).to(torch.bfloat16).requires_grad_(True)
    xin = x.clone().requires_grad_(True)
    routed, src_row, inv, layout = moe_dispatch_padded(xin, gates, ids, counts)
    assert routed.shape[0] % 128 == 0 and int(layout[3]) == sum(max((int(c) + 127) // 128, 1) for c in counts)
    y = grouped_mm_device(routed, w, layout)
    g = torch.randn_like(y) * (src_row >= 0).unsqueeze(1)
    y.backward(g)
    # oracle: rows of the padded buffer, expert by expert
    offsets = layout[0].tolist()
    wr = w.detach().float().requires_grad_(True)
    rr = routed.detach().float().requires_grad_(True)
    ref = torch.zeros(routed.shape[0], N, device="cuda")
    for e in range(E):
        ref[offsets[e]:offsets[e + 1]] = rr[offsets[e]:offsets[e + 1]] @ wr[e]
    ref.backward(g.float())
    used = int(layout[3]) * 128                # rows past the last tile are never written (nor read by a consumer)
    assert offsets[-1] == used
    assert _rel_err(y[:used].float(), ref[:used].detach()) < 1e-2
    assert _rel_err(w.grad.float(), wr.grad) < 1.5e-2
    assert float(w.grad[E - 1].abs().max()) == 0.0                                 # the empty expert gets a zero gradient
    # gradient reaching x through dispatch: sum_j gate * d_routed[inv]
    dxr = torch.zeros(T, K, device="cuda")
    for j in range(k):
        dxr += gates[:, j:j + 1] * rr.grad[inv[:, j].long()]
    assert _rel_err(xin.grad.float(), dxr) < 1.5e-2


@pytest.mark.gpu
def test_embed_vocab_parallel_kernel() -> None:
    from fairseq2_b200.ops.embedding import embed_vocab_parallel, embed_vocab_parallel_reference

    torch.manual_seed(0)
    V, D, lo = 1000, 256, 250
    shard = torch.randn(250, D, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    ids = torch.randint(0, V, (7, 123), device="cuda")
    out = embed_vocab_parallel(ids, shard, lo)
    sr = shard.detach().float().requires_grad_(True)
    ref = embed_vocab_parallel_reference(ids, sr, lo)
    assert torch.equal(out.float(), ref.detach())
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    assert _rel_err(shard.grad.float(), sr.grad) < 1e-2


@pytest.mark.gpu
def test_swiglu_gate_up_and_bounded_copy() -> None:
    """Two-input SwiGLU bounded by a device-resident tile count (fp32 oracle on the rows that hold data; rows beyond
    the bound are neither read nor written) and the bounded row copy."""
    from fairseq2_b200.ops import require_ext
    from fairseq2_b200.ops.moe import swiglu_gate_up

    torch.manual_seed(0)
    rows, F, tiles = 1024, 768, 5
    g = torch.randn(rows, F, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    u = torch.randn(rows, F, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    with torch.no_grad():
        g[tiles * 128:] = float("nan")                          # must never be looked at
    nt = torch.tensor([tiles], device="cuda", dtype=torch.int32)
    y = swiglu_gate_up(g, u, nt)
    n = tiles * 128
    gr, ur = g.detach()[:n].float().cpu().requires_grad_(True), u.detach()[:n].float().cpu().requires_grad_(True)
    ref = torch.nn.functional.silu(gr) * ur
    assert _rel_err(y[:n].float().cpu(), ref.detach()) < 1e-2
    dy = torch.randn(rows, F, device="cuda", dtype=torch.bfloat16)
    y.backward(dy)
    ref.backward(dy[:n].float().cpu())
    assert _rel_err(g.grad[:n].float().cpu(), gr.grad) < 1.5e-2 and _rel_err(u.grad[:n].float().cpu(), ur.grad) < 1.5e-2
    # unbounded form
    y2 = swiglu_gate_up(g.detach()[:n], u.detach()[:n])
    assert torch.equal(y2, y[:n])
    src = torch.randn(rows, 256, device="cuda", dtype=torch.bfloat16)
    dst = torch.full_like(src, 7.0)
    require_ext().copy_rows_bounded(dst, src, nt)
    assert torch.equal(dst[:n], src[:n]) and bool((dst[n:] == 7.0).all())
    require_ext().copy_rows_bounded(dst, src)
    assert torch.equal(dst, src)


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,C,G,k", [(3, 200, 1024, 16, 128), (2, 77, 256, 4, 9)])
def test_grouped_conv1d_channels_last(B: int, T: int, C: int, G: int, k: int) -> None:
    """The grouped same-padded convolution of the wav2vec 2.0 position encoder as one view GEMM per group: output
    and all gradients against ``F.conv1d`` in fp32 on the CPU."""
    from fairseq2_b200.ops.conv import grouped_conv1d_channels_last, grouped_conv1d_supported

    torch.manual_seed(0)
    x = torch.randn(B, T, C, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    w = (torch.randn(C, C // G, k, device="cuda") * (k * C // G) ** -0.5).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(C, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    assert grouped_conv1d_supported(x, w, G)
    y = grouped_conv1d_channels_last(x, w, b, G, k // 2)
    xr, wr, br = (t.detach().float().cpu().requires_grad_(True) for t in (x, w, b))
    ref = torch.nn.functional.conv1d(xr.transpose(1, 2), wr, br, padding=k // 2, groups=G).transpose(1, 2)
    assert y.shape == ref.shape
    assert _rel_err(y.float().cpu(), ref.detach()) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float().cpu())
    assert _rel_err(x.grad.float().cpu(), xr.grad) < 2e-2
    assert _rel_err(w.grad.float().cpu(), wr.grad) < 2e-2
    assert _rel_err(b.grad.float().cpu(), br.grad) < 2e-2
