"""Position encoders against their closed forms, for padded and packed layouts and with an incremental state bag
(cf. the reference's ``tests/unit/nn/test_position_encoder.py``)."""
from __future__ import annotations

import math

import pytest
import torch

from fairseq2_b200.nn import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.nn.position_encoder import (LearnedPositionEncoder, ReferenceRotaryEncoder, RotaryEncoder,
                                               SinusoidalPositionEncoder)


def test_sinusoidal_table_and_padding() -> None:
    enc = SinusoidalPositionEncoder(8, max_seq_len=16)
    x = torch.zeros(2, 5, 8)
    layout = BatchLayout.of(x, [5, 3])
    y = enc(x, layout)
    half = 4
    for pos in range(5):
        for i in range(half):
            ang = pos * math.exp(-i * math.log(10000.0) / (half - 1))
            assert float(y[0, pos, i]) == pytest.approx(math.sin(ang), abs=1e-6)
            assert float(y[0, pos, half + i]) == pytest.approx(math.cos(ang), abs=1e-6)
    assert torch.equal(y[1, :3], y[0, :3]) and float(y[1, 3:].abs().sum()) == 0.0      # padding gets no encoding
    with pytest.raises(ValueError):
        enc(torch.zeros(1, 17, 8), BatchLayout.of(torch.zeros(1, 17, 8)))


def test_sinusoidal_packed_positions_restart_per_sequence() -> None:
    enc = SinusoidalPositionEncoder(8, max_seq_len=16)
    x = torch.zeros(7, 8)
    layout = BatchLayout.of(x, [3, 4], packed=True)
    y = enc(x, layout)
    assert torch.equal(y[3:6], y[0:3])                        # the second document starts again at position 0


def test_learned_encoder_incremental_matches_full() -> None:
    torch.manual_seed(0)
    enc = LearnedPositionEncoder(4, max_seq_len=8).eval()      # the state bag is only honoured in evaluation mode
    x = torch.randn(1, 6, 4)
    full = enc(x, BatchLayout.of(x))
    bag = IncrementalStateBag(max_num_steps=8)
    outs = []
    for t in range(6):
        step = x[:, t: t + 1]
        outs.append(enc(step, BatchLayout.of(step), state_bag=bag))
        bag.increment_step_nr()
    assert torch.allclose(torch.cat(outs, dim=1), full)


@pytest.mark.parametrize("kls", [RotaryEncoder, ReferenceRotaryEncoder])
def test_rotary_is_a_rotation_and_depends_on_relative_position(kls) -> None:  # type: ignore[no-untyped-def]
    torch.manual_seed(1)
    enc = kls(8, max_seq_len=32, theta=10000.0)
    q, k = torch.randn(1, 12, 2, 8), torch.randn(1, 12, 2, 8)
    layout = BatchLayout.of(q)
    rq, rk = enc(q, layout), enc(k, layout)
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1), atol=1e-5)                 # norms are preserved
    assert torch.allclose(rq[:, 0], q[:, 0], atol=1e-6)                               # position 0 is the identity
    # <R(m) q, R(n) k> depends on m - n only: shifting both positions by 5 leaves the score unchanged
    qq, kk = q[:, :1].expand(1, 12, 2, 8).contiguous(), k[:, :1].expand(1, 12, 2, 8).contiguous()
    rqq, rkk = enc(qq, layout), enc(kk, layout)
    s_a = (rqq[:, 7] * rkk[:, 2]).sum(-1)
    s_b = (rqq[:, 11] * rkk[:, 6]).sum(-1)
    assert torch.allclose(s_a, s_b, atol=1e-4)


def test_rotary_pairing_conventions() -> None:
    enc_i, enc_h = RotaryEncoder(4, max_seq_len=4, theta=10000.0), ReferenceRotaryEncoder(4, max_seq_len=4, theta=10000.0)
    x = torch.tensor([1.0, 0.0, 0.0, 0.0]).view(1, 1, 1, 4).expand(1, 2, 1, 4).contiguous()
    layout = BatchLayout.of(x)
    yi, yh = enc_i(x, layout)[0, 1, 0], enc_h(x, layout)[0, 1, 0]
    c, s = math.cos(1.0), math.sin(1.0)
    assert yi.tolist() == pytest.approx([c, s, 0.0, 0.0], abs=1e-6)      # interleaved pairs (x0, x1)
    assert yh.tolist() == pytest.approx([c, 0.0, s, 0.0], abs=1e-6)      # half-rotation pairs (x0, x2)


def test_rotary_incremental_matches_full() -> None:
    torch.manual_seed(2)
    enc = RotaryEncoder(8, max_seq_len=16).eval()
    x = torch.randn(2, 5, 2, 8)
    full = enc(x, BatchLayout.of(x))
    bag = IncrementalStateBag(max_num_steps=16)
    outs = []
    for t in range(5):
        step = x[:, t: t + 1].contiguous()
        outs.append(enc(step, BatchLayout.of(step), state_bag=bag))
        bag.increment_step_nr()
    assert torch.allclose(torch.cat(outs, dim=1), full, atol=1e-6)


def test_dual_rotary_encoder_equals_two_half_width_encoders() -> None:
    """One table with two frequency bands must equal RoPE(theta) on the first half of the features and
    RoPE(dual_theta) on the second half, concatenated; incremental decoding offsets the positions."""
    import pytest
    import torch

    from fairseq2_b200.nn import BatchLayout, DualRotaryEncoder, IncrementalStateBag, RotaryEncoder

    torch.manual_seed(0)
    E, S = 16, 9
    enc = DualRotaryEncoder(E, 32, theta=10_000.0, dual_theta=100_000.0)
    std, long = RotaryEncoder(E // 2, 32, theta=10_000.0), RotaryEncoder(E // 2, 32, theta=100_000.0)
    x = torch.randn(2, S, 3, E)
    layout = BatchLayout.of(x[:, :, 0, 0])
    want = torch.cat([std(x[..., : E // 2], layout), long(x[..., E // 2:], layout)], dim=-1)
    assert torch.allclose(enc(x, layout), want, atol=1e-6)
    bag = IncrementalStateBag(32)
    bag.increment_step_nr(5)
    step = x[:, :1]
    one = BatchLayout.of(step[:, :, 0, 0])
    want = torch.cat([std(step[..., : E // 2], one, state_bag=bag), long(step[..., E // 2:], one, state_bag=bag)], -1)
    assert torch.allclose(enc(step, one, state_bag=bag), want, atol=1e-6)
    with pytest.raises(ValueError):
        DualRotaryEncoder(6, 32)
