"""Checkpoint resharding: unit cases of ``reshard_tensor`` (uneven and empty data-parallel shards, tensor-parallel
merges and splits) and an end-to-end round trip -- a model trained and saved by FSDP over two gloo ranks is read
back at (dp=1), at (dp=3) and at (tp=2) and must equal slices of the gathered state."""
from __future__ import annotations

from pathlib import Path

import pytest
import torch

from fairseq2_b200.model_checkpoint.common import reshard_tensor
from tests.dist_utils import run_distributed


def _dp_split(t: torch.Tensor, dp: int) -> list[torch.Tensor]:
    chunk = -(-t.shape[0] // dp)
    return [t[min(r * chunk, t.shape[0]): min((r + 1) * chunk, t.shape[0])] for r in range(dp)]


@pytest.mark.parametrize("d0,src_dp,tgt_dp", [(10, 4, 1), (10, 4, 3), (2, 4, 1), (2, 4, 3), (7, 1, 4), (8, 2, 8)])
def test_dp_resharding_with_uneven_and_empty_shards(d0: int, src_dp: int, tgt_dp: int) -> None:
    full = torch.arange(d0 * 3, dtype=torch.float32).view(d0, 3)
    splits = [_dp_split(full, src_dp)]
    # the source layout really contains short and empty shards, as FSDP2's DTensor.to_local() gives them
    want_shapes = [c.shape[0] for c in torch.chunk(full, src_dp, dim=0)] + [0] * src_dp
    assert [s.shape[0] for s in splits[0]] == want_shapes[:src_dp]
    for r in range(tgt_dp):
        got = reshard_tensor("w", splits, (1, src_dp), (1, tgt_dp), (0, r), {})
        assert torch.equal(got, _dp_split(full, tgt_dp)[r])


@pytest.mark.parametrize("src_tp,tgt_tp", [(2, 1), (1, 2), (4, 2), (2, 4), (3, 2)])
@pytest.mark.parametrize("dim", [0, 1])
def test_tp_resharding(src_tp: int, tgt_tp: int, dim: int) -> None:
    full = torch.arange(12 * 12, dtype=torch.float32).view(12, 12)
    src = list(full.chunk(src_tp, dim=dim))
    splits = [_dp_split(s, 2) for s in src]
    for r in range(tgt_tp):
        got = reshard_tensor("w", splits, (src_tp, 2), (tgt_tp, 1), (r, 0), {"w": dim})
        assert torch.equal(got, full.chunk(tgt_tp, dim=dim)[r])
    # a parameter without a shard dim is replicated over tp
    rep = reshard_tensor("b", [[full[:6], full[6:]]] * src_tp, (src_tp, 2), (tgt_tp, 1), (0, 0), {"w": dim})
    assert torch.equal(rep, full)


def _save_worker(rank: int, world: int, out_dir: str):
    from fairseq2_b200.checkpoint import CheckpointManager
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model, get_llama_config
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.nn.data_parallel import DataParallelFacade
    from fairseq2_b200.optim import AdamW
    from fairseq2_b200.parallel.fsdp import FSDP

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_fsdp_gangs(create_parallel_gangs(root))
    cfg = get_llama_config("tiny")
    cfg.num_layers = 1
    cfg.vocab_size = 8191                  # odd: the embedding and the output projection shard unevenly
    torch.manual_seed(9)
    model = create_llama_model(cfg)
    fsdp = FSDP(model, gangs, param_dtype=torch.float32)
    opt = AdamW(fsdp.parameters(), lr=1e-2)
    b = torch.randint(0, 8191, (2, 16), generator=torch.Generator().manual_seed(rank))
    fsdp.zero_grad()
    fsdp(b, BatchLayout.of(b), targets=b).backward()
    fsdp.finish_backward()
    opt.step()
    fsdp.after_optimizer_step()
    ckpt = CheckpointManager(Path(out_dir), gangs)
    ckpt.save_model_only(1, DataParallelFacade(fsdp), blocking=True)
    local = {k: tuple(v.shape) for k, v in fsdp.state_dict().items()}
    full = fsdp.full_state_dict()
    ckpt.close()
    root.close()
    return local, {k: v.numpy() for k, v in full.items()}


def test_save_at_dp2_load_at_dp1_dp3_and_tp2(tmp_path: Path) -> None:
    from fairseq2_b200.gang import FakeGang, Gangs
    from fairseq2_b200.model_checkpoint.loader import NativeModelCheckpointLoader

    results = run_distributed(_save_worker, 2, str(tmp_path))
    full = {k: torch.from_numpy(v) for k, v in results[0][1].items()}
    # local shards = what FSDP2's dim-0 DTensor sharding yields (ceil-sized chunks, short tail)
    for r, (local, _) in enumerate(results):
        for k, shape in local.items():
            chunks = torch.chunk(torch.empty(full[k].shape[0]), 2)
            want0 = chunks[r].shape[0] if r < len(chunks) else 0
            assert shape == (want0, *full[k].shape[1:]), k
    model_dir = tmp_path / "step_1" / "model"
    loader = NativeModelCheckpointLoader()
    dev = torch.device("cpu")

    def gangs(tp_rank: int, tp: int, dp_rank: int, dp: int) -> Gangs:
        one = FakeGang(dev)
        root = FakeGang(dev, rank=tp_rank + tp * dp_rank, size=tp * dp)
        return Gangs(root=root, dp=FakeGang(dev, rank=dp_rank, size=dp), rdp=one,
                     sdp=FakeGang(dev, rank=dp_rank, size=dp), tp=FakeGang(dev, rank=tp_rank, size=tp), pp=one)

    # dp = 1: the consolidated state
    got = dict(loader.lazy_load(model_dir, {}, gangs=gangs(0, 1, 0, 1)))
    assert set(got) == set(full)
    for k, v in full.items():
        assert torch.equal(got[k], v), k
    # dp = 3: uneven shards of an odd-sized vocabulary
    for r in range(3):
        got = dict(loader.lazy_load(model_dir, {}, gangs=gangs(0, 1, r, 3)))
        for k, v in full.items():
            assert torch.equal(got[k], _dp_split(v, 3)[r]), k
    # tp = 2: column-sharded q_proj (dim 0), row-sharded output_proj (dim 1), the rest replicated
    dims = {"decoder.layers.0.self_attn.q_proj.weight": 0, "decoder.layers.0.self_attn.output_proj.weight": 1}
    for r in range(2):
        got = dict(loader.lazy_load(model_dir, dims, gangs=gangs(r, 2, 0, 1)))
        for k, v in full.items():
            want = v.chunk(2, dim=dims[k])[r] if k in dims else v
            assert torch.equal(got[k], want), k


def _load_then_shard_worker(rank: int, world: int, full_file: str, sharded_dir: str):
    """What a fine-tuning job does: build the model, load pretrained weights into it, then hand it to the
    data-parallel engine. The model holds whole parameters while it is loaded, whatever the FSDP size."""
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.family import get_model_family
    from fairseq2_b200.parallel.fsdp import FSDP

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_fsdp_gangs(create_parallel_gangs(root))
    fam = get_model_family("llama")
    cfg = fam.get_arch_config("tiny")
    cfg.num_layers = 1
    cfg.vocab_size = 8191
    out = []
    for path in (full_file, sharded_dir):
        model = fam.create_new_model(cfg, gangs)
        fam.load_into(model, Path(path), cfg, gangs)
        fsdp = FSDP(model, gangs, param_dtype=torch.float32)
        out.append({k: v.numpy() for k, v in fsdp.full_state_dict().items()})
    root.close()
    return out


def test_pretrained_weights_load_into_a_model_that_fsdp_shards_afterwards(tmp_path: Path) -> None:
    results = run_distributed(_save_worker, 2, str(tmp_path / "ckpt"))
    full = {k: torch.from_numpy(v) for k, v in results[0][1].items()}
    full_file = tmp_path / "consolidated.pt"
    torch.save({"model": full}, full_file)
    sharded_dir = tmp_path / "ckpt" / "step_1" / "model"
    for per_source in run_distributed(_load_then_shard_worker, 2, str(full_file), str(sharded_dir)):
        for got in per_source:                              # a single file, then a directory written at dp = 2
            assert set(got) == set(full)
            for k, v in full.items():
                assert torch.equal(torch.from_numpy(got[k]), v), k
