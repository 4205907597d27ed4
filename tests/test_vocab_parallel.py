"""Vocabulary-parallel output projection + cross entropy and embedding on two gloo ranks (CPU)."""
import torch

from tests.dist_utils import run_distributed


def _worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang
    from fairseq2_b200.nn.embedding import StandardEmbedding, VocabShardedEmbedding
    from fairseq2_b200.ops.cross_entropy import cross_entropy_reference, vocab_parallel_linear_cross_entropy

    gang = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    torch.manual_seed(0)
    T, D, V = 37, 16, 40
    h = torch.randn(T, D, requires_grad=True)
    w = torch.randn(V, D) * 0.3
    t = torch.randint(0, V, (T,))
    mask = (torch.rand(T) > 0.3).float()
    ws = w[rank * V // world:(rank + 1) * V // world].clone().requires_grad_(True)
    loss = vocab_parallel_linear_cross_entropy(h, ws, t, gang, target_mask=mask, chunk_size=16)
    loss.backward()
    wr = w.clone().requires_grad_(True)
    hr = h.detach().clone().requires_grad_(True)
    ref = cross_entropy_reference(hr @ wr.t(), t, None, target_mask=mask, reduction="sum")
    ref.backward()
    out = {"loss": float((loss - ref).abs()),
           "dh": float((h.grad - hr.grad).abs().max()),
           "dw": float((ws.grad - wr.grad[rank * V // world:(rank + 1) * V // world]).abs().max())}
    # vocabulary-sharded embedding against the plain table
    full = StandardEmbedding(V, D)
    with torch.no_grad():
        full.weight.copy_(w)
    sharded = VocabShardedEmbedding(gang, V, D)
    with torch.no_grad():
        sharded.weight.copy_(w[rank * V // world:(rank + 1) * V // world])
    ids = torch.randint(0, V, (3, 5))
    out["embed"] = float((sharded(ids) - full(ids)).abs().max())
    gang.close()
    return out


def test_vocab_parallel_cross_entropy_and_embedding() -> None:
    for r in run_distributed(_worker, 2):
        assert r["loss"] < 1e-3 and r["dh"] < 1e-4 and r["dw"] < 1e-4 and r["embed"] < 1e-6, r
