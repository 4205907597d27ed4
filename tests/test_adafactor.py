"""Adafactor against ``torch.optim.Adafactor`` (what the reference configures), on plain parameters and on the
dim-0 shards of FSDP units over two gloo ranks."""
from __future__ import annotations

import torch

from fairseq2_b200.optim import Adafactor
from tests.dist_utils import run_distributed


def _params(seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(12, 8, generator=g), torch.randn(16, generator=g), torch.randn(3, 6, 4, generator=g)]


def test_matches_torch_adafactor_on_plain_parameters() -> None:
    ours = [torch.nn.Parameter(p.clone()) for p in _params()]
    ref = [torch.nn.Parameter(p.clone()) for p in _params()]
    a = Adafactor(ours, lr=1e-2, weight_decay=0.01)
    b = torch.optim.Adafactor(ref, lr=1e-2, weight_decay=0.01)
    g = torch.Generator().manual_seed(1)
    for _ in range(5):
        for p, q in zip(ours, ref):
            grad = torch.randn(p.shape, generator=g)
            p.grad, q.grad = grad.clone(), grad.clone()
        a.step()
        b.step()
    for p, q in zip(ours, ref):
        assert torch.allclose(p, q, atol=1e-6, rtol=1e-5)


def test_recipe_builds_adafactor() -> None:
    from fairseq2_b200.recipe.config import AdafactorConfig

    cfg = AdafactorConfig()
    opt = Adafactor([torch.nn.Parameter(torch.zeros(4, 4))], lr=cfg.lr, beta2_decay=cfg.beta2_decay, eps=cfg.eps,
                    d=cfg.d, weight_decay=cfg.weight_decay)
    assert opt.param_groups[0]["eps"] == (None, 0.001)


def _fsdp_worker(rank: int, world: int):
    from fairseq2_b200.gang import ProcessGroupGang, create_fsdp_gangs, create_parallel_gangs
    from fairseq2_b200.models.llama import create_llama_model, get_llama_config
    from fairseq2_b200.nn import BatchLayout
    from fairseq2_b200.parallel.fsdp import FSDP

    root = ProcessGroupGang.create_default_process_group(torch.device("cpu"))
    gangs = create_fsdp_gangs(create_parallel_gangs(root))
    cfg = get_llama_config("tiny")
    cfg.num_layers = 1
    torch.manual_seed(7)
    model = create_llama_model(cfg)
    fsdp = FSDP(model, gangs, param_dtype=torch.float32)
    opt = Adafactor(fsdp.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(3)
    for _ in range(2):
        batches = [torch.randint(0, 8192, (2, 16), generator=g) for _ in range(world)]
        fsdp.zero_grad()
        b = batches[rank]
        fsdp(b, BatchLayout.of(b), targets=b).backward()
        fsdp.finish_backward()
        fsdp.scale_grads(float(world) / sum(x.numel() for x in batches))
        opt.step(grad_scale=fsdp.grad_scale)
        fsdp.after_optimizer_step()
    full = fsdp.full_state_dict()
    root.close()
    return {k: v.numpy() for k, v in full.items()}


def test_fsdp_shards_follow_the_unsharded_run() -> None:
    from fairseq2_b200.models.llama import create_llama_model, get_llama_config
    from fairseq2_b200.nn import BatchLayout

    world = 2
    cfg = get_llama_config("tiny")
    cfg.num_layers = 1
    torch.manual_seed(7)
    model = create_llama_model(cfg)
    opt = Adafactor(model.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(3)
    for _ in range(2):
        batches = [torch.randint(0, 8192, (2, 16), generator=g) for _ in range(world)]
        opt.zero_grad()
        n = sum(x.numel() for x in batches)
        for b in batches:
            (model(b, BatchLayout.of(b), targets=b) / n).backward()
        opt.step()
    ref = model.state_dict()
    for full in run_distributed(_fsdp_worker, world):
        for k, v in ref.items():
            assert torch.allclose(torch.from_numpy(full[k]), v, atol=2e-4, rtol=1e-3), k
