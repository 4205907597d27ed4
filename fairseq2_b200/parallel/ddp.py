"""Distributed data parallelism with flat gradient buckets (cf. fairseq2
``nn/ddp.py:30-152``).

Parameters keep their dtype and stay replicated. Gradients of each bucket live
in one flat buffer (``param.grad`` are views); as soon as the last gradient of
a bucket has been produced during backward the bucket is all-reduced on a side
stream, so communication overlaps the rest of the backward pass. The 1/size
factor is not applied here (``normalize_grads`` semantics of the reference's
custom comm hook, ``nn/ddp.py:141-152``): the caller scales by the global
number of targets afterwards.

On one NVSwitch box (``comm="symm"``, the default when available) the buckets
are allocated inside a symmetric arena and reduced IN PLACE by the in-tree
two-shot all-reduce kernel, which applies the averaging factor while the data
moves: no staging copy, no library call and no separate scaling pass.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Iterator

import torch
from torch import Tensor
from torch.nn import Module

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.gang import Gang, Gangs, ReduceOperation
from fairseq2_b200.nn.utils.module import broadcast_module


class _Bucket:
    def __init__(self, params: list[torch.nn.Parameter], arena: Any | None = None, index: int = 0) -> None:
        self.params = params
        n = sum(p.numel() for p in params)
        p0 = params[0]
        self.index = index
        self.numel = n
        self.byte_off = -1
        if arena is not None:
            per = 16 // p0.element_size()
            padded = (n + per - 1) // per * per              # whole 16-byte vectors
            self.byte_off, raw = arena.alloc_tensor(padded, p0.dtype)
            raw.zero_()
            self.flat = raw[:n]
            self.padded = padded
        else:
            self.flat = torch.zeros(n, device=p0.device, dtype=p0.dtype)
        self.views: list[Tensor] = []
        off = 0
        for p in params:
            self.views.append(self.flat[off: off + p.numel()].view_as(p))
            off += p.numel()
        self.pending = len(params)
        self.event: torch.cuda.Event | None = None
        self.epoch = 0            # reductions of this bucket so far (every reduction gets an epoch of its own)
        self.reduced_in_step = 0  # reductions since the last ``zero_grad``


class DDP(Module):
    #: first flag slot used by the bucket all-reduces (two slots per bucket)
    SLOT_BASE = 64

    def __init__(self, module: Module, gangs: Gangs, *, bucket_bytes: int = 64 * 1024 * 1024,
                 broadcast_parameters: bool = True, average: bool = True, comm: str = "auto",
                 allreduce: str = "auto") -> None:
        """``allreduce`` picks the kernel of the symmetric-memory path: "multimem" reduces inside the NVSwitch
        (``multimem.ld_reduce`` / ``multimem.st`` on the multicast mapping of the arena), "p2p" is the two-shot
        kernel on plain peer loads and stores. "auto" takes "multimem" where the arena has a multicast mapping and
        "p2p" otherwise; ``FAIRSEQ2_B200_DDP_ALLREDUCE`` overrides it.

        Gradient accumulation: a bucket is reduced whenever all of its gradients have been produced, i.e. once per
        micro-batch unless the backward pass runs under :meth:`no_sync`. Reducing the running sum again is exact for
        ``average=True`` (the mean of a value that is already identical on every rank is that value); with
        ``average=False`` the earlier micro-batches would be counted ``size`` times, so a second reduction of a
        bucket within one step raises -- accumulate under ``no_sync`` there."""
        super().__init__()
        if allreduce not in ("auto", "multimem", "p2p"):
            raise ValueError(f"`allreduce` must be 'auto', 'multimem' or 'p2p', but is '{allreduce}' instead.")
        import os

        self._allreduce = os.environ.get("FAIRSEQ2_B200_DDP_ALLREDUCE", allreduce)
        if any(getattr(m, "sequence_parallel", False) for m in module.modules()):
            # token-sharded activations leave partial gradients on every parameter that is replicated over the
            # tensor-parallel gang; only the flat-unit engine adds them up
            raise NotSupportedError("A model built with sequence-parallel activations needs the flat-unit engine "
                                    "(`fairseq2_b200.parallel.fsdp.FSDP`), not `DDP`.")
        self.module = module
        self.gang: Gang = gangs.rdp if gangs.rdp.size > 1 else gangs.dp
        self.average = average
        self._require_sync = True
        if broadcast_parameters:
            broadcast_module(module, self.gang)
        params = [p for p in module.parameters() if p.requires_grad]
        dev = params[0].device if params else torch.device("cpu")
        self.device = dev
        self.comm_stream = torch.cuda.Stream(dev) if dev.type == "cuda" and self.gang.size > 1 else None
        # buckets in reverse registration order ~ order in which gradients become ready
        groups: list[list[torch.nn.Parameter]] = []
        cur: list[torch.nn.Parameter] = []
        size = 0
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if cur and (size + nbytes > bucket_bytes or p.dtype != cur[0].dtype):
                groups.append(cur)
                cur, size = [], 0
            cur.append(p)
            size += nbytes
        if cur:
            groups.append(cur)
        self.arena = self._maybe_create_arena(groups, comm)
        self._counter_off = -1
        if self.arena is not None:
            # two zeroed words per bucket: "last CTA" counters of the two phases of the in-place kernel
            self._counter_off, c = self.arena.alloc(8 * len(groups), align=16)
            c.zero_()
        self.buckets: list[_Bucket] = [_Bucket(g, self.arena, i) for i, g in enumerate(groups)]
        if self.arena is not None:
            torch.cuda.synchronize(dev)
            self.gang.barrier()
        self._bucket_of: dict[int, tuple[_Bucket, int]] = {}
        for b in self.buckets:
            for i, p in enumerate(b.params):
                self._bucket_of[id(p)] = (b, i)
                p.register_post_accumulate_grad_hook(self._on_grad)

    def _maybe_create_arena(self, groups: list[list[torch.nn.Parameter]], comm: str) -> Any | None:
        if comm not in ("auto", "symm", "nccl"):
            raise ValueError(f"`comm` must be 'auto', 'symm' or 'nccl', but is '{comm}' instead.")
        from fairseq2_b200.gang import ProcessGroupGang

        usable = (self.device.type == "cuda" and self.gang.size > 1 and self.gang.size <= 8
                  and isinstance(self.gang.base_gang(), ProcessGroupGang)
                  and all(g[0].dtype in (torch.float32, torch.bfloat16) for g in groups))
        if comm == "nccl" or not usable:
            if comm == "symm":
                raise RuntimeError("The symmetric-memory all-reduce needs 2 to 8 CUDA ranks of one process group and "
                                   "fp32/bf16 parameters.")
            return None
        try:
            from fairseq2_b200.parallel.symm import SymmetricArena

            total = sum(sum(p.numel() * p.element_size() for p in g) + 512 for g in groups) + 4096
            return SymmetricArena(self.gang, total)
        except Exception:  # noqa: BLE001 - peer access unavailable: fall back to the process group
            if comm == "symm":
                raise
            return None

    def forward(self, *a: Any, **kw: Any) -> Any:
        return self.module(*a, **kw)

    def _on_grad(self, p: torch.nn.Parameter) -> None:
        b, i = self._bucket_of[id(p)]
        if p.grad is not None and p.grad.data_ptr() != b.views[i].data_ptr():
            b.views[i].copy_(p.grad)
            p.grad = b.views[i]
        b.pending -= 1
        if b.pending == 0:
            b.pending = len(b.params)          # the next micro-batch counts from the top again
            if self._require_sync:
                self._reduce(b)

    def _reduce(self, b: _Bucket) -> None:
        if self.gang.size == 1:
            return
        b.reduced_in_step += 1
        if b.reduced_in_step > 1 and not self.average:
            raise RuntimeError("A gradient bucket was summed over the ranks twice in one step, which counts the "
                               "earlier micro-batches `size` times; accumulate under `no_sync()` or use "
                               "`average=True`.")
        if self.arena is not None:
            self._reduce_symm(b)
            return
        op = ReduceOperation.MEAN if self.average else ReduceOperation.SUM
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.comm_stream):
                self.gang.all_reduce(b.flat, op)
        else:
            self.gang.all_reduce(b.flat, op)

    def _reduce_symm(self, b: _Bucket) -> None:
        a = self.arena
        assert a is not None and self.comm_stream is not None
        # every reduction of a bucket has an epoch of its own (the flags only grow; a repeated epoch would let both
        # waits of the kernel pass without synchronising); all ranks reduce a bucket equally often
        b.epoch += 1
        epoch = b.epoch
        scale = 1.0 / self.gang.size if self.average else 1.0
        blocks = max(1, min(64, b.padded * b.flat.element_size() // (512 * 16 * 4)))
        use_mm = self._allreduce == "multimem" or (self._allreduce == "auto" and a.multicast_ptr != 0)
        if use_mm and a.multicast_ptr == 0:
            raise RuntimeError("The symmetric arena has no NVSwitch multicast mapping; use allreduce='p2p'.")
        self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.comm_stream):
            fn = a.ext.comm_allreduce_multimem if use_mm else a.ext.comm_allreduce_inplace
            args = (a.multicast_ptr,) if use_mm else ()
            fn(a.peer_ptrs, a.rank, *args, b.byte_off, b.padded, b.flat.dtype == torch.float32, scale,
               self.SLOT_BASE + 2 * b.index, self.SLOT_BASE + 2 * b.index + 1, epoch, self._counter_off + 8 * b.index,
               a.device_index, blocks, a.wait_limit_s)

    def finish_backward(self) -> None:
        for b in self.buckets:
            if self._require_sync and b.pending != len(b.params):
                # some parameters of the bucket received no gradient in the last backward pass
                for i, p in enumerate(b.params):
                    if p.grad is None:
                        b.views[i].zero_()
                        p.grad = b.views[i]
                self._reduce(b)
            elif self._require_sync and b.reduced_in_step == 0 and any(p.grad is not None for p in b.params):
                # gradients accumulated under ``no_sync`` only: reduce them now
                for i, p in enumerate(b.params):
                    if p.grad is None:
                        b.views[i].zero_()
                        p.grad = b.views[i]
                self._reduce(b)
            b.pending = len(b.params)
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

    @contextmanager
    def no_sync(self) -> Iterator[None]:
        old = self._require_sync
        self._require_sync = False
        try:
            yield
        finally:
            self._require_sync = old

    def zero_grad(self, set_to_none: bool = True) -> None:  # type: ignore[override]
        for b in self.buckets:
            for p in b.params:
                p.grad = None
            b.pending = len(b.params)
            b.reduced_in_step = 0


def convert_batch_norms(module: Module, gangs: Gangs) -> Module:
    """Buffers are not broadcast during training, so batch-norm statistics have to be computed over the whole
    replicated gang: every ``BatchNorm`` becomes a ``SyncBatchNorm`` over it (cf. fairseq2 ``nn/ddp.py:92-94``).
    A module without batch norms, or a gang without a process group (single rank, fake gang), is returned as is."""
    from torch.nn.modules.batchnorm import _BatchNorm

    gang = gangs.rdp
    if gang.size == 1 or not any(isinstance(m, _BatchNorm) for m in module.modules()):
        return module
    try:
        group = gang.as_process_group()
    except Exception:  # noqa: BLE001 - fake gangs have no process group
        return module
    return torch.nn.SyncBatchNorm.convert_sync_batchnorm(module, group)


def to_ddp(module: Module, gangs: Gangs, **kw: Any) -> DDP:
    module = convert_batch_norms(module, gangs)
    return DDP(module, gangs, **kw)
