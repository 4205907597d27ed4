"""Symmetric-memory communication for one NVSwitch box.

``SymmetricArena`` allocates one buffer per rank through
``torch.distributed._symmetric_memory`` (CUDA VMM allocation + handle exchange
over the process group -- the plumbing), maps every peer's buffer, and hands out
sub-allocations at identical offsets on every rank. The collectives themselves
are the in-tree kernels of ``csrc/comm.cu``: peer loads/stores over NVLink,
flag-based synchronisation with bounded waits, no NCCL on the data path.

``SymmGang`` implements the :class:`~fairseq2_b200.gang.Gang` interface on top:
tensors are staged into the arena, reduced/gathered by the kernels and copied
out. FSDP uses the arena directly (its shards and flat gradients *live* in it),
so its all-gathers and reduce-scatters are zero-copy.

Flag slots (each slot holds one epoch counter per source rank):
``0`` generic collectives of ``SymmGang``, ``1`` "parameters ready", ``2 + u``
gradient readiness of FSDP unit ``u``.
"""
from __future__ import annotations

import pickle
from typing import Sequence

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup

from fairseq2_b200.gang import Gang, GangError, ProcessGroupGang, ReduceOperation
from fairseq2_b200.ops._ext import require_ext
from fairseq2_b200.typing import Device

FLAG_BYTES = 64 * 1024
MAX_RANKS = 8
SLOT_GENERIC = 0
SLOT_PARAMS = 1
SLOT_UNIT0 = 2

_OPS = {ReduceOperation.SUM: 0, ReduceOperation.MEAN: 1, ReduceOperation.PRODUCT: 2, ReduceOperation.MIN: 3,
        ReduceOperation.MAX: 4}


def symmetric_memory_available(gang: Gang) -> bool:
    gang = gang.base_gang()
    if not isinstance(gang, ProcessGroupGang) or gang.device.type != "cuda" or gang.size > MAX_RANKS:
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except ImportError:
        return False
    return True


class SymmetricArena:
    """One symmetric buffer per rank with a bump allocator (offsets are the
    same on every rank because every rank performs the same allocations)."""

    def __init__(self, gang: ProcessGroupGang, nbytes: int, *, wait_limit_s: float = 5.0) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.gang = gang
        self.device = gang.device
        self.rank, self.world = gang.rank, gang.size
        self.wait_limit_s = wait_limit_s
        nbytes = FLAG_BYTES + ((nbytes + 4095) // 4096) * 4096
        pg = gang.as_process_group()
        try:
            symm_mem.enable_symm_mem_for_group(pg.group_name)
        except Exception:  # noqa: BLE001 - newer releases enable groups implicitly
            pass
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, pg.group_name)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        # NVSwitch multicast mapping of the same buffer (0 where the fabric does not offer one): one address whose
        # loads can be reduced and whose stores are replicated inside the switch (``multimem.*`` instructions)
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.nbytes = nbytes
        self._top = FLAG_BYTES
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        gang.barrier()                       # every rank's flags are zero before anyone signals
        self._generic_epoch = 0
        self.ext = require_ext()

    def alloc(self, nbytes: int, align: int = 256) -> tuple[int, Tensor]:
        off = ((self._top + align - 1) // align) * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"The symmetric arena ({self.nbytes} bytes) cannot hold another {nbytes} bytes.")
        self._top = off + nbytes
        return off, self.buf[off: off + nbytes]

    def alloc_tensor(self, numel: int, dtype: torch.dtype) -> tuple[int, Tensor]:
        off, raw = self.alloc(numel * torch.empty((), dtype=dtype).element_size())
        return off, raw.view(dtype)

    @property
    def device_index(self) -> int:
        return self.device.index if self.device.index is not None else torch.cuda.current_device()

    # ---- primitives (launched on the current stream)
    def barrier(self, slot: int, epoch: int) -> None:
        self.ext.comm_barrier(self.peer_ptrs, self.rank, slot, epoch, self.device_index, self.wait_limit_s)

    def signal(self, slot: int, epoch: int) -> None:
        self.ext.comm_signal(self.peer_ptrs, self.rank, slot, epoch, self.device_index)

    def barrier_next(self, slot: int) -> None:
        """Barrier on ``slot`` with the arena-wide next epoch of that slot, so that several operators may share
        a slot (epochs only grow; a repeated epoch would let a barrier pass without synchronising)."""
        epochs = self.__dict__.setdefault("_slot_epochs", {})
        epochs[slot] = epochs.get(slot, 0) + 1
        self.barrier(slot, epochs[slot])

    def next_generic_epoch(self) -> int:
        self._generic_epoch += 1
        return self._generic_epoch


class SymmGang(Gang):
    """Gang whose CUDA collectives run on the in-tree peer-memory kernels.

    Control-plane calls (object broadcast, sub-gang creation, CPU tensors) are
    delegated to the wrapped process-group gang.
    """

    def __init__(self, base: ProcessGroupGang, *, staging_bytes: int = 64 * 1024 * 1024,
                 arena: SymmetricArena | None = None, wait_limit_s: float = 5.0) -> None:
        """``wait_limit_s``: how long a collective waits for its slowest peer before it gives up and records a
        time-out in the status word (the next ``barrier()`` raises); a training job sets it to the gang timeout,
        since ranks legitimately wait for one another during checkpoint writes and evaluation."""
        self._base = base
        self.arena = arena if arena is not None else SymmetricArena(base, 2 * staging_bytes + 4096,
                                                                    wait_limit_s=wait_limit_s)
        self._stage_bytes = staging_bytes
        # two staging halves alternate so that a rank that races ahead into the next collective
        # cannot overwrite data a slower peer is still reading
        self._stage = [self.arena.alloc(staging_bytes) for _ in range(2)]
        self._which = 0
        self._offs_dev: Tensor | None = None

    # ---- helpers
    def _stage_in(self, t: Tensor) -> tuple[int, Tensor, int]:
        nbytes = t.numel() * t.element_size()
        if nbytes > self._stage_bytes:
            raise GangError(f"A tensor of {nbytes} bytes exceeds the staging area ({self._stage_bytes} bytes).")
        off, raw = self._stage[self._which]
        self._which ^= 1
        view = raw[:nbytes].view(t.dtype).view(t.shape)
        view.copy_(t)
        return off, view, self.arena.next_generic_epoch()

    def close(self) -> None:
        self._base.close()

    def base_gang(self) -> Gang:
        return self._base

    def _on_kernels(self, t: Tensor, *, reduce: bool = False) -> bool:
        """Whether a collective on ``t`` runs on the peer-memory kernels; otherwise it goes to the wrapped gang:
        CPU tensors, tensors beyond the staging area, and reductions of types that fp32 cannot hold exactly."""
        if not t.is_cuda or t.numel() == 0:
            return False
        nbytes = t.numel() * (4 if reduce else t.element_size())
        if nbytes + 16 > self._stage_bytes:
            return False
        return not reduce or t.dtype in (torch.float32, torch.bfloat16, torch.float16)

    def create_gang(self, ranks: Sequence[int]) -> "Gang | None":
        return self._base.create_gang(ranks)

    def as_process_group(self) -> ProcessGroup:
        return self._base.as_process_group()

    def barrier(self) -> None:
        self.arena.barrier(SLOT_GENERIC, self.arena.next_generic_epoch())
        torch.cuda.current_stream(self.device).synchronize()
        self.arena.ext.check_status()

    def all_reduce(self, tensor: Tensor, op: ReduceOperation) -> None:
        if not self._on_kernels(tensor, reduce=True):
            self._base.all_reduce(tensor, op)
            return
        src = tensor if tensor.dtype == torch.float32 else tensor.float()
        src = src.contiguous()
        off, _, epoch = self._stage_in(src)
        out = torch.empty_like(src)
        a = self.arena
        a.ext.comm_allreduce_f32(a.peer_ptrs, a.rank, off, out, _OPS[op], SLOT_GENERIC, epoch, a.wait_limit_s)
        tensor.copy_(out.view_as(tensor))

    def all_gather(self, output_tensor: Tensor, input_tensor: Tensor) -> None:
        if not self._on_kernels(input_tensor):
            self._base.all_gather(output_tensor, input_tensor)
            return
        if not output_tensor.is_contiguous():
            raise ValueError("`output_tensor` must be contiguous.")
        inp = input_tensor.contiguous()
        nbytes = inp.numel() * inp.element_size()
        pad = (-nbytes) % 16
        flat = inp.view(-1).view(torch.uint8)
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        off, _, epoch = self._stage_in(flat)
        a = self.arena
        tmp = torch.empty((self.size, nbytes + pad), dtype=torch.uint8, device=inp.device)
        for r in range(self.size):
            a.ext.comm_pull(a.peer_ptrs, a.rank, r, off, tmp[r], SLOT_GENERIC, epoch, a.wait_limit_s)
        output_tensor.view(self.size, -1).view(torch.uint8).copy_(tmp[:, :nbytes])

    def all_gather_to_list(self, output_tensors: list[Tensor], input_tensor: Tensor) -> None:
        out = input_tensor.new_empty((self.size, *input_tensor.shape))
        self.all_gather(out, input_tensor)
        for o, s in zip(output_tensors, out.unbind(0)):
            o.copy_(s)

    def reduce_scatter(self, output_tensor: Tensor, input_tensor: Tensor, op: ReduceOperation) -> None:
        if not self._on_kernels(input_tensor, reduce=True):
            self._base.reduce_scatter(output_tensor, input_tensor, op)
            return
        tmp = input_tensor.float().contiguous()
        self.all_reduce(tmp, op)
        output_tensor.copy_(tmp[self.rank])

    def all_to_all(self, output_tensor: Tensor, input_tensor: Tensor,
                   output_split_sizes: Sequence[int] | None = None,
                   input_split_sizes: Sequence[int] | None = None) -> None:
        if not self._on_kernels(input_tensor):
            self._base.all_to_all(output_tensor, input_tensor, output_split_sizes, input_split_sizes)
            return
        W = self.size
        isz = list(input_split_sizes) if input_split_sizes is not None else [input_tensor.shape[0] // W] * W
        sizes = torch.tensor(isz, dtype=torch.int64, device=input_tensor.device)
        all_sizes = torch.empty((W, W), dtype=torch.int64, device=input_tensor.device)
        self.all_gather(all_sizes, sizes)
        offs = torch.zeros((W, W + 1), dtype=torch.int64, device=input_tensor.device)
        offs[:, 1:] = all_sizes.cumsum(dim=1)
        off, _, epoch = self._stage_in(input_tensor.contiguous())
        a = self.arena
        a.ext.comm_alltoall(a.peer_ptrs, a.rank, off, output_tensor, offs, SLOT_GENERIC, epoch, a.wait_limit_s)

    def broadcast(self, tensor: Tensor, source_rank: int = 0) -> None:
        if not 0 <= source_rank < self.size:
            raise ValueError(f"`source_rank` must be in [0, {self.size}), but is {source_rank} instead.")
        if not self._on_kernels(tensor):
            self._base.broadcast(tensor, source_rank)
            return
        src = tensor.contiguous()
        nbytes = src.numel() * src.element_size()
        pad = (-nbytes) % 16
        flat = src.view(-1).view(torch.uint8)
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        off, _, epoch = self._stage_in(flat)
        a = self.arena
        out = torch.empty_like(flat)
        a.ext.comm_pull(a.peer_ptrs, a.rank, source_rank, off, out, SLOT_GENERIC, epoch, a.wait_limit_s)
        tensor.copy_(out[:nbytes].view(tensor.dtype).view(tensor.shape))

    def broadcast_objects(self, objects: list[object], source_rank: int = 0) -> None:
        self._base.broadcast_objects(objects, source_rank)

    @property
    def rank(self) -> int:
        return self._base.rank

    @property
    def size(self) -> int:
        return self._base.size

    @property
    def device(self) -> Device:
        return self._base.device

    @property
    def supports_process_group(self) -> bool:
        return True
