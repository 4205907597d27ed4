"""Collective communication over sets of processes ("gangs").

Capability parity with fairseq2's ``src/fairseq2/gang.py``: ``Gang`` ABC
(:55-227), ``ReduceOperation`` (:230), ``FakeGang`` (:252), ``ProcessGroupGang``
(:396), ``Gangs`` (:647), topology builders ``create_parallel_gangs`` (:907) /
``create_fsdp_gangs`` (:1034) / ``create_fake_gangs`` (:1183), helpers
``broadcast_flag`` (:1214) and ``all_sum`` (:1244) and the per-thread gang
context (:716-904).

Differences by design:

* ``reduce_scatter`` and ``all_to_all`` are first-class members of the ABC
  (FSDP gradient sync and MoE dispatch need them; the reference emulates the
  former with all-reduce and has no all-to-all).
* Sub-gangs are described by a rank *mesh* so that a symmetric-memory gang
  (``fairseq2_b200.parallel.symm``) can reuse the same peer pointer table for
  every sub-gang without a communicator split.
* One process drives one GPU; NCCL is used for CUDA tensors, Gloo for CPU.
"""
from __future__ import annotations

import os
import threading
import warnings
from abc import ABC, abstractmethod
from contextlib import contextmanager
from dataclasses import dataclass
from datetime import timedelta
from enum import Enum
from typing import Any, Iterator, Sequence, final

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup

from fairseq2_b200.device import CPU, META_DEVICE, get_current_device
from fairseq2_b200.error import InternalError, InvalidOperationError, NotSupportedError, OperationalError
from fairseq2_b200.logging import log
from fairseq2_b200.typing import Device
from fairseq2_b200.world_info import WorldInfo


class GangError(OperationalError):
    """A collective failed (peer died, timeout, transport error)."""


class ReduceOperation(Enum):
    SUM = 1
    MEAN = 2
    PRODUCT = 3
    MIN = 4
    MAX = 5


class Gang(ABC):
    """A set of processes that communicate collectively."""

    @abstractmethod
    def close(self) -> None: ...

    @abstractmethod
    def create_gang(self, ranks: Sequence[int]) -> "Gang | None":
        """Creates a sub-gang of ``ranks`` (unique, in ``[0, size)``). Must be
        called by every process of this gang; returns ``None`` on processes
        that are not in ``ranks``."""

    @abstractmethod
    def as_process_group(self) -> ProcessGroup: ...

    @abstractmethod
    def barrier(self) -> None: ...

    @abstractmethod
    def all_reduce(self, tensor: Tensor, op: ReduceOperation) -> None:
        """In-place reduction of ``tensor`` over the gang."""

    @abstractmethod
    def all_gather(self, output_tensor: Tensor, input_tensor: Tensor) -> None:
        """``output_tensor`` (contiguous, ``[size, *input.shape]``) receives
        every rank's ``input_tensor`` in rank order."""

    @abstractmethod
    def all_gather_to_list(self, output_tensors: list[Tensor], input_tensor: Tensor) -> None: ...

    @abstractmethod
    def reduce_scatter(self, output_tensor: Tensor, input_tensor: Tensor, op: ReduceOperation) -> None:
        """``input_tensor`` (contiguous, ``[size, *output.shape]``) is reduced
        over ranks and slice ``rank`` lands in ``output_tensor``."""

    @abstractmethod
    def all_to_all(self, output_tensor: Tensor, input_tensor: Tensor,
                   output_split_sizes: Sequence[int] | None = None,
                   input_split_sizes: Sequence[int] | None = None) -> None:
        """Personalised exchange along dim 0 (equal splits if sizes are None)."""

    @abstractmethod
    def broadcast(self, tensor: Tensor, source_rank: int = 0) -> None: ...

    @abstractmethod
    def broadcast_objects(self, objects: list[object], source_rank: int = 0) -> None: ...

    @property
    @abstractmethod
    def rank(self) -> int: ...

    @property
    @abstractmethod
    def size(self) -> int: ...

    @property
    @abstractmethod
    def device(self) -> Device: ...

    @property
    @abstractmethod
    def supports_process_group(self) -> bool: ...

    def base_gang(self) -> "Gang":
        """The gang that owns the process group: ``self``, except for gangs that wrap another one to run its
        collectives on other kernels."""
        return self

    def __enter__(self) -> "Gang":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()


def _check_ranks(ranks: Sequence[int], size: int) -> None:
    if len(set(ranks)) != len(ranks):
        raise ValueError("The ranks in ``ranks`` must be all unique.")
    for i, r in enumerate(ranks):
        if r < 0 or r >= size:
            raise ValueError(
                f"The rank at index {i} in `ranks` must be in [0, {size}), but is {r} instead.")


@final
class FakeGang(Gang):
    """Single-process stand-in that answers as rank ``rank`` of ``size``.

    Collectives behave as if every peer held the same tensor as the caller:
    SUM multiplies by ``size``, PRODUCT raises to the power ``size``,
    MEAN/MIN/MAX are identities, all_gather replicates the input, reduce_scatter
    reduces ``size`` copies of slice ``rank``. Used by unit tests and by
    single-GPU runs (cf. reference ``gang.py:252-392``).
    """

    def __init__(self, device: Device, *, rank: int = 0, size: int = 1) -> None:
        if size <= 0:
            raise ValueError(f"`size` must be positive, but is {size} instead.")
        if not 0 <= rank < size:
            raise ValueError(f"`rank` must be in [0, {size}), but is {rank} instead.")
        if device.type == "meta":
            raise ValueError("`device` must be a real device.")
        self._rank, self._size, self._device = rank, size, device

    def close(self) -> None:
        pass

    def create_gang(self, ranks: Sequence[int]) -> "FakeGang | None":
        _check_ranks(ranks, self._size)
        try:
            idx = list(ranks).index(self._rank)
        except ValueError:
            return None
        return FakeGang(self._device, rank=idx, size=len(ranks))

    def as_process_group(self) -> ProcessGroup:
        raise NotSupportedError("`FakeGang` does not support conversion to a process group.")

    def barrier(self) -> None:
        pass

    def _reduce_like(self, t: Tensor, op: ReduceOperation) -> None:
        if op == ReduceOperation.SUM:
            t.mul_(self._size)
        elif op == ReduceOperation.PRODUCT:
            t.pow_(self._size)
        elif op in (ReduceOperation.MEAN, ReduceOperation.MIN, ReduceOperation.MAX):
            pass
        else:
            raise ValueError(f"`op` must be a `ReduceOperation`, but is {op!r} instead.")

    def all_reduce(self, tensor: Tensor, op: ReduceOperation) -> None:
        self._reduce_like(tensor, op)

    def all_gather(self, output_tensor: Tensor, input_tensor: Tensor) -> None:
        if not output_tensor.is_contiguous():
            raise ValueError("`output_tensor` must be contiguous.")
        if output_tensor.shape[0] != self._size or output_tensor.shape[1:] != input_tensor.shape:
            raise ValueError(
                f"`output_tensor` must have shape [{self._size}, *input_tensor.shape].")
        for i in range(self._size):
            output_tensor[i].copy_(input_tensor)

    def all_gather_to_list(self, output_tensors: list[Tensor], input_tensor: Tensor) -> None:
        if len(output_tensors) != self._size:
            raise ValueError(f"`output_tensors` must have {self._size} element(s).")
        for t in output_tensors:
            t.copy_(input_tensor)

    def reduce_scatter(self, output_tensor: Tensor, input_tensor: Tensor, op: ReduceOperation) -> None:
        if input_tensor.shape[0] != self._size or input_tensor.shape[1:] != output_tensor.shape:
            raise ValueError(f"`input_tensor` must have shape [{self._size}, *output_tensor.shape].")
        output_tensor.copy_(input_tensor[self._rank])
        self._reduce_like(output_tensor, op)

    def all_to_all(self, output_tensor: Tensor, input_tensor: Tensor,
                   output_split_sizes: Sequence[int] | None = None,
                   input_split_sizes: Sequence[int] | None = None) -> None:
        if self._size == 1:
            output_tensor.copy_(input_tensor)
            return
        # Every peer is assumed to send what we would send to ourselves.
        if input_split_sizes is None:
            chunk = input_tensor.shape[0] // self._size
            mine = input_tensor[self._rank * chunk:(self._rank + 1) * chunk]
        else:
            off = sum(input_split_sizes[: self._rank])
            mine = input_tensor[off: off + input_split_sizes[self._rank]]
        outs = output_tensor.split(list(output_split_sizes) if output_split_sizes is not None
                                   else output_tensor.shape[0] // self._size)
        for o in outs:
            o.copy_(mine[: o.shape[0]])

    def broadcast(self, tensor: Tensor, source_rank: int = 0) -> None:
        if not 0 <= source_rank < self._size:
            raise ValueError(f"`source_rank` must be in [0, {self._size}), but is {source_rank} instead.")

    def broadcast_objects(self, objects: list[object], source_rank: int = 0) -> None:
        if not 0 <= source_rank < self._size:
            raise ValueError(f"`source_rank` must be in [0, {self._size}), but is {source_rank} instead.")

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def size(self) -> int:
        return self._size

    @property
    def device(self) -> Device:
        return self._device

    @property
    def supports_process_group(self) -> bool:
        return False


_TORCH_OPS = {
    ReduceOperation.SUM: dist.ReduceOp.SUM,
    ReduceOperation.PRODUCT: dist.ReduceOp.PRODUCT,
    ReduceOperation.MIN: dist.ReduceOp.MIN,
    ReduceOperation.MAX: dist.ReduceOp.MAX,
}


@final
class ProcessGroupGang(Gang):
    """Gang over a ``torch.distributed`` process group (NCCL for CUDA devices,
    Gloo for CPU). Every failed collective surfaces as :class:`GangError`."""

    def __init__(self, pg: ProcessGroup, device: Device, *, owns_default: bool = False) -> None:
        self._pg, self._device, self._owns_default = pg, device, owns_default
        self._rank, self._size = dist.get_rank(pg), dist.get_world_size(pg)

    @classmethod
    def create_default_process_group(cls, device: Device, *, timeout: timedelta | None = None,
                                     high_priority: bool = False, world_info: WorldInfo | None = None,
                                     ) -> "ProcessGroupGang":
        """Initialises the default process group from torchrun-style env vars.

        NCCL communicators are created eagerly (``device_id``) so that the
        first collective of the training loop does not pay for rendezvous.
        """
        if not dist.is_available():
            raise NotSupportedError("`torch.distributed` is not available.")
        if dist.is_initialized():
            raise InvalidOperationError("The default process group is already initialized.")
        if device.type == "cpu":
            backend = "gloo"
        elif device.type == "cuda":
            backend = "nccl"
        else:
            raise NotSupportedError(f"`device` must be of type cpu or cuda, but is of type {device.type}.")
        if timeout is None:
            timeout = timedelta(minutes=15)
        kwargs: dict[str, Any] = {}
        if device.type == "cuda":
            os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
            if device.index is None:
                device = torch.device("cuda", torch.cuda.current_device())
            kwargs["device_id"] = device
            if high_priority:
                try:
                    opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
                    kwargs["pg_options"] = opts
                except AttributeError:
                    pass
        if world_info is None:
            world_info = WorldInfo.from_env()
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        try:
            dist.init_process_group(backend, timeout=timeout, rank=world_info.rank,
                                    world_size=world_info.size, **kwargs)
        except (RuntimeError, ValueError) as ex:
            raise GangError("The default process group cannot be initialized.") from ex
        pg = dist.group.WORLD
        if pg is None:
            raise InternalError("`dist.group.WORLD` is `None`.")
        return cls(pg, device, owns_default=True)

    def close(self) -> None:
        if self._owns_default and dist.is_initialized():
            try:
                dist.destroy_process_group()
            except RuntimeError:
                pass
            self._owns_default = False

    def create_gang(self, ranks: Sequence[int]) -> "ProcessGroupGang | None":
        _check_ranks(ranks, self._size)
        if self._pg is not dist.group.WORLD:
            # torch can only create groups out of global ranks.
            glob = [dist.get_global_rank(self._pg, r) for r in ranks]
        else:
            glob = list(ranks)
        backend = "gloo" if self._device.type == "cpu" else "nccl"
        try:
            pg = dist.new_group(glob, backend=backend)
        except RuntimeError as ex:
            raise GangError("The sub process group cannot be created.") from ex
        if self._rank not in ranks:
            return None
        return ProcessGroupGang(pg, self._device)

    def as_process_group(self) -> ProcessGroup:
        return self._pg

    def _run(self, fn: Any, *a: Any, **kw: Any) -> Any:
        try:
            return fn(*a, **kw)
        except RuntimeError as ex:
            raise GangError(f"The collective `{getattr(fn, '__name__', fn)}` has failed: {ex}") from ex

    def barrier(self) -> None:
        if self._device.type == "cuda":
            self._run(dist.barrier, group=self._pg, device_ids=[self._device.index])
        else:
            self._run(dist.barrier, group=self._pg)

    def all_reduce(self, tensor: Tensor, op: ReduceOperation) -> None:
        if op == ReduceOperation.MEAN:
            if self._device.type == "cuda":
                self._run(dist.all_reduce, tensor, dist.ReduceOp.AVG, group=self._pg)
            else:
                self._run(dist.all_reduce, tensor, dist.ReduceOp.SUM, group=self._pg)
                tensor.div_(self._size) if tensor.is_floating_point() else tensor.floor_divide_(self._size)
            return
        self._run(dist.all_reduce, tensor, _TORCH_OPS[op], group=self._pg)

    def all_gather(self, output_tensor: Tensor, input_tensor: Tensor) -> None:
        if not output_tensor.is_contiguous():
            raise ValueError("`output_tensor` must be contiguous.")
        if output_tensor.shape[0] != self._size or output_tensor.shape[1:] != input_tensor.shape:
            raise ValueError(f"`output_tensor` must have shape [{self._size}, *input_tensor.shape].")
        self._run(dist.all_gather_into_tensor, output_tensor.view(-1), input_tensor.contiguous().view(-1),
                  group=self._pg)

    def all_gather_to_list(self, output_tensors: list[Tensor], input_tensor: Tensor) -> None:
        if len(output_tensors) != self._size:
            raise ValueError(f"`output_tensors` must have {self._size} element(s).")
        self._run(dist.all_gather, output_tensors, input_tensor, group=self._pg)

    def reduce_scatter(self, output_tensor: Tensor, input_tensor: Tensor, op: ReduceOperation) -> None:
        if input_tensor.shape[0] != self._size or input_tensor.shape[1:] != output_tensor.shape:
            raise ValueError(f"`input_tensor` must have shape [{self._size}, *output_tensor.shape].")
        if self._device.type == "cpu":
            # Gloo has no reduce-scatter: all-reduce a copy and keep our slice.
            tmp = input_tensor.clone()
            self.all_reduce(tmp, op)
            output_tensor.copy_(tmp[self._rank])
            return
        top = dist.ReduceOp.AVG if op == ReduceOperation.MEAN else _TORCH_OPS[op]
        self._run(dist.reduce_scatter_tensor, output_tensor.view(-1), input_tensor.contiguous().view(-1), top,
                  group=self._pg)

    def all_to_all(self, output_tensor: Tensor, input_tensor: Tensor,
                   output_split_sizes: Sequence[int] | None = None,
                   input_split_sizes: Sequence[int] | None = None) -> None:
        if self._device.type == "cpu":
            # Gloo lacks all_to_all_single on some builds; emulate with all_gather of padded chunks.
            self._cpu_all_to_all(output_tensor, input_tensor, output_split_sizes, input_split_sizes)
            return
        self._run(dist.all_to_all_single, output_tensor, input_tensor,
                  list(output_split_sizes) if output_split_sizes is not None else None,
                  list(input_split_sizes) if input_split_sizes is not None else None, group=self._pg)

    def _cpu_all_to_all(self, out: Tensor, inp: Tensor, osz: Sequence[int] | None, isz: Sequence[int] | None) -> None:
        n = self._size
        isz = list(isz) if isz is not None else [inp.shape[0] // n] * n
        osz = list(osz) if osz is not None else [out.shape[0] // n] * n
        sizes = torch.tensor(isz, dtype=torch.int64)
        all_sizes = torch.empty((n, n), dtype=torch.int64)
        self._run(dist.all_gather_into_tensor, all_sizes, sizes, group=self._pg)
        mx = int(all_sizes.max())
        rest = inp.shape[1:]
        padded = inp.new_zeros((n, mx, *rest))
        off = 0
        for j, s in enumerate(isz):
            padded[j, :s] = inp[off: off + s]
            off += s
        gathered = inp.new_empty((n, n, mx, *rest))
        self._run(dist.all_gather_into_tensor, gathered, padded, group=self._pg)
        off = 0
        for src in range(n):
            s = int(all_sizes[src, self._rank])
            if s != osz[src]:
                raise GangError(f"all_to_all split mismatch: rank {src} sends {s}, expected {osz[src]}.")
            out[off: off + s] = gathered[src, self._rank, :s]
            off += s

    def broadcast(self, tensor: Tensor, source_rank: int = 0) -> None:
        if not 0 <= source_rank < self._size:
            raise ValueError(f"`source_rank` must be in [0, {self._size}), but is {source_rank} instead.")
        self._run(dist.broadcast, tensor, group=self._pg, group_src=source_rank)

    def broadcast_objects(self, objects: list[object], source_rank: int = 0) -> None:
        if not 0 <= source_rank < self._size:
            raise ValueError(f"`source_rank` must be in [0, {self._size}), but is {source_rank} instead.")
        self._run(dist.broadcast_object_list, objects, group=self._pg, group_src=source_rank)

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def size(self) -> int:
        return self._size

    @property
    def device(self) -> Device:
        return self._device

    @property
    def supports_process_group(self) -> bool:
        return True


@dataclass(kw_only=True, frozen=True)
class Gangs:
    """The gangs of every parallelism dimension of a job.

    ``dp`` = data parallel; ``rdp``/``sdp`` = its replicated and sharded
    factors (HSDP: rdp inter-node, sdp intra-node; pure FSDP: sdp == dp; DDP:
    rdp == dp); ``tp`` = tensor parallel; ``pp`` = pipeline parallel (always
    size 1: pipeline parallelism is not offered, as in the reference).
    """

    root: Gang
    dp: Gang
    rdp: Gang
    sdp: Gang
    tp: Gang
    pp: Gang

    def __post_init__(self) -> None:
        if self.root.rank == 0 and (self.dp.rank != 0 or self.tp.rank != 0 or self.pp.rank != 0):
            raise ValueError("The coordinator process (root rank 0) must be rank 0 in every parallel gang.")

    @property
    def device(self) -> Device:
        return self.root.device

    def __enter__(self) -> "Gangs":
        _ctx_push(self, meta=False)
        return self

    def __exit__(self, *exc: Any) -> None:
        _ctx_pop(self.device)

    def close(self) -> None:
        self.root.close()


# --------------------------------------------------------------------- context
_tls = threading.local()
_defaults: dict[str, Gangs] = {}


def _key(device: Device) -> str:
    if device.type == "cuda" and device.index is None and torch.cuda.is_available():
        return f"cuda:{torch.cuda.current_device()}"
    return str(device)


def _stacks() -> dict[str, list[Gangs]]:
    s = getattr(_tls, "stacks", None)
    if s is None:
        s = _tls.stacks = {}
    return s


def _ctx_push(gangs: Gangs, meta: bool) -> None:
    st = _stacks()
    st.setdefault(_key(gangs.device), []).append(gangs)
    if meta:
        st.setdefault("meta", []).append(gangs)


def _ctx_pop(device: Device, meta: bool = False) -> None:
    st = _stacks()
    st[_key(device)].pop()
    if meta:
        st["meta"].pop()


def get_default_gangs(device: Device | None = None) -> Gangs:
    device = device or get_current_device()
    g = _defaults.get(_key(device))
    if g is None:
        real = CPU if device.type == "meta" else device
        g = create_fake_gangs(real)
    return g


def set_default_gangs(gangs: Gangs, *, meta: bool = False) -> None:
    _defaults[_key(gangs.device)] = gangs
    if meta:
        _defaults["meta"] = gangs


def get_current_gangs(device: Device | None = None) -> Gangs:
    device = device or get_current_device()
    st = _stacks().get(_key(device))
    if st:
        return st[-1]
    return get_default_gangs(device)


@contextmanager
def set_gangs(gangs: Gangs, *, meta: bool = False) -> Iterator[None]:
    _ctx_push(gangs, meta)
    try:
        yield
    finally:
        _ctx_pop(gangs.device, meta)


# -------------------------------------------------------------------- topology
def create_fake_gangs(device: Device) -> Gangs:
    g = FakeGang(device)
    return Gangs(root=g, dp=g, rdp=g, sdp=g, tp=g, pp=g)


def _sub_gang(root: Gang, groups: Sequence[Sequence[int]]) -> Gang:
    """Every process creates every group (collective contract of ``create_gang``)
    and keeps the one it belongs to."""
    mine: Gang | None = None
    for ranks in groups:
        if len(ranks) == 1:
            if ranks[0] == root.rank:
                mine = FakeGang(root.device)
            continue
        if len(ranks) == root.size and list(ranks) == list(range(root.size)):
            mine = root
            continue
        g = root.create_gang(ranks)
        if g is not None:
            mine = g
    if mine is None:
        raise InternalError("The process is not part of any sub-gang.")
    return mine


def create_parallel_gangs(root_gang: Gang, *, tp_size: int = 1) -> Gangs:
    """Splits ``root_gang`` into data- and tensor-parallel gangs.

    Mesh = ``arange(world).view(dp, tp)``: tensor-parallel peers are contiguous
    ranks (they share NVSwitch bandwidth for the activation collectives), data
    parallel peers are strided by ``tp_size``. ``rdp = dp`` and ``sdp`` is a
    size-1 gang until :func:`create_fsdp_gangs` refines them.
    """
    if tp_size <= 0:
        raise ValueError(f"`tp_size` must be positive, but is {tp_size} instead.")
    if root_gang.size % tp_size != 0:
        raise ValueError(
            f"The size of the root gang ({root_gang.size}) must be a multiple of `tp_size` ({tp_size}).")
    dp_size = root_gang.size // tp_size
    mesh = torch.arange(root_gang.size).view(dp_size, tp_size)
    fake = FakeGang(root_gang.device)
    if tp_size == 1:
        dp, tp = root_gang, fake
    elif dp_size == 1:
        dp, tp = fake, root_gang
    else:
        dp = _sub_gang(root_gang, [mesh[:, j].tolist() for j in range(tp_size)])
        tp = _sub_gang(root_gang, [mesh[i, :].tolist() for i in range(dp_size)])
    log.debug("Parallel gangs created: dp={} tp={}", dp.size, tp.size)
    return Gangs(root=root_gang, dp=dp, rdp=dp, sdp=fake, tp=tp, pp=fake)


def create_fsdp_gangs(gangs: Gangs, intra_node_size: int | None = None) -> Gangs:
    """Refines ``gangs.dp`` into replicated (``rdp``) and sharded (``sdp``) parts.

    ``intra_node_size=None`` → fully sharded over ``dp`` (``sdp = dp``,
    ``rdp`` size 1). Otherwise hybrid sharding: ``dp`` mesh
    ``view(inter, intra)`` with ``sdp`` = the ``intra`` (contiguous) axis.
    """
    dp = gangs.dp
    fake = FakeGang(gangs.root.device)
    if intra_node_size is None:
        return Gangs(root=gangs.root, dp=dp, rdp=fake, sdp=dp, tp=gangs.tp, pp=gangs.pp)
    if intra_node_size <= 1:
        raise ValueError(f"`intra_node_size` must be greater than 1, but is {intra_node_size} instead.")
    tp_size = gangs.tp.size
    if intra_node_size % tp_size != 0:
        raise ValueError(
            f"`intra_node_size` ({intra_node_size}) must be a multiple of the tensor parallel size ({tp_size}).")
    intra = intra_node_size // tp_size
    if dp.size % intra != 0:
        raise ValueError(
            f"The data parallel size ({dp.size}) must be a multiple of the intra-node data parallel size ({intra}).")
    inter = dp.size // intra
    if inter == 1:
        return Gangs(root=gangs.root, dp=dp, rdp=fake, sdp=dp, tp=gangs.tp, pp=gangs.pp)
    if intra == 1:
        return Gangs(root=gangs.root, dp=dp, rdp=dp, sdp=fake, tp=gangs.tp, pp=gangs.pp)
    mesh = torch.arange(dp.size).view(inter, intra)
    rdp = _sub_gang(dp, [mesh[:, j].tolist() for j in range(intra)])
    sdp = _sub_gang(dp, [mesh[i, :].tolist() for i in range(inter)])
    return Gangs(root=gangs.root, dp=dp, rdp=rdp, sdp=sdp, tp=gangs.tp, pp=gangs.pp)


def setup_root_gang(device: Device, *, timeout: timedelta | None = None, high_priority: bool = False,
                    collectives: str = "auto") -> Gang:
    """Root gang from the environment: fake when ``WORLD_SIZE`` is 1.

    ``collectives``: ``"nccl"`` keeps the process-group gang; ``"symm"`` wraps it into a
    :class:`~fairseq2_b200.parallel.symm.SymmGang`, whose CUDA collectives (loss / metric / gradient-norm
    reductions, flag broadcasts, data-reader synchronisation) run on the peer-memory kernels of a symmetric arena
    and raises if that is not possible; ``"auto"`` does so when all ranks sit in one NVSwitch domain (2 to 8 CUDA
    ranks of one node) and keeps NCCL otherwise."""
    if collectives not in ("auto", "nccl", "symm"):
        raise ValueError(f"`collectives` must be 'auto', 'nccl' or 'symm', but is '{collectives}' instead.")
    info = WorldInfo.from_env()
    if info.size == 1:
        return FakeGang(device)
    root = ProcessGroupGang.create_default_process_group(device, timeout=timeout, high_priority=high_priority,
                                                         world_info=info)
    if collectives == "nccl" or device.type != "cuda":
        if collectives == "symm":
            raise NotSupportedError("`collectives='symm'` needs CUDA devices.")
        return root
    from fairseq2_b200.parallel.symm import SymmGang, symmetric_memory_available

    single_node = info.local_size == info.size
    if not (single_node and symmetric_memory_available(root)):
        if collectives == "symm":
            raise NotSupportedError("`collectives='symm'` needs 2 to 8 CUDA ranks on one node with peer access.")
        return root
    try:
        limit = timeout.total_seconds() if timeout is not None else 900.0
        return SymmGang(root, wait_limit_s=limit)
    except Exception as ex:  # noqa: BLE001 - no peer access between the devices
        if collectives == "symm":
            raise
        log.warning("Symmetric memory is not usable for the root gang ({}); using NCCL collectives.", ex)
        return root


# --------------------------------------------------------------------- helpers
def broadcast_flag(gang: Gang, flag: bool, source_rank: int = 0) -> bool:
    t = torch.tensor(1 if flag else 0, device=gang.device, dtype=torch.int32)
    gang.broadcast(t, source_rank)
    return bool(t.item())


def all_sum(gang: Gang, value: float | int | Tensor) -> Tensor:
    """Sum of a scalar over the gang, returned as a 0-dim tensor on the gang's device."""
    if isinstance(value, Tensor):
        if value.ndim != 0:
            raise ValueError(f"`value` must be a scalar tensor, but has {value.ndim} dimension(s).")
        t = value.detach().clone().to(gang.device)
    else:
        t = torch.tensor(value, device=gang.device)
    gang.all_reduce(t, ReduceOperation.SUM)
    return t


def maybe_get_current_gangs() -> Gangs | None:
    warnings.warn("`maybe_get_current_gangs` is deprecated; use `get_current_gangs`.", DeprecationWarning)
    return get_current_gangs()
