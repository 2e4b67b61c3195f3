"""Symmetric (peer-accessible) device memory for the fused compute+collective kernels.

``SymmGroup`` wraps one process group whose ranks sit on GPUs with NVLink peer access.  It
hands out *symmetric tensors*: the same shape on every rank, with the device addresses of all
ranks' copies known everywhere, so that a kernel can load from / store to a peer's copy.

Two providers, tried in order:

1. ``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged by PyTorch, also gives
   an NVLS multicast address when the fabric supports it);
2. CUDA IPC handles of ordinary allocations, exchanged with ``all_gather_object``.

The group's barrier is a kernel (``csrc/comm_p2p.cu: symm_barrier_kernel``) that signals through
words in the peers' memory; its wait is bounded and reports ``ST_TIMEOUT_PEER`` in the device
status word instead of hanging.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops._ext import extension

_SIGNAL_WORDS = 16 * 64  # 64 channels x 16 peers
_CANARY_BYTES = 4096     # guard band on each side of a symmetric buffer when OLB_SYMM_CANARY=1
_CANARY_VALUE = 0xA5


def canaries_enabled() -> bool:
    """``OLB_SYMM_CANARY=1``: every symmetric buffer gets a guard band of ``_CANARY_BYTES`` on both sides, filled with a
    pattern; ``SymmGroup.check_canaries`` then tells whether a kernel (of this or of another rank: peers store into these
    buffers) wrote outside a buffer.  The stand-in for a memory checker on the multi-GPU paths; the tests switch it on."""
    return os.environ.get("OLB_SYMM_CANARY", "0") == "1"


class SymmTensor:
    """Local tensor + the addresses of every rank's copy."""

    __slots__ = ("local", "ptrs", "multicast_ptr", "_keep", "_guards")

    def __init__(self, local: torch.Tensor, ptrs: List[int], multicast_ptr: int = 0, keep=None, guards=None):
        self.local = local
        self.ptrs = ptrs
        self.multicast_ptr = multicast_ptr
        self._keep = keep
        self._guards = guards      # (front, back) uint8 views of the guard bands, or None

    def guards_intact(self) -> bool:
        if self._guards is None:
            return True
        return all(bool((g == _CANARY_VALUE).all().item()) for g in self._guards)

    def offset_ptrs(self, elem_offset: int) -> List[int]:
        b = elem_offset * self.local.element_size()
        return [p + b for p in self.ptrs]


class SymmGroup:
    _instances: Dict[int, "SymmGroup"] = {}

    def __init__(self, group):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.provider = os.environ.get("OLB_SYMM_PROVIDER", "auto")
        self._epochs: Dict[int, int] = {}
        self._named: Dict[str, SymmTensor] = {}
        self._all: List[SymmTensor] = []
        self.pads = self.empty((_SIGNAL_WORDS,), torch.int32, zero=True)
        # every rank must have zeroed its signal words before anyone signals
        dist.barrier(group=group)
        torch.cuda.synchronize()

    @classmethod
    def all_canaries_intact(cls) -> bool:
        return all(g.check_canaries() for g in cls._instances.values())

    @classmethod
    def get(cls, group) -> "SymmGroup":
        key = id(group)
        inst = cls._instances.get(key)
        if inst is None:
            inst = cls._instances[key] = SymmGroup(group)
        return inst

    # ------------------------------------------------------------------ allocation
    def _alloc_symm_mem(self, shape, dtype) -> SymmTensor:
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(*shape, dtype=dtype, device=self.device)
        hdl = symm_mem.rendezvous(t, self.group)
        delta = t.data_ptr() - int(hdl.buffer_ptrs[hdl.rank])
        ptrs = [int(p) + delta for p in hdl.buffer_ptrs]
        mc = 0
        try:
            mc = int(hdl.multicast_ptr or 0)
            if mc:
                mc += delta
        except Exception:
            mc = 0
        return SymmTensor(t, ptrs, mc, keep=hdl)

    def _alloc_ipc(self, shape, dtype) -> SymmTensor:
        t = torch.empty(shape, dtype=dtype, device=self.device)
        storage = t.untyped_storage()
        handle = storage._share_cuda_()
        gathered = [None] * self.size
        dist.all_gather_object(gathered, (handle, t.storage_offset() * t.element_size()), group=self.group)
        ptrs, keep = [], []
        for r, (h, byte_off) in enumerate(gathered):
            if r == self.rank:
                ptrs.append(t.data_ptr())
                continue
            st = torch.UntypedStorage._new_shared_cuda(*h)
            keep.append(st)
            ptrs.append(st.data_ptr() + byte_off)
        return SymmTensor(t, ptrs, 0, keep=keep)

    def _alloc(self, shape, dtype) -> SymmTensor:
        st = None
        if self.provider in ("auto", "symm_mem"):
            try:
                st = self._alloc_symm_mem(tuple(shape), dtype)
            except Exception as exc:  # noqa: BLE001 - provider fallback
                if self.provider == "symm_mem":
                    raise
                self._symm_mem_error = exc
                self.provider = "ipc"
        if st is None:
            st = self._alloc_ipc(tuple(shape), dtype)
        return st

    def empty(self, shape, dtype, zero=False) -> SymmTensor:
        if not canaries_enabled():
            st = self._alloc(shape, dtype)
        else:
            # one flat allocation [guard | payload | guard]; the tensor handed out is the payload
            esz = torch.empty((), dtype=dtype).element_size()
            numel = 1
            for d in shape:
                numel *= int(d)
            pad = _CANARY_BYTES // esz
            raw = self._alloc((numel + 2 * pad,), dtype)
            flat = raw.local
            bytes_view = flat.view(torch.uint8)
            front, back = bytes_view[:_CANARY_BYTES], bytes_view[_CANARY_BYTES + numel * esz:]
            front.fill_(_CANARY_VALUE)
            back.fill_(_CANARY_VALUE)
            st = SymmTensor(flat[pad:pad + numel].view(tuple(shape)), [p + _CANARY_BYTES for p in raw.ptrs],
                            raw.multicast_ptr + _CANARY_BYTES if raw.multicast_ptr else 0, keep=(raw, raw._keep),
                            guards=(front, back))
        if zero:
            st.local.zero_()
        self._all.append(st)
        return st

    def check_canaries(self) -> bool:
        """True when no guard band of this group's buffers has been written (always true without canaries).  Call it
        after a barrier, when the peers' stores of the step under test are complete."""
        return all(st.guards_intact() for st in self._all)

    def named(self, name: str, shape, dtype, zero=False) -> SymmTensor:
        """Cached symmetric tensor (all ranks must request the same names in the same order)."""
        st = self._named.get(name)
        if st is None or tuple(st.local.shape) != tuple(shape) or st.local.dtype != dtype:
            st = self._named[name] = self.empty(shape, dtype, zero=zero)
        return st

    # ------------------------------------------------------------------ synchronisation
    def side_stream(self) -> "torch.cuda.Stream":
        """A second stream of this group for peer-memory kernels that run underneath compute of the main stream."""
        s = getattr(self, "_side_stream", None)
        if s is None:
            s = self._side_stream = torch.cuda.Stream(device=self.device)
        return s

    def barrier(self, channel: int = 0):
        """All ranks' preceding work on the current stream is complete and visible to peers when
        the kernels enqueued after this call start."""
        e = self._epochs.get(channel, 0) + 1
        self._epochs[channel] = e
        extension().symm_barrier(self.pads.ptrs, self.rank, channel, e, OF.status_word(self.device))


def peer_access_ok(group) -> bool:
    """True if every pair of GPUs of this node-local group can address each other's memory."""
    if not torch.cuda.is_available() or not dist.is_initialized():
        return False
    try:
        n = torch.cuda.device_count()
        me = torch.cuda.current_device()
        ok = all(torch.cuda.can_device_access_peer(me, d) for d in range(n) if d != me)
    except Exception:
        ok = False
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())
