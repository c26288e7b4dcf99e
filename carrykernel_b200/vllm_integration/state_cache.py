"""Slot cache for the quantized recurrent state: who owns which slot, and the
copies that keep a request's state alive across an engine's cache events.

carrykernel's slot-indexed step works on a paged pool addressed through
``ssm_state_indices`` and leaves the cache wiring open, with one requirement
spelled out (``vllm_integration/quantized_packed_decode.py:50-54``): the
error-feedback residual is per-request persistent state -- it has to survive
paging, preemption, prefix-cache reuse and speculative-decode rollback together
with the state codes and both sets of scales.  This module is that wiring for
an engine that drives the decode calls itself:

* slot ownership: :meth:`SlotCache.allocate` / :meth:`free`, slot 0 reserved as
  the padding id (``NULL_BLOCK_ID``), :meth:`indices` for the decode calls;
* page accounting from ``state_bytes_per_slot``
  (``quantized_packed_decode.py:355-369``): one page = one slot of one layer;
* preemption: :meth:`preempt` moves a request's slot of every layer into a
  spill pool and releases the slot, :meth:`resume` brings it back (to whatever
  slot is free then);
* prefix reuse: :meth:`fork` gives a new request a copy of another request's
  state (codes, scales, residual: a request that continues from a cached prefix
  continues from the cached residual too);
* speculative decoding: :meth:`checkpoint` before the speculative tokens,
  :meth:`rollback` when some are rejected, :meth:`release_checkpoint` when all
  are accepted.

Every move is ``state_pool.copy_slots`` -- one launch per layer, all four
tensors of the slot bit for bit, on the current stream, nothing allocated and
nothing read back -- so an interrupted request ends with exactly the pool
contents of an uninterrupted one.  The bookkeeping is host-side Python, the
engine's scheduler thread being its only caller (no locking).  Registration
with vLLM's own cache manager (``MambaSpec``) is engine code and not part of
this library.
"""

from __future__ import annotations

from typing import Dict, Hashable, Iterable, List, Optional

import torch

from . import quantized_packed_decode as qpd
from . import state_pool

NULL_SLOT = qpd.NULL_BLOCK_ID


class CacheFull(RuntimeError):
    """No free slot (or spill slot) is left."""


class _Pools:
    """One pool per layer plus the free list of its slot ids (shared by all layers: a request has
    the same slot id in every layer)."""

    def __init__(self, num_layers, num_slots, HV, V, K, device, resid_fmt, resid_scale):
        self.layers = [qpd.init_quantized_state(num_slots, HV, V, K, device, resid_fmt=resid_fmt,
                                                resid_scale=resid_scale) for _ in range(num_layers)]
        self.num_slots = num_slots
        self.free = list(range(num_slots - 1, 0, -1))     # pop() hands out 1, 2, 3, ...

    def take(self, what):
        if not self.free:
            raise CacheFull(f"no free {what}")
        return self.free.pop()

    def give(self, slot):
        if not (0 < slot < self.num_slots) or slot in self.free:
            raise ValueError(f"slot {slot} is not in use")
        self.free.append(slot)


class SlotCache:
    """Slots of ``num_layers`` stacked GDN layers for up to ``num_slots - 1`` running requests,
    with ``spill_slots - 1`` places for preempted requests and checkpoints.

    ``pools[layer]`` is the ``(state_codes, state_scale, resid_codes, resid_scale)`` tuple to pass
    to ``quantized_gated_delta_rule_packed_decode`` together with ``indices(request_ids)``."""

    def __init__(self, num_layers: int, num_slots: int, HV: int, V: int, K: int, device,
                 resid_fmt: int = qpd.RESID_INT4, resid_scale: str = "head", spill_slots: int = 0):
        if num_layers < 1 or num_slots < 2:
            raise ValueError("need at least one layer and one real slot besides the padding slot 0")
        self.device = torch.device(device)
        self.resid_fmt, self.resid_scale = resid_fmt, resid_scale
        self.shape = (HV, V, K)
        self._main = _Pools(num_layers, num_slots, HV, V, K, device, resid_fmt, resid_scale)
        self._spill = _Pools(num_layers, max(spill_slots, 1), HV, V, K, device, resid_fmt, resid_scale)
        self.pools = self._main.layers
        self._slot_of: Dict[Hashable, int] = {}           # running requests
        self._spilled: Dict[Hashable, int] = {}           # preempted requests -> spill slot
        self._checkpoints: Dict[int, tuple] = {}          # token -> (request, spill slot)
        self._next_token = 1

    # ---- accounting -------------------------------------------------------
    @property
    def num_layers(self) -> int:
        return len(self.pools)

    def page_size_bytes(self) -> int:
        """Bytes of one slot of one layer: the page an engine's block table accounts in."""
        HV, V, K = self.shape
        return qpd.state_bytes_per_slot(HV, V, K, True, resid_fmt=self.resid_fmt, resid_scale=self.resid_scale)

    def bytes_per_request(self) -> int:
        return self.page_size_bytes() * self.num_layers

    def pages_in_use(self) -> int:
        used_main = self._main.num_slots - 1 - len(self._main.free)
        used_spill = self._spill.num_slots - 1 - len(self._spill.free)
        return (used_main + used_spill) * self.num_layers

    def bytes_in_use(self) -> int:
        return self.pages_in_use() * self.page_size_bytes()

    def capacity_bytes(self) -> int:
        """Bytes the pools hold on the device, padding slots included."""
        return (self._main.num_slots + self._spill.num_slots) * self.bytes_per_request()

    def free_slots(self) -> int:
        return len(self._main.free)

    # ---- slot ownership ---------------------------------------------------
    def allocate(self, request) -> int:
        """A slot for a new request.  Its contents are whatever the slot held: seed it with
        ``state_pool.store_state`` (prefill hand-off) or :meth:`fork` before decoding."""
        if request in self._slot_of or request in self._spilled:
            raise ValueError(f"request {request!r} already has state")
        slot = self._main.take("slot")
        self._slot_of[request] = slot
        return slot

    def free(self, request) -> None:
        """Release everything the request holds: its slot or spill slot, and its checkpoints."""
        if request in self._slot_of:
            self._main.give(self._slot_of.pop(request))
        elif request in self._spilled:
            self._spill.give(self._spilled.pop(request))
        else:
            raise KeyError(request)
        for token in [t for t, (r, _) in self._checkpoints.items() if r == request]:
            self._spill.give(self._checkpoints.pop(token)[1])

    def slot(self, request) -> int:
        return self._slot_of[request]

    def is_running(self, request) -> bool:
        return request in self._slot_of

    def indices(self, requests: Iterable, pad_to: Optional[int] = None) -> torch.Tensor:
        """``ssm_state_indices`` (int32, on the pools' device) for a batch of running requests;
        ``None`` entries and the tail up to ``pad_to`` become the padding id 0."""
        ids: List[int] = [NULL_SLOT if r is None else self._slot_of[r] for r in requests]
        if pad_to is not None:
            if pad_to < len(ids):
                raise ValueError("pad_to is shorter than the batch")
            ids += [NULL_SLOT] * (pad_to - len(ids))
        return torch.tensor(ids, dtype=torch.int32, device=self.device)

    # ---- moves ------------------------------------------------------------
    def _copy(self, src: _Pools, src_slot: int, dst: _Pools, dst_slot: int) -> None:
        s = torch.tensor([src_slot], dtype=torch.int32, device=self.device)
        d = torch.tensor([dst_slot], dtype=torch.int32, device=self.device)
        for sp, dp in zip(src.layers, dst.layers):
            state_pool.copy_slots(sp, s, d, dst_pool=dp, resid_fmt=self.resid_fmt)

    def preempt(self, request) -> None:
        """Move a running request's state to the spill pool and release its slot."""
        slot = self._slot_of[request]
        spill = self._spill.take("spill slot")
        self._copy(self._main, slot, self._spill, spill)
        del self._slot_of[request]
        self._main.give(slot)
        self._spilled[request] = spill

    def resume(self, request) -> int:
        """Bring a preempted request back into a free slot (not necessarily its old one)."""
        spill = self._spilled[request]
        slot = self._main.take("slot")
        self._copy(self._spill, spill, self._main, slot)
        del self._spilled[request]
        self._spill.give(spill)
        self._slot_of[request] = slot
        return slot

    def fork(self, src_request, dst_request) -> int:
        """A new request that continues from ``src_request``'s state (prefix-cache reuse): its slot
        starts as a bit-for-bit copy, residual included."""
        src = self._slot_of[src_request]
        dst = self.allocate(dst_request)
        self._copy(self._main, src, self._main, dst)
        return dst

    def checkpoint(self, request) -> int:
        """Save a running request's state before speculative tokens are applied; returns a token
        for :meth:`rollback` / :meth:`release_checkpoint`."""
        slot = self._slot_of[request]
        spill = self._spill.take("spill slot")
        self._copy(self._main, slot, self._spill, spill)
        token, self._next_token = self._next_token, self._next_token + 1
        self._checkpoints[token] = (request, spill)
        return token

    def rollback(self, token: int) -> None:
        """Restore the state saved by :meth:`checkpoint` (rejected speculative tokens) and drop the
        checkpoint.  The request must be running."""
        request, spill = self._checkpoints.pop(token)
        self._copy(self._spill, spill, self._main, self._slot_of[request])
        self._spill.give(spill)

    def release_checkpoint(self, token: int) -> None:
        """All speculative tokens were accepted: drop the checkpoint."""
        _, spill = self._checkpoints.pop(token)
        self._spill.give(spill)
