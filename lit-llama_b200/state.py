"""Per-sequence state on the device: a pool of slots, one per live request.

Every layer of a model declares what it carries from token to token as `StateSpec`s (a recurrent matrix per
head, the last inputs of a short convolution, a ring of cached keys and values, ...).  The pool allocates one
tensor `[n_slots, *shape]` per spec, hands slots to requests, zeroes what must start at zero when a slot is
taken (a slot that another request used before is as good as a fresh one), and keeps the position of every
sequence.  Kernels address a slot through the device int32 pair {slot, position} (`meta`), so a captured step
replays for any slot."""
from dataclasses import dataclass
from typing import Dict, Hashable, List, Tuple

import torch

from . import _seqlib as S


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]          # per slot
    dtype: torch.dtype
    zero_on_acquire: bool = True    # recurrent state: must start at zero; ring caches are overwritten before they are read


class PoolFull(RuntimeError):
    """No free slot, or the token budget of the pool is used up."""


class SequenceStatePool:
    def __init__(self, specs: Dict[str, StateSpec], n_slots: int, device: torch.device, max_tokens: int = 0) -> None:
        if n_slots < 1:
            raise ValueError("n_slots must be at least 1")
        self.specs = dict(specs)
        self.n_slots = n_slots
        self.device = torch.device(device)
        self.max_tokens = int(max_tokens)           # 0 = no budget: recurrent state does not grow with the sequence
        self.tensors: Dict[str, torch.Tensor] = {
            name: torch.zeros((n_slots,) + tuple(sp.shape), dtype=sp.dtype, device=self.device) for name, sp in specs.items()}
        self._free: List[int] = list(range(n_slots - 1, -1, -1))   # slot 0 first
        self._slot_of: Dict[Hashable, int] = {}
        self._pos: Dict[int, int] = {}
        self.acquired = 0                            # lifetime counters (tests and diagnostics)
        self.reused = 0
        self._used_before = set()

    # ------------------------------------------------------------------ slots
    def has(self, request_id: Hashable) -> bool:
        return request_id in self._slot_of

    def live_tokens(self) -> int:
        return sum(self._pos.values())

    def free_slots(self) -> int:
        return len(self._free)

    def acquire(self, request_id: Hashable) -> int:
        if request_id in self._slot_of:
            raise KeyError(f"request {request_id!r} already holds slot {self._slot_of[request_id]}")
        if not self._free:
            raise PoolFull(f"all {self.n_slots} state slots are in use")
        slot = self._free.pop()
        for name, sp in self.specs.items():
            if sp.zero_on_acquire:
                t = self.tensors[name]
                S.check(S.lib().b2l_seq_zero_slot(t.data_ptr(), t[0].numel() * t.element_size(), slot, S.stream_ptr()), "b2l_seq_zero_slot")
        self._slot_of[request_id] = slot
        self._pos[slot] = 0
        self.acquired += 1
        if slot in self._used_before:
            self.reused += 1
        self._used_before.add(slot)
        return slot

    def release(self, request_id: Hashable) -> None:
        slot = self._slot_of.pop(request_id)
        del self._pos[slot]
        self._free.append(slot)

    def slot(self, request_id: Hashable) -> int:
        return self._slot_of[request_id]

    def position(self, request_id: Hashable) -> int:
        return self._pos[self._slot_of[request_id]]

    def reserve(self, request_id: Hashable, n_tokens: int) -> None:
        """Raises PoolFull when n_tokens more tokens would exceed the pool's token budget."""
        if self.max_tokens and self.live_tokens() + n_tokens > self.max_tokens:
            raise PoolFull(f"{self.live_tokens()} live tokens + {n_tokens} exceed the budget of {self.max_tokens}")

    def advance(self, request_id: Hashable, n_tokens: int) -> None:
        self._pos[self._slot_of[request_id]] += n_tokens

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())
