"""The cache on the device: keys and values in pages, and fixed-size state per sequence.

The reference gives every request one tensor [buf, nblk, 2, nkvh, dh] that the caller owns
(models/llama/common/src/lib.rs:98-107, args.rs:19-25) and sizes it by the context length or half
the free memory (models/llama/cuda/src/infer.rs:74-79).  Here one pool serves all sequences:

* a **slot** per live sequence (its length, its list of pages, its row in every state tensor);
* **pages** of 64 tokens; a sequence holds ceil(length / 64) of them, so the pool is sized by the
  most tokens that live sequences hold, each rounded up to 64;
* **groups**: runs of the model whose mixers need the same kind of storage (kind, heads, head
  size, the kind's own parameters) share one storage object; another need gets a group of its own.
  The storage class is looked up by the need's ``kind`` in :data:`CACHE_KINDS`.  Kind "full" keeps
  keys and values of every position in one pair of tensors K, V [runs, pages, nkvh, 64, dh]; page
  numbers are common to the groups of kind "full".  Another kind (a window of the last W tokens, a
  compressed cache) is a class registered under another name: see :class:`CacheStorage`;
* **state**: for each run whose mixer asks for it, a tensor [slots, *shape], zeroed when a slot
  is opened.

Slots and pages are given back by :meth:`close` and used again by later sequences.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, Registry, StateNeed
from .slots import PAGE, CacheError, SequenceTable

CACHE_KINDS = Registry("cache")     # CacheNeed.kind -> storage class


@dataclass
class CacheView:
    """What one run of a mixer sees of the cache."""
    k: torch.Tensor          # [pages, nkvh, PAGE, dh]
    v: torch.Tensor
    writable: bool           # False when the run reads the cache another run wrote
    kind: str = "full"

    def tensors(self):
        """The device tensors of this view, in a fixed order (what a replayed layer's pointers are moved between)."""
        return [self.k, self.v]


@dataclass
class LatentView:
    """What one run of a latent-attention mixer sees: one row per token for all heads."""
    kv: torch.Tensor         # [pages, PAGE, width]
    writable: bool
    kind: str = "latent"

    def tensors(self):
        return [self.kv]


class CacheStorage:
    """What a storage class must offer.  One object serves all runs with the same :class:`CacheNeed`.

    ``__init__(need, runs, *, n_pages, max_slots, max_context, dtype, device)``: allocate for ``len(runs)`` runs;
    ``n_pages`` pages of 64 tokens are what the cache's common page pool holds, ``max_slots`` the sequences that
    can be live.  ``view(i, writable)``: what the i-th of these runs hands its mixer as ``cache`` (any object;
    ``writable`` is False for a run that reads another run's cache).  ``open(slot)`` / ``close(slot)``: a
    sequence starts or ends in this slot (storage addressed by slot, not by pages, puts itself in order here)."""

    def __init__(self, need: CacheNeed, runs: List[int], *, n_pages: int, max_slots: int, max_context: int,
                 dtype, device):
        self.need = need
        self.runs = runs

    def view(self, index: int, writable: bool):
        raise NotImplementedError

    def open(self, slot: int) -> None:
        pass

    def close(self, slot: int) -> None:
        pass

    @property
    def nbytes(self) -> int:
        return 0


@CACHE_KINDS.register("full")
class CacheGroup(CacheStorage):
    """Keys and values of every position, in the pages of the common pool.  ``need.params`` may give ``dv``, the size of
    a value head where it differs from a key head's (``need.dh``)."""

    def __init__(self, need: CacheNeed, runs: List[int], *, n_pages: int, max_slots: int, max_context: int,
                 dtype, device):
        super().__init__(need, runs, n_pages=n_pages, max_slots=max_slots, max_context=max_context, dtype=dtype,
                         device=device)
        dv = int(need.get().get("dv", need.dh))      # value heads of a size of their own
        self.k = torch.zeros((len(runs), n_pages, need.nkvh, PAGE, need.dh), dtype=dtype, device=device)
        self.v = torch.zeros((len(runs), n_pages, need.nkvh, PAGE, dv), dtype=dtype, device=device)

    def view(self, index: int, writable: bool) -> CacheView:
        return CacheView(self.k[index], self.v[index], writable=writable, kind=self.need.kind)

    @property
    def nbytes(self) -> int:
        return (self.k.numel() + self.v.numel()) * self.k.element_size()


@CACHE_KINDS.register("latent")
class LatentGroup(CacheStorage):
    """One row of ``need.dh`` values per position (a compressed latent and whatever travels with it), shared by
    all heads, in the pages of the common pool."""

    def __init__(self, need: CacheNeed, runs: List[int], *, n_pages: int, max_slots: int, max_context: int,
                 dtype, device):
        super().__init__(need, runs, n_pages=n_pages, max_slots=max_slots, max_context=max_context, dtype=dtype,
                         device=device)
        if need.nkvh != 1:
            raise CacheError(f"a latent cache holds one row per token, not {need.nkvh}")
        self.kv = torch.zeros((len(runs), n_pages, PAGE, need.dh), dtype=dtype, device=device)

    def view(self, index: int, writable: bool) -> LatentView:
        return LatentView(self.kv[index], writable=writable, kind=self.need.kind)

    @property
    def nbytes(self) -> int:
        return self.kv.numel() * self.kv.element_size()


class Cache:
    def __init__(self, cache_needs: Sequence[Optional[CacheNeed]], state_needs: Sequence[Optional[StateNeed]],
                 reads_from: Sequence[Optional[int]], *, max_tokens: int, max_context: int,
                 max_slots: Optional[int], dtype: torch.dtype, device: torch.device,
                 named_states: Optional[Dict[str, StateNeed]] = None):
        """cache_needs[r] / state_needs[r]: what run r's mixer asks for (state_needs[r] may be a dict, part name ->
        StateNeed, for a block in which several parts carry state); reads_from[r]: the run whose
        cache run r reads instead of owning one; named_states: per-sequence state of parts that are not a run's
        mixer (the embedding), by name."""
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        n_pages = (max_tokens + PAGE - 1) // PAGE
        if max_slots is None:
            max_slots = min(n_pages, 1024)
        self.table = SequenceTable(max_slots, n_pages, max_context)
        self.dtype = dtype
        self.device = device
        self.groups: List[CacheStorage] = []
        self._where: Dict[int, Tuple[int, int]] = {}     # run -> (group, index in group)
        self._reads_from = list(reads_from)
        by_need: Dict[CacheNeed, List[int]] = {}
        for r, need in enumerate(cache_needs):
            if need is None or reads_from[r] is not None:
                continue
            by_need.setdefault(need, []).append(r)
        for need, runs in by_need.items():
            try:
                storage_cls = CACHE_KINDS.get(need.kind)
            except ValueError as e:
                raise CacheError(str(e)) from None
            g = storage_cls(need, runs, n_pages=n_pages, max_slots=max_slots, max_context=max_context, dtype=dtype,
                            device=device)
            for i, r in enumerate(runs):
                self._where[r] = (len(self.groups), i)
            self.groups.append(g)
        for r, src in enumerate(reads_from):
            if src is not None and cache_needs[r] is not None:
                if src not in self._where:
                    raise CacheError(f"run {r} reads the cache of run {src}, which owns none")
                if cache_needs[src] != cache_needs[r]:
                    raise CacheError(f"run {r} reads the cache of run {src}, but they need different storage")
        self.state: Dict[int, object] = {}    # run -> tensor, or {part name: tensor} for a block with several
        for r, need in enumerate(state_needs):
            if isinstance(need, dict):
                if need:
                    self.state[r] = {n: torch.zeros((max_slots, *v.shape), dtype=v.dtype, device=device)
                                     for n, v in need.items()}
            elif need is not None:
                self.state[r] = torch.zeros((max_slots, *need.shape), dtype=need.dtype, device=device)
        self.named: Dict[str, torch.Tensor] = {}
        for name, need in (named_states or {}).items():
            self.named[name] = torch.zeros((max_slots, *need.shape), dtype=need.dtype, device=device)

    # ---- sequences ------------------------------------------------------------------------
    def open(self) -> int:
        slot = self.table.open()
        for t in self._state_tensors():
            t[slot].zero_()
        for t in self.named.values():
            t[slot].zero_()
        for g in self.groups:
            g.open(slot)
        return slot

    def _state_tensors(self):
        for t in self.state.values():
            if isinstance(t, dict):
                yield from t.values()
            else:
                yield t

    def close(self, slot: int) -> None:
        self.table.close(slot)
        for g in self.groups:
            g.close(slot)

    def extend(self, slot: int, new_tokens: int) -> int:
        return self.table.extend(slot, new_tokens)

    def truncate(self, slot: int, length: int) -> None:
        self.table.truncate(slot, length)

    def length(self, slot: int) -> int:
        return self.table.length[slot]

    def pages_of(self, slot: int) -> List[int]:
        return self.table.page_list[slot]

    # ---- what a run sees ----------------------------------------------------------------------
    def view(self, run: int) -> Optional[CacheView]:
        src = self._reads_from[run]
        owner = run if src is None else src
        if owner not in self._where:
            return None
        g, i = self._where[owner]
        return self.groups[g].view(i, src is None)

    def state_of(self, run: int):
        """The run's state tensor [slots, ...], or a dict of them by part name, or None."""
        return self.state.get(run)

    @property
    def nbytes(self) -> int:
        return sum(g.nbytes for g in self.groups) + sum(t.numel() * t.element_size() for t in self._state_tensors()) + \
            sum(t.numel() * t.element_size() for t in self.named.values())
