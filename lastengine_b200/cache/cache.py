"""The cache: per-sequence keys/values and fixed-size state, for every layer that keeps any.

A sequence gets a slot when it starts and gives it back when it ends; slots and pages are
reused.  Layers are grouped by what they need:

* a KV group per distinct (kv heads, key head size, value head size, window): pools of pages of
  `page_size` positions, keys `[entry, page, kv_head, position in page, head_dim]` and values
  `[entry, page, kv_head, value_dim, position in page]`, with a page pool and a page list per
  sequence of its own.  A windowed group gives pages back once every position in
  them has left the window.
  A group whose spec pools blocks of positions has a second pair of pools of the same layout, one row per
  complete block, with pages and a page list per sequence of their own; they are never given back before
  the sequence ends.
* a latent group per distinct (rank, rotated key width) is a KV group with one "head" whose key row is
  the cached row `[latent | rotated key part]` and whose value pool is empty (the values are read out
  of the same row); pages, tables, export and import are those of any KV group.
* a state group per distinct (shape, dtype): `[entry, slot, *shape]`, zeroed when a slot is
  given out (the reference zeroes its convolution state on reset, src/gpu/dense.rs:264-267); an entry may
  keep several states of different shapes (a recurrent state and a convolution's memory).

The reference keeps one sequence: K/V `[ctx][kv_head][head_dim]` per attention layer and a
float convolution state per conv layer (src/gpu/dense.rs:91-107).  Lengths live on the host;
each step carries the positions, slots and page tables it needs to the device, so the device
holds nothing per sequence but the data itself.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import KVSpec, LatentSpec, StateSpec
from .allocator import CacheError, CacheFull, IdPool

PAGE_SIZE = 64


@dataclass
class CacheView:
    """What one schedule entry's mixer sees of the cache during a step."""
    writable: bool
    page_size: int = PAGE_SIZE
    k: torch.Tensor | None = None            # [page, kv_head, page_size, head_dim]
    v: torch.Tensor | None = None            # [page, kv_head, value_dim, page_size] (positions contiguous)
    block_table: torch.Tensor | None = None  # int32 [sequences of the step, pages]
    state: torch.Tensor | None = None        # [slot, *shape]: the entry's first (or only) state
    states: list = field(default_factory=list)   # every state of the entry, in the order its mixer names them
    pooled_k: torch.Tensor | None = None     # [page, kv_head, page_size, head_dim]: row b is block b's pooled key
    pooled_v: torch.Tensor | None = None     # [page, kv_head, value_dim, page_size]
    pooled_table: torch.Tensor | None = None  # int32 [sequences of the step, pages of pooled rows]


def pooled_table_key(group: int) -> int:
    """Under which key a step's tables hold the page lists of a group's pooled rows (the group's own
    number is the key of its positions' page lists)."""
    return -1 - group


class KVGroup:
    def __init__(self, spec: KVSpec, entries: list[int], n_pages: int, page_size: int,
                 dtype: torch.dtype, device, max_seqs: int | None = None):
        self.spec, self.entries = spec, list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.page_size = page_size
        # keys as [.., position, dim], values as [.., dim, position]
        self.k_pool = torch.zeros((len(entries), n_pages, spec.n_kv_heads, page_size, spec.head_dim),
                                  dtype=dtype, device=device)
        self.v_pool = torch.zeros((len(entries), n_pages, spec.n_kv_heads, spec.value_dim, page_size),
                                  dtype=dtype, device=device)
        self.pages = IdPool(n_pages, "cache page")
        self.seq_pages: dict[int, list[int]] = {}   # slot -> page of each page index (-1: given back)
        # pooled rows: a sequence of n positions holds n // pool of them, rounded up to whole pages
        self.pool = int(getattr(spec, "pool", 0) or 0)
        self.pooled_k = self.pooled_v = self.pooled_pages = None
        self.seq_pooled_pages: dict[int, list[int]] = {}
        if self.pool > 0:
            n_pooled = -(-n_pages // self.pool) + min(max_seqs or n_pages, n_pages)
            self.pooled_k = torch.zeros((len(entries), n_pooled, spec.n_kv_heads, page_size, spec.head_dim),
                                        dtype=dtype, device=device)
            self.pooled_v = torch.zeros((len(entries), n_pooled, spec.n_kv_heads, spec.value_dim, page_size),
                                        dtype=dtype, device=device)
            self.pooled_pages = IdPool(n_pooled, "page of pooled rows")

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self.seq_pages.get(slot, ()))
        return max(0, -(-new_len // self.page_size) - have)

    def pooled_pages_needed(self, slot: int, new_len: int) -> int:
        if self.pool <= 0:
            return 0
        have = len(self.seq_pooled_pages.get(slot, ()))
        return max(0, -(-(new_len // self.pool) // self.page_size) - have)

    def grow(self, slot: int, new_len: int) -> None:
        lst = self.seq_pages.setdefault(slot, [])
        lst.extend(self.pages.alloc_many(self.pages_needed(slot, new_len)))
        if self.pool > 0:
            self.seq_pooled_pages.setdefault(slot, []).extend(
                self.pooled_pages.alloc_many(self.pooled_pages_needed(slot, new_len)))

    def trim(self, slot: int, length: int) -> None:
        """Gives back the pages no later query can reach (windowed groups only)."""
        w = self.spec.window
        if w <= 0:
            return
        first_needed = length + 1 - w     # the next query, at position `length`, reaches back to here
        if self.pool > 0:                 # the block that is still filling is pooled from its cached rows
            first_needed = min(first_needed, length // self.pool * self.pool)
        lst = self.seq_pages.get(slot, [])
        for j, p in enumerate(lst):
            if p >= 0 and (j + 1) * self.page_size - 1 < first_needed:
                self.pages.free(p)
                lst[j] = -1

    def release(self, slot: int) -> None:
        for p in self.seq_pages.pop(slot, []):
            if p >= 0:
                self.pages.free(p)
        for p in self.seq_pooled_pages.pop(slot, []):
            self.pooled_pages.free(p)

    def table(self, slots: list[int], width: int, pooled: bool = False) -> np.ndarray:
        """The page list of every sequence of a step (-1 where it holds none); `pooled`: of its pooled rows."""
        t = np.full((len(slots), max(width, 1)), -1, dtype=np.int32)
        for i, s in enumerate(slots):
            if s < 0:
                continue
            lst = (self.seq_pooled_pages if pooled else self.seq_pages).get(s, [])
            if len(lst) > width:
                raise CacheError(f"sequence in slot {s} holds {len(lst)} pages, the step's table has {width}")
            t[i, :len(lst)] = lst
        return t


class StateGroup:
    def __init__(self, spec: StateSpec, entries: list[int], max_seqs: int, device):
        self.spec, self.entries = spec, list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.data = torch.zeros((len(entries), max_seqs, *spec.shape), dtype=spec.dtype, device=device)


class Cache:
    def __init__(self, specs: dict[int, KVSpec | StateSpec], max_tokens: int, max_seqs: int | None,
                 dtype: torch.dtype, device, page_size: int = PAGE_SIZE):
        """`specs`: cache entry id -> what it keeps.  `max_tokens`: positions all live sequences
        may hold together, each sequence rounded up to whole pages."""
        if page_size % 32 != 0:
            raise ValueError("page size must be a multiple of 32")
        self.page_size = page_size
        self.n_pages = max(1, -(-int(max_tokens) // page_size))
        self.max_seqs = int(max_seqs) if max_seqs else self.n_pages
        self.dtype, self.device = dtype, device
        self.slots = IdPool(self.max_seqs, "sequence slot")
        self.lens: dict[int, int] = {}
        self.state_version = 0      # bumped by every change of lengths, pages or slots
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        # entry -> its places, each (kind, group): one for most mixers, keys/values and a state for
        # a mixer that keeps both
        self._where: dict[int, list[tuple[str, int]]] = {}
        self._state_order: dict[int, list[StateSpec]] = {}     # entry -> its states in the order its mixer names them
        by_spec: dict[object, list[int]] = {}
        for entry, spec in sorted(specs.items()):
            if spec is None:
                continue
            several = list(spec) if isinstance(spec, (tuple, list)) else [spec]
            kinds = [type(s) for s in several]
            states = [s for s in several if isinstance(s, StateSpec)]
            if kinds.count(KVSpec) + kinds.count(LatentSpec) > 1 or len(set(states)) != len(states):
                raise TypeError(f"cache entry {entry}: at most one KVSpec, and states of different shapes, got {spec!r}")
            self._state_order[entry] = states
            for s in several:
                by_spec.setdefault(s, []).append(entry)
        for spec, entries in by_spec.items():
            if isinstance(spec, (KVSpec, LatentSpec)):
                self.kv_groups.append(KVGroup(spec, entries, self.n_pages, page_size, dtype, device, self.max_seqs))
                for e in entries:
                    self._where.setdefault(e, []).append(("kv", len(self.kv_groups) - 1))
            elif isinstance(spec, StateSpec):
                self.state_groups.append(StateGroup(spec, entries, self.max_seqs, device))
                for e in entries:
                    self._where.setdefault(e, []).append(("state", len(self.state_groups) - 1))
            else:
                raise TypeError(f"unknown cache spec {spec!r}")
        for places in self._where.values():
            places.sort()        # keys and values before the state, whatever order the groups were made in

    # ---- sequences -----------------------------------------------------------------------
    def alloc_seq(self) -> int:
        slot = self.slots.alloc()
        self.state_version += 1
        self.lens[slot] = 0
        for g in self.state_groups:
            g.data[:, slot].zero_()
        return slot

    def free_seq(self, slot: int) -> None:
        if not self.slots.holds(slot):
            raise CacheError(f"sequence slot {slot} is not held (freed twice, or never given out)")
        self.state_version += 1
        for g in self.kv_groups:
            g.release(slot)
        del self.lens[slot]
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        try:
            return self.lens[slot]
        except KeyError:
            raise CacheError(f"sequence slot {slot} is not held") from None

    def reserve(self, grow: dict[int, int]) -> None:
        """Makes room for `grow[slot]` more positions per sequence, or raises CacheFull and
        leaves everything as it was."""
        for g in self.kv_groups:
            need = sum(g.pages_needed(s, self.length(s) + n) for s, n in grow.items())
            if need > g.pages.n_free:
                raise CacheFull(f"the step needs {need} more cache pages of {self.page_size} positions, "
                                f"{g.pages.n_free} of {g.pages.n} are free")
            if g.pool > 0:
                need = sum(g.pooled_pages_needed(s, self.length(s) + n) for s, n in grow.items())
                if need > g.pooled_pages.n_free:
                    raise CacheFull(f"the step needs {need} more pages of pooled rows, "
                                    f"{g.pooled_pages.n_free} of {g.pooled_pages.n} are free")
        for g in self.kv_groups:
            for s, n in grow.items():
                g.grow(s, self.lens[s] + n)

    def commit(self, grow: dict[int, int]) -> None:
        """After the step ran: the sequences are `grow[slot]` positions longer."""
        self.state_version += 1
        for s, n in grow.items():
            self.lens[s] += n
            for g in self.kv_groups:
                g.trim(s, self.lens[s])

    def pages_held(self, slot: int) -> int:
        return max((len(g.seq_pages.get(slot, ())) for g in self.kv_groups), default=0)

    # ---- a sequence as bytes --------------------------------------------------------------
    def _places(self) -> list[tuple[int, str, int]]:
        """(entry, kind, group) of everything the cache holds, in the order it is written out."""
        return [(e, kind, gi) for e in sorted(self._where) for kind, gi in self._where[e]]

    def _entry_nbytes(self, entry: int, length: int, kind: str | None = None, gi: int = 0) -> int:
        if kind is None:
            return sum(self._entry_nbytes(entry, length, k, g) for k, g in self._where[entry])
        if kind == "state":
            g = self.state_groups[gi]
            return int(np.prod(g.spec.shape, dtype=np.int64)) * g.data.element_size()
        g = self.kv_groups[gi]
        sp = g.spec
        rows = length + (length // g.pool if g.pool > 0 else 0)      # the positions, then the pooled rows
        return rows * sp.n_kv_heads * (sp.head_dim + sp.value_dim) * g.k_pool.element_size()

    @staticmethod
    def _sections(g: KVGroup, i: int, slot: int, n: int):
        """(key pool, value pool, the sequence's pages, rows held) of an entry's positions and of its pooled rows."""
        yield g.k_pool[i], g.v_pool[i], g.seq_pages.get(slot, []), n
        if g.pool > 0:
            yield g.pooled_k[i], g.pooled_v[i], g.seq_pooled_pages.get(slot, []), n // g.pool

    def _rows_of_pages(self, sp, kp: torch.Tensor, vp: torch.Tensor, pages: list[int]):
        """Keys [rows, kv head, dim] and values [rows, kv head, value dim] of a page list (zeros for pages given back)."""
        ps = self.page_size
        k = torch.zeros((len(pages) * ps, sp.n_kv_heads, sp.head_dim), dtype=self.dtype, device=self.device)
        v = torch.zeros((len(pages) * ps, sp.n_kv_heads, sp.value_dim), dtype=self.dtype, device=self.device)
        for j, p in enumerate(pages):
            if p >= 0:
                k[j * ps:(j + 1) * ps] = kp[p].permute(1, 0, 2)
                v[j * ps:(j + 1) * ps] = vp[p].permute(2, 0, 1)
        return k, v

    def export_seq(self, slot: int) -> bytes:
        """What a sequence holds, as bytes: its length (u64, little-endian), then for every cache
        entry in order its state, or its keys and then its values as `[position][kv head][dim]`
        in the cache's dtype.  The reference writes one sequence the same way: position count,
        then per layer the state or K and V up to that position (src/gpu/dense.rs:391-399).
        Positions that a windowed group has given back are written as zeros.  An entry that pools
        blocks of positions writes its pooled rows (keys, then values) after those of the positions."""
        n = self.length(slot)
        out = [struct.pack("<Q", n)]
        raw = lambda t: t.contiguous().view(torch.uint8).cpu().numpy().tobytes()
        ps = self.page_size
        for entry, kind, gi in self._places():
            if kind == "state":
                g = self.state_groups[gi]
                out.append(raw(g.data[g.index[entry], slot].reshape(-1)))
                continue
            g = self.kv_groups[gi]
            i = g.index[entry]
            for kp, vp, pages, rows in self._sections(g, i, slot, n):
                k, v = self._rows_of_pages(g.spec, kp, vp, pages)
                out.append(raw(k[:rows].reshape(-1)))
                out.append(raw(v[:rows].reshape(-1)))
        return b"".join(out)

    def import_seq(self, data: bytes) -> int:
        """A new sequence that holds what `export_seq` wrote (same model, same dtype).  Raises
        CacheError when the bytes do not fit this model and CacheFull when there is no room; the
        cache is then as it was (the reference checks the same two things, src/gpu/dense.rs:400-412)."""
        if len(data) < 8:
            raise CacheError("sequence data is too short to hold a length")
        (n,) = struct.unpack_from("<Q", data, 0)
        need = 8 + sum(self._entry_nbytes(e, n) for e in self._where)
        if len(data) != need:
            raise CacheError(f"sequence data of {len(data)} bytes does not match this model and dtype "
                             f"({need} bytes for {n} positions)")
        slot = self.alloc_seq()
        try:
            self.reserve({slot: n})
        except CacheFull:
            self.free_seq(slot)
            raise
        ps, o = self.page_size, 8
        buf = torch.frombuffer(bytearray(data), dtype=torch.uint8).to(self.device)
        for entry, kind, gi in self._places():
            nb = self._entry_nbytes(entry, n, kind, gi)
            if kind == "state":
                g = self.state_groups[gi]
                dst = g.data[g.index[entry], slot]
                dst.copy_(buf[o:o + nb].clone().view(g.data.dtype).view(dst.shape))
                o += nb
                continue
            g = self.kv_groups[gi]
            i, sp = g.index[entry], g.spec
            for kp, vp, pages, rows in self._sections(g, i, slot, n):
                for which, width in ((0, sp.head_dim), (1, sp.value_dim)):
                    part = rows * sp.n_kv_heads * width * g.k_pool.element_size()
                    t = torch.zeros((len(pages) * ps, sp.n_kv_heads, width), dtype=self.dtype, device=self.device)
                    if rows:
                        t[:rows] = buf[o:o + part].clone().view(self.dtype).view(rows, sp.n_kv_heads, width)
                    o += part
                    for j, p in enumerate(pages):
                        block = t[j * ps:(j + 1) * ps]
                        if which == 0:
                            kp[p] = block.permute(1, 0, 2)
                        else:
                            vp[p] = block.permute(1, 2, 0)
        self.commit({slot: n})
        return slot

    # ---- views ---------------------------------------------------------------------------
    def group_of(self, entry: int) -> tuple[str, int] | None:
        """(kind, group) of the entry's first place (its keys and values, if it has any)."""
        w = self._where.get(entry)
        return w[0] if w else None

    def view(self, entry: int, writable: bool, tables: dict[int, torch.Tensor]) -> CacheView:
        view = CacheView(writable=writable, page_size=self.page_size)
        for kind, gi in self._where.get(entry, ()):
            if kind == "kv":
                g = self.kv_groups[gi]
                i = g.index[entry]
                view.k, view.v, view.block_table = g.k_pool[i], g.v_pool[i], tables[gi]
                if g.pool > 0:
                    view.pooled_k, view.pooled_v = g.pooled_k[i], g.pooled_v[i]
                    view.pooled_table = tables[pooled_table_key(gi)]
            else:
                g = self.state_groups[gi]
                at = self._state_order[entry].index(g.spec)
                while len(view.states) <= at:
                    view.states.append(None)
                view.states[at] = g.data[g.index[entry]]
        if view.states:
            view.state = view.states[0]
        return view

    def check(self) -> None:
        """Bookkeeping invariants (used by tests): nothing lost, nothing held twice."""
        self.slots.check()
        assert set(self.lens) == self.slots._held
        for g in self.kv_groups:
            g.pages.check()
            held = [p for lst in g.seq_pages.values() for p in lst if p >= 0]
            assert len(held) == len(set(held)), "a page belongs to two sequences"
            assert set(held) == g.pages._held, "held pages and page lists disagree"
            assert set(g.seq_pages) <= self.slots._held, "a freed sequence still owns pages"
            if g.pool > 0:
                g.pooled_pages.check()
                held = [p for lst in g.seq_pooled_pages.values() for p in lst]
                assert len(held) == len(set(held)) and set(held) == g.pooled_pages._held, "pages of pooled rows are off"
                assert set(g.seq_pooled_pages) <= self.slots._held, "a freed sequence still owns pages of pooled rows"

    def nbytes(self) -> int:
        n = sum((g.k_pool.numel() + g.v_pool.numel()) * g.k_pool.element_size() for g in self.kv_groups)
        n += sum((g.pooled_k.numel() + g.pooled_v.numel()) * g.k_pool.element_size() for g in self.kv_groups if g.pool > 0)
        return n + sum(g.data.numel() * g.data.element_size() for g in self.state_groups)
