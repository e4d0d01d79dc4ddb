"""The cache of a model: page pools with their tensors, state slots, step metadata.

Bookkeeping (which page belongs to whom) is native code (``csrc/host``); this
module owns the device tensors the ids index and turns a list of
``(request slot, tokens, wanted places)`` into the device-side ``StepBatch``.

A mixer declares what it caches per token as a list of tensors (keys and values
for attention; a mixer with one latent vector per token declares one).  Layout
of each: ``[pages + 1, heads, page_size, width]``; a page of one head is a
contiguous ``page_size x width`` tile.  The last page is a sink that padded rows
write to; the pool never hands it out.  Calls whose window and page size agree
form a group with one pool of page ids and one block table per request.
"""
from __future__ import annotations

import torch

from ..build import load_host
from ..parts.base import GroupView, PagedView, StepBatch


class ModelCache:
    def __init__(self, model, *, page_size: int = 64, num_pages: int | None = None, max_tokens: int | None = None,
                 num_slots: int = 64):
        """``num_pages`` pages per group, or enough for ``max_tokens`` tokens held at once."""
        host = load_host()
        self.host = host
        rt = model.rt
        self.rt = rt
        self.page_size = int(page_size)
        if num_pages is None:
            if max_tokens is None:
                raise ValueError("give num_pages or max_tokens")
            num_pages = -(-int(max_tokens) // self.page_size)
        self.num_pages = int(num_pages)
        self.num_slots = int(num_slots)
        needs = model.cache_needs()
        # groups: one per distinct (window, page size) among the calls that own paged tensors
        self.group_windows: list[int] = []
        self.group_page_size: list[int] = []
        self.group_pages: list[int] = []
        self.call_group: dict[int, int] = {}
        self.call_owner: dict[int, int] = {}
        self.tensors: dict[int, dict[str, torch.Tensor]] = {}
        self.state: dict[int, torch.Tensor] = {}
        keys: list[tuple[int, int]] = []
        for ci, (need, st, owner) in enumerate(needs):
            self.call_owner[ci] = owner
            if need is not None and owner == ci:
                ps = int(need.page_size or self.page_size)
                key = (int(need.window or 0), ps)
                if key not in keys:
                    keys.append(key)
                    self.group_windows.append(key[0])
                    self.group_page_size.append(ps)
                    # the same number of tokens in every pool
                    self.group_pages.append(max(1, -(-self.num_pages * self.page_size // ps)))
                g = keys.index(key)
                self.call_group[ci] = g
                self.tensors[ci] = {
                    t.name: torch.zeros((self.group_pages[g] + 1, t.heads, ps, t.width), dtype=rt.dtype, device=rt.device)
                    for t in need.tensors}
            if st is not None:
                # one slot more than requests can hold: the sink that padded rows of a step use
                self.state[ci] = torch.zeros((self.num_slots + 1, *st.shape), dtype=st.dtype, device=rt.device)
        for ci, (need, st, owner) in enumerate(needs):
            if need is not None and owner != ci:
                self.call_group[ci] = self.call_group[owner]
        if not self.group_windows:
            self.group_windows.append(0)     # a model without paged caches still counts tokens
            self.group_page_size.append(self.page_size)
            self.group_pages.append(self.num_pages)
        self.manager = host.CacheManager(
            [host.GroupSpec(ps, w, n) for ps, w, n in zip(self.group_page_size, self.group_windows, self.group_pages)],
            self.num_slots)
        self._pinned = []
        self._ring = 0
        self.last_h2d_bytes = 0      # size of the last step's metadata copy

    # ------------------------------------------------------------ requests
    def open(self) -> int:
        """Takes a state slot for a new request (its per-request state is zeroed).  -1: none free."""
        slot = self.manager.open()
        if slot >= 0:
            self.reset_state(slot)
        return slot

    def reset_state(self, slot: int) -> None:
        """Zeroes the per-request state of a slot (a request starts, or starts over)."""
        for t in self.state.values():
            t[slot].zero_()

    def close(self, slot: int) -> None:
        self.manager.close(slot)

    def append(self, slot_and_n) -> None:
        self.manager.append(list(slot_and_n))

    @property
    def k(self) -> dict[int, torch.Tensor]:
        """The ``k`` tensors of the calls that have one, by call."""
        return {ci: t["k"] for ci, t in self.tensors.items() if "k" in t}

    @property
    def v(self) -> dict[int, torch.Tensor]:
        return {ci: t["v"] for ci, t in self.tensors.items() if "v" in t}

    def bytes_per_token(self) -> int:
        """Bytes of cache one token takes over all calls (what the declared tensors add up to)."""
        return sum(t.shape[1] * t.shape[3] * t.element_size() for ts in self.tensors.values() for t in ts.values())

    # ---------------------------------------------------------- step views
    def paged_view(self, call: int, batch: StepBatch):
        if call not in self.call_group:
            return None
        owner = self.call_owner[call]
        return PagedView(self.tensors[owner], batch.groups[self.call_group[call]], write=(owner == call))

    def state_tensor(self, call: int):
        return self.state.get(call)

    # ------------------------------------------------------------ metadata
    def _staging(self, n: int):
        """A pinned int32 buffer that no copy still in flight reads (ring of four)."""
        if self.rt.device.type != "cuda":
            return torch.empty(n, dtype=torch.int32), None
        if not self._pinned:
            self._pinned = [[torch.empty(max(n, 4096), dtype=torch.int32).pin_memory(), None] for _ in range(4)]
        self._ring = (self._ring + 1) % len(self._pinned)
        ent = self._pinned[self._ring]
        if ent[1] is not None:
            ent[1].synchronize()
        if ent[0].numel() < n:
            ent[0] = torch.empty(max(n, 2 * ent[0].numel()), dtype=torch.int32).pin_memory()
        return ent[0], ent

    def make_batch(self, items, fixed_table_width: int = 0, into: torch.Tensor | None = None) -> StepBatch:
        """``items``: list of ``(slot, tokens, want)``; the requests' lengths must already
        include these tokens (``append`` first).  ``into``: a device int32 buffer to reuse
        (replayed graphs); its layout must not change between calls."""
        host = self.host
        sitems = [host.StepItem(int(s), list(t), list(w)) for s, t, w in items]
        lay = self.manager.plan_layout(sitems, fixed_table_width)
        stage, ent = self._staging(lay.total)
        self.last_h2d_bytes = 4 * lay.total
        self.manager.pack(sitems, lay, stage.data_ptr(), stage.numel())
        if into is not None:
            if into.numel() < lay.total:
                raise ValueError("metadata buffer too small")
            into[:lay.total].copy_(stage[:lay.total], non_blocking=True)
            dev = into
        else:
            dev = stage[:lay.total].to(self.rt.device, non_blocking=True)
        if ent is not None:
            ev = torch.cuda.Event()
            ev.record()
            ent[1] = ev
        return self.batch_from_layout(lay, dev)

    def fill_metadata(self, sitems, lay, dev: torch.Tensor) -> None:
        """Packs a step's metadata with a layout fixed earlier and copies it into ``dev`` (a device
        buffer that a captured graph reads).  The items must give the same layout sizes; fewer
        requests than the layout has rows are padded with rows that belong to nobody."""
        now = self.manager.plan_layout(sitems, lay.table_width[0] if lay.table_width else 0, lay.num_requests)
        if (now.total, now.num_tokens, now.num_requests, now.num_wanted) != \
                (lay.total, lay.num_tokens, lay.num_requests, lay.num_wanted):
            raise ValueError("the step does not fit the fixed metadata layout")
        stage, ent = self._staging(lay.total)
        self.last_h2d_bytes = 4 * lay.total
        self.manager.pack(sitems, lay, stage.data_ptr(), stage.numel())
        dev[:lay.total].copy_(stage[:lay.total], non_blocking=True)
        if ent is not None:
            ev = torch.cuda.Event()
            ev.record()
            ent[1] = ev

    def batch_from_layout(self, lay, dev: torch.Tensor) -> StepBatch:
        T, R, N = lay.num_tokens, lay.num_requests, lay.num_wanted

        def sl(off, n):
            return dev[off:off + n]

        groups = []
        for g, w in enumerate(self.group_windows):
            width = lay.table_width[g]
            groups.append(GroupView(slots=sl(lay.off_slots[g], T),
                                    block_table=sl(lay.off_table[g], R * width).view(R, width),
                                    page_size=self.group_page_size[g], window=w))
        return StepBatch(num_tokens=T, num_requests=R, tokens=sl(lay.off_tokens, T),
                         positions=sl(lay.off_positions, T), token_req=sl(lay.off_token_req, T),
                         cu_q=sl(lay.off_cu_q, R + 1), kv_len=sl(lay.off_kv_len, R),
                         state_slot=sl(lay.off_state_slot, R), logit_rows=sl(lay.off_logit_rows, N),
                         groups=groups, max_q_len=lay.max_q_len, max_kv_len=lay.max_kv_len,
                         num_single=lay.num_single)

    def stats(self):
        return [self.manager.stats(g) for g in range(len(self.group_windows))]
