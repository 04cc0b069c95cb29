"""CPU oracle for the expert-residency policy.  TEST INFRASTRUCTURE ONLY.

A tensor-free restatement of the bookkeeping in the reference's ExpertCache
(expert_cache.py:20-52 for the per-group LRU, :93-118 for placement,
:120-179 for the order in which experts are yielded and swaps are issued,
:181-201 for a swap).  It tracks only *where* each expert is, so that the
C++ policy in the product can be checked against it trace for trace.  It is
pinned against traces recorded from the reference's own ExpertCache
(tests/golden/lru_traces.json).
"""
from __future__ import annotations

from collections import OrderedDict


class LruOracle:
    def __init__(self, main_size: int, offload_size: int, buffer_size: int):
        self.main = [None] * main_size          # device slot -> uid
        self.off = [None] * offload_size        # host slot -> uid
        self.buffers = buffer_size
        self.where = {}                         # uid -> [group, offloaded, slot]
        self.lru_main = {}                      # group -> OrderedDict(uid) least recent first
        self.lru_off = {}
        self.hits = {}
        self.misses = {}

    # expert_cache.py:93-118
    def add(self, uid, group=0, offload=None):
        assert uid not in self.where, f"expert {uid} already registered"
        placed = None
        if not offload:
            for i, u in enumerate(self.main):
                if u is None:
                    self.main[i] = uid
                    placed = [group, False, i]
                    break
        if placed is None and (offload is None or offload):
            for i, u in enumerate(self.off):
                if u is None:
                    self.off[i] = uid
                    placed = [group, True, i]
                    break
        if placed is None:
            raise ValueError("Cache is full")
        self.where[uid] = placed
        self.lru_main.setdefault(group, OrderedDict())
        self.lru_off.setdefault(group, OrderedDict())
        self.hits.setdefault(group, 0)
        self.misses.setdefault(group, 0)
        (self.lru_off if placed[1] else self.lru_main)[group][uid] = True

    def _swap(self, group, uid_in):
        """expert_cache.py:181-201: the least recently used resident expert of the
        group leaves, uid_in takes its device slot."""
        lm, lo = self.lru_main[group], self.lru_off[group]
        if not lm:
            raise ValueError("No evictable experts")
        uid_out = next(iter(lm))
        win, wout = self.where[uid_in], self.where[uid_out]
        assert win[1] and not wout[1]
        self.main[wout[2]], self.off[win[2]] = uid_in, uid_out
        win[1], wout[1] = False, True
        win[2], wout[2] = wout[2], win[2]
        del lo[uid_in]
        lm[uid_in] = True                       # most recently used
        del lm[uid_out]
        lo[uid_out] = True
        return (uid_in, uid_out, win[2])

    # expert_cache.py:120-179
    def load(self, uids, unordered=False):
        """Returns (yield order, list of swaps (uid_in, uid_out, device_slot) in issue order,
        and for each yielded uid the number of swaps that had been issued when it was yielded)."""
        uids = list(uids)
        assert len(set(uids)) == len(uids)
        if unordered:
            uids = sorted(uids, key=lambda u: self.where[u][1])          # resident first, stable
        groups = {self.where[u][0] for u in uids}
        assert len(groups) == 1, "experts must be in the same evicton group"
        group = groups.pop()
        lm, lo = self.lru_main[group], self.lru_off[group]
        for u in uids:                                                    # expert_cache.py:142-143
            if u in lm:
                lm.move_to_end(u)
                self.hits[group] += 1
            else:
                lo.move_to_end(u)
                self.misses[group] += 1
        resident = [u for u in uids if not self.where[u][1]]
        to_load = [u for u in uids if self.where[u][1]]
        window = min(self.buffers - 1, len(lm), len(to_load))             # expert_cache.py:155-157
        swaps, loading, order, issued = [], [], [], []
        for _ in range(window):
            u = to_load.pop(0)
            loading.append(u)
            swaps.append(self._swap(group, u))
        for u in uids:
            if resident and u == resident[0]:
                resident.pop(0)
                order.append(u)
                issued.append(len(swaps))
            elif loading and u == loading[0]:
                loading.pop(0)
                order.append(u)
                issued.append(len(swaps))
                if to_load:                                               # expert_cache.py:171-175
                    nxt = to_load.pop(0)
                    loading.append(nxt)
                    swaps.append(self._swap(group, nxt))
            else:
                raise RuntimeError("internal error: caching algorithm failed")
        return order, swaps, issued

    def prefetch(self, uids):
        """NOT in the reference (its README.md:24-27 lists speculative loading as upcoming).  Defined here in the
        reference's own terms so that the product's prefetch can be checked: each offloaded uid is swapped in as
        expert_cache.py:181-201 would do it for a miss; hits, misses and resident experts' order are untouched.
        Returns the swaps."""
        swaps = []
        for u in uids:
            group, offloaded, _ = self.where[u]
            if offloaded and self.lru_main[group]:
                swaps.append(self._swap(group, u))
        return swaps

    def resident(self, group=0):
        return list(self.lru_main[group].keys())
