"""ExpertCache: the reference's per-layer LRU of expert slabs (src/expert_cache.py) with
the same constructor, add_expert / add_expert_storage / load_experts protocol, exceptions
and hit/miss counters, driven by the C++ runtime in csrc/expert_cache.cpp.

Differences that matter on a B200 box (plenty of pinned host memory, copy engines beside
the SMs): every expert keeps its pinned host copy, so an eviction moves no bytes; the
host->device copy of a missing expert runs on a side stream and is ordered against the
compute stream with events, instead of being queued in front of the compute that needs it.
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Dict, Iterator, Optional, Tuple

import torch

from . import _cabi
from .expert_wrapper import MixtralExpertWrapper

ExpertUID = Any


class _GroupStats:
    """group_infos[g].hits / .misses (expert_cache.py:25-26), read from the runtime."""

    def __init__(self, cache, group):
        self._cache, self._group = cache, group

    def _stats(self):
        vals = [C.c_int64() for _ in range(4)]
        _cabi.check(_cabi.lib().hqm_cache_stats(self._cache._handle, self._group, *[C.byref(v) for v in vals]))
        return [v.value for v in vals]

    hits = property(lambda self: self._stats()[0])
    misses = property(lambda self: self._stats()[1])

    @property
    def resident(self):
        buf = (C.c_int64 * 4096)()
        n = _cabi.lib().hqm_cache_resident(self._cache._handle, self._group, buf, 4096)
        return [self._cache._uids[buf[i]] for i in range(min(n, 4096))]


class _GroupInfos(dict):
    def __init__(self, cache):
        super().__init__()
        self._cache = cache

    def __missing__(self, group):
        self[group] = _GroupStats(self._cache, group)
        return self[group]


class ExpertCache:
    def __init__(self, make_module: callable, main_size: int, offload_size: int, buffer_size: int):
        """Dynamically loads an array of modules with identical hyperparameters (expert_cache.py:56-74).
        make_module() is called main_size + buffer_size times; each result's slab is one device buffer."""
        self.module_type = self.module_size = self.device = None
        self._handle = None
        self.main_modules = [self._check_module(make_module()) for _ in range(main_size + buffer_size)]
        assert self.module_size is not None
        if self.device.type != "cuda":
            raise RuntimeError("ExpertCache needs its modules on a CUDA device (no CPU path exists)")
        self.main_size, self.offload_size, self.buffer_size = main_size, offload_size, buffer_size
        slabs = (C.c_void_p * len(self.main_modules))(*[m.storage.data_ptr() for m in self.main_modules])
        handle = C.c_void_p()
        _cabi.check(_cabi.lib().hqm_cache_create(C.byref(handle), main_size, offload_size, buffer_size,
                                                 self.module_size, slabs, self.device.index or 0))
        self._handle = handle
        self._keys: Dict[ExpertUID, int] = {}
        self._uids = []
        self._host: Dict[ExpertUID, torch.Tensor] = {}          # pinned copies, one per expert
        self.group_infos = _GroupInfos(self)
        self.active = False

    def __del__(self):
        if getattr(self, "_handle", None):
            _cabi.lib().hqm_cache_destroy(self._handle)
            self._handle = None

    def _check_module(self, module: MixtralExpertWrapper):
        assert isinstance(module.storage, torch.UntypedStorage)
        if self.module_type is None:
            self.module_type = type(module)
            self.module_size = len(module.storage)
            self.device = module.storage.device
        else:
            assert isinstance(module, self.module_type)
            assert len(module.storage) == self.module_size
            assert module.storage.device == self.device
        return module

    @property
    def registered_experts(self):
        return self._keys

    def add_expert(self, uid: ExpertUID, module: MixtralExpertWrapper, eviction_group: int = 0,
                   offload: Optional[bool] = None):
        """Register an expert to the cache and associate it with uid (expert_cache.py:86-91)."""
        assert self.module_type is not None
        assert isinstance(module, self.module_type)
        return self.add_expert_storage(uid, module.storage, eviction_group=eviction_group, offload=offload)

    def add_expert_storage(self, uid: ExpertUID, storage: torch.UntypedStorage, eviction_group: int = 0,
                           offload: Optional[bool] = None):
        """expert_cache.py:93-118."""
        assert uid not in self._keys, f"expert {uid} already registered"
        assert isinstance(storage, torch.UntypedStorage)
        assert len(storage) == self.module_size
        host = torch.empty(self.module_size, dtype=torch.uint8).pin_memory()
        host.copy_(torch.as_tensor(storage, dtype=torch.uint8, device=storage.device))
        key = len(self._uids)
        flag = -1 if offload is None else int(bool(offload))
        placed = C.c_int32()
        _cabi.check(_cabi.lib().hqm_cache_add(self._handle, key, int(eviction_group), flag, _cabi.ptr(host),
                                              C.byref(placed), _cabi.stream_ptr(self.device)))
        self._keys[uid] = key
        self._uids.append(uid)
        self._host[uid] = host

    def load_experts(self, *uids: ExpertUID, unordered: bool = False) -> Iterator[Tuple[ExpertUID, MixtralExpertWrapper]]:
        """Iterate (uid, expert) over the requested experts; usable only inside the for loop
        (expert_cache.py:120-179).  With unordered=True resident experts come first."""
        lib = _cabi.lib()
        n = len(uids)
        keys = (C.c_int64 * max(n, 1))(*[self._keys[u] for u in uids])
        stream = _cabi.stream_ptr(self.device)
        _cabi.check(lib.hqm_cache_begin(self._handle, keys, n, int(bool(unordered)), None, stream))
        self.active = True
        try:
            key, slab, slot = C.c_int64(), C.c_void_p(), C.c_int32()
            while True:
                rc = lib.hqm_cache_next(self._handle, C.byref(key), C.byref(slab), C.byref(slot), stream)
                if rc == 1:
                    break
                _cabi.check(rc)
                yield self._uids[key.value], self.main_modules[slot.value]
        finally:
            self.active = False
            lib.hqm_cache_end(self._handle, stream)

    def prefetch(self, *uids: ExpertUID) -> int:
        """Speculative loading (the reference lists it as upcoming, README.md:24-27): start bringing the offloaded ones
        among `uids` onto the device now, as a miss would, so that a later load_experts() finds them resident.
        Only between load_experts() loops.  Returns the number of copies started."""
        n = len(uids)
        if n == 0:
            return 0
        keys = (C.c_int64 * n)(*[self._keys[u] for u in uids])
        issued = C.c_int32()
        _cabi.check(_cabi.lib().hqm_cache_prefetch(self._handle, keys, n, C.byref(issued)))
        return issued.value

    def prefetch_stats(self):
        """(copies started by prefetch, guesses that were then requested, guesses evicted unused)."""
        vals = [C.c_int64() for _ in range(3)]
        _cabi.check(_cabi.lib().hqm_cache_prefetch_stats(self._handle, *[C.byref(v) for v in vals]))
        return tuple(v.value for v in vals)

    def stats(self):
        """Copy counters of the runtime: (host->device bytes moved by swaps, number of swaps)."""
        vals = [C.c_int64() for _ in range(4)]
        _cabi.check(_cabi.lib().hqm_cache_stats(self._handle, 0, *[C.byref(v) for v in vals]))
        return vals[2].value, vals[3].value
