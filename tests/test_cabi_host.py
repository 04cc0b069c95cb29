"""Host-side checks that need no GPU: the library loads, exports what the header declares,
the residency policy replays the reference's recorded traces, and the slab order matches."""
import ctypes as C
import json
import os
import re

import pytest
import torch

from mixtral_offloading_b200 import _cabi
from mixtral_offloading_b200 import build as libbuild

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    libbuild.build()
    return _cabi.lib()


def test_header_symbols_exported(lib):
    header = open(os.path.join(ROOT, "include", "hqq_moe.h")).read()
    declared = set(re.findall(r"\b(hqm_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/hqq_moe.h but not exported"
    assert declared == set(_cabi.SIGNATURES), "ctypes table and header disagree"
    assert lib.hqm_version() >= 1


def test_argument_errors_are_reported_not_raised_in_c(lib):
    w = _cabi.HqmWeight(N=128, K=256, nbits=5, group_size=64, meta_group=256)
    assert lib.hqm_dequantize(None, 0, C.byref(w), None) == _cabi.HQM_ERR_ARG
    assert "nbits == 5" in _cabi.last_error()
    w = _cabi.HqmWeight(N=100, K=256, nbits=4, group_size=64, meta_group=256)
    assert lib.hqm_linear(None, None, 1, C.byref(w), None, None, 0, None) == _cabi.HQM_ERR_ARG
    with pytest.raises(ValueError):
        _cabi.check(_cabi.HQM_ERR_ARG)
    assert lib.hqm_pack_4bit_u8(None, None, 3, 16, None) == _cabi.HQM_ERR_ARG      # odd row count
    assert lib.hqm_unpack_2bit_u8(None, None, 4, 16, None) == _cabi.HQM_ERR_ARG    # null pointers
    assert lib.hqm_unpack_2bit_u8(None, None, 0, 16, None) == 0                    # nothing to do


class PolicyHandle:
    """Bookkeeping-only cache handle (no device slabs, no CUDA calls)."""

    def __init__(self, lib, main_size, offload_size, buffer_size):
        self.lib = lib
        self.h = C.c_void_p()
        assert lib.hqm_cache_create(C.byref(self.h), main_size, offload_size, buffer_size, 64, None, 0) == 0

    def close(self):
        self.lib.hqm_cache_destroy(self.h)

    def add(self, key, group, offload):
        flag = -1 if offload is None else int(bool(offload))
        placed = C.c_int32()
        rc = self.lib.hqm_cache_add(self.h, key, group, flag, None, C.byref(placed), None)
        return rc, placed.value

    def load(self, keys, unordered, consume=None):
        arr = (C.c_int64 * max(len(keys), 1))(*keys)
        planned = (C.c_int64 * max(len(keys), 1))()
        rc = self.lib.hqm_cache_begin(self.h, arr, len(keys), int(unordered), planned, None)
        if rc != 0:
            return rc, []
        order = []
        k, slab, slot = C.c_int64(), C.c_void_p(), C.c_int32()
        while True:
            rc = self.lib.hqm_cache_next(self.h, C.byref(k), C.byref(slab), C.byref(slot), None)
            if rc != 0:
                break
            order.append((k.value, slot.value))
            if consume is not None and len(order) >= consume:
                self.lib.hqm_cache_end(self.h, None)
                return 0, order
        if rc < 0:
            return rc, order
        assert [o[0] for o in order] == list(planned)[:len(keys)]
        return 0, order

    def resident(self, group):
        buf = (C.c_int64 * 256)()
        n = self.lib.hqm_cache_resident(self.h, group, buf, 256)
        return [buf[i] for i in range(n)]

    def stats(self, group):
        v = [C.c_int64() for _ in range(4)]
        assert self.lib.hqm_cache_stats(self.h, group, *[C.byref(x) for x in v]) == 0
        return [x.value for x in v]


def test_cache_policy_replays_reference_traces(lib, golden_dir):
    traces = json.load(open(os.path.join(golden_dir, "lru_traces.json")))
    for tr in traces:
        pol = PolicyHandle(lib, tr["main_size"], tr["offload_size"], tr["buffer_size"])
        keyof = {}
        for uid, group, offload in tr["placement"]:
            keyof[tuple(uid)] = len(keyof)
            rc, placed = pol.add(keyof[tuple(uid)], group, offload)
            assert rc == 0 and placed == int(offload)
        uidof = {v: k for k, v in keyof.items()}
        for step in tr["steps"]:
            keys = [keyof[tuple(u)] for u in step["request"]]
            rc, order = pol.load(keys, step["unordered"])
            assert rc == 0, _cabi.last_error()
            group = step["request"][0][0]
            if all(step["intact"]):
                # (when the reference itself corrupts a slab the runtime protects it by
                #  evicting a different expert, so residency may differ from that point on)
                assert [list(uidof[k]) for k, _ in order] == step["order"]
                assert [list(uidof[k]) for k in pol.resident(group)] == step["resident"]
                hits, misses, _, _ = pol.stats(group)
                assert (hits, misses) == (step["hits"], step["misses"])
            else:
                assert [list(uidof[k]) for k, _ in order] == step["order"]
                break
        pol.close()


def test_cache_never_hands_out_an_overwritten_slab(lib):
    """Track slab contents on the host: every yielded (uid, slot) must still hold that uid."""
    import random
    rng = random.Random(1)
    for buffers in (2, 3, 4):
        pol = PolicyHandle(lib, 3, 5, buffers)
        for e in range(8):
            assert pol.add(e, 0, e >= 3)[0] == 0
        for _ in range(200):
            k = rng.choice([1, 2, 3, 5, 8])
            req = rng.sample(range(8), k)
            rc, order = pol.load(req, rng.random() < 0.5)
            assert rc == 0, _cabi.last_error()
            assert sorted(o[0] for o in order) == sorted(req)
            assert len(pol.resident(0)) == 3
        pol.close()


def test_prefetch_bookkeeping_matches_oracle(lib):
    """Prefetch = the reference's swap applied early: residency follows the oracle, hits and misses only count
    requests, and the used / wasted counters add up."""
    import random
    from oracle.lru_oracle import LruOracle
    rng = random.Random(5)
    for buffers in (2, 4):
        pol, orc = PolicyHandle(lib, 4, 4, buffers), LruOracle(4, 4, buffers)
        for e in range(8):
            assert pol.add(e, 0, e >= 4)[0] == 0
            orc.add(e, 0, e >= 4)
        issued_total = 0
        for step in range(300):
            if rng.random() < 0.6:
                guess = rng.sample(range(8), rng.choice([1, 2]))
                arr, issued = (C.c_int64 * len(guess))(*guess), C.c_int32()
                before = pol.stats(0)[:2]
                assert lib.hqm_cache_prefetch(pol.h, arr, len(guess), C.byref(issued)) == 0
                assert issued.value == len(orc.prefetch(guess))
                assert pol.stats(0)[:2] == before
                issued_total += issued.value
            req = rng.sample(range(8), 2)
            rc, order = pol.load(req, True)
            want_order, _, _ = orc.load(req, unordered=True)
            assert rc == 0 and [o[0] for o in order] == want_order
            assert pol.resident(0) == orc.resident(0)
            assert pol.stats(0)[:2] == [orc.hits[0], orc.misses[0]]
        v = [C.c_int64() for _ in range(3)]
        assert lib.hqm_cache_prefetch_stats(pol.h, *[C.byref(x) for x in v]) == 0
        n_issued, used, wasted = [x.value for x in v]
        assert n_issued == issued_total and used > 0 and wasted > 0
        assert used + wasted <= n_issued <= used + wasted + 4       # at most the resident set is still undecided
        # not while a request is running
        rc, order = pol.load([0, 1], True, consume=1)
        arr = (C.c_int64 * 1)(0)
        assert lib.hqm_cache_begin(pol.h, arr, 1, 0, None, None) == 0
        assert lib.hqm_cache_prefetch(pol.h, arr, 1, None) == _cabi.HQM_ERR_STATE
        lib.hqm_cache_end(pol.h, None)
        pol.close()


def test_cache_errors_match_reference(lib):
    pol = PolicyHandle(lib, 1, 1, 2)
    assert pol.add(0, 0, False)[0] == 0
    assert pol.add(1, 0, True)[0] == 0
    rc, _ = pol.add(2, 0, None)
    assert rc == _cabi.HQM_ERR_STATE and _cabi.last_error() == "Cache is full"
    with pytest.raises(ValueError):
        _cabi.check(rc)
    rc, _ = pol.add(0, 0, None)
    assert rc == _cabi.HQM_ERR_STATE and "already registered" in _cabi.last_error()
    rc, _ = pol.load([0, 0], False)
    assert rc == _cabi.HQM_ERR_STATE
    # re-entrant request
    rc, order = pol.load([0, 1], True, consume=1)
    assert rc == 0 and len(order) == 1
    arr = (C.c_int64 * 1)(0)
    assert lib.hqm_cache_begin(pol.h, arr, 1, 0, None, None) == 0      # previous request was ended
    assert lib.hqm_cache_begin(pol.h, arr, 1, 0, None, None) == _cabi.HQM_ERR_STATE
    assert "already loading experts" in _cabi.last_error()
    with pytest.raises(AssertionError):
        _cabi.check(_cabi.HQM_ERR_STATE)
    lib.hqm_cache_end(pol.h, None)
    pol.close()
    # mixed eviction groups
    pol = PolicyHandle(lib, 2, 2, 2)
    pol.add(0, 0, False)
    pol.add(1, 1, False)
    rc, _ = pol.load([0, 1], False)
    assert rc == _cabi.HQM_ERR_STATE and "same evicton group" in _cabi.last_error()
    pol.close()
    # a single buffer cannot serve a miss (window of buffer_size - 1 == 0 copies), as in the reference
    pol = PolicyHandle(lib, 1, 1, 1)
    pol.add(0, 0, False)
    pol.add(1, 0, True)
    rc, _ = pol.load([1], False)
    assert rc == _cabi.HQM_ERR_STATE and _cabi.last_error().startswith("internal error")
    with pytest.raises(RuntimeError):
        _cabi.check(rc)
    pol.close()


def test_slab_order_matches_reference(golden_dir):
    """Same tensor order as MixtralExpertWrapper.replace_layer_storage; offsets differ only by alignment."""
    from mixtral_offloading_b200 import BaseQuantizeConfig, HQQLinearTritonSavable
    from mixtral_offloading_b200.expert_wrapper import SLAB_ALIGN, MixtralExpertWrapper, slab_layout
    ref = json.load(open(os.path.join(golden_dir, "slab_layout.json")))
    hidden, ffn = 128, 256
    cfg = BaseQuantizeConfig(nbits=2, group_size=16, quant_zero=True, quant_scale=True)

    class Expert:
        pass
    ex = Expert()
    named = {}
    for name, shape in (("w1", (hidden, ffn)), ("w2", (ffn, hidden)), ("w3", (hidden, ffn))):
        lyr = HQQLinearTritonSavable(None, cfg, HQQLinearTritonSavable.get_hqq_meta(shape, cfg))
        N, K = lyr.meta["shape"]
        C_ = (N // 16) * K // 256
        lyr.W_q = torch.randint(0, 255, (N // 4, K), dtype=torch.uint8)
        lyr.meta["scale_q"] = torch.randint(0, 255, (256, C_), dtype=torch.uint8)
        lyr.meta["zero_q"] = torch.randint(0, 255, (256, C_), dtype=torch.uint8)
        for mm in ("meta_scale", "meta_zero"):
            lyr.meta[mm]["scale"] = torch.rand(1, C_).half()
            lyr.meta[mm]["zero"] = torch.rand(1, C_).half()
        setattr(ex, name, lyr)
        named[name] = lyr
    before = {n: (l.W_q.clone(), l.meta["scale_q"].clone()) for n, l in named.items()}
    state = {n: {"W_q": l.W_q, "meta": l.meta, "bias": l.bias} for n, l in named.items()}
    placed, size = slab_layout(state)
    sizes = [t.nbytes for t, _ in placed]
    ref_sizes = [b - a for a, b in zip(ref["offsets"], ref["offsets"][1:] + [ref["total"]])]
    assert sizes == ref_sizes                                  # same tensors in the same order
    assert all(off % SLAB_ALIGN == 0 for _, off in placed)
    wrapper = MixtralExpertWrapper(ex, torch.device("cpu"))
    assert len(wrapper.storage) == size
    base = wrapper.storage.data_ptr()
    assert named["w1"].W_q.data_ptr() == base
    for n, l in named.items():
        assert torch.equal(l.W_q, before[n][0]) and torch.equal(l.meta["scale_q"], before[n][1])
        assert base <= l.W_q.data_ptr() < base + size
    assert len(list(wrapper.parameters())) == 0 and list(wrapper.state_dict().keys()) == ["storage"]
