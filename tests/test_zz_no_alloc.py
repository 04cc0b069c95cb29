"""hqm_linear_static_scratch: the entry point for callers that cannot allocate a workspace
(stream capture in progress, foreign hosts without a device allocator, frozen memory plans).

Collected last on purpose: if it fails, a run that stops at the first failure has already
run every other test.  It must also pass alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

from mixtral_offloading_b200 import _cabi
from oracle import hqq_oracle as O
from tests.helpers import layer_from_oracle, random_layer, random_layer_fast

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = 1e-2


def _both(layer, x):
    """(existing entry point with a torch-owned workspace, new entry point with the built-in one)."""
    lib = _cabi.lib()
    d = layer.descriptor()
    M, N = x.shape[0], layer.meta["shape"][0]
    need = lib.hqm_linear_scratch_bytes(M, C.byref(d))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    if need:
        _cabi.check(lib.hqm_scratch_init(_cabi.ptr(ws), _cabi.stream_ptr(DEV)))
    y_ref = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    y_new = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    stream = _cabi.stream_ptr(DEV)
    _cabi.check(lib.hqm_linear(_cabi.ptr(y_ref), _cabi.ptr(x), M, C.byref(d), None, _cabi.ptr(ws), need, stream))
    _cabi.check(lib.hqm_linear_static_scratch(_cabi.ptr(y_new), _cabi.ptr(x), M, C.byref(d), None, stream))
    torch.cuda.synchronize(DEV)
    return need, y_ref, y_new


@pytest.mark.parametrize("nbits,group,N,K", [(2, 16, 1792, 1024), (4, 64, 1024, 4096)])
def test_static_scratch_matches_caller_scratch_twice(nbits, group, N, K):
    od = random_layer(N, K, nbits, group, seed=nbits)
    layer = layer_from_oracle(od, DEV)
    g = torch.Generator().manual_seed(0)
    for call, M in enumerate((1, 8)):                       # two calls in a row share the workspace
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        need, y_ref, y_new = _both(layer, x.to(DEV))
        assert need > 0, "this shape must take the path that uses scratch memory"
        assert not torch.isnan(y_new.float()).any()
        assert O.rel_err(y_new.cpu(), y_ref.cpu()) < TOL, f"call {call}"
        assert O.rel_err(y_new.cpu(), O.linear(x, od)) < TOL, f"call {call}"


@pytest.mark.parametrize("nbits,group,N,K,Ms", [(2, 16, 14336, 4096, (24, 17)), (3, 64, 1792, 512, (1, 4)),
                                                 (3, 64, 1792, 512, (16, 5))])
def test_static_scratch_other_kernels(nbits, group, N, K, Ms):
    """The built-in workspace also serves the tensor-core path (M >= 17, 2-bit) and both 3-bit paths."""
    od = random_layer(N, K, nbits, group, seed=7 * nbits)
    layer = layer_from_oracle(od, DEV)
    g = torch.Generator().manual_seed(1)
    for call, M in enumerate(Ms):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        need, y_ref, y_new = _both(layer, x.to(DEV))
        assert 0 < need <= _cabi.lib().hqm_static_scratch_capacity()
        assert not torch.isnan(y_new.float()).any()
        assert O.rel_err(y_new.cpu(), y_ref.cpu()) < TOL, f"call {call}"
        assert O.rel_err(y_new.cpu(), O.linear(x, od)) < TOL, f"call {call}"
    assert _cabi.lib().hqm_device_error() == 0


def test_static_scratch_rejects_oversized_calls():
    lib = _cabi.lib()
    cap = lib.hqm_static_scratch_capacity()
    assert cap == 2 << 20
    N = 28672
    od = random_layer_fast(N, 4096, 2, 16, seed=1)
    layer = layer_from_oracle(od, DEV)
    d = layer.descriptor()
    M = 16
    assert lib.hqm_linear_scratch_bytes(M, C.byref(d)) > cap
    x = torch.zeros((M, 4096), dtype=torch.bfloat16, device=DEV)
    y = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    rc = lib.hqm_linear_static_scratch(_cabi.ptr(y), _cabi.ptr(x), M, C.byref(d), None, _cabi.stream_ptr(DEV))
    assert rc == _cabi.HQM_ERR_SCRATCH
    assert "workspace" in _cabi.last_error() and str(cap) in _cabi.last_error()
    # one row of the same layer fits
    rc = lib.hqm_linear_static_scratch(_cabi.ptr(y), _cabi.ptr(x), 1, C.byref(d), None, _cabi.stream_ptr(DEV))
    assert rc == 0
    torch.cuda.synchronize(DEV)
