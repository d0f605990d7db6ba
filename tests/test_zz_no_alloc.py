"""The allocation-free attention backward (bsp_attn_bwd_static).

Some callers of the library cannot allocate device memory (a runtime with a
pre-planned memory pool, a plug-in that only sees its input and output
tensors), so they cannot supply the scratch bsp_attn_bwd asks for.  The static
variant keeps that scratch inside the library.  This test drives both entry
points through the C ABI on the same inputs and expects identical gradients,
twice in a row (the second call finds the previous call's data in the shared
scratch), and checks the size limit.  It is collected last on purpose.
"""
import pytest
import torch

import workloads
from tests.util import Guarded, assert_close
from torch_blocksparse_b200 import _lib, tables

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def _tile_args(tiles, device):
    """(header, device buffer) of the tcgen05 tile lists, or two NULLs for the mma.sync kernels."""
    if tiles is None:
        return [None, None]
    return [tiles.hdr.data_ptr(), tiles.on(device).data_ptr()]


def _code(x):
    return _lib.F16 if x.dtype == torch.float16 else _lib.BF16


def _backward(entry, t, meta, block, scale, delta=None, tiles=None):
    q, k, v, o, do, lse = t
    Z, H, L, D = q.shape
    guards = [Guarded(q.shape, q.dtype, q.device) for _ in range(3)]       # NaN margins around dq, dk, dv
    grads = [g.t for g in guards]
    st = lambda x: (x.stride(0), x.stride(1), x.stride(2))
    head = [q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr()]
    if delta is not None:
        head.append(delta.data_ptr())
    args = head + [g.data_ptr() for g in grads] + [_code(q), block, Z, H, L, D] \
        + [*st(q), *st(k), *st(v), *st(o), *st(do)] \
        + [meta.hdr.data_ptr(), meta.on(q.device).data_ptr()] + _tile_args(tiles, q.device) + [scale] \
        + [None, 0, 0, 0, None, 0, 0, None, 0, 0] \
        + [torch.cuda.current_stream().cuda_stream]
    _lib.check(entry(*args))
    torch.cuda.synchronize()
    for g, name in zip(guards, ('dq', 'dk', 'dv')):
        g.check(name)
    return grads


def _forward(c, meta, tiles=None):
    q, k, v, do = (c[n].to(DEV) for n in ('q', 'k', 'v', 'do'))
    Z, H, L, D = q.shape
    o = torch.empty_like(q)
    lse = torch.empty((Z, H, L), dtype=torch.float32, device=DEV)
    st = lambda x: (x.stride(0), x.stride(1), x.stride(2))
    _lib.check(_lib.lib().bsp_attn_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), _code(q), c['block'], Z, H, L, D,
        *st(q), *st(k), *st(v), *st(o), meta.hdr.data_ptr(), meta.on(q.device).data_ptr(), *_tile_args(tiles, q.device), c['scale'],
        None, 0, 0, 0, None, 0, 0, None, 0, 0, torch.cuda.current_stream().cuda_stream))
    return q, k, v, o, do, lse


@pytest.mark.parametrize('with_tiles', [False, True])
def test_static_scratch_backward_matches_caller_scratch_backward_twice(with_tiles):
    """Without tile lists the mma.sync kernels read the built-in scratch; with them the tcgen05
    dK/dV kernel fetches it by bulk copies and the dQ kernel by plain loads."""
    from torch_blocksparse_b200 import fused
    L = _lib.lib()
    cases = [workloads.config4('unidirectional', small=True), workloads.config4('bidirectional', small=True),
             workloads.config5(small=True)]                      # FP16 head_dim 64 twice, then BF16 head_dim 128
    for c in cases:                                              # different problems back to back
        meta = tables.build_meta(c['layout'])
        tiles = tables.build_attn_tiles(c['layout'], c['block']) if with_tiles else None
        assert (tiles is not None) == with_tiles
        t = _forward(c, meta, tiles)
        Z, H, Ln, _ = t[0].shape
        delta = torch.empty((Z, H, Ln), dtype=torch.float32, device=DEV)
        want = _backward(L.bsp_attn_bwd, t, meta, c['block'], c['scale'], delta, tiles)
        for call in range(2):
            got = _backward(L.bsp_attn_bwd_static, t, meta, c['block'], c['scale'], None, tiles)
            for name, g, w in zip(('dq', 'dk', 'dv'), got, want):
                assert torch.equal(g, w), '%s differs on call %d' % (name, call)
                assert_close(g, w, name)
    assert fused.device_status() == 0, 'a bounded device-side wait expired'


def test_static_scratch_size_limit_is_reported():
    L = _lib.lib()
    c = workloads.config4('unidirectional', small=True)
    meta = tables.build_meta(c['layout'])
    rows = _lib.ATTN_STATIC_ROWS
    # Z * H * L one past the limit: rejected before anything is launched or dereferenced
    Z = rows // (2 * 1024) + 1
    rc = L.bsp_attn_bwd_static(16, 16, 16, 16, 16, 16, 16, 16, 16, _lib.F16, 64, Z, 2, 1024, 64,
                               *([8] * 15), meta.hdr.data_ptr(), meta.on(torch.device(DEV)).data_ptr(), None, None, 0.125,
                               None, 0, 0, 0, None, 0, 0, None, 0, 0, None)
    assert rc == _lib.ERR_UNSUPPORTED
    msg = L.bsp_last_error().decode()
    assert 'exceed the built-in scratch' in msg and str(rows) in msg
