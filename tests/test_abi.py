"""The C-ABI library: loads, exports every symbol include/bsp.h declares, and
rejects bad arguments before touching the GPU (no compute call needs a device here)."""
import ctypes
import os
import re

import pytest
import torch

from torch_blocksparse_b200 import _build, _lib, tables

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'include', 'bsp.h')


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(bsp_[a-z0-9_]+)\s*\(', text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_build.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), 'libbsp_b200.so does not export ' + n
    assert sorted(_lib.exported_symbols()) == names, 'ctypes signatures and header disagree'
    assert lib.bsp_abi_version() == 1


def test_library_is_sm100a_only_and_self_contained():
    # cudart is linked statically: the library must load on a box without a GPU
    assert _lib.lib().bsp_abi_version() == 1
    flags = ' '.join(_build.NVCC_FLAGS)
    assert 'arch=compute_100a,code=sm_100a' in flags and '-lineinfo' in flags


def _call_sdd(hdr, meta, K=32, dtype=_lib.F16, block=16, a=16, b=16, c=16):
    L = _lib.lib()
    return L.bsp_sdd(a, b, c, dtype, block, 1, 1, K, 8, 8, 8, 1, 8, 8, 8, 1, 256, hdr, meta, None)


def test_bad_arguments_are_rejected_with_messages():
    L = _lib.lib()
    m = tables.build_meta(torch.ones((1, 1, 1), dtype=torch.long))
    hdr = m.hdr.data_ptr()
    fake_dev = m.host.data_ptr()            # never dereferenced: every call below fails validation first
    assert _call_sdd(None, fake_dev) == _lib.ERR_INVALID and b'NULL' in L.bsp_last_error()
    bad = m.hdr.clone()
    bad[0] = 0
    assert _call_sdd(bad.data_ptr(), fake_dev) == _lib.ERR_INVALID and b'magic' in L.bsp_last_error()
    assert _call_sdd(hdr, fake_dev, K=24) == _lib.ERR_INVALID
    assert b'Reduction size for SDD must be a multiple of 16' in L.bsp_last_error()
    assert _call_sdd(hdr, fake_dev, dtype=7) == _lib.ERR_INVALID
    assert _call_sdd(hdr, fake_dev, block=48) == _lib.ERR_INVALID
    assert _call_sdd(hdr, fake_dev, a=None) == _lib.ERR_INVALID
    assert _call_sdd(hdr, fake_dev, a=24) == _lib.ERR_INVALID and b'aligned' in L.bsp_last_error()
    # softmax: row limit and NULL checks
    rc = L.bsp_softmax_fwd(16, _lib.F16, 1, 256, 16, 1, 1, 16, 2048, 1.0, None, 0, 0, 0, None, 0, 0, None, 0, 0, None)
    assert rc == _lib.ERR_UNSUPPORTED and b'32768' in L.bsp_last_error()
    rc = L.bsp_softmax_fwd(None, _lib.F16, 1, 256, 16, 1, 1, 16, 1, 1.0, None, 0, 0, 0, None, 0, 0, None, 0, 0, None)
    assert rc == _lib.ERR_INVALID
    # fused attention: dtype / head-dimension limits
    args = [16] * 4 + [16, _lib.F32, 16, 1, 1, 16, 64] + [8] * 12 + [hdr, fake_dev, None, None, 1.0] + [None, 0, 0, 0, None, 0, 0, None, 0, 0, None]
    assert L.bsp_attn_fwd(*args) == _lib.ERR_UNSUPPORTED
    args[5], args[10] = _lib.F16, 48
    assert L.bsp_attn_fwd(*args) == _lib.ERR_UNSUPPORTED
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_INVALID)
    with pytest.raises(NotImplementedError):
        _lib.check(_lib.ERR_UNSUPPORTED)
