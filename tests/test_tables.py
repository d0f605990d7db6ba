"""The native table builders (through the C ABI) against the reference's tables
(fixtures), the CPU restatement (random layouts) and the live reference when mounted."""
import ctypes
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import lut as olut
import workloads
from tests.util import GOLDEN, load_npz
from torch_blocksparse_b200 import layouts
from torch_blocksparse_b200 import _lib, tables


def _flat(luts):
    return np.concatenate([l.numpy() for l in luts]) if luts else np.zeros(0, np.int32)


def test_builders_match_reference_fixtures():
    z = load_npz('lut_small.npz')
    for name in sorted({k.split('/')[0] for k in z.files}):
        lay = torch.from_numpy(z[name + '/layout'])
        before = lay.clone()
        for block in (16, 32, 64):
            luts, none, widths, packs = tables.make_sdd_lut(lay, block)
            assert none is None
            assert np.array_equal(_flat(luts), z['%s/sdd_b%d_lut' % (name, block)]), (name, block)
            assert widths == list(z['%s/sdd_b%d_widths' % (name, block)])
            assert packs == list(z['%s/sdd_b%d_packs' % (name, block)])
            for step in (8, 16):
                for trans in (0, 1):
                    key = '%s/dxx_b%d_s%d_t%d' % (name, block, step, trans)
                    lut, nlocks, width, none = tables.make_dxx_lut(lay, block, step, bool(trans))
                    assert lut.dtype == torch.int32 and none is None
                    assert np.array_equal(lut.numpy(), z[key + '_lut']), key
                    assert [nlocks, width] == list(z[key + '_meta']), key
        lut, maxlut = tables.make_softmax_lut(lay)
        assert np.array_equal(lut.numpy(), z[name + '/softmax_lut'])
        assert maxlut == int(z[name + '/softmax_maxlut'][0])
        assert torch.equal(lay, before), 'the layout must never be modified'


def test_int32_layout_is_not_consumed():
    """The reference zeroes an int32 layout in place while packing; this build copies."""
    lay = torch.ones((1, 4, 4), dtype=torch.int32)
    tables.make_sdd_lut(lay, 16)
    assert int(lay.sum()) == 16


@pytest.mark.parametrize('seed', range(6))
def test_builders_match_restatement_on_random_layouts(seed):
    rng = np.random.default_rng(seed)
    for _ in range(25):
        H, Mb, Nb = (int(rng.integers(1, 5)), int(rng.integers(1, 24)), int(rng.integers(1, 24)))
        lay = (rng.random((H, Mb, Nb)) < rng.choice([0.1, 0.3, 0.5, 0.8, 0.97])).astype(np.int64)
        for h in range(H):
            if lay[h].sum() == 0:
                lay[h, rng.integers(Mb), rng.integers(Nb)] = 1
        t = torch.from_numpy(lay)
        for block in (16, 32, 64, 128):
            luts, _, widths, packs = tables.make_sdd_lut(t, block)
            ol, ow, op = olut.make_sdd_lut(lay, block)
            assert widths == ow and packs == op
            assert np.array_equal(_flat(luts), np.concatenate(ol) if ol else np.zeros(0, np.int32))
            for step in (8, 16):
                for trans in (False, True):
                    lut, nlocks, width, _ = tables.make_dxx_lut(t, block, step, trans)
                    o = olut.make_dxx_lut(lay, block, step, trans)
                    assert np.array_equal(lut.numpy(), o[0]) and (nlocks, width) == (o[1], o[2])
        lut, maxlut = tables.make_softmax_lut(t)
        o = olut.make_softmax_lut(lay)
        assert np.array_equal(lut.numpy(), o[0]) and maxlut == o[1]


def test_block128_has_no_sdd_table():
    luts, _, widths, packs = tables.make_sdd_lut(torch.ones((2, 3, 3), dtype=torch.long), 128)
    assert luts == [] and widths == [] and packs == []


def test_empty_head_is_an_error_for_dxx():
    lay = torch.zeros((2, 3, 3), dtype=torch.long)
    lay[0, 0, 0] = 1
    with pytest.raises(RuntimeError):
        tables.make_dxx_lut(lay, 16, 16, True)


def test_fixed_layout_matches_restatement():
    for args in [(4, 16, 'fixed', 4, 'unidirectional', 1, 1), (4, 16, 'fixed', 4, 'bidirectional', 2, 2),
                 (3, 32, 'fixed', 8, 'unidirectional', 4, 2), (2, 8, 'dense', 4, 'unidirectional', 1, 1),
                 (16, 128, 'fixed', 4, 'bidirectional', 1, 1)]:
        assert np.array_equal(tables.make_fixed_layout(*args).numpy(), olut.make_fixed_layout(*args))
    with pytest.raises(ValueError):
        tables.make_fixed_layout(2, 8, 'fixed', 4, 'unidirectional', 1, 3)
    with pytest.raises(ValueError):
        tables.make_fixed_layout(2, 8, 'fixed', 4, 'unidirectional', 5, 1)
    with pytest.raises(NotImplementedError):
        tables.make_fixed_layout(2, 8, 'variable', 4, 'unidirectional', 1, 1)


def test_fixed_layout_matches_reference_fixture():
    """Native generator and CPU restatement against layouts the reference's own
    _make_layout (deepspeedsparseselfattention.py:51-65) returned."""
    z = load_npz('fixed_layouts.npz')
    assert len(z.files) == 6
    for key in z.files:
        f = key.split('_')
        args = (int(f[0]), int(f[1]), f[2], int(f[3]), f[4], int(f[5]), int(f[6]))
        want = z[key].astype(np.int64)
        assert np.array_equal(tables.make_fixed_layout(*args).numpy(), want), key
        assert np.array_equal(olut.make_fixed_layout(*args), want), key


def test_native_builders_hash_to_reference_on_config_layouts():
    """The native builders on the full-size layouts of the benchmark configurations against
    SHA-256 digests of the reference's own tables (matmul.py:281-297, 372-458; softmax.py:201-221)."""
    cfg = json.load(open(os.path.join(GOLDEN, 'lut_configs.json')))
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    cases = {
        'c1': workloads.config1()['layout'],
        'c2': torch.bernoulli(torch.full((8, 64, 64), 0.25), generator=torch.Generator().manual_seed(0)).long(),
        'c3_full': layouts.causal_band(16, 64, 4, 1),
        'c4_uni_full': layouts.fixed(16, 128, 4, 'unidirectional'),
        'c4_bi_full': layouts.fixed(16, 128, 4, 'bidirectional'),
        'c5_full': layouts.bigbird(16, 128, 3, 3, 2, seed=0),
    }
    for name, layout in cases.items():
        e = cfg[name]
        assert sha(layout.numpy()) == e['layout_sha'], name + ': generator drifted from the fixture'
        assert int(layout.sum()) == e['nnz']
        block = e['block']
        luts, _, widths, packs = tables.make_sdd_lut(layout, block)
        assert sha(_flat(luts)) == e['sdd_b%d_lut' % block]['sha'], name
        assert _flat(luts).size == e['sdd_b%d_lut' % block]['size'], name
        for step in (8, 16):
            for trans in (0, 1):
                lut, _, _, _ = tables.make_dxx_lut(layout, block, step, bool(trans))
                assert sha(lut.numpy()) == e['dxx_b%d_s%d_t%d_lut' % (block, step, trans)]['sha'], (name, step, trans)
        lut, _ = tables.make_softmax_lut(layout)
        assert sha(lut.numpy()) == e['softmax_lut']['sha'], name


def test_meta_is_consistent_csr_and_csc():
    g = torch.Generator().manual_seed(3)
    lay = (torch.rand((3, 7, 5), generator=g) > 0.5).long()
    m = tables.build_meta(lay)
    H, Mb, Nb = lay.shape
    nnz = int(lay.sum())
    assert (m.H, m.Mb, m.Nb, m.nnz) == (H, Mb, Nb, nnz)
    buf = m.host.numpy()
    p = _lib.META_HEADER
    row_ptr = buf[p:p + H * Mb + 1]; p += H * Mb + 1
    blk_row = buf[p:p + nnz]; p += nnz
    blk_col = buf[p:p + nnz]; p += nnz
    blk_head = buf[p:p + nnz]; p += nnz
    col_ptr = buf[p:p + H * Nb + 1]; p += H * Nb + 1
    col_row = buf[p:p + nnz]; p += nnz
    col_bid = buf[p:p + nnz]; p += nnz
    row_order = buf[p:p + H * Mb]; p += H * Mb
    col_order = buf[p:p + H * Nb]; p += H * Nb
    assert p == buf.size
    nz = lay.nonzero().numpy()
    assert np.array_equal(blk_head, nz[:, 0]) and np.array_equal(blk_row, nz[:, 1]) and np.array_equal(blk_col, nz[:, 2])
    assert np.array_equal(np.diff(row_ptr), lay.sum(2).reshape(-1).numpy())
    assert np.array_equal(np.diff(col_ptr), lay.sum(1).reshape(-1).numpy())
    for c in range(H * Nb):
        ids = col_bid[col_ptr[c]:col_ptr[c + 1]]
        assert np.all(blk_head[ids] == c // Nb) and np.all(blk_col[ids] == c % Nb)
        assert np.array_equal(blk_row[ids], col_row[col_ptr[c]:col_ptr[c + 1]])
        assert np.all(np.diff(col_row[col_ptr[c]:col_ptr[c + 1]]) > 0)
    assert sorted(row_order.tolist()) == list(range(H * Mb)) and sorted(col_order.tolist()) == list(range(H * Nb))
    assert np.all(np.diff(np.diff(row_ptr)[row_order]) <= 0) and np.all(np.diff(np.diff(col_ptr)[col_order]) <= 0)
    assert m.max_row == int(lay.sum(2).max()) and m.max_col == int(lay.sum(1).max())


def test_capacity_error_reports_needed_size():
    lay = torch.ones((1, 4, 4), dtype=torch.int64)
    L = _lib.lib()
    total = ctypes.c_int64(0)
    maxlut = ctypes.c_int(0)
    small = torch.zeros(4, dtype=torch.int32)
    rc = L.bsp_softmax_lut_build(lay.data_ptr(), 1, 4, 4, small.data_ptr(), small.numel(), ctypes.byref(total),
                                 ctypes.byref(maxlut))
    assert rc == _lib.ERR_CAPACITY and total.value == 2 * 4 + 4 * 16
    assert b'needs' in L.bsp_last_error()


def test_live_reference_when_mounted():
    """With the reference checkout present, compare against its builders directly
    on fresh random layouts (skipped elsewhere; the fixtures cover that case)."""
    from oracle import build_ref
    ref = build_ref.import_reference() if build_ref.reference_present() else None
    if ref is None:
        pytest.skip('reference checkout not mounted')
    RM = ref.matmul._sparse_matmul
    rng = np.random.default_rng(99)
    for _ in range(20):
        lay = torch.from_numpy((rng.random((2, 16, 32)) < 0.5).astype(np.int64))
        for block in (16, 32):
            rl, _, rw, rp = RM.make_sdd_lut(lay.clone(), block, torch.float16, 'cpu')
            luts, _, widths, packs = tables.make_sdd_lut(lay, block)
            assert widths == rw and packs == rp and all(torch.equal(a, b) for a, b in zip(luts, rl))
            for trans in (False, True):
                r = RM.make_dxx_lut(lay.clone(), block, 16, trans, 'cpu')
                o = tables.make_dxx_lut(lay, block, 16, trans)
                assert torch.equal(r[0], o[0]) and int(r[1]) == o[1] and r[2] == o[2]
