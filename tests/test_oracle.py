"""Pins the CPU oracle (oracle/) against fixtures generated from the reference itself."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

import workloads
from oracle import dense_masked as dm
from oracle import lut as olut
from tests.util import GOLDEN, load_npz
from torch_blocksparse_b200 import layouts


def _names(z):
    return sorted({k.split('/')[0] for k in z.files})


def test_lut_restatement_matches_reference_tables():
    z = load_npz('lut_small.npz')
    names = _names(z)
    assert 'bogus_entries' in names and 'tiny_rows' in names and 'holes' in names
    for name in names:
        lay = z[name + '/layout']
        for block in (16, 32, 64):
            luts, widths, packs = olut.make_sdd_lut(lay, block)
            flat = np.concatenate(luts) if luts else np.zeros(0, np.int32)
            assert np.array_equal(flat, z['%s/sdd_b%d_lut' % (name, block)]), (name, block)
            assert list(widths) == list(z['%s/sdd_b%d_widths' % (name, block)])
            assert list(packs) == list(z['%s/sdd_b%d_packs' % (name, block)])
            for step in (8, 16):
                for trans in (0, 1):
                    key = '%s/dxx_b%d_s%d_t%d' % (name, block, step, trans)
                    lut, nlocks, width = olut.make_dxx_lut(lay, block, step, bool(trans))
                    assert np.array_equal(lut, z[key + '_lut']), key
                    assert [nlocks, width] == list(z[key + '_meta']), key
        lut, maxlut = olut.make_softmax_lut(lay)
        assert np.array_equal(lut, z[name + '/softmax_lut'])
        assert maxlut == int(z[name + '/softmax_maxlut'][0])


def test_bogus_entries_fixture_has_duplicate_block_ids():
    """The reference's 4x4 packing can emit positions outside the layout; the
    fixture must contain such a table (more entries than nonzero blocks)."""
    z = load_npz('lut_small.npz')
    lay = z['bogus_entries/layout']
    assert z['bogus_entries/sdd_b16_lut'].size // 4 > lay.sum()


def test_tiny_rows_worked_example():
    """Layout [[[1,0],[1,1]]], block 16, step 16, per-row reductions: the table
    quoted from the reference run, including the extra zero-length segment."""
    lut, nlocks, width = olut.make_dxx_lut(np.array([[[1, 0], [1, 1]]]), 16, 16, True)
    assert lut.tolist() == [18, 16, 0, 0, 0, 0, 20, 32, 1, 0, 0, 0, 22, 0, 1, 0, 0, 0, 0, 0, 0, 1, 16, 256, 0, 0]
    assert (nlocks, width) == (1, 3)


def test_config_layout_tables_hash_to_reference():
    cfg = json.load(open(os.path.join(GOLDEN, 'lut_configs.json')))
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    cases = {
        'c1': workloads.config1()['layout'],
        'c3_full': layouts.causal_band(16, 64, 4, 1),
        'c4_uni': workloads.config4('unidirectional', small=True)['layout'],
        'c4_bi': workloads.config4('bidirectional', small=True)['layout'],
        'c5': workloads.config5(small=True)['layout'],
    }
    for name, layout in cases.items():
        e = cfg[name]
        lay = layout.numpy()
        assert sha(lay) == e['layout_sha'], name + ': generator drifted from the fixture'
        block = e['block']
        luts, widths, packs = olut.make_sdd_lut(lay, block)
        flat = np.concatenate(luts) if luts else np.zeros(0, np.int32)
        assert sha(flat) == e['sdd_b%d_lut' % block]['sha'], name
        for step in (8, 16):
            for trans in (0, 1):
                lut, _, _ = olut.make_dxx_lut(lay, block, step, bool(trans))
                assert sha(lut) == e['dxx_b%d_s%d_t%d_lut' % (block, step, trans)]['sha'], name
        lut, _ = olut.make_softmax_lut(lay)
        assert sha(lut) == e['softmax_lut']['sha'], name
    assert cfg['c5']['sdd_b128_lut']['size'] == 0        # block 128: the reference builds no SDD table
    assert cfg['c4_uni_full']['nnz'] == 36864 and cfg['c4_bi_full']['nnz'] == 71680
    assert cfg['c3_full']['nnz'] == 4960


def test_fixed_layout_restatement():
    a = olut.make_fixed_layout(16, 128, 'fixed', 4, 'unidirectional', 1, 1)
    assert a.sum() == 36864 and a[0].sum(1).max() == 35 and a[0].sum(0).max() == 125
    b = olut.make_fixed_layout(16, 128, 'fixed', 4, 'bidirectional', 1, 1)
    assert b.sum() == 71680
    with pytest.raises(ValueError):
        olut.make_fixed_layout(2, 8, 'fixed', 4, 'unidirectional', 1, 3)


def test_dense_masked_oracle_matches_reference_helpers():
    d = load_npz('dense_masked.npz')
    lay = torch.from_numpy(d['fmt_layout'])
    w = torch.from_numpy(d['fmt_w'])
    assert np.array_equal(dm.dense_to_sparse(w, lay, 16).numpy(), d['fmt_sparse'])
    assert np.array_equal(dm.mask_dense(w, lay, 16, float('-inf')).numpy(), d['fmt_dense_ninf'])
    back = dm.sparse_to_dense(dm.dense_to_sparse(w, lay, 16), lay, 16, float('-inf'))
    assert np.array_equal(back.numpy(), d['fmt_dense_ninf'])
    for mode in ('sdd', 'dsd', 'dds'):
        for ta in (0, 1):
            for tb in (0, 1):
                key = 'mm_%s_%d%d_' % (mode, ta, tb)
                layout = torch.from_numpy(d[key + 'layout'])
                x, w, dy = (torch.from_numpy(d[key + n]) for n in ('x', 'w', 'dy'))
                a = dm.dense_to_sparse(x, layout, 16) if mode == 'dsd' else x
                b = dm.dense_to_sparse(w, layout, 16) if mode == 'dds' else w
                dc = dm.dense_to_sparse(dy, layout, 16) if mode == 'sdd' else dy
                c, da, db = dm.matmul_reference(a, b, mode, bool(ta), bool(tb), layout, 16, dc)
                # inputs sit on a 1/8 grid: FP32 sums are exact, so equality is exact
                assert np.array_equal(c.numpy(), d[key + 'y']), key
                assert np.array_equal(da.numpy(), d[key + 'dx']), key
                assert np.array_equal(db.numpy(), d[key + 'dw']), key
    layout = torch.from_numpy(d['sm_layout'])
    x = dm.dense_to_sparse(torch.from_numpy(d['sm_x']), layout, 16)
    dy = dm.dense_to_sparse(torch.from_numpy(d['sm_dy']), layout, 16)
    y, dx = dm.softmax_reference(x, layout, 16, scale=float(d['sm_scale'][0]),
                                 key_padding_mask=torch.from_numpy(d['sm_kp']), attn_mask=torch.from_numpy(d['sm_am']),
                                 key_padding_mask_mode='add', attn_mask_mode='mul', dy=dy)
    assert torch.allclose(y, torch.from_numpy(d['sm_y']), rtol=1e-6, atol=1e-7)
    assert torch.allclose(dx, torch.from_numpy(d['sm_dx']), rtol=1e-5, atol=1e-7)


def test_attention_oracle_equals_three_op_oracle_chain():
    """attention_reference is the composition of the three op oracles."""
    g = torch.Generator().manual_seed(0)
    H, nb, block, D = 2, 4, 16, 32
    layout = (torch.rand((H, nb, nb), generator=g) > 0.4).long()
    layout[:, :, 0] = 1
    q, k, v = (torch.randn((2, H, nb * block, D), generator=g) for _ in range(3))
    s, _, _ = dm.matmul_reference(q, k, 'sdd', False, True, layout, block)
    p, _ = dm.softmax_reference(s, layout, block, scale=0.3)
    o, _, _ = dm.matmul_reference(p, v, 'dsd', False, False, layout, block)
    o2, _, _, _ = dm.attention_reference(q, k, v, layout, block, 0.3)
    assert torch.allclose(o, o2, rtol=1e-5, atol=1e-6)
