"""Execution metadata built on the device against the host builder (bit-exact), and the
process-wide cache keyed by the layout's content."""
import numpy as np
import pytest
import torch

import workloads
from tests.util import assert_close, load_npz
from torch_blocksparse_b200 import MatMul, Softmax, SparseSelfAttention, layouts, tables

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def _host_meta(lay):
    tables.clear_cache()
    return tables.build_meta(lay)


def _check_equal(lay_cpu, dtype=torch.int64):
    want = _host_meta(lay_cpu)
    dev_layout = lay_cpu.to(DEV).to(dtype) if dtype != torch.bool else (lay_cpu != 0).to(DEV)
    got = tables.build_meta_device(dev_layout)
    assert torch.equal(got.hdr, want.hdr), 'header differs'
    assert torch.equal(got.on(DEV).cpu(), want.host), 'metadata buffer differs'
    assert (got.H, got.Mb, got.Nb, got.nnz, got.max_row, got.max_col) == \
           (want.H, want.Mb, want.Nb, want.nnz, want.max_row, want.max_col)


def test_device_build_equals_host_build_on_fixture_layouts():
    z = load_npz('lut_small.npz')
    for name in sorted({k.split('/')[0] for k in z.files}):
        _check_equal(torch.from_numpy(z[name + '/layout']))
    for lay in (layouts.fixed(16, 128, 4, 'unidirectional'), layouts.fixed(16, 128, 4, 'bidirectional'),
                layouts.bigbird(16, 128, 3, 3, 2, seed=0), layouts.causal_band(16, 64, 4, 1),
                torch.zeros((2, 3, 5), dtype=torch.long), torch.ones((1, 1, 1), dtype=torch.long)):
        _check_equal(lay)


def test_device_build_equals_host_build_on_1000_random_layouts():
    rng = np.random.default_rng(2024)
    dtypes = [torch.int64, torch.int32, torch.uint8, torch.bool]
    for i in range(1000):
        H, Mb, Nb = int(rng.integers(1, 6)), int(rng.integers(1, 40)), int(rng.integers(1, 40))
        if i % 50 == 0:
            H, Mb, Nb = 3, int(rng.integers(300, 500)), int(rng.integers(300, 500))     # more than one scan chunk
        p = rng.choice([0.0, 0.05, 0.3, 0.6, 0.95, 1.0])
        lay = torch.from_numpy((rng.random((H, Mb, Nb)) < p).astype(np.int64))
        _check_equal(lay, dtypes[i % 4])


def test_softmax_table_from_device_metadata_equals_the_host_table():
    """bsp_softmax_lut_from_meta (the table written by a kernel from the metadata built on the
    device) against bsp_softmax_lut_build on the host: fixtures, the benchmark layouts, 200
    random layouts (odd and even numbers of block-rows, empty rows, an empty layout)."""
    rng = np.random.default_rng(5)
    z = load_npz('lut_small.npz')
    lays = [torch.from_numpy(z[name + '/layout']) for name in sorted({k.split('/')[0] for k in z.files})]
    lays += [layouts.fixed(16, 128, 4, 'unidirectional'), layouts.bigbird(16, 128, 3, 3, 2, seed=0),
             layouts.causal_band(16, 64, 4, 1), torch.zeros((2, 3, 5), dtype=torch.long),
             torch.ones((1, 1, 1), dtype=torch.long)]
    for i in range(200):
        H, Mb, Nb = int(rng.integers(1, 6)), int(rng.integers(1, 40)), int(rng.integers(1, 40))
        p = rng.choice([0.0, 0.05, 0.3, 0.6, 1.0])
        lays.append(torch.from_numpy((rng.random((H, Mb, Nb)) < p).astype(np.int64)))
    for lay in lays:
        tables.clear_cache()
        want, want_max = tables.make_softmax_lut(lay)
        got, got_max = tables.make_softmax_lut_device(lay.to(DEV))
        assert got_max == want_max and got.is_cuda and torch.equal(got.cpu(), want), tuple(lay.shape)


def test_softmax_with_a_device_layout_matches_the_host_layout_path(monkeypatch):
    c = workloads.config3(small=True)
    tables.clear_cache()
    x = c['x'].to(DEV)
    kw = dict(scale=c['scale'], rpe=c['rpe'].to(DEV), key_padding_mask=c['key_padding_mask'].to(DEV),
              attn_mask=c['attn_mask'].to(DEV), key_padding_mask_mode='add', attn_mask_mode='mul')
    want = Softmax(c['layout'], c['block'])(x.clone(), **kw)
    tables.clear_cache()
    before = dict(tables.CACHE_STATS)

    def host_builder(*args, **kwargs):
        raise AssertionError('the host builder must not run for a device layout')
    monkeypatch.setattr(tables, 'make_softmax_lut', host_builder)
    got = Softmax(c['layout'].to(DEV), c['block'])(x.clone(), **kw)
    assert torch.equal(got, want)
    assert tables.CACHE_STATS['host_builds'] == before['host_builds']          # nor the metadata


def test_ops_on_one_layout_share_one_buffer_and_a_changed_layout_is_rebuilt():
    tables.clear_cache()
    g = torch.Generator().manual_seed(1)
    layout = (torch.rand((2, 4, 4), generator=g) > 0.4).long()
    layout[:, :, 0] = 1
    a = MatMul(layout, 64, 'sdd', trans_b=True)
    b = MatMul(layout.clone(), 64, 'dsd')                      # another tensor object, same content
    assert a.meta is b.meta and a.meta.on(DEV).data_ptr() == b.meta.on(DEV).data_ptr()
    m1 = SparseSelfAttention(layout=layout, block=64)
    m2 = SparseSelfAttention(layout=layout.clone(), block=64)
    m1.get_ops(2, 256), m2.get_ops(2, 256)
    assert m1.tiles[(2, 256)] is m2.tiles[(2, 256)] and m1.ops[(2, 256)][0].meta is a.meta
    s1, s2 = Softmax(layout, 64), Softmax(layout.clone(), 64)
    assert s1.make_lut(torch.device(DEV))[0].data_ptr() == s2.make_lut(torch.device(DEV))[0].data_ptr()
    changed = layout.clone()
    changed[0, 3, 3] = 1 - changed[0, 3, 3]
    c = MatMul(changed, 64, 'sdd', trans_b=True)
    assert c.meta is not a.meta and c.meta.nnz != a.meta.nnz


def test_matmul_with_a_device_layout_matches_the_host_layout_path():
    tables.clear_cache()
    g = torch.Generator().manual_seed(5)
    layout = (torch.rand((2, 4, 6), generator=g) > 0.5).long()
    layout[:, 0, 0] = 1
    before = dict(tables.CACHE_STATS)
    x = torch.randn((2, 2, 256, 128), generator=g).half().to(DEV)
    y = torch.randn((2, 2, 128, 384), generator=g).half().to(DEV)
    on_host = MatMul(layout, 64, 'sdd')(x, y)
    on_dev = MatMul(layout.to(DEV), 64, 'sdd')(x, y)
    assert tables.CACHE_STATS['device_builds'] == before['device_builds'] + 1
    assert torch.equal(on_host, on_dev)
    s = torch.randn((2, int(layout.sum()), 64, 64), generator=g).half().to(DEV)
    w = torch.randn((2, 2, 384, 128), generator=g).half().to(DEV)
    assert_close(MatMul(layout.to(DEV), 64, 'dsd')(s, w), MatMul(layout, 64, 'dsd')(s, w), 'dsd')


def test_validation_accepts_built_buffers_and_names_the_corrupt_entry():
    """The debug-time validation kernels: buffers from the builders pass; a block column, a block
    id, a row pointer, a chunk id or a tile order out of range is reported with its check
    number and position."""
    tables.clear_cache()
    for lay, block in ((layouts.fixed(4, 16, 4, 'unidirectional'), 64), (layouts.bigbird(3, 12, 2, 3, 1, seed=1), 128),
                       (layouts.fixed(2, 16, 4, 'bidirectional'), 16)):
        m = tables.build_meta(lay)
        tables.validate_device_buffer(m.on(DEV))
        tables.validate_device_buffer(tables.build_meta_device(lay.to(DEV)).on(DEV))
        t = tables.build_attn_tiles(lay, block)
        tables.validate_device_buffer(t.on(DEV), tiles=True)
    lay = layouts.fixed(2, 8, 4, 'unidirectional')
    m = tables.build_meta(lay)
    H, Mb, Nb, nnz = m.H, m.Mb, m.Nb, m.nnz
    base = 8 + (H * Mb + 1)
    for offset, value, code in ((base + nnz + 3, Nb, 6),               # blk_col out of range
                                (base + 3 * nnz + (H * Nb + 1) + nnz + 1, nnz, 7),   # col_bid out of range
                                (8 + 2, 10 ** 6, 3)):                  # row_ptr jumps
        bad = m.on(DEV).clone()
        bad[offset] = value
        with pytest.raises(ValueError, match='check %d failed' % code):
            tables.validate_device_buffer(bad)
    t = tables.build_attn_tiles(lay, 64)
    n = int(t.hdr[1]) * int(t.hdr[4])
    bad = t.on(DEV).clone()
    bad[8 + 2 * n + (n + 1) + 1] = 10 ** 4                            # a chunk id of the row tiles
    with pytest.raises(ValueError, match='check 16 failed'):
        tables.validate_device_buffer(bad, tiles=True)


def test_device_tile_lists_equal_host_tile_lists():
    """Attention tile lists built on the device (greedy pairing of block-rows by similarity, one CTA
    per head and side) against the host builder: fixtures, the benchmark layouts, random layouts
    with odd counts, empty and identical rows, blocks 16, 32, 64 and 128."""
    rng = np.random.default_rng(77)
    cases = [(layouts.fixed(16, 128, 4, 'unidirectional'), 64), (layouts.fixed(16, 128, 4, 'bidirectional'), 64),
             (layouts.bigbird(16, 128, 3, 3, 2, seed=0), 128), (layouts.causal_band(4, 64, 4, 1), 64),
             (torch.zeros((2, 5, 5), dtype=torch.long), 64), (torch.ones((1, 1, 1), dtype=torch.long), 128),
             (torch.ones((3, 7, 7), dtype=torch.long), 64)]
    for i in range(300):
        H, nb = int(rng.integers(1, 5)), int(rng.integers(1, 40))
        if i % 60 == 0:
            nb = int(rng.integers(200, 300))
        p = rng.choice([0.0, 0.05, 0.3, 0.6, 0.95, 1.0])
        lay = torch.from_numpy((rng.random((H, nb, nb)) < p).astype(np.int64))
        if i % 7 == 0 and nb > 3:
            lay[:, 2] = lay[:, 1]                                # identical rows
        cases.append((lay, 64 if i % 3 else 128))
    # blocks 16 and 32: coarsened on the device, with the piece masks of every entry
    for i in range(120):
        block = 16 if i % 2 else 32
        f = 64 // block
        H, nb = int(rng.integers(1, 4)), f * int(rng.integers(1, 24))
        p = rng.choice([0.0, 0.02, 0.1, 0.4, 0.9, 1.0])
        cases.append((torch.from_numpy((rng.random((H, nb, nb)) < p).astype(np.int64)), block))
    cases += [(layouts.fixed(4, 512, 16, 'unidirectional'), 16), (layouts.causal_band(4, 128, 8, 2), 32)]
    for lay, block in cases:
        tables.clear_cache()
        want = tables.build_attn_tiles(lay, block)
        got = tables.build_attn_tiles_device(lay.to(DEV), block)
        assert torch.equal(got.hdr, want.hdr), (tuple(lay.shape), block, got.hdr.tolist(), want.hdr.tolist())
        assert torch.equal(got.on(DEV).cpu(), want.host), (tuple(lay.shape), block)


def test_attention_with_a_device_layout_builds_everything_on_the_device():
    tables.clear_cache()
    c = workloads.config4('unidirectional', small=True)
    before = dict(tables.CACHE_STATS)
    mod = SparseSelfAttention(layout=c['layout'].to(DEV), block=c['block'], fused=True)
    q, k, v = (c[n].to(DEV) for n in ('q', 'k', 'v'))
    with torch.no_grad():
        o = mod(q, k, v)
    assert tables.CACHE_STATS['device_builds'] == before['device_builds'] + 2        # metadata and tile lists
    assert tables.CACHE_STATS['host_builds'] == before['host_builds']
    from oracle import dense_masked as dm
    want = dm.attention_reference(c['q'], c['k'], c['v'], c['layout'], c['block'], c['scale'])[0]
    assert_close(o, want, 'attention on a device layout')


@pytest.mark.parametrize('block', [16, 32])
def test_attention_with_a_device_layout_at_small_blocks(block):
    """Blocks 16 / 32 with the layout in device memory: metadata and the coarsened tile lists
    are built there (no host build), and the tcgen05 kernels run on them."""
    from oracle import dense_masked as dm
    from torch_blocksparse_b200 import fused
    tables.clear_cache()
    g = torch.Generator().manual_seed(block)
    H, L, D = 2, 512, 64
    nb = L // block
    layout = (torch.rand((H, nb, nb), generator=g) < 0.2).long()
    layout[:, torch.arange(nb), torch.arange(nb)] = 1
    q, k, v = ((torch.randn((2, H, L, D), generator=g)).half() for _ in range(3))
    before = dict(tables.CACHE_STATS)
    mod = SparseSelfAttention(layout=layout.to(DEV), block=block, fused=True)
    with torch.no_grad():
        o = mod(q.to(DEV), k.to(DEV), v.to(DEV))
    assert tables.CACHE_STATS['device_builds'] == before['device_builds'] + 2
    assert tables.CACHE_STATS['host_builds'] == before['host_builds']
    want = dm.attention_reference(q, k, v, layout, block, D ** -0.5)[0]
    assert_close(o, want, 'attention on a device layout, block %d' % block)
    assert fused.device_status() == 0
