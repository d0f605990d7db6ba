"""GPU parity of the block-sparse MatMul (sdd / dsd / dds, forward and both
gradients) against the dense-masked CPU oracle."""
import pytest
import torch

import workloads
from oracle import dense_masked as dm
from tests.util import assert_close, head_blocks, load_npz
from torch_blocksparse_b200 import MatMul

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def run_both(layout, block, mode, ta, tb, a, b, dc, what=''):
    want_c, want_da, want_db = dm.matmul_reference(a, b, mode, ta, tb, layout, block, dc)
    op = MatMul(layout, block, mode, trans_a=ta, trans_b=tb)
    ag = a.to(DEV).requires_grad_()
    bg = b.to(DEV).requires_grad_()
    c = op(ag, bg)
    c.backward(dc.to(DEV))
    assert_close(c, want_c, what + ' c')
    assert_close(ag.grad, want_da, what + ' da')
    assert_close(bg.grad, want_db, what + ' db')


def make_case(mode, ta, tb, block, dtype, Z=3, H=2, M=256, N=512, K=384, rho=0.5, seed=1, dist='rand'):
    """Inputs shaped as in the reference's test (tests/test_matmul.py:44-65)."""
    g = torch.Generator().manual_seed(seed)
    AS = (K, M) if ta else (M, K)
    BS = (N, K) if tb else (K, N)
    shape = {'sdd': (M, N), 'dsd': AS, 'dds': BS}[mode]
    layout = (torch.rand((H, shape[0] // block, shape[1] // block), generator=g) > rho).long()
    layout[:, 0, 0] = 1
    draw = (lambda s: torch.rand(s, generator=g)) if dist == 'rand' else (lambda s: torch.randn(s, generator=g) * 0.1)
    x = draw((Z, H) + AS).to(dtype)
    w = draw((Z, H) + BS).to(dtype)
    dy = draw((Z, H, M, N)).to(dtype)
    a = dm.dense_to_sparse(x, layout, block) if mode == 'dsd' else x
    b = dm.dense_to_sparse(w, layout, block) if mode == 'dds' else w
    dc = dm.dense_to_sparse(dy, layout, block) if mode == 'sdd' else dy
    return layout, a, b, dc


# the reference's own grid (tests/test_matmul.py:87-103): 3 modes x 4 transpose
# combinations at block 32, and 3 modes x blocks 16/32/64, FP16, Z=3 H=2 M=256 N=512 K=384
@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('ta', [False, True])
@pytest.mark.parametrize('tb', [False, True])
def test_reference_grid_transposes(mode, ta, tb):
    layout, a, b, dc = make_case(mode, ta, tb, 32, torch.float16)
    run_both(layout, 32, mode, ta, tb, a, b, dc, '%s ta=%d tb=%d' % (mode, ta, tb))


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('block', [16, 32, 64, 128])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.float32])
def test_blocks_and_dtypes(mode, block, dtype):
    layout, a, b, dc = make_case(mode, False, False, block, dtype, Z=2, dist='randn' if dtype != torch.float32 else 'rand')
    run_both(layout, block, mode, False, False, a, b, dc, '%s block %d %s' % (mode, block, dtype))


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('ta', [False, True])
@pytest.mark.parametrize('tb', [False, True])
def test_fp32_transposes_block16(mode, ta, tb):
    layout, a, b, dc = make_case(mode, ta, tb, 16, torch.float32, Z=2, M=64, N=96, K=48)
    run_both(layout, 16, mode, ta, tb, a, b, dc, '%s fp32 ta=%d tb=%d' % (mode, ta, tb))


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
def test_golden_reference_oracle_cases(mode):
    """Fixtures produced by the reference's own run_mm_reference (FP32, block 16)."""
    d = load_npz('dense_masked.npz')
    for ta in (0, 1):
        for tb in (0, 1):
            key = 'mm_%s_%d%d_' % (mode, ta, tb)
            layout = torch.from_numpy(d[key + 'layout'])
            x, w, dy = (torch.from_numpy(d[key + n]) for n in ('x', 'w', 'dy'))
            y, dx, dw = (torch.from_numpy(d[key + n]) for n in ('y', 'dx', 'dw'))
            a = dm.dense_to_sparse(x, layout, 16) if mode == 'dsd' else x
            b = dm.dense_to_sparse(w, layout, 16) if mode == 'dds' else w
            dc = dm.dense_to_sparse(dy, layout, 16) if mode == 'sdd' else dy
            op = MatMul(layout, 16, mode, trans_a=bool(ta), trans_b=bool(tb))
            ag, bg = a.to(DEV).requires_grad_(), b.to(DEV).requires_grad_()
            c = op(ag, bg)
            c.backward(dc.to(DEV))
            assert_close(c, y, key + 'y')
            assert_close(ag.grad, dx, key + 'dx')
            assert_close(bg.grad, dw, key + 'dw')


def test_empty_rows_are_zero_filled_and_every_block_written():
    """Dense outputs are allocated uninitialised: block-rows / columns of the
    layout without a nonzero block must come back as zeros."""
    block = 32
    layout = torch.zeros((2, 4, 4), dtype=torch.long)
    layout[0, 1, 2] = layout[0, 1, 3] = layout[1, 3, 0] = 1
    g = torch.Generator().manual_seed(4)
    s = torch.randn((2, 3, block, block), generator=g).half()
    d = torch.randn((2, 2, 128, 64), generator=g).half()
    for ta in (False, True):
        want, _, _ = dm.matmul_reference(s, d, 'dsd', ta, False, layout, block)
        got = MatMul(layout, block, 'dsd', trans_a=ta)(s.to(DEV), d.to(DEV))
        assert_close(got, want, 'dsd ta=%d' % ta)
    dd = torch.randn((2, 2, 64, 128), generator=g).half()
    want, _, _ = dm.matmul_reference(dd, s, 'dds', False, False, layout, block)
    assert_close(MatMul(layout, block, 'dds')(dd.to(DEV), s.to(DEV)), want, 'dds')


def test_bogus_sdd_table_layout_still_matches_the_oracle():
    """A layout for which the reference's 4x4 packing emits entries outside the
    layout: the table is reproduced, the kernel must not execute from it."""
    z = load_npz('lut_small.npz')
    layout = torch.from_numpy(z['bogus_entries/layout'])
    block = 16
    g = torch.Generator().manual_seed(8)
    a = torch.rand((1, 2, 256, 64), generator=g)
    b = torch.rand((1, 2, 64, 512), generator=g)
    want, _, _ = dm.matmul_reference(a, b, 'sdd', False, False, layout, block)
    assert_close(MatMul(layout, block, 'sdd')(a.to(DEV), b.to(DEV)), want, 'sdd')


def test_non_contiguous_and_odd_inputs():
    """Permuted views, K not a multiple of 32, dense widths that are not tile multiples."""
    block = 32
    g = torch.Generator().manual_seed(6)
    layout = (torch.rand((2, 4, 3), generator=g) > 0.3).long()
    layout[:, 0, 0] = 1
    a = torch.randn((2, 2, 128, 48), generator=g).half()          # K = 48
    bt = torch.randn((2, 2, 96, 48), generator=g).half()
    want, _, _ = dm.matmul_reference(a, bt, 'sdd', False, True, layout, block)
    got = MatMul(layout, block, 'sdd', trans_b=True)(a.to(DEV), bt.to(DEV))
    assert_close(got, want, 'sdd K=48')
    # the same product with b handed over as a permuted view of a [.., K, N] tensor
    b_kn = bt.transpose(2, 3).contiguous().to(DEV)
    got = MatMul(layout, block, 'sdd', trans_b=True)(a.to(DEV), b_kn.transpose(2, 3))
    assert_close(got, want, 'sdd permuted view')
    # dsd with a dense width of 72 (not a multiple of the 64-wide tile)
    s = torch.randn((2, int(layout.sum()), block, block), generator=g).half()
    d = torch.randn((2, 2, 96, 72), generator=g).half()
    want, _, _ = dm.matmul_reference(s, d, 'dsd', False, False, layout, block)
    assert_close(MatMul(layout, block, 'dsd')(s.to(DEV), d.to(DEV)), want, 'dsd N=72')
    with pytest.raises(ValueError):
        MatMul(layout, block, 'sdd')(torch.zeros((1, 2, 128, 40), device=DEV), torch.zeros((1, 2, 40, 96), device=DEV))


@pytest.mark.parametrize('block', [32, 64, 128])
def test_layout_without_blocks_gives_zeros(block):
    """dsd / dds with an all-zero layout: the sparse operand has no block and the dense result
    is all zeros (the reference zero-fills through zero-length segments, matmul.py:246-264)."""
    H, nb, Z, N = 2, 2, 2, 128
    layout = torch.zeros((H, nb, nb), dtype=torch.long)
    s = torch.zeros((Z, 0, block, block), dtype=torch.float16, device=DEV)
    d = torch.randn((Z, H, nb * block, N), dtype=torch.float16, device=DEV)
    out = MatMul(layout, block, 'dsd')(s, d)
    assert out.shape == (Z, H, nb * block, N) and float(out.abs().max()) == 0.0
    out = MatMul(layout, block, 'dds')(d.transpose(2, 3).contiguous(), s)
    assert out.shape == (Z, H, N, nb * block) and float(out.abs().max()) == 0.0


@pytest.mark.parametrize('mode', ['dsd', 'dds'])
@pytest.mark.parametrize('ta', [False, True])
@pytest.mark.parametrize('tb', [False, True])
@pytest.mark.parametrize('dtype', [torch.float16, torch.float32])
def test_free_dimension_that_is_not_a_multiple_of_the_vector_width(mode, ta, tb, dtype):
    """The reference's kernels bounds-check the dense operand's free dimension and accept any
    size; here an odd width / height (77 = 72 + 5) is padded and cut off again."""
    g = torch.Generator().manual_seed(3)
    block, H, Z, F = 16, 2, 2, 77
    layout = (torch.rand((H, 4, 6), generator=g) > 0.4).long()
    layout[:, 0, 0] = 1
    sp_rows, sp_cols = 4 * block, 6 * block
    s_ = torch.randn((Z, int(layout.sum()), block, block), generator=g).to(dtype)
    if mode == 'dsd':                                    # C = op(S) . op(B): the free dimension is N
        K = sp_rows if ta else sp_cols
        d_ = torch.randn((Z, H, F, K) if tb else (Z, H, K, F), generator=g).to(dtype)
        a, b = s_, d_
        M = sp_cols if ta else sp_rows
        dc = torch.randn((Z, H, M, F), generator=g).to(dtype)
    else:                                                # C = op(A) . op(S): the free dimension is M
        K = sp_cols if tb else sp_rows
        d_ = torch.randn((Z, H, K, F) if ta else (Z, H, F, K), generator=g).to(dtype)
        a, b = d_, s_
        N = sp_rows if tb else sp_cols
        dc = torch.randn((Z, H, F, N), generator=g).to(dtype)
    # forward only: the gradient of the sparse operand is an sdd product whose reduction runs over
    # this dimension and must be a multiple of 16, in the reference as here (matmul.py:318-319)
    want_c, _, _ = dm.matmul_reference(a, b, mode, ta, tb, layout, block)
    got = MatMul(layout, block, mode, trans_a=ta, trans_b=tb)(a.to(DEV), b.to(DEV))
    assert_close(got, want_c, 'odd free dimension')


def test_config1():
    c = workloads.config1()
    want, _, _ = dm.matmul_reference(c['a'], c['b'], 'sdd', True, False, c['layout'], 16)
    got = MatMul(c['layout'], 16, 'sdd', trans_a=True, trans_b=False)(c['a'].to(DEV), c['b'].to(DEV))
    assert got.shape == (4, int(c['layout'].sum()), 16, 16)
    assert_close(got, want, 'config 1')


@pytest.mark.parametrize('mode', ['dsd', 'dds'])
@pytest.mark.parametrize('ta', [False, True])
@pytest.mark.parametrize('tb', [False, True])
def test_config2_small(mode, ta, tb):
    c = workloads.config2(mode, ta, tb, small=True)
    run_both(c['layout'], 32, mode, ta, tb, c['a'], c['b'], c['dc'], 'config 2 small')


@pytest.mark.parametrize('mode', ['dsd', 'dds'])
@pytest.mark.parametrize('ta', [False, True])
@pytest.mark.parametrize('tb', [False, True])
def test_config2_full_slice(mode, ta, tb):
    """Full-size configuration 2 on the GPU; the oracle checks one (batch, head)
    slice of the result and of both gradients."""
    c = workloads.config2(mode, ta, tb, small=False)
    layout, block = c['layout'], 32
    op = MatMul(layout, block, mode, trans_a=ta, trans_b=tb)
    ag, bg = c['a'].to(DEV).requires_grad_(), c['b'].to(DEV).requires_grad_()
    out = op(ag, bg)
    out.backward(c['dc'].to(DEV))
    z, h = 7, 5
    b0, b1 = head_blocks(layout, h)
    sl = lambda t, sparse: (t[z:z + 1, b0:b1] if sparse else t[z:z + 1, h:h + 1])
    a_s, b_s = sl(c['a'], mode == 'dsd'), sl(c['b'], mode == 'dds')
    want_c, want_da, want_db = dm.matmul_reference(a_s, b_s, mode, ta, tb, layout[h:h + 1], block, sl(c['dc'], False))
    assert_close(sl(out, False), want_c, 'c')
    assert_close(sl(ag.grad, mode == 'dsd'), want_da, 'da')
    assert_close(sl(bg.grad, mode == 'dds'), want_db, 'db')


@pytest.mark.parametrize('mode', ['dsd', 'dds'])
@pytest.mark.parametrize('ta', [False, True])
@pytest.mark.parametrize('tb', [False, True])
@pytest.mark.parametrize('block', [32, 64, 128])
@pytest.mark.parametrize('dtype,width', [(torch.float16, 256), (torch.bfloat16, 384)])
def test_dsd_dds_tcgen05_kernel(mode, ta, tb, block, dtype, width):
    """Block 32 / 64 / 128 on the tcgen05 kernel, result tiles 256 and 128 wide.  A number of
    block-rows that does not fill the last tile (block 32: three of four, block 64: one of two), a
    block-row and a block-column without blocks, an odd number of columns in a tile's union;
    checked against the dense-masked oracle and against the mma.sync kernels on the same inputs."""
    from torch_blocksparse_b200 import _lib, fused
    Z, H, K = 2, 2, 384
    big = {32: 7 * 32, 64: 5 * 64, 128: 384}[block]           # extent of the sparse operand's non-K side
    M, N = (big, width) if mode == 'dsd' else (width, big)
    g = torch.Generator().manual_seed(block + 3)
    AS = (K, M) if ta else (M, K)
    BS = (N, K) if tb else (K, N)
    sshape = AS if mode == 'dsd' else BS
    layout = (torch.rand((H, sshape[0] // block, sshape[1] // block), generator=g) > 0.5).long()
    layout[1, 1, :] = 0
    layout[0, :, 2] = 0
    layout[:, 0, 0] = 1
    x = (torch.randn((Z, H) + AS, generator=g) * 0.1).to(dtype)
    w = (torch.randn((Z, H) + BS, generator=g) * 0.1).to(dtype)
    dc = (torch.randn((Z, H, M, N), generator=g) * 0.1).to(dtype)
    a = dm.dense_to_sparse(x, layout, block) if mode == 'dsd' else x
    b = dm.dense_to_sparse(w, layout, block) if mode == 'dds' else w
    run_both(layout, block, mode, ta, tb, a, b, dc, '%s ta=%d tb=%d block %d' % (mode, ta, tb, block))
    op = MatMul(layout, block, mode, trans_a=ta, trans_b=tb)
    L = _lib.lib()
    try:
        c_tc = op(a.to(DEV), b.to(DEV))
        _lib.check(L.bsp_matmul_use_tcgen05(0))
        c_mma = op(a.to(DEV), b.to(DEV))
    finally:
        _lib.check(L.bsp_matmul_use_tcgen05(1))
    assert_close(c_tc.cpu(), c_mma.cpu(), 'tcgen05 vs mma.sync')
    assert fused.device_status() == 0


def test_tcgen05_kernels_against_mma_sync_on_random_shapes():
    """Sixty random cases (mode, transposes, block 32 / 64 / 128, layout shape and density, batch,
    dense extent, dtype): the tcgen05 kernels against the mma.sync kernels on the same device
    tensors.  Covers tiles with empty block-rows, single blocks, empty heads' neighbours, tails."""
    import random
    from torch_blocksparse_b200 import _lib, fused
    rnd = random.Random(11)
    L = _lib.lib()
    for case in range(60):
        mode = rnd.choice(['sdd', 'dsd', 'dds'])
        ta, tb = rnd.random() < 0.5, rnd.random() < 0.5
        block = rnd.choice([32, 64, 128])
        dtype = rnd.choice([torch.float16, torch.bfloat16])
        Z, H = rnd.randint(1, 3), rnd.randint(1, 3)
        n1, n2 = rnd.randint(1, 9), rnd.randint(1, 20)          # blocks of the sparse tensor's two sides
        dense = rnd.choice([128, 256, 384, 512])
        g = torch.Generator().manual_seed(1000 + case)
        p = rnd.choice([0.1, 0.3, 0.6, 1.0])
        if mode == 'sdd':
            M, N, K = n1 * block, n2 * block, rnd.choice([64, 128, 320])
            lshape = (H, n1, n2)
        elif mode == 'dsd':
            M, K, N = n1 * block, n2 * block, dense
            lshape = (H, n2, n1) if ta else (H, n1, n2)
        else:
            K, N, M = n1 * block, n2 * block, dense
            lshape = (H, n2, n1) if tb else (H, n1, n2)
        layout = (torch.rand(lshape, generator=g) < p).long()
        layout[:, 0, 0] = 1
        AS = (K, M) if ta else (M, K)
        BS = (N, K) if tb else (K, N)
        x = (torch.randn((Z, H) + AS, generator=g) * 0.2).to(dtype)
        w = (torch.randn((Z, H) + BS, generator=g) * 0.2).to(dtype)
        a = dm.dense_to_sparse(x, layout, block) if mode == 'dsd' else x
        b = dm.dense_to_sparse(w, layout, block) if mode == 'dds' else w
        op = MatMul(layout, block, mode, trans_a=ta, trans_b=tb)
        try:
            c_tc = op(a.to(DEV), b.to(DEV))
            _lib.check(L.bsp_matmul_use_tcgen05(0))
            c_mma = op(a.to(DEV), b.to(DEV))
        finally:
            _lib.check(L.bsp_matmul_use_tcgen05(1))
        assert_close(c_tc.cpu(), c_mma.cpu(), 'case %d: %s ta=%d tb=%d block %d layout %s' % (case, mode, ta, tb, block, lshape))
    assert fused.device_status() == 0


@pytest.mark.parametrize('mode,ta,tb', [('dsd', False, False), ('dsd', True, False), ('dds', False, True)])
@pytest.mark.parametrize('block,nred', [(32, 200), (64, 160), (128, 140), (32, 1024), (32, 1056)])
def test_dsd_dds_long_reduction_side(mode, ta, tb, block, nred):
    """Many blocks on the reduction side: a tile whose plan does not fit one buffer of the
    tcgen05 kernel (more than 64 entries: it is handed over in several pieces), the 1024 blocks
    that kernel plans for at most, and 1056 (the mma.sync kernel takes the call).  Rows that are
    nearly full, one empty block-row; forward against the dense-masked oracle."""
    from torch_blocksparse_b200 import fused
    Z, H = 1, 2
    nout = 5                                                    # block-rows on the other side: the last tile is not full
    K, big = nred * block, nout * block
    M, N = (big, 128) if mode == 'dsd' else (128, big)
    g = torch.Generator().manual_seed(nred + block)
    AS = (K, M) if ta else (M, K)
    BS = (N, K) if tb else (K, N)
    sshape = AS if mode == 'dsd' else BS
    layout = (torch.rand((H, sshape[0] // block, sshape[1] // block), generator=g) < 0.7).long()
    red = (1 if ta else 2) if mode == 'dsd' else (2 if tb else 1)   # the layout dimension that is summed over
    if red == 2:
        layout[1, 1, :] = 0
    else:
        layout[1, :, 1] = 0
    x = (torch.randn((Z, H) + AS, generator=g) * K ** -0.5).half()
    w = (torch.randn((Z, H) + BS, generator=g)).half()
    a = dm.dense_to_sparse(x, layout, block) if mode == 'dsd' else x
    b = dm.dense_to_sparse(w, layout, block) if mode == 'dds' else w
    want = dm.matmul_reference(a, b, mode, ta, tb, layout, block)[0]
    got = MatMul(layout, block, mode, trans_a=ta, trans_b=tb)(a.to(DEV), b.to(DEV))
    assert_close(got.cpu(), want, '%s block %d, %d blocks summed' % (mode, block, nred))
    assert fused.device_status() == 0


@pytest.mark.parametrize('ta', [False, True])
@pytest.mark.parametrize('tb', [False, True])
@pytest.mark.parametrize('block', [32, 64, 128])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_sdd_tcgen05_kernel(ta, tb, block, dtype):
    """Block 32 / 64 / 128 with K a multiple of 64: sdd on the tcgen05 kernel, every transpose (K-
    and MN-major tiles of both operands).  Numbers of block-rows and of block-columns that do not
    fill the last tile / column group at block 32 and 64, a block-row and a block-column without
    blocks, rows with one block; checked against the dense-masked oracle and against the mma.sync
    kernel on the same inputs."""
    from torch_blocksparse_b200 import _lib, fused
    Z, H, K = 2, 2, 192
    M, N = {32: (7 * 32, 13 * 32), 64: (5 * 64, 7 * 64), 128: (384, 256)}[block]
    g = torch.Generator().manual_seed(block + 11)
    layout = (torch.rand((H, M // block, N // block), generator=g) > 0.5).long()
    layout[1, 1, :] = 0
    layout[0, :, 1] = 0
    layout[0, 2, :] = 0
    layout[0, 2, 0] = 1
    layout[:, 0, 0] = 1
    x = (torch.randn((Z, H) + ((K, M) if ta else (M, K)), generator=g) * 0.1).to(dtype)
    w = (torch.randn((Z, H) + ((N, K) if tb else (K, N)), generator=g) * 0.1).to(dtype)
    dc = dm.dense_to_sparse((torch.randn((Z, H, M, N), generator=g) * 0.1).to(dtype), layout, block)
    run_both(layout, block, 'sdd', ta, tb, x, w, dc, 'sdd ta=%d tb=%d block %d' % (ta, tb, block))
    op = MatMul(layout, block, 'sdd', trans_a=ta, trans_b=tb)
    L = _lib.lib()
    try:
        c_tc = op(x.to(DEV), w.to(DEV))
        _lib.check(L.bsp_matmul_use_tcgen05(0))
        c_mma = op(x.to(DEV), w.to(DEV))
    finally:
        _lib.check(L.bsp_matmul_use_tcgen05(1))
    assert_close(c_tc.cpu(), c_mma.cpu(), 'tcgen05 vs mma.sync')
    assert fused.device_status() == 0


@pytest.mark.parametrize('block,dtype', [(16, torch.float32), (32, torch.float16), (64, torch.float16), (128, torch.bfloat16)])
def test_linear_layer(block, dtype):
    """Linear (the layer torch_blocksparse/matmul.py:693-709 describes): forward and gradients
    against a dense layer whose weight is the sparse weight scattered into zeros; inputs of
    rank 3 with a row count that is not a multiple of 8."""
    from torch_blocksparse_b200 import Linear
    fin, fout = 3 * block if block >= 64 else 256, 2 * block if block >= 64 else 128
    g = torch.Generator().manual_seed(block)
    layout = (torch.rand((fin // block, fout // block), generator=g) > 0.4).long()
    layout[0, 0] = 1
    lin = Linear(fin, fout, block, layout).to(DEV)
    x = (torch.randn((3, 7, fin), generator=g) * 0.5).to(dtype)
    dy = (torch.randn((3, 7, fout), generator=g) * 0.5).to(dtype)
    xg = x.to(DEV).requires_grad_()
    y = lin(xg)
    assert y.shape == (3, 7, fout) and y.dtype == dtype
    y.backward(dy.to(DEV))
    w = lin.weight.detach().cpu().float()
    wd = dm.sparse_to_dense(w[None].to(dtype), layout[None], block)[0, 0].float()      # [fin, fout]
    xr = x.float().requires_grad_()
    yr = xr @ wd
    yr.backward(dy.float())
    assert_close(y, yr.to(dtype), 'linear y')
    assert_close(xg.grad, xr.grad.to(dtype), 'linear dx')
    dwd = x.float().reshape(-1, fin).t() @ dy.float().reshape(-1, fout)
    want_dw = dm.dense_to_sparse(dwd[None, None], layout[None], block)[0]
    assert_close(lin.weight.grad.to(dtype), want_dw.to(dtype), 'linear dw')
    with pytest.raises(ValueError):
        Linear(fin, fout + 1, block, layout)
