"""GPU parity of the block-sparse softmax against the dense-masked CPU oracle."""
import pytest
import torch

import workloads
from oracle import dense_masked as dm
from tests.util import Guarded, assert_close, load_npz
from torch_blocksparse_b200 import Softmax

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def run_both(layout, block, x, dy, dtype, **kw):
    """Runs the CUDA op (forward + backward through autograd) and the oracle."""
    want_y, want_dx = dm.softmax_reference(x, layout, block, dy=dy, **kw)
    op = Softmax(layout, block)
    gkw = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in kw.items()}
    # forward alone on an input inside a NaN-margined allocation: nothing is written outside it
    gx = Guarded(x.shape, x.dtype, DEV, fill=x.to(DEV))
    with torch.no_grad():
        y0 = op(gx.t, **gkw)
    torch.cuda.synchronize()
    gx.check('x')
    assert_close(y0, want_y, 'y (guarded input)')
    xg = x.to(DEV).requires_grad_()
    xin = xg * 1                      # non-leaf: the op works in place
    y = op(xin, **gkw)
    assert y.data_ptr() == xin.data_ptr(), 'softmax must overwrite its input'
    y_copy = y.detach().clone()
    gdy = Guarded(dy.shape, dy.dtype, DEV, fill=dy.to(DEV))
    y.backward(gdy.t)                 # the backward overwrites the incoming gradient
    torch.cuda.synchronize()
    gdy.check('dy')
    assert_close(y_copy, want_y, 'y')
    assert_close(xg.grad, want_dx, 'dx')


def make_inputs(Z, H, M, N, block, rho, dtype, seed=0, masks=True):
    g = torch.Generator().manual_seed(seed)
    layout = (torch.rand((H, M // block, N // block), generator=g) > rho).long()
    layout[:, :, 0] = 1
    nnz = int(layout.sum())
    x = torch.rand((Z, nnz, block, block), generator=g).to(dtype)
    dy = torch.rand((Z, nnz, block, block), generator=g).to(dtype)
    kw = {}
    if masks:
        am = torch.randint(0, 2, (M, N), generator=g).to(dtype)
        am[:, 0] = 1
        kp = torch.randint(0, 2, (Z, N), generator=g).to(dtype)
        kp[:, 0] = 0
        kp[kp == 1] = float('-inf')
        kw = dict(key_padding_mask=kp, key_padding_mask_mode='add', attn_mask=am, attn_mask_mode='mul')
    return layout, x, dy, kw


# the reference's own test grid (tests/test_softmax.py:80-90): block 16, widths 256 / 576,
# FP16 and FP32, Z=2, H=4, scale 0.4, rho 0.4, kp 'add' with -inf, attention mask 'mul'
@pytest.mark.parametrize('dtype', [torch.float16, torch.float32, torch.bfloat16])
@pytest.mark.parametrize('width', [256, 576])
def test_reference_grid(width, dtype):
    layout, x, dy, kw = make_inputs(2, 4, width, width, 16, 0.4, dtype)
    run_both(layout, 16, x, dy, dtype, scale=0.4, **kw)


@pytest.mark.parametrize('block', [16, 32, 64, 128])
@pytest.mark.parametrize('dtype', [torch.float16, torch.float32])
def test_blocks_no_masks(block, dtype):
    layout, x, dy, _ = make_inputs(2, 2, 4 * block, 6 * block, block, 0.5, dtype, seed=block, masks=False)
    run_both(layout, block, x, dy, dtype, scale=1.0)


@pytest.mark.parametrize('kp_mode,am_mode', [('add', 'add'), ('mul', 'mul'), ('mul', 'add')])
def test_mask_modes_and_rpe(kp_mode, am_mode):
    Z, H, M, N, block, dtype = 2, 3, 128, 192, 32, torch.float16
    g = torch.Generator().manual_seed(5)
    layout = (torch.rand((H, M // block, N // block), generator=g) > 0.4).long()
    layout[:, :, 0] = 1
    nnz = int(layout.sum())
    x = torch.randn((Z, nnz, block, block), generator=g).to(dtype)
    dy = torch.randn((Z, nnz, block, block), generator=g).to(dtype)
    rpe = (0.5 * torch.randn((Z, H, M, N), generator=g)).to(dtype)
    keep_k = torch.randint(0, 2, (Z, N), generator=g).bool()
    keep_k[:, 0] = True
    keep_a = torch.randint(0, 2, (M, N), generator=g).bool()
    keep_a[:, 0] = True
    ninf = float('-inf')
    kp = keep_k.to(dtype) if kp_mode == 'mul' else torch.where(keep_k, 0.0, ninf).to(dtype)
    am = keep_a.to(dtype) if am_mode == 'mul' else torch.where(keep_a, 0.0, ninf).to(dtype)
    run_both(layout, block, x, dy, dtype, scale=0.3, rpe=rpe, key_padding_mask=kp, attn_mask=am,
             key_padding_mask_mode=kp_mode, attn_mask_mode=am_mode)


def test_rpe_3d_broadcast_and_unaligned_masks():
    """rpe given as [H, M, N]; masks whose storage offset breaks 16-byte alignment
    take the scalar load path."""
    Z, H, M, N, block, dtype = 2, 2, 64, 64, 16, torch.float16
    layout, x, dy, kw = make_inputs(Z, H, M, N, block, 0.3, dtype, seed=9)
    g = torch.Generator().manual_seed(3)
    rpe = torch.randn((H, M, N), generator=g).to(dtype)
    want_y, _ = dm.softmax_reference(x, layout, block, scale=0.5, rpe=rpe, **kw)
    op = Softmax(layout, block)
    pad = torch.zeros(Z * N + 1, dtype=dtype, device=DEV)
    kp_dev = pad[1:].view(Z, N)
    kp_dev.copy_(kw['key_padding_mask'])
    y = op(x.to(DEV).clone(), scale=0.5, rpe=rpe.to(DEV), key_padding_mask=kp_dev,
           attn_mask=kw['attn_mask'].to(DEV), key_padding_mask_mode='add', attn_mask_mode='mul')
    assert_close(y, want_y, 'y')


def test_long_rows_use_loop_kernel():
    """Rows of 160 blocks of 64 (10240 elements) exceed the register variants."""
    H, nb, block, dtype = 1, 160, 64, torch.float16
    layout = torch.ones((H, 1, nb), dtype=torch.long)
    g = torch.Generator().manual_seed(1)
    x = torch.randn((2, nb, block, block), generator=g).to(dtype)
    dy = torch.randn((2, nb, block, block), generator=g).to(dtype)
    run_both(layout, block, x, dy, dtype, scale=0.7)


def test_empty_rows_and_row_limit():
    block = 16
    layout = torch.zeros((2, 4, 4), dtype=torch.long)
    layout[0, 1, 2] = layout[0, 1, 3] = layout[1, 3, 0] = 1
    g = torch.Generator().manual_seed(2)
    x = torch.randn((3, 3, block, block), generator=g)
    dy = torch.randn((3, 3, block, block), generator=g)
    run_both(layout, block, x, dy, torch.float32, scale=2.0)
    big = torch.ones((1, 1, 2048), dtype=torch.long)      # 2048 * 16 = 32768 elements per row
    with pytest.raises(NotImplementedError):
        Softmax(big, 16)(torch.zeros((1, 2048, 16, 16), device=DEV))


def test_fully_masked_row_is_nan_like_the_reference():
    block = 16
    layout = torch.ones((1, 1, 2), dtype=torch.long)
    x = torch.zeros((1, 2, block, block), device=DEV)
    kp = torch.full((1, 32), float('-inf'), device=DEV)
    y = Softmax(layout, block)(x, key_padding_mask=kp)
    assert bool(torch.isnan(y).all())


def test_golden_reference_oracle_case():
    """The fixture produced by the reference's own run_softmax_reference."""
    d = load_npz('dense_masked.npz')
    layout = torch.from_numpy(d['sm_layout'])
    block = 16
    x = dm.dense_to_sparse(torch.from_numpy(d['sm_x']), layout, block)
    dy = dm.dense_to_sparse(torch.from_numpy(d['sm_dy']), layout, block)
    op = Softmax(layout, block)
    xg = x.to(DEV).requires_grad_()
    y = op(xg * 1, scale=float(d['sm_scale'][0]), key_padding_mask=torch.from_numpy(d['sm_kp']).to(DEV),
           attn_mask=torch.from_numpy(d['sm_am']).to(DEV), key_padding_mask_mode='add', attn_mask_mode='mul')
    y_copy = y.detach().clone()
    y.backward(dy.to(DEV))
    assert_close(y_copy, torch.from_numpy(d['sm_y']), 'y')
    assert_close(xg.grad, torch.from_numpy(d['sm_dx']), 'dx')


def test_config3_small_and_full():
    """Benchmark configuration 3: small against the oracle, full size through
    properties that need no oracle (rows sum to one, masked entries are zero,
    backward rows sum to zero) plus an oracle check of one (z, head) slice."""
    c = workloads.config3(small=True)
    run_both(c['layout'], c['block'], c['x'], c['dy'], c['dtype'], scale=c['scale'], rpe=c['rpe'],
             key_padding_mask=c['key_padding_mask'], attn_mask=c['attn_mask'],
             key_padding_mask_mode='add', attn_mask_mode='mul')
    c = workloads.config3(small=False)
    layout, block = c['layout'], c['block']
    op = Softmax(layout, block)
    x = c['x'].to(DEV)
    rpe = c['rpe'].to(DEV)
    y = op(x, scale=c['scale'], rpe=rpe[None].expand(x.size(0), -1, -1, -1),
           key_padding_mask=c['key_padding_mask'].to(DEV), attn_mask=c['attn_mask'].to(DEV),
           key_padding_mask_mode='add', attn_mask_mode='mul')
    torch.cuda.synchronize()
    # every row of every block-row sums to one
    lut, _ = op.make_lut(torch.device('cpu'))
    H, Mb, _ = layout.shape
    sizes = lut[:2 * H * Mb:2].long()
    rowsum = torch.zeros((y.size(0), H * Mb, block), device=DEV)
    owner = torch.repeat_interleave(torch.arange(H * Mb), sizes).to(DEV)
    rowsum.index_add_(1, owner, y.float().sum(-1))
    assert float((rowsum - 1).abs().max()) < 2e-2
    # oracle on the last batch entry, last head
    z, h = y.size(0) - 1, H - 1
    from tests.util import head_blocks
    b0, b1 = head_blocks(layout, h)
    want, _ = dm.softmax_reference(c['x'][z:z + 1, b0:b1], layout[h:h + 1], block, scale=c['scale'],
                                   rpe=c['rpe'][h:h + 1], key_padding_mask=c['key_padding_mask'][z:z + 1],
                                   attn_mask=c['attn_mask'], key_padding_mask_mode='add', attn_mask_mode='mul')
    assert_close(y[z:z + 1, b0:b1], want, 'config3 slice')
    # backward at full size: dx = y (dy - sum_row y dy) scale, written over dy; rows of dx sum to
    # zero, and the same slice against the oracle
    dy = c['dy'].to(DEV)
    _, want_dx = dm.softmax_reference(c['x'][z:z + 1, b0:b1], layout[h:h + 1], block, scale=c['scale'],
                                      rpe=c['rpe'][h:h + 1], key_padding_mask=c['key_padding_mask'][z:z + 1],
                                      attn_mask=c['attn_mask'], key_padding_mask_mode='add', attn_mask_mode='mul',
                                      dy=c['dy'][z:z + 1, b0:b1])
    xg = c['x'].to(DEV).requires_grad_()
    y2 = op(xg * 1, scale=c['scale'], rpe=rpe[None].expand(x.size(0), -1, -1, -1),
            key_padding_mask=c['key_padding_mask'].to(DEV), attn_mask=c['attn_mask'].to(DEV),
            key_padding_mask_mode='add', attn_mask_mode='mul')
    y2.backward(dy)
    dx = xg.grad
    rowsum.zero_()
    rowsum.index_add_(1, owner, dx.float().sum(-1))
    assert float(rowsum.abs().max()) < 2e-2
    assert_close(dx[z:z + 1, b0:b1], want_dx, 'config3 backward slice')
