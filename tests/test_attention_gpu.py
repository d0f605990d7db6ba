"""GPU parity of the sparse self-attention wrapper (fused kernel and the
three-op chain) against the dense-masked CPU oracle."""
import pytest
import torch

import workloads
from oracle import dense_masked as dm
from tests.util import assert_close
from torch_blocksparse_b200 import DeepSpeedSparseSelfAttention, SparseSelfAttention, SparsityConfig, layouts

pytestmark = pytest.mark.gpu
DEV = 'cuda'


@pytest.fixture(autouse=True)
def no_device_side_timeout():
    """A bounded wait that expired inside a tcgen05 kernel is reported through the
    device status word; every test must leave it at zero."""
    yield
    from torch_blocksparse_b200 import fused
    assert fused.device_status() == 0, 'a bounded device-side wait expired'


def run_module(mod, q, k, v, do, **kw):
    qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
    gkw = {n: (t.to(DEV) if torch.is_tensor(t) else t) for n, t in kw.items()}
    o = mod(qg, kg, vg, **gkw)
    o.backward(do.to(DEV))
    return o, qg.grad, kg.grad, vg.grad


def check(layout, block, q, k, v, do, fused, kp_mode='add', am_mode='mul', **kw):
    scale = q.size(-1) ** -0.5
    want = dm.attention_reference(q, k, v, layout, block, scale, do=do, key_padding_mask_mode=kp_mode,
                                  attn_mask_mode=am_mode, **kw)
    mod = SparseSelfAttention(layout=layout, block=block, fused=fused, key_padding_mask_mode=kp_mode,
                              attn_mask_mode=am_mode)
    got = run_module(mod, q, k, v, do, **kw)
    for name, g, w in zip(('o', 'dq', 'dk', 'dv'), got, want):
        assert_close(g, w, '%s (fused=%s)' % (name, fused))


def rand_qkv(Z, H, L, D, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn((Z, H, L, D), generator=g).to(dtype) for _ in range(4))


@pytest.mark.parametrize('fused', [True, False])
@pytest.mark.parametrize('block,D', [(16, 64), (32, 64), (64, 64), (128, 64), (32, 128), (64, 128), (128, 128)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_random_layouts(block, D, dtype, fused):
    H, nb = 2, 6
    g = torch.Generator().manual_seed(block + D)
    layout = (torch.rand((H, nb, nb), generator=g) > 0.5).long()
    layout[:, :, 0] = 1
    layout[0, 3, :] = 0                       # a block-row without any block
    layout[1, :, 4] = 0                       # a block-column without any block
    q, k, v, do = rand_qkv(2, H, nb * block, D, dtype, seed=block)
    check(layout, block, q, k, v, do, fused)


@pytest.mark.parametrize('fused', [True, False])
@pytest.mark.parametrize('kp_mode,am_mode', [('add', 'mul'), ('mul', 'add')])
def test_masks_and_rpe(kp_mode, am_mode, fused):
    Z, H, L, D, block, dtype = 2, 2, 256, 64, 32, torch.float16
    g = torch.Generator().manual_seed(17)
    layout = (torch.rand((H, L // block, L // block), generator=g) > 0.4).long()
    layout[:, :, 0] = 1
    q, k, v, do = rand_qkv(Z, H, L, D, dtype, seed=3)
    rpe = (0.5 * torch.randn((Z, H, L, L), generator=g)).to(dtype)
    keep_k = torch.randint(0, 2, (Z, L), generator=g).bool()
    keep_k[:, 0] = True
    keep_a = torch.tril(torch.ones((L, L))).bool()
    ninf = float('-inf')
    kp = keep_k.to(dtype) if kp_mode == 'mul' else torch.where(keep_k, 0.0, ninf).to(dtype)
    am = keep_a.to(dtype) if am_mode == 'mul' else torch.where(keep_a, 0.0, ninf).to(dtype)
    check(layout, block, q, k, v, do, fused, kp_mode, am_mode, rpe=rpe, key_padding_mask=kp, attn_mask=am)


@pytest.mark.parametrize('what', ['rpe', 'rpe3d+am_mul', 'am_add', 'rpe+am_add+kpm', 'am_mul+kpm_mul'])
@pytest.mark.parametrize('block,D,dtype', [(64, 64, torch.float16), (128, 128, torch.bfloat16), (32, 64, torch.float16),
                                            (64, 128, torch.float16), (16, 64, torch.bfloat16)])
def test_rpe_and_attention_masks_on_tcgen05_path(block, D, dtype, what):
    """A relative position bias and an arbitrary attention mask (added or 'mul') travel with
    the chunks of the tcgen05 kernels (softmax.py:48-56, 63-70, 114-128 of the reference fuse them
    into its softmax).  Against the dense-masked definition and against the mma.sync kernels; an
    odd number of block-rows leaves a tile with a single half."""
    from torch_blocksparse_b200 import fused as F
    Z, H = 2, 2
    nb = {16: 12, 32: 6, 64: 5, 128: 3}[block]
    L = nb * block
    g = torch.Generator().manual_seed(block + D + len(what))
    layout = (torch.rand((H, nb, nb), generator=g) > 0.45).long()
    layout[:, :, 0] = 1
    layout[1, nb - 1, 1:] = 0
    q, k, v, do = rand_qkv(Z, H, L, D, dtype, seed=block + 11)
    kw, kp_mode, am_mode = {}, 'add', 'mul'
    if 'rpe3d' in what:
        kw['rpe'] = (0.5 * torch.randn((H, L, L), generator=g)).to(dtype)          # broadcast over the batch
    elif 'rpe' in what:
        kw['rpe'] = (0.5 * torch.randn((Z, H, L, L), generator=g)).to(dtype)
    if 'am_mul' in what:
        keep = torch.rand((L, L), generator=g) > 0.3
        keep[:, 0] = True
        kw['attn_mask'] = keep.to(dtype)
    if 'am_add' in what:
        am_mode = 'add'
        keep = torch.rand((L, L), generator=g) > 0.2
        keep[:, 0] = True
        kw['attn_mask'] = torch.where(keep, 0.3 * torch.randn((L, L), generator=g), torch.tensor(float('-inf'))).to(dtype)
    if 'kpm_mul' in what:
        kp_mode = 'mul'
        keepk = torch.rand((Z, L), generator=g) > 0.3
        keepk[:, 0] = True
        kw['key_padding_mask'] = keepk.to(dtype)
    elif 'kpm' in what:
        keepk = torch.rand((Z, L), generator=g) > 0.3
        keepk[:, 0] = True
        kw['key_padding_mask'] = torch.where(keepk, 0.0, float('-inf')).to(dtype)
    check(layout, block, q, k, v, do, True, kp_mode, am_mode, **kw)
    mod = SparseSelfAttention(layout=layout, block=block, fused=True, key_padding_mask_mode=kp_mode, attn_mask_mode=am_mode)
    try:
        tc = run_module(mod, q, k, v, do, **kw)
        F.PATH = 'mma'
        mma = run_module(mod, q, k, v, do, **kw)
    finally:
        F.PATH = 'tc'
    for name, a, b in zip(('o', 'dq', 'dk', 'dv'), tc, mma):
        assert_close(a.cpu(), b.cpu(), name + ' tcgen05 vs mma.sync')


@pytest.mark.parametrize('kp_mode', ['add', 'mul'])
@pytest.mark.parametrize('block,D', [(16, 64), (32, 64), (64, 64), (128, 64), (16, 128), (32, 128), (64, 128), (128, 128)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_key_padding_mask_on_tcgen05_path(block, D, dtype, kp_mode):
    """A key-padding mask alone (the BERT-style call of the reference's wrapper) stays on the
    tcgen05 kernels at every block size.  Checked against the dense-masked definition and against
    the mma.sync kernels; the first column block is kept and never masked, so that no row is
    masked out entirely (the reference's softmax gives NaN there)."""
    from torch_blocksparse_b200 import fused as F
    Z, H, nb = 3, 2, 8
    L = nb * block
    g = torch.Generator().manual_seed(block * 3 + D)
    layout = (torch.rand((H, nb, nb), generator=g) > 0.5).long()
    layout[:, :, 0] = 1
    layout[0, 2, 1:] = 0
    q, k, v, do = rand_qkv(Z, H, L, D, dtype, seed=block + 1)
    keep = torch.rand((Z, L), generator=g) > 0.3
    keep[:, :block] = True
    keep[1, L // 2:] = False                      # a padded tail, as with variable-length batches
    if kp_mode == 'mul':
        kp = keep.to(dtype)
    else:
        kp = torch.where(keep, 0.25 * torch.randn((Z, L), generator=g), torch.tensor(float('-inf'))).to(dtype)
    check(layout, block, q, k, v, do, True, kp_mode, 'mul', key_padding_mask=kp)
    mod = SparseSelfAttention(layout=layout, block=block, fused=True, key_padding_mask_mode=kp_mode)
    try:
        tc = run_module(mod, q, k, v, do, key_padding_mask=kp)
        F.PATH = 'mma'
        mma = run_module(mod, q, k, v, do, key_padding_mask=kp)
    finally:
        F.PATH = 'tc'
    for name, a, b in zip(('o', 'dq', 'dk', 'dv'), tc, mma):
        assert_close(a.cpu(), b.cpu(), name + ' tcgen05 vs mma.sync')


@pytest.mark.parametrize('D', [64, 128])
@pytest.mark.parametrize('with_kpm', [False, True])
def test_odd_number_of_block_rows_on_tcgen05_path(D, with_kpm):
    """Block 64 with an odd number of block-rows: one 128-row tile of every head has a single
    64-row chunk; heads with one-block and empty rows / columns; chunk lists of one to five."""
    block, H, nb, Z = 64, 3, 5, 2
    g = torch.Generator().manual_seed(D)
    layout = (torch.rand((H, nb, nb), generator=g) > 0.4).long()
    layout[:, :, 0] = 1
    layout[1] = torch.eye(nb, dtype=torch.long)
    layout[2, 4, :] = 0
    layout[2, :, 3] = 0
    q, k, v, do = rand_qkv(Z, H, nb * block, D, torch.float16, seed=D + 7)
    kw = {}
    if with_kpm:
        keep = torch.ones((Z, nb * block), dtype=torch.bool)
        keep[0, 70:90] = False
        keep[1, 200:] = False
        keep[1, 256:264] = True                   # the diagonal block of head 1 keeps one key per row block
        keep[:, ::64] = True
        kw['key_padding_mask'] = torch.where(keep, 0.0, float('-inf')).to(torch.float16)
    check(layout, block, q, k, v, do, True, **kw)


@pytest.mark.parametrize('block', [16, 32])
@pytest.mark.parametrize('D', [64, 128])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_small_blocks_on_tcgen05_path(block, D, dtype):
    """Blocks 16 and 32 run on the tcgen05 kernels through 64-wide lists of the coarsened layout,
    with absent 16 x 16 pieces masked out.  Random fine layout; a fine block-row without any
    block inside a coarse row that has some; a coarse position with a single fine block; a
    whole coarse row and column without blocks.  Against the oracle and the mma.sync kernels."""
    from torch_blocksparse_b200 import fused as F
    f = 64 // block
    H, nbc, Z = 2, 5, 2
    nb = nbc * f
    g = torch.Generator().manual_seed(block + D)
    layout = (torch.rand((H, nb, nb), generator=g) > 0.55).long()
    layout[:, :, 0] = 1
    layout[0, 1, :] = 0                                      # a fine row without blocks, neighbours have some
    layout[1, 2 * f:3 * f, :] = 0                            # a coarse row without blocks
    layout[1, :, 3 * f:4 * f] = 0                            # a coarse column without blocks
    layout[0, 3 * f:4 * f, f:2 * f] = 0
    layout[0, 3 * f, f + 1 if f > 1 else f] = 1              # a coarse position with one fine block
    q, k, v, do = rand_qkv(Z, H, nb * block, D, dtype, seed=block + D)
    check(layout, block, q, k, v, do, True)
    mod = SparseSelfAttention(layout=layout, block=block, fused=True)
    assert mod.get_ops(H, nb * block) and mod.tiles[(H, nb * block)] is not None
    try:
        tc = run_module(mod, q, k, v, do)
        F.PATH = 'mma'
        mma = run_module(mod, q, k, v, do)
    finally:
        F.PATH = 'tc'
    for name, a, b in zip(('o', 'dq', 'dk', 'dv'), tc, mma):
        assert_close(a.cpu(), b.cpu(), name + ' tcgen05 vs mma.sync')


@pytest.mark.parametrize('block,D', [(16, 64), (32, 64), (64, 64), (128, 64), (64, 128), (128, 128)])
@pytest.mark.parametrize('with_kpm', [False, True])
def test_causal_mask_on_tcgen05_path(block, D, with_kpm):
    """A 'mul' attention mask that is exactly lower triangular (the usual causal mask given
    with a unidirectional layout) is recognised and derived from the indices on the tcgen05
    kernels; any other mask is read as given.  Against the oracle and the mma.sync kernels."""
    from torch_blocksparse_b200 import fused as F
    Z, H, nbc = 2, 2, 4
    L = nbc * 128
    nb = L // block
    dtype = torch.float16
    g = torch.Generator().manual_seed(block + D + 5)
    layout = torch.tril((torch.rand((H, nb, nb), generator=g) > 0.3).long())
    layout[:, torch.arange(nb), torch.arange(nb)] = 1          # every row sees itself
    layout[:, :, 0] = 1
    q, k, v, do = rand_qkv(Z, H, L, D, dtype, seed=block + 2)
    am = torch.tril(torch.ones((L, L))).to(dtype)
    kw = dict(attn_mask=am)
    if with_kpm:
        keep = torch.rand((Z, L), generator=g) > 0.2
        keep[:, 0] = True
        kw['key_padding_mask'] = torch.where(keep, 0.0, float('-inf')).to(dtype)
    check(layout, block, q, k, v, do, True, 'add', 'mul', **kw)
    mod = SparseSelfAttention(layout=layout, block=block, fused=True)
    assert mod._is_causal(am.to(DEV))
    try:
        tc = run_module(mod, q, k, v, do, **kw)
        F.PATH = 'mma'
        mma = run_module(mod, q, k, v, do, **kw)
    finally:
        F.PATH = 'tc'
    for name, a, b in zip(('o', 'dq', 'dk', 'dv'), tc, mma):
        assert_close(a.cpu(), b.cpu(), name + ' tcgen05 vs mma.sync')
    am2 = am.clone()
    am2[5, 3] = 0                                              # not causal any more: read as given
    assert not mod._is_causal(am2.to(DEV))
    check(layout, block, q, k, v, do, True, 'add', 'mul', attn_mask=am2)


def test_causal_check_runs_once_per_mask_tensor():
    """forward() squeezes and casts the caller's mask into a new tensor object on every call; the
    comparison against the causal mask is still made once per tensor the caller holds, and again
    after the caller modifies it in place."""
    Z, H, L, D, block = 1, 2, 256, 64, 64
    layout = torch.tril(torch.ones((H, L // block, L // block), dtype=torch.long))
    mod = SparseSelfAttention(layout=layout, block=block, fused=True)
    q, k, v, _ = (t.to(DEV) for t in rand_qkv(Z, H, L, D, torch.float16))
    am = torch.tril(torch.ones((1, 1, L, L))).to(DEV)          # 4-D and FP32, as a model would hold it
    for _ in range(3):
        mod(q, k, v, attn_mask=am)
    assert mod.causal_checks == 1
    am[0, 0, 0, 5] = 1                                          # in-place change: checked again, no longer causal
    mod(q, k, v, attn_mask=am)
    assert mod.causal_checks == 2 and not mod._is_causal(am.squeeze(), am)


def test_operands_expanded_over_the_batch_fall_back_to_mma_sync():
    """q, k, v expanded over the batch (stride 0) cannot be described to the tensor-map encoder:
    the call still succeeds (on the mma.sync kernels) and matches the oracle."""
    Z, H, L, D, block = 3, 2, 256, 64, 64
    g = torch.Generator().manual_seed(4)
    layout = (torch.rand((H, L // block, L // block), generator=g) > 0.4).long()
    layout[:, :, 0] = 1
    q, k, v, do = rand_qkv(1, H, L, D, torch.float16, seed=9)
    mod = SparseSelfAttention(layout=layout, block=block, fused=True)
    o = mod(*(t.to(DEV).expand(Z, -1, -1, -1) for t in (q, k, v)))
    want = dm.attention_reference(q, k, v, layout, block, D ** -0.5)[0]
    for z in range(Z):
        assert_close(o[z:z + 1], want, 'expanded batch entry %d' % z)


def test_bounded_wait_expires_into_a_status_code_and_the_context_stays_usable():
    """A wait inside a tcgen05 kernel that can never complete (the loads of one chunk of every
    tile are withheld through the test hook, and the waits get a short limit) ends the kernel
    with the status word set: no hang, no trap.  Reading the status reports BSP_ERR_TIMEOUT once
    and clears it; the next launch on the same context is correct."""
    from torch_blocksparse_b200 import _lib
    c = workloads.config4('unidirectional', small=True)
    mod = SparseSelfAttention(layout=c['layout'], block=c['block'], fused=True)
    q, k, v = (c[n].to(DEV) for n in ('q', 'k', 'v'))
    L = _lib.lib()
    try:
        _lib.check(L.bsp_debug_attn_wait(4000, 1))
        with torch.no_grad():
            mod(q, k, v)
        torch.cuda.synchronize()                       # the launch returns by itself
        import ctypes
        st = ctypes.c_int(0)
        assert L.bsp_device_status(ctypes.byref(st)) == _lib.ERR_TIMEOUT and st.value == 1
        assert b'bounded wait expired' in L.bsp_last_error()
        with pytest.raises(RuntimeError):              # what the Python layer raises where it synchronises
            with torch.no_grad():
                mod(q, k, v)
            _lib.check_device()
    finally:
        _lib.check(L.bsp_debug_attn_wait(0, -1))
    assert _lib.device_status() == 0                   # reading cleared it
    with torch.no_grad():
        o = mod(q, k, v)
    want = dm.attention_reference(c['q'], c['k'], c['v'], c['layout'], c['block'], c['scale'])[0]
    assert_close(o, want, 'forward after a timed-out launch')


@pytest.mark.parametrize('attention', ['unidirectional', 'bidirectional'])
def test_graphed_step_equals_the_eager_step_bit_for_bit(attention):
    """module.graphed(): forward + backward captured in a CUDA graph (the dQ kernel on its second
    stream included) and replayed on changed inputs gives what module(q, k, v).backward(do) gives."""
    c = workloads.config4(attention, small=True, Z=2)
    mod = SparseSelfAttention(layout=c['layout'], block=c['block'], fused=True)
    q, k, v, do = (c[n].to(DEV) for n in ('q', 'k', 'v', 'do'))
    step = mod.graphed(q, k, v, do)
    for trial in range(2):
        if trial == 1:                                   # new values in the same buffers
            for t in (q, k, v, do):
                t.copy_(torch.randn_like(t))
        step.replay()
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        o = mod(qg, kg, vg)
        o.backward(do)
        for name, a, b in zip(('o', 'dq', 'dk', 'dv'), (step.o, step.dq, step.dk, step.dv), (o, qg.grad, kg.grad, vg.grad)):
            assert torch.equal(a, b), '%s differs on trial %d' % (name, trial)


def test_sparsity_config_path_and_key_transposed():
    """The reference's constructor path: SparsityConfig 'fixed', key handed over
    pre-transposed as [.., head_dim, L] (deepspeedsparseselfattention.py:119-123)."""
    cfg = SparsityConfig(mode='fixed', block=16, stride=64, attention='unidirectional', numverts=2, vertsize=1)
    Z, H, L, D = 2, 4, 256, 64
    q, k, v, do = rand_qkv(Z, H, L, D, torch.float16, seed=5)
    layout = layouts.fixed(H, L // 16, 4, 'unidirectional', 2, 1)
    want = dm.attention_reference(q, k, v, layout, 16, D ** -0.5, do=do)
    for fused in (True, False):
        mod = DeepSpeedSparseSelfAttention(cfg, fused=fused)
        qg, kg, vg = (t.to(DEV).requires_grad_() for t in (q, k, v))
        o = mod(qg, kg.transpose(2, 3), vg)
        o.backward(do.to(DEV))
        for name, g, w in zip(('o', 'dq', 'dk', 'dv'), (o, qg.grad, kg.grad, vg.grad), want):
            assert_close(g, w, '%s (fused=%s)' % (name, fused))
    with pytest.raises(NotImplementedError):
        DeepSpeedSparseSelfAttention(cfg)(q.to(DEV), k[:, :, :128].to(DEV), v.to(DEV))
    with pytest.raises(ValueError):
        DeepSpeedSparseSelfAttention(SparsityConfig(block=16, stride=64))(
            torch.zeros((1, 1, 40, 64), device=DEV, dtype=torch.float16),
            torch.zeros((1, 1, 40, 64), device=DEV, dtype=torch.float16),
            torch.zeros((1, 1, 40, 64), device=DEV, dtype=torch.float16))


@pytest.mark.parametrize('attention', ['unidirectional', 'bidirectional'])
def test_config4_small(attention):
    c = workloads.config4(attention, small=True)
    for fused in (True, False):
        check(c['layout'], c['block'], c['q'], c['k'], c['v'], c['do'], fused)


def test_config5_small():
    c = workloads.config5(small=True)
    for fused in (True, False):
        check(c['layout'], c['block'], c['q'], c['k'], c['v'], c['do'], fused)


def test_config4_full_fused_matches_chain_and_oracle_slice():
    """Full-size configuration 4 (Z reduced to 2 to bound host memory): the fused
    kernel against the three-op chain everywhere, and against the oracle on one
    (batch, head) slice."""
    c = workloads.config4('unidirectional', small=False, Z=2)
    layout, block = c['layout'], c['block']
    outs = {}
    for fused in (True, False):
        mod = SparseSelfAttention(layout=layout, block=block, fused=fused)
        outs[fused] = run_module(mod, c['q'], c['k'], c['v'], c['do'])
    for name, a, b in zip(('o', 'dq', 'dk', 'dv'), outs[True], outs[False]):
        assert_close(a, b, 'fused vs chain ' + name)
    z, h = 1, 15
    want = dm.attention_reference(c['q'][z:z + 1, h:h + 1], c['k'][z:z + 1, h:h + 1], c['v'][z:z + 1, h:h + 1],
                                  layout[h:h + 1], block, c['scale'], do=c['do'][z:z + 1, h:h + 1])
    for name, g, w in zip(('o', 'dq', 'dk', 'dv'), outs[True], want):
        assert_close(g[z:z + 1, h:h + 1], w, 'oracle slice ' + name)


@pytest.mark.parametrize('block,nb', [(64, 5), (64, 8), (128, 3)])
@pytest.mark.parametrize('dtype,D', [(torch.float16, 64), (torch.bfloat16, 128)])
def test_tcgen05_and_mma_sync_paths_agree(block, nb, dtype, D):
    """The same call on both kernel families (odd block counts leave a tile with a
    single block-row), each against the oracle, and against each other."""
    from torch_blocksparse_b200 import fused
    H = 3
    g = torch.Generator().manual_seed(block * nb + D)
    layout = (torch.rand((H, nb, nb), generator=g) > 0.45).long()
    layout[:, :, 0] = 1
    layout[2, 1, :] = 0
    q, k, v, do = rand_qkv(2, H, nb * block, D, dtype, seed=nb)
    want = dm.attention_reference(q, k, v, layout, block, D ** -0.5, do=do)
    outs = {}
    try:
        for path in ('tc', 'mma'):
            fused.PATH = path
            mod = SparseSelfAttention(layout=layout, block=block, fused=True)
            outs[path] = run_module(mod, q, k, v, do)
            for name, got, w in zip(('o', 'dq', 'dk', 'dv'), outs[path], want):
                assert_close(got, w, '%s on path %s' % (name, path))
    finally:
        fused.PATH = 'tc'
    for name, a, b in zip(('o', 'dq', 'dk', 'dv'), outs['tc'], outs['mma']):
        assert_close(a, b, 'tc vs mma ' + name)


def test_config5_full_layout_slice():
    """Benchmark configuration 5 at its full layout and length (L = 16384, block 128,
    head_dim 128, BF16), batch reduced to 1: oracle on three heads, both kernel families."""
    from torch_blocksparse_b200 import fused
    c = workloads.config5(small=False, Z=1)
    layout, block = c['layout'], c['block']
    heads = (0, 7, 15)
    want = {h: dm.attention_reference(c['q'][:, h:h + 1], c['k'][:, h:h + 1], c['v'][:, h:h + 1], layout[h:h + 1], block,
                                      c['scale'], do=c['do'][:, h:h + 1]) for h in heads}
    try:
        for path in ('tc', 'mma'):
            fused.PATH = path
            mod = SparseSelfAttention(layout=layout, block=block, fused=True)
            got = run_module(mod, c['q'], c['k'], c['v'], c['do'])
            for h in heads:
                for name, g_, w in zip(('o', 'dq', 'dk', 'dv'), got, want[h]):
                    assert_close(g_[:, h:h + 1], w, 'config 5 head %d %s on path %s' % (h, name, path))
    finally:
        fused.PATH = 'tc'


def test_multihead_attention_matches_torch_dense():
    """The reference's own test (tests/test_attention.py:13-49): all-ones layout against
    torch.nn.MultiheadAttention, FP16, block 16, B=2, H=2, L=128, E=128, key-padding mask
    given additively (-inf) to the sparse module and as bool to the dense one."""
    from torch_blocksparse_b200 import MultiheadAttention, replace_mha
    torch.manual_seed(0)
    block, B, H, L, E = 16, 2, 2, 128, 128
    layout = torch.ones(H, L // block, L // block).long()
    sparse = MultiheadAttention(E, H, layout, block).to(DEV).half()
    torch.manual_seed(0)
    dense = torch.nn.MultiheadAttention(E, H).to(DEV).half()
    for ps, pd in zip(sparse.parameters(), dense.parameters()):
        ps.data.copy_(pd.data)
    x = torch.rand(L, B, E, device=DEV).half()
    mul_mask = torch.randint(0, 2, (B, L), dtype=torch.bool, device=DEV)
    mul_mask[:, 0] = False
    add_mask = torch.zeros((B, L), device=DEV).half()
    add_mask[mul_mask] = float('-inf')
    got, _ = sparse(x, x, x, key_padding_mask=add_mask, need_weights=False)
    want, _ = dense(x, x, x, key_padding_mask=mul_mask, need_weights=False)
    assert_close(got, want, 'MultiheadAttention')
    # model surgery keeps the parameters
    model = torch.nn.Sequential(torch.nn.MultiheadAttention(E, H)).to(DEV).half()
    ref_w = model[0].in_proj_weight.detach().clone()
    replace_mha(model, (layout, block))
    assert isinstance(model[0], MultiheadAttention) and torch.equal(model[0].in_proj_weight, ref_w)


@pytest.mark.parametrize('kp_mode', ['add', 'mul'])
@pytest.mark.parametrize('block,D', [(64, 64), (128, 128), (32, 64)])
def test_fully_padded_window_gives_zeros_on_both_paths(block, D, kp_mode):
    """Query rows whose every visible key is padded out (a padded tail inside a local window):
    both kernel families return zeros for them, a log-sum-exp of -inf and finite gradients
    everywhere (the reference's softmax would give NaN for such rows); the unpadded batch
    entry still matches the oracle."""
    from torch_blocksparse_b200 import fused as F
    Z, H, nb = 2, 2, 6
    L = nb * block
    dtype = torch.float16
    layout = torch.zeros((H, nb, nb), dtype=torch.long)
    for i in range(nb):
        layout[:, i, max(0, i - 1):i + 1] = 1                 # a band of two blocks, no global column
    q, k, v, do = rand_qkv(Z, H, L, D, dtype, seed=block + D)
    keep = torch.ones((Z, L), dtype=torch.bool)
    keep[1, 3 * block:] = False                               # rows from block 4 on see padded keys only
    kp = keep.to(dtype) if kp_mode == 'mul' else torch.where(keep, 0.0, float('-inf')).to(dtype)
    mod = SparseSelfAttention(layout=layout, block=block, fused=True, key_padding_mask_mode=kp_mode)
    try:
        tc = run_module(mod, q, k, v, do, key_padding_mask=kp)
        F.PATH = 'mma'
        mma = run_module(mod, q, k, v, do, key_padding_mask=kp)
    finally:
        F.PATH = 'tc'
    for name, a, b in zip(('o', 'dq', 'dk', 'dv'), tc, mma):
        assert bool(torch.isfinite(a).all()) and bool(torch.isfinite(b).all()), name + ' has non-finite values'
        assert_close(a.cpu(), b.cpu(), name + ' tcgen05 vs mma.sync')
    assert float(tc[0].detach()[1, :, 4 * block:].abs().max()) == 0.0
    assert float(mma[0].detach()[1, :, 4 * block:].abs().max()) == 0.0
    want = dm.attention_reference(q[:1], k[:1], v[:1], layout, block, D ** -0.5, do=do[:1], key_padding_mask=kp[:1],
                                  key_padding_mask_mode=kp_mode)
    for name, g_, w in zip(('o', 'dq', 'dk', 'dv'), tc, want):
        assert_close(g_[:1], w, 'unpadded batch entry ' + name)


def test_config4_bidirectional_full_slices():
    """Configuration 4 with the bidirectional layout at full length (L = 8192, 71 680 blocks),
    batch reduced to 1: the oracle on two (batch, head) slices."""
    c = workloads.config4('bidirectional', small=False, Z=1)
    layout, block = c['layout'], c['block']
    assert int(layout.sum()) == 71680
    mod = SparseSelfAttention(layout=layout, block=block, fused=True)
    got = run_module(mod, c['q'], c['k'], c['v'], c['do'])
    for h in (0, 11):
        want = dm.attention_reference(c['q'][:, h:h + 1], c['k'][:, h:h + 1], c['v'][:, h:h + 1], layout[h:h + 1], block,
                                      c['scale'], do=c['do'][:, h:h + 1])
        for name, g_, w in zip(('o', 'dq', 'dk', 'dv'), got, want):
            assert_close(g_[:, h:h + 1], w, 'bidirectional head %d %s' % (h, name))


def test_multihead_attention_backward_matches_torch_dense():
    """Gradients of the seq-first drop-in (input and every parameter) against
    torch.nn.MultiheadAttention on an all-ones layout."""
    from torch_blocksparse_b200 import MultiheadAttention
    torch.manual_seed(1)
    block, B, H, L, E = 16, 2, 2, 128, 128
    layout = torch.ones(H, L // block, L // block).long()
    sparse = MultiheadAttention(E, H, layout, block).to(DEV).half()
    dense = torch.nn.MultiheadAttention(E, H).to(DEV).half()
    for ps, pd in zip(sparse.parameters(), dense.parameters()):
        ps.data.copy_(pd.data)
    x0 = torch.rand(L, B, E, device=DEV).half()
    dy = (torch.rand(L, B, E, device=DEV) - 0.5).half()
    grads = []
    for mod in (sparse, dense):
        x = x0.clone().requires_grad_()
        y, _ = mod(x, x, x, need_weights=False)
        y.backward(dy)
        grads.append([x.grad] + [p.grad for p in mod.parameters()])
    names = ['x'] + [n for n, _ in sparse.named_parameters()]
    for name, a, b in zip(names, *grads):
        assert_close(a, b, 'MultiheadAttention backward: ' + name)


def test_host_pipeline_matches_device_path():
    """HostAttention (pinned host operands streamed by batch slices over three streams) gives
    bit for bit what the module gives on device tensors, on two runs in a row (the second one
    reuses the slice buffers while the first is still draining)."""
    from torch_blocksparse_b200 import HostAttention
    c = workloads.config4('unidirectional', small=True, Z=5)
    Z, H, L, D = c['q'].shape
    mod = SparseSelfAttention(layout=c['layout'], block=c['block'], fused=True)
    q, k, v = (c[n].cuda().requires_grad_() for n in ('q', 'k', 'v'))
    o = mod(q, k, v)
    o.backward(c['do'].cuda())
    want = [o.detach().cpu(), q.grad.cpu(), k.grad.cpu(), v.grad.cpu()]
    pipe = HostAttention(mod, H, L, D, torch.float16, 'cuda', slice_batch=2, depth=2)
    host = [c[n].pin_memory() for n in ('q', 'k', 'v', 'do')]
    for attempt in range(2):
        outs = [torch.zeros_like(host[0]).pin_memory() for _ in range(4)]
        pipe.run(*host, *outs).synchronize()
        for name, got, ref in zip(('o', 'dq', 'dk', 'dv'), outs, want):
            assert torch.equal(got, ref), '%s differs on run %d' % (name, attempt)
    with pytest.raises(ValueError):
        pipe.run(*[t.clone() for t in host], *outs)          # unpinned operands
