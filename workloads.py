"""Seeded synthetic inputs for the five benchmark configurations.

The reference measures on no dataset; every configuration is random data of a
stated shape and distribution.  All tensors are drawn on the CPU from an
explicit torch.Generator so that the CPU oracle and the GPU kernels see the
same bits; callers move them to the device.  Each generator takes a `small`
flag that shrinks the batch / size to something the dense-masked CPU oracle
finishes in seconds (same layout family, same distributions).
"""
import torch

# Layout generators: the package's native ones, or (LAYOUT_SOURCE = 'oracle') the CPU restatement
# under oracle/, so that the CPU reference arm of the benchmark needs nothing of the product.
LAYOUT_SOURCE = 'package'


def _fixed_layout(H, nb, stride, attention):
    if LAYOUT_SOURCE == 'oracle':
        from oracle import lut
        return torch.from_numpy(lut.make_fixed_layout(H, nb, 'fixed', stride, attention, 1, 1)).long()
    from torch_blocksparse_b200 import layouts
    return layouts.fixed(H, nb, stride, attention, 1, 1)


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def config1(small=False):
    """sdd FP32, trans_a=True, block 16: A [4,2,384,256] (stored K x M), B [4,2,384,512],
    U[0,1) seed 0; layout [2,16,32] Bernoulli(0.5)."""
    g = _gen(0)
    layout = torch.bernoulli(torch.full((2, 16, 32), 0.5), generator=g).long()
    Z = 2 if small else 4
    a = torch.rand((Z, 2, 384, 256), generator=g)
    b = torch.rand((Z, 2, 384, 512), generator=g)
    return dict(layout=layout, block=16, mode='sdd', trans_a=True, trans_b=False, a=a, b=b, dtype=torch.float32)


def config2(mode='dsd', trans_a=False, trans_b=False, small=False):
    """dsd / dds FP16, block 32, Z=8, H=8, M=N=K=2048; layout [8,64,64] Bernoulli(0.25);
    values N(0,1)/sqrt(K)."""
    g = _gen(0)
    if small:
        Z, H, S = 2, 2, 256
    else:
        Z, H, S = 8, 8, 2048
    nb = S // 32
    layout = torch.bernoulli(torch.full((H, nb, nb), 0.25), generator=g).long()
    for h in range(H):                         # the table builders reject an empty head
        if layout[h].sum() == 0:
            layout[h, 0, 0] = 1
    nnz = int(layout.sum())
    sc = S ** -0.5
    sparse = (torch.randn((Z, nnz, 32, 32), generator=g) * sc).half()
    dense = (torch.randn((Z, H, S, S), generator=g) * sc).half()
    grad = (torch.randn((Z, H, S, S), generator=g) * sc).half()
    a, b = (sparse, dense) if mode == 'dsd' else (dense, sparse)
    return dict(layout=layout, block=32, mode=mode, trans_a=trans_a, trans_b=trans_b, a=a, b=b, dc=grad,
                dtype=torch.float16)


def config3(small=False):
    """Softmax FP16 fwd+bwd, block 64, Z=8, H=16, 4096 x 4096; causal band of 4 blocks plus
    the first block-column; scale 1/8; rpe [H,4096,4096] N(0,0.1) broadcast over Z; key-padding
    mask with valid lengths in [2048,4096] ('add', -inf); causal attention mask ('mul')."""
    g = _gen(0)
    if small:
        Z, H, L = 2, 2, 512
    else:
        Z, H, L = 8, 16, 4096
    nb = L // 64
    from torch_blocksparse_b200 import layouts
    layout = layouts.causal_band(H, nb, 4, 1)
    nnz = int(layout.sum())
    x = torch.randn((Z, nnz, 64, 64), generator=g).half()
    rpe = (0.1 * torch.randn((H, L, L), generator=g)).half()
    lengths = torch.randint(L // 2, L + 1, (Z,), generator=g)
    kpm = torch.zeros((Z, L), dtype=torch.float16)
    kpm[torch.arange(L)[None, :] >= lengths[:, None]] = float('-inf')
    am = torch.tril(torch.ones((L, L), dtype=torch.float16))
    dy = torch.randn((Z, nnz, 64, 64), generator=g).half()
    return dict(layout=layout, block=64, x=x, scale=0.125, rpe=rpe, key_padding_mask=kpm, attn_mask=am,
                key_padding_mask_mode='add', attn_mask_mode='mul', dy=dy, dtype=torch.float16)


def config4(attention='unidirectional', small=False, Z=None, seed=0):
    """Sparse self-attention FP16 fwd+bwd: Z=8, H=16, L=8192, head_dim 64, block 64, fixed
    layout with local windows of 4 blocks whose last block is global.  `seed` selects
    the shard (rank) the tensors are drawn for."""
    g = _gen(seed)
    if small:
        z, H, L = 1, 2, 1024
    else:
        z, H, L = 8, 16, 8192
    if Z is not None:
        z = Z
    layout = _fixed_layout(H, L // 64, 4, attention)
    q, k, v, do = (torch.randn((z, H, L, 64), generator=g).half() for _ in range(4))
    return dict(layout=layout, block=64, q=q, k=k, v=v, do=do, scale=64 ** -0.5, dtype=torch.float16,
                attention=attention)


def config5(small=False, Z=None):
    """BigBird-style attention BF16 fwd+bwd: Z=32, H=16, L=16384, head_dim 128, block 128;
    per head 3 random blocks per row, a sliding window of 3 blocks, 2 global rows and columns."""
    g = _gen(0)
    if small:
        z, H, L = 1, 2, 2048
    else:
        z, H, L = 32, 16, 16384
    if Z is not None:
        z = Z
    from torch_blocksparse_b200 import layouts
    layout = layouts.bigbird(H, L // 128, 3, 3, 2, seed=0)
    q, k, v, do = (torch.randn((z, H, L, 128), generator=g).bfloat16() for _ in range(4))
    return dict(layout=layout, block=128, q=q, k=k, v=v, do=do, scale=128 ** -0.5, dtype=torch.bfloat16)


def attention_flops(layout, block, Z, D):
    """Counted FLOPs of one attention fwd+bwd: the six nonzero-block products
    (QK^T, PV; dP, dV, dQ, dK), 2*Z*nnz*block^2*D each; softmax and any
    recomputation are not counted."""
    return 6 * 2 * Z * int(layout.sum()) * block * block * D
