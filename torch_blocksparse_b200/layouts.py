"""Layout generators: int64 CPU tensors [H, L/block, L/block] of 0/1.

`fixed` is the reference's sparse-transformer layout
(torch_blocksparse/deepspeedsparseselfattention.py:33-65); the others cover
layouts the reference's SparsityConfig cannot express and are passed to the
ops through their explicit `layout` argument.
"""
import torch

from . import _lib, tables


def fixed(num_heads, num_blocks, block_stride, attention='unidirectional', numverts=1, vertsize=1):
    """Local windows of `block_stride` blocks plus vertical stripes (the last
    `vertsize` block-columns of every window, rotated over `numverts` heads)."""
    return tables.make_fixed_layout(num_heads, num_blocks, 'fixed', block_stride, attention, numverts, vertsize)


def dense(num_heads, num_blocks):
    return torch.ones((num_heads, num_blocks, num_blocks), dtype=torch.int64)


def window(num_heads, num_blocks, below, above, global_rows=0, global_cols=0, random_cols=None):
    """Sliding-window layout built natively: block-row i sees block-columns
    [i - below, i + above], the first `global_cols` block-columns and the columns
    `random_cols[h, i, :]` (int tensor [H, nb, r], optional); the first
    `global_rows` block-rows see everything."""
    out = torch.empty((num_heads, num_blocks, num_blocks), dtype=torch.int64)
    if random_cols is not None:
        random_cols = random_cols.to(torch.int32).contiguous()
        if random_cols.dim() != 3 or tuple(random_cols.shape[:2]) != (num_heads, num_blocks):
            raise ValueError('random_cols must be [num_heads, num_blocks, r]')
    _lib.check(_lib.lib().bsp_window_layout_build(
        num_heads, num_blocks, below, above, global_rows, global_cols,
        random_cols.data_ptr() if random_cols is not None else None,
        random_cols.size(2) if random_cols is not None else 0, out.data_ptr()))
    return out


def causal_band(num_heads, num_blocks, band, global_cols=1):
    """Block-row i sees block-columns max(0, i-band+1) .. i and the first
    `global_cols` block-columns."""
    return window(num_heads, num_blocks, band - 1, 0, 0, global_cols)


def bigbird(num_heads, num_blocks, num_random=3, window_blocks=3, num_global=2, seed=0):
    """BigBird-style layout: a sliding window of `window_blocks` blocks, `num_random`
    random block-columns per block-row (head h drawn from torch.Generator(seed + h),
    one randperm per block-row) and `num_global` global block-rows and block-columns."""
    cols = torch.empty((num_heads, num_blocks, num_random), dtype=torch.int32)
    for h in range(num_heads):
        g = torch.Generator().manual_seed(seed + h)
        for r in range(num_blocks):
            cols[h, r] = torch.randperm(num_blocks, generator=g)[:num_random]
    half = window_blocks // 2
    return window(num_heads, num_blocks, half, half, num_global, num_global, cols)
