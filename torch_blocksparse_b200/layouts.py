"""Layout generators: int64 CPU tensors [H, L/block, L/block] of 0/1.

`fixed` is the reference's sparse-transformer layout
(torch_blocksparse/deepspeedsparseselfattention.py:33-65); the others cover
layouts the reference's SparsityConfig cannot express and are passed to the
ops through their explicit `layout` argument.
"""
import torch

from . import tables


def fixed(num_heads, num_blocks, block_stride, attention='unidirectional', numverts=1, vertsize=1):
    """Local windows of `block_stride` blocks plus vertical stripes (the last
    `vertsize` block-columns of every window, rotated over `numverts` heads)."""
    return tables.make_fixed_layout(num_heads, num_blocks, 'fixed', block_stride, attention, numverts, vertsize)


def dense(num_heads, num_blocks):
    return torch.ones((num_heads, num_blocks, num_blocks), dtype=torch.int64)


def causal_band(num_heads, num_blocks, band, global_cols=1):
    """Block-row i sees block-columns max(0, i-band+1) .. i and the first
    `global_cols` block-columns."""
    i = torch.arange(num_blocks)[:, None]
    j = torch.arange(num_blocks)[None, :]
    lay = ((j <= i) & (j > i - band)) | (j < global_cols)
    return lay.to(torch.int64)[None].repeat(num_heads, 1, 1)


def bigbird(num_heads, num_blocks, num_random=3, window=3, num_global=2, seed=0):
    """BigBird-style layout: a sliding window of `window` blocks, `num_random`
    random block-columns per block-row (head h drawn from seed + h) and
    `num_global` global block-rows and block-columns."""
    half = window // 2
    i = torch.arange(num_blocks)[:, None]
    j = torch.arange(num_blocks)[None, :]
    base = ((j - i).abs() <= half) | (i < num_global) | (j < num_global)
    out = torch.zeros((num_heads, num_blocks, num_blocks), dtype=torch.int64)
    for h in range(num_heads):
        g = torch.Generator().manual_seed(seed + h)
        lay = base.clone()
        for r in range(num_blocks):
            lay[r, torch.randperm(num_blocks, generator=g)[:num_random]] = True
        out[h] = lay.to(torch.int64)
    return out
