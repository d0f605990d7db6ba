"""Sparse self-attention wrapper with the reference's interface.

Mirrors torch_blocksparse/deepspeedsparseselfattention.py:
  SparsityConfig(mode, block, stride, attention, numverts, vertsize)          (8-26)
  DeepSpeedSparseSelfAttention(sparsity_config, key_padding_mask_mode='add',
                               attn_mask_mode='mul')                          (109-117)
  forward(query, key, value, rpe=None, key_padding_mask=None, attn_mask=None) (135-166)
and is also exported as SparseSelfAttention.

Differences, all additive:
  * an explicit `layout` (with `block`) may be given instead of a SparsityConfig,
    for layouts the config cannot describe (e.g. BigBird-style);
  * the op cache is per instance and keyed on (heads, sequence length), not a
    class-level dict keyed on the length alone (deepspeedsparseselfattention.py:67-106),
    so two modules with different layouts never share tables;
  * `fused=True` (default) computes scores, softmax and the product with V in
    one kernel without storing the score tensor; `fused=False` runs the
    reference's three-op chain sdd -> softmax -> dsd.
"""
import weakref

import torch
import torch.nn as nn

from . import tables
from .matmul import MatMul
from .softmax import Softmax


class SparsityConfig:
    """deepspeedsparseselfattention.py:8-26."""

    def __init__(self, mode='fixed', block=16, stride=64, attention='unidirectional', numverts=1, vertsize=1):
        if mode != 'dense' and mode != 'fixed':
            raise NotImplementedError('only "dense" and "fixed" modes are supported for now')
        self.mode = mode
        self.block = block
        self.stride = stride
        if attention != 'unidirectional' and attention != 'bidirectional':
            raise NotImplementedError('only "uni/bi-directional" attentions are supported for now')
        self.attention = attention
        self.numverts = numverts
        self.vertsize = vertsize


class DeepSpeedSparseSelfAttention(nn.Module):

    @staticmethod
    def _make_layout(num_heads, num_blocks, mode, block_stride, attention, numverts, vertsize):
        """deepspeedsparseselfattention.py:51-65, built natively."""
        return tables.make_fixed_layout(num_heads, num_blocks, mode, block_stride, attention, numverts, vertsize)

    def __init__(self, sparsity_config=None, key_padding_mask_mode='add', attn_mask_mode='mul',
                 layout=None, block=None, fused=True):
        super().__init__()
        if layout is not None:
            if block is None:
                raise ValueError('an explicit layout needs its block size')
            if layout.dim() != 3 or layout.size(1) != layout.size(2):
                raise ValueError('an attention layout must be [heads, L/block, L/block]')
        self.sparsity_config = sparsity_config if sparsity_config is not None else SparsityConfig()
        self.layout = layout
        self.block = block if layout is not None else self.sparsity_config.block
        self.key_padding_mask_mode = key_padding_mask_mode
        self.attn_mask_mode = attn_mask_mode
        self.fused = fused
        self.ops = dict()
        self.tiles = dict()
        self._causal_cache = dict()
        self.causal_checks = 0            # comparisons of a mask against the causal one made so far

    def get_layout(self, H, L):
        """The [H, L/block, L/block] layout used for H heads and sequence length L."""
        block = self.block
        if L % block != 0:
            raise ValueError(f'Sequence length {L} must be dividable by block size {block}')
        if self.layout is not None:
            if self.layout.size(0) != H or self.layout.size(1) * block != L:
                raise ValueError(f'layout {tuple(self.layout.shape)} with block {block} does not fit {H} heads of length {L}')
            return self.layout
        cfg = self.sparsity_config
        if cfg.stride % block != 0:
            raise ValueError(f'Stride {cfg.stride} must be dividable by block size {block}')
        return DeepSpeedSparseSelfAttention._make_layout(H, L // block, cfg.mode, cfg.stride // block,
                                                         cfg.attention, cfg.numverts, cfg.vertsize)

    def get_ops(self, H, L):
        """(sdd_nt, dsd_nn, softmax) for H heads of length L, built once
        (deepspeedsparseselfattention.py:67-106)."""
        key = (H, L)
        if key not in self.ops:
            layout = self.get_layout(H, L)
            sdd_nt = MatMul(layout, self.block, 'sdd', trans_a=False, trans_b=True)
            dsd_nn = MatMul(layout, self.block, 'dsd', trans_a=False, trans_b=False)
            dsd_nn._meta = sdd_nt.meta            # one metadata buffer per layout
            self.ops[key] = (sdd_nt, dsd_nn, Softmax(layout, self.block))
            self.tiles[key] = tables.build_attn_tiles(layout, self.block) if self.fused else None
        return self.ops[key]

    def _is_causal(self, attn_mask, owner=None):
        """True when a 'mul' attention mask is exactly the lower-triangular (causal) mask: the
        fused kernels then derive it from the indices.  The answer is remembered per tensor
        object and version (not per address: a freed tensor's address is reused).  `owner` is
        the tensor the caller handed in when `attn_mask` is a view or a converted copy made from
        it on the way here (forward() squeezes and casts the mask, which creates a new tensor
        object on every call): the answer is then remembered for the caller's tensor.  A caller
        that builds a new mask tensor for every call pays the comparison every time."""
        key = attn_mask if owner is None else owner
        entry = self._causal_cache.get(id(key))
        if entry is not None and entry[0]() is key and entry[1] == key._version:
            return entry[2]
        self.causal_checks += 1
        L = attn_mask.size(-1)
        hit = (attn_mask.dim() == 2 and attn_mask.size(0) == L and
               bool(torch.equal(attn_mask != 0, torch.ones((L, L), dtype=torch.bool, device=attn_mask.device).tril())))
        if len(self._causal_cache) > 16:
            self._causal_cache.clear()
        self._causal_cache[id(key)] = (weakref.ref(key), key._version, hit)
        return hit

    def graphed(self, query, key, value, dout, scale=None):
        """Forward + backward on the given [bsz, heads, L, head_dim] buffers as one CUDA graph (see
        fused.GraphedStep): `step = module.graphed(q, k, v, do)`, then `step.replay()` per step;
        results in step.o, step.dq, step.dk, step.dv.  No rpe / masks."""
        from .fused import GraphedStep
        bsz, num_heads, tgt_len, head_dim = query.size()
        sdd_nt, _, _ = self.get_ops(num_heads, tgt_len)
        tiles = self.tiles.get((num_heads, tgt_len))
        return GraphedStep(sdd_nt.meta, tiles, self.block, float(head_dim) ** -0.5 if scale is None else float(scale),
                           query, key, value, dout)

    def transpose_key_for_scores(self, x, L):
        """deepspeedsparseselfattention.py:119-123: a key given as [.., hd, L] is
        viewed back as [.., L, hd]."""
        bsz, num_heads, seq_len, head_dim = x.size()
        if seq_len != L:
            return x.permute(0, 1, 3, 2)
        return x

    def transpose_mask_for_sparse(self, qtype, x, is_key_padding_mask=False):
        """deepspeedsparseselfattention.py:125-132."""
        x = x.type(qtype)
        if is_key_padding_mask:
            xdim = x.dim()
            for d in range(xdim - 1, 0, -1):
                x = x.squeeze(dim=d)
            return x
        return x.squeeze()

    def forward(self, query, key, value, rpe=None, key_padding_mask=None, attn_mask=None):
        bsz, num_heads, tgt_len, head_dim = query.size()
        key = self.transpose_key_for_scores(key, tgt_len)
        if query.shape != key.shape or key.shape != value.shape:
            raise NotImplementedError('only self-attention is supported for now')
        if key_padding_mask is not None:
            key_padding_mask = self.transpose_mask_for_sparse(query.dtype, key_padding_mask, is_key_padding_mask=True)
            if key_padding_mask.dim() == 1:
                key_padding_mask = key_padding_mask.unsqueeze(0)
        mask_owner = attn_mask
        if attn_mask is not None:
            attn_mask = self.transpose_mask_for_sparse(query.dtype, attn_mask)
        return self.attend(query, key, value, float(head_dim) ** -0.5, rpe, key_padding_mask, attn_mask,
                           mask_owner=mask_owner)

    def attend(self, query, key, value, scaling, rpe=None, key_padding_mask=None, attn_mask=None, mask_owner=None,
               seq_first_out=False):
        """The attention core on [bsz, heads, L, head_dim] operands with an explicit score scale
        (masks already in the dtype of the operands).  `mask_owner`: the caller's own attention
        mask tensor when `attn_mask` was derived from it (see _is_causal).  `seq_first_out`: the
        fused kernel writes its result in [L, bsz, heads * head_dim] memory order (returned as the
        [bsz, heads, L, head_dim] view of it)."""
        bsz, num_heads, tgt_len, head_dim = query.size()
        if key_padding_mask is not None and key_padding_mask.dtype != query.dtype:
            key_padding_mask = key_padding_mask.to(query.dtype)
        if attn_mask is not None and attn_mask.dtype != query.dtype:
            if mask_owner is None:
                mask_owner = attn_mask
            attn_mask = attn_mask.to(query.dtype)
        sdd_nt, dsd_nn, softmax = self.get_ops(num_heads, tgt_len)
        if self.fused:
            from .fused import fused_attention, fused_supported
            if fused_supported(query, self.block):
                am_mode = self.attn_mask_mode
                if attn_mask is not None and am_mode == 'mul' and self._is_causal(attn_mask, mask_owner):
                    am_mode = 'causal'
                return fused_attention(query, key, value, sdd_nt.meta, self.block, scaling, rpe,
                                       key_padding_mask, attn_mask,
                                       self.key_padding_mask_mode, am_mode,
                                       tiles=self.tiles[(num_heads, tgt_len)], seq_first_out=seq_first_out)
        w = sdd_nt(query, key)
        w = softmax(w, scale=scaling, rpe=rpe, key_padding_mask=key_padding_mask, attn_mask=attn_mask,
                    key_padding_mask_mode=self.key_padding_mask_mode, attn_mask_mode=self.attn_mask_mode)
        return dsd_nn(w, value)


SparseSelfAttention = DeepSpeedSparseSelfAttention
