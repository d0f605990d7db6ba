"""Block-sparse drop-in for torch.nn.MultiheadAttention (sequence-first [L, B, E]).

Mirrors torch_blocksparse/attention.py:
  MultiheadAttention(embed_dim, num_heads, layout, block, dropout=0., bias=True,
                     add_bias_kv=False, add_zero_attn=False, kdim=None, vdim=None,
                     key_padding_mask_mode='add', attn_mask_mode='mul')          (attention.py:207-232)
  forward(query, key, value, key_padding_mask=None, need_weights=True, attn_mask=None)
                                                                                 (attention.py:234-265)
  replace_mha(model, info)                                                       (attention.py:267-281)
  make_layout(num_heads, num_blocks, mode, block_stride, unidirectional, numverts, vertsize)
                                                                                 (attention.py:205)

The projections are plain F.linear calls (dense GEMMs, as in the reference); the
attention core between them -- q scaled by head_dim^-1/2, sparse scores, masked
softmax without further scale, product with v (attention.py:127, 190-198) -- runs
in the fused kernel.  As in the reference only self-attention without dropout is
supported and no attention weights are returned.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import tables
from .attention import DeepSpeedSparseSelfAttention


def make_layout(num_heads, num_blocks, mode, block_stride, unidirectional, numverts, vertsize):
    """The reference exports its native generator under this name (attention.py:205)."""
    return tables.make_fixed_layout(num_heads, num_blocks, mode, block_stride,
                                    'unidirectional' if unidirectional else 'bidirectional', numverts, vertsize)


class MultiheadAttention(nn.modules.activation.MultiheadAttention):

    def __init__(self, embed_dim, num_heads, layout, block, dropout=0., bias=True, add_bias_kv=False,
                 add_zero_attn=False, kdim=None, vdim=None, key_padding_mask_mode='add', attn_mask_mode='mul'):
        if dropout != 0:
            raise NotImplementedError('dropout is not supported for now')
        super().__init__(embed_dim, num_heads, dropout, bias, add_bias_kv, add_zero_attn, kdim, vdim)
        if add_bias_kv or add_zero_attn:
            raise NotImplementedError('add_bias_kv / add_zero_attn change the key length and are not supported')
        self.layout = layout
        self.block = block
        self.key_padding_mask_mode = key_padding_mask_mode
        self.attn_mask_mode = attn_mask_mode
        # the core: scores are not scaled again (q is pre-scaled), masks follow the softmax op's modes
        self.core = DeepSpeedSparseSelfAttention(layout=layout, block=block,
                                                 key_padding_mask_mode=key_padding_mask_mode,
                                                 attn_mask_mode=attn_mask_mode)

    def forward(self, query, key, value, key_padding_mask=None, need_weights=True, attn_mask=None):
        if query.shape != key.shape or key.shape != value.shape:
            raise NotImplementedError('only self-attention is supported for now')
        tgt_len, bsz, embed_dim = query.shape
        H = self.num_heads
        head_dim = embed_dim // H
        if self._qkv_same_embed_dim:
            w, b = self.in_proj_weight, self.in_proj_bias
            if (query is key or torch.equal(query, key)) and (key is value or torch.equal(key, value)):
                q, k, v = F.linear(query, w, b).chunk(3, dim=-1)
            else:
                E = embed_dim
                bq, bk, bv = (None, None, None) if b is None else (b[:E], b[E:2 * E], b[2 * E:])
                q = F.linear(query, w[:E], bq)
                k = F.linear(key, w[E:2 * E], bk)
                v = F.linear(value, w[2 * E:], bv)
        else:
            E = embed_dim
            b = self.in_proj_bias
            bq, bk, bv = (None, None, None) if b is None else (b[:E], b[E:2 * E], b[2 * E:])
            q = F.linear(query, self.q_proj_weight, bq)
            k = F.linear(key, self.k_proj_weight, bk)
            v = F.linear(value, self.v_proj_weight, bv)
        q = q * (float(head_dim) ** -0.5)
        # [L, B, E] -> [B, H, L, head_dim] as views: the kernels address their operands through
        # batch / head / row strides, so the projections are used where they lie, and the result
        # is written in [L, B, E] order by the kernel (no transposed copies on the way in or out)
        to_heads = lambda t: t.view(tgt_len, bsz, H, head_dim).permute(1, 2, 0, 3)
        out = self.core.attend(to_heads(q), to_heads(k), to_heads(v), 1.0, None, key_padding_mask, attn_mask,
                               seq_first_out=True)
        out = out.permute(2, 0, 1, 3).reshape(tgt_len, bsz, embed_dim)
        return F.linear(out, self.out_proj.weight, self.out_proj.bias), None


def replace_mha(model, info):
    """Replaces every nn.MultiheadAttention of `model` by the block-sparse module built from
    `info` = (layout, block), copying the parameters (attention.py:267-281)."""
    layout, block = info
    for child_name, child in model.named_children():
        if isinstance(child, nn.modules.activation.MultiheadAttention) and not isinstance(child, MultiheadAttention):
            device = child.in_proj_weight.device if child.in_proj_weight is not None else child.q_proj_weight.device
            mha = MultiheadAttention(child.embed_dim, child.num_heads, layout, block, dropout=child.dropout,
                                     bias=child.in_proj_bias is not None, add_bias_kv=child.bias_k is not None,
                                     add_zero_attn=child.add_zero_attn, kdim=child.kdim, vdim=child.vdim,
                                     key_padding_mask_mode='mul', attn_mask_mode='add').to(device)
            for yparam, xparam in zip(mha.parameters(), child.parameters()):
                yparam.data.copy_(xparam.data)
            setattr(model, child_name, mha)
        else:
            replace_mha(child, info)
