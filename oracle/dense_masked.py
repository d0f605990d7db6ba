"""CPU restatement of the reference's dense-masked definitions of each op (torch, CPU).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file;
only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may.

The reference defines the result of every sparse op as "what dense PyTorch
gives on the densified operands, re-sparsified":
  * block format <-> dense          tests/utils.py:5-25
  * MatMul (sdd / dsd / dds)        tests/test_matmul.py:10-27
  * Softmax                         tests/test_softmax.py:21-34, extended with the
                                    relative-position bias and the 'add'/'mul' mask
                                    modes exactly as the kernel applies them
                                    (torch_blocksparse/softmax.py:104-128)
  * attention chain                 torch_blocksparse/deepspeedsparseselfattention.py:157-166
The Python loops of the reference helpers are replaced by index arithmetic;
tests/golden/ holds outputs of the reference helpers themselves against which
this file is pinned (tests/test_oracle.py).

All arithmetic runs in `compute_dtype` (float32 by default, float64 on request)
on inputs that were first rounded to the op's storage dtype, so the CPU result
does not depend on CPU half-precision matmul behaviour.
"""
import torch


def _nnz(layout):
    nz = (layout != 0).nonzero(as_tuple=False)
    return nz[:, 0], nz[:, 1], nz[:, 2]


def dense_to_sparse(w, layout, block):
    """[Z,H,R,C] -> [Z,nnz,block,block]; block b is the b-th nonzero of `layout`
    in (h,i,j) row-major order (tests/utils.py:5-13)."""
    Z, H, R, C = w.shape
    h, i, j = _nnz(layout)
    t = w.reshape(Z, H, R // block, block, C // block, block).permute(0, 1, 2, 4, 3, 5)
    return t[:, h, i, j].contiguous()


def sparse_to_dense(ws, layout, block, fill=0.0):
    """[Z,nnz,block,block] -> [Z,H,R,C] with `fill` outside the layout."""
    H, Mb, Nb = layout.shape
    Z = ws.shape[0]
    h, i, j = _nnz(layout)
    t = torch.full((Z, H, Mb, Nb, block, block), fill, dtype=ws.dtype)
    t[:, h, i, j] = ws
    return t.permute(0, 1, 2, 4, 3, 5).reshape(Z, H, Mb * block, Nb * block)


def mask_dense(w, layout, block, fill=0.0):
    """Dense tensor with everything outside the layout replaced by `fill`
    (tests/utils.py:16-25)."""
    m = (layout != 0).repeat_interleave(block, 1).repeat_interleave(block, 2)
    return torch.where(m[None], w, torch.full((), fill, dtype=w.dtype))


def matmul_reference(a, b, mode, trans_a, trans_b, layout, block, dc=None,
                     compute_dtype=torch.float32):
    """tests/test_matmul.py:10-27.  `a`/`b`/`dc` are given in the op's own
    formats (block format for the sparse operand).  Returns (c, da, db) in the
    op's formats and in the storage dtype of `a`; da/db are None without `dc`."""
    st = a.dtype
    x = a.detach().to(compute_dtype).clone()
    w = b.detach().to(compute_dtype).clone()
    if mode == 'dsd':
        x = sparse_to_dense(x, layout, block)
    if mode == 'dds':
        w = sparse_to_dense(w, layout, block)
    x.requires_grad_(dc is not None)
    w.requires_grad_(dc is not None)
    xx = x.transpose(2, 3) if trans_a else x
    ww = w.transpose(2, 3) if trans_b else w
    y = torch.matmul(xx, ww)
    if mode == 'sdd':
        y = mask_dense(y, layout, block)
    da = db = None
    if dc is not None:
        g = dc.to(compute_dtype)
        if mode == 'sdd':
            g = sparse_to_dense(g, layout, block)
        y.backward(g)
        da, db = x.grad, w.grad
        if mode == 'dsd':
            da = dense_to_sparse(da, layout, block)
        if mode == 'dds':
            db = dense_to_sparse(db, layout, block)
        da, db = da.to(st), db.to(st)
    y = y.detach()
    if mode == 'sdd':
        y = dense_to_sparse(y, layout, block)
    return y.to(st), da, db


def _mask_term(m, mode):
    """softmax.py:104-110: in 'mul' mode a mask value of 0 becomes -inf and
    anything else 0; in 'add' mode the mask is added as is."""
    if mode == 'mul':
        return torch.where(m == 0, torch.full_like(m, float('-inf')), torch.zeros_like(m))
    return m


def softmax_reference(xs, layout, block, scale=1.0, rpe=None, key_padding_mask=None,
                      attn_mask=None, key_padding_mask_mode='add', attn_mask_mode='add',
                      dy=None, compute_dtype=torch.float32):
    """tests/test_softmax.py:21-34 generalised.  `xs`, `dy` in block format
    [Z,nnz,block,block]; rpe [Z,H,M,N] (or [H,M,N]); key_padding_mask [Z,N];
    attn_mask [M,N].  Order: x*scale + rpe + kpm + attn (softmax.py:112-128).
    Returns (y, dx) in block format in xs.dtype (dx None without dy)."""
    st = xs.dtype
    x = sparse_to_dense(xs.detach().to(compute_dtype), layout, block, fill=float('-inf'))
    x.requires_grad_(dy is not None)
    f = x * scale
    if rpe is not None:
        r = rpe.to(compute_dtype)
        f = f + (r if r.dim() == 4 else r[None])
    if key_padding_mask is not None:
        f = f + _mask_term(key_padding_mask.to(compute_dtype), key_padding_mask_mode)[:, None, None, :]
    if attn_mask is not None:
        f = f + _mask_term(attn_mask.to(compute_dtype), attn_mask_mode)[None, None, :, :]
    y = torch.softmax(f, -1)
    dx = None
    if dy is not None:
        g = sparse_to_dense(dy.to(compute_dtype), layout, block)
        # rows that are entirely outside the layout are NaN in y; they are not
        # part of the block format, keep them out of the backward pass
        valid = (layout != 0).any(-1).repeat_interleave(block, 1)[None, :, :, None]
        torch.where(valid, y, torch.zeros_like(y)).backward(g)
        dx = dense_to_sparse(x.grad, layout, block).to(st)
    return dense_to_sparse(y.detach(), layout, block).to(st), dx


def attention_reference(q, k, v, layout, block, scale, rpe=None, key_padding_mask=None,
                        attn_mask=None, key_padding_mask_mode='add', attn_mask_mode='mul',
                        do=None, compute_dtype=torch.float32):
    """deepspeedsparseselfattention.py:157-166: sdd(q, k^T) -> softmax(scale, rpe,
    masks) -> dsd(p, v), as dense-masked math.  Returns (o, dq, dk, dv)."""
    st = q.dtype
    qq, kk, vv = (t.detach().to(compute_dtype).clone().requires_grad_(do is not None) for t in (q, k, v))
    s = torch.matmul(qq, kk.transpose(2, 3))
    s = mask_dense(s, layout, block, fill=float('-inf'))
    f = s * scale
    if rpe is not None:
        r = rpe.to(compute_dtype)
        f = f + (r if r.dim() == 4 else r[None])
    if key_padding_mask is not None:
        f = f + _mask_term(key_padding_mask.to(compute_dtype), key_padding_mask_mode)[:, None, None, :]
    if attn_mask is not None:
        f = f + _mask_term(attn_mask.to(compute_dtype), attn_mask_mode)[None, None, :, :]
    p = torch.softmax(f, -1)
    # a block-row without any nonzero block contributes nothing: the dsd product
    # zero-fills such rows (matmul.py: zero-length segment of the DSD table)
    valid = (layout != 0).any(-1).repeat_interleave(block, 1)[None, :, :, None]
    p = torch.where(valid, p, torch.zeros_like(p))
    o = torch.matmul(p, vv)
    if do is None:
        return o.detach().to(st), None, None, None
    o.backward(do.to(compute_dtype))
    return o.detach().to(st), qq.grad.to(st), kk.grad.to(st), vv.grad.to(st)
