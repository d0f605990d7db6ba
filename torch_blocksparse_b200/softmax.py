"""Block-sparse softmax with the reference's Python interface.

Mirrors torch_blocksparse/softmax.py:
  Softmax(layout, block, bench=False)                                  (softmax.py:338-343)
  Softmax.__call__(x, scale=1., rpe=None, key_padding_mask=None, attn_mask=None,
                   key_padding_mask_mode='add', attn_mask_mode='add')  (softmax.py:345-361)
  _sparse_softmax: autograd function                                   (softmax.py:197-326)

Semantics kept from the reference: the result overwrites `x` and `x` itself
is returned (softmax.py:301,313); the backward overwrites the incoming
gradient and returns it (softmax.py:325-326); rpe and the masks receive no
gradient; masks in 'mul' mode turn 0 into -inf and anything else into 0.
rpe is addressed as [Z, H, M, N] (softmax.py:50-55); a 3-D [H, M, N] tensor is
accepted as well and broadcast over the batch.
"""
import torch

from . import _lib, tables
from .matmul import _Timer, _dtype_code, _require_cuda, _stream


def _inner_contiguous(x, block):
    return x.stride(3) == 1 and x.stride(2) == block and x.stride(1) == block * block \
        and x.data_ptr() % 16 == 0 and (x.size(0) == 1 or x.stride(0) % (16 // x.element_size()) == 0)


class _sparse_softmax(torch.autograd.Function):

    @staticmethod
    def make_lut(layout, block, device):
        """softmax.py:201-221: returns (lut, maxlut).  A layout in device memory gets its table
        there (from the metadata built on the device), without a copy to the host."""
        if layout.is_cuda and torch.device(device).type == 'cuda':
            return tables.make_softmax_lut_device(layout, device)
        return tables.make_softmax_lut(layout, device)

    @staticmethod
    def forward(ctx, x, scale, rpe, key_padding_mask, attn_mask, kp_mask_mode, attn_mask_mode,
                spdims, block, lut, maxlut, bench, time):
        _require_cuda(x)
        if maxlut * block >= 32768:
            raise NotImplementedError('Reductions larger than 32768 elements are not yet implemented')
        if x.dim() != 4 or x.size(2) != block or x.size(3) != block or x.size(1) * 4 + 2 * spdims[0] * spdims[1] != lut.numel():
            raise ValueError('x of shape %s is not a block-format tensor for this layout' % (tuple(x.shape),))
        H, Mb, Nb = spdims
        M, N = Mb * block, Nb * block
        Z = x.size(0)
        work = x if _inner_contiguous(x, block) else x.contiguous()

        rpe_ptr, rz, rh, rr = None, 0, 0, 0
        if rpe is not None:
            if rpe.dim() == 3:
                rpe = rpe.unsqueeze(0).expand(Z, -1, -1, -1)
            if rpe.dim() != 4 or rpe.size(1) != H or rpe.size(2) != M or rpe.size(3) != N or rpe.size(0) not in (1, Z):
                raise ValueError('rpe must be [Z, H, %d, %d] (got %s)' % (M, N, tuple(rpe.shape)))
            if rpe.stride(3) != 1 and rpe.size(3) != 1:
                rpe = rpe.contiguous()
            rpe_ptr = rpe.data_ptr()
            rz, rh, rr = (0 if rpe.size(0) == 1 else rpe.stride(0)), rpe.stride(1), rpe.stride(2)
        kpm_ptr, kz = None, 0
        if key_padding_mask is not None:
            if key_padding_mask.dim() != 2 or key_padding_mask.size(1) != N or key_padding_mask.size(0) not in (1, Z):
                raise ValueError('key_padding_mask must be [Z, %d] (got %s)' % (N, tuple(key_padding_mask.shape)))
            if key_padding_mask.stride(1) != 1:
                key_padding_mask = key_padding_mask.contiguous()
            kpm_ptr = key_padding_mask.data_ptr()
            kz = 0 if key_padding_mask.size(0) == 1 else key_padding_mask.stride(0)
        am_ptr, ar = None, 0
        if attn_mask is not None:
            if attn_mask.dim() != 2 or attn_mask.size(0) != M or attn_mask.size(1) != N:
                raise ValueError('attn_mask must be [%d, %d] (got %s)' % (M, N, tuple(attn_mask.shape)))
            if attn_mask.stride(1) != 1:
                attn_mask = attn_mask.contiguous()
            am_ptr = attn_mask.data_ptr()
            ar = attn_mask.stride(0)
        for name, mode in (('key_padding_mask_mode', kp_mask_mode), ('attn_mask_mode', attn_mask_mode)):
            if mode not in ('add', 'mul'):
                raise ValueError("%s must be 'add' or 'mul'" % name)

        with _Timer(bench, None, time):
            _lib.check(_lib.lib().bsp_softmax_fwd(
                work.data_ptr(), _dtype_code(x), Z, work.stride(0), block, H, Mb, lut.data_ptr(), maxlut, float(scale),
                rpe_ptr, rz, rh, rr, kpm_ptr, kz, 1 if kp_mask_mode == 'mul' else 0,
                am_ptr, ar, 1 if attn_mask_mode == 'mul' else 0, _stream(x)))
        if work is not x:
            x.copy_(work)
        ctx.mark_dirty(x)
        ctx.save_for_backward(x, lut)
        ctx.spdims, ctx.block, ctx.maxlut, ctx.scale = spdims, block, maxlut, float(scale)
        return x

    @staticmethod
    def backward(ctx, dx):
        y, lut = ctx.saved_tensors
        block = ctx.block
        H, Mb, _ = ctx.spdims
        if not _inner_contiguous(dx, block):
            dx = dx.contiguous()
        yy = y if _inner_contiguous(y, block) else y.contiguous()
        _lib.check(_lib.lib().bsp_softmax_bwd(
            yy.data_ptr(), dx.data_ptr(), _dtype_code(y), y.size(0), yy.stride(0), dx.stride(0),
            block, H, Mb, lut.data_ptr(), ctx.maxlut, ctx.scale, _stream(y)))
        return (dx,) + (None,) * 12


class Softmax:

    sparse_softmax = _sparse_softmax.apply

    def make_lut(self, device):
        """Table cache per device (softmax.py:332-336)."""
        key = (device, )
        if key not in self.lut_cache:
            # (one table per layout content and device for the whole process: ops on the same layout share it)
            self.lut_cache[key] = tables._cached('softmax_lut', self.layout, (str(device),),
                                                 lambda: _sparse_softmax.make_lut(self.layout, self.block, device))
        return self.lut_cache[key]

    def __init__(self, layout, block, bench=False):
        self.spdims = layout.shape
        self.layout = layout
        self.block = block
        self.bench = bench
        self.lut_cache = dict()
        self.time_y = None

    def __call__(self, x, scale=1., rpe=None, key_padding_mask=None, attn_mask=None,
                 key_padding_mask_mode='add', attn_mask_mode='add'):
        time_y = [None]
        if rpe is not None and rpe.dtype != x.dtype:
            raise ValueError('relative position embedding must be %s' % x.dtype)
        if attn_mask is not None and attn_mask.dtype != x.dtype:
            raise ValueError('Attention mask must be %s' % x.dtype)
        if key_padding_mask is not None and key_padding_mask.dtype != x.dtype:
            raise ValueError('Key padding mask must be %s' % x.dtype)
        lut, maxlut = self.make_lut(x.device)
        x = Softmax.sparse_softmax(x, scale, rpe, key_padding_mask, attn_mask,
                                   key_padding_mask_mode, attn_mask_mode,
                                   self.spdims, self.block, lut, maxlut, self.bench, time_y)
        self.time_y = time_y[0]
        return x
