"""Fused sparse self-attention: scores, softmax and the product with V in one
kernel, with a matching three-kernel backward.

The reference computes the same result with three ops and keeps the score
tensor [Z, nnz, block, block] in memory
(torch_blocksparse/deepspeedsparseselfattention.py:157-166); this path never
materialises it.  rpe and the masks follow the softmax op's conventions
(torch_blocksparse/softmax.py:104-128) and receive no gradient.
"""
import torch

from . import _lib
from .matmul import _dtype_code, _require_cuda, _stream


# When set to a list, every forward / backward appends (name, start_event,
# end_event) triples around each kernel launch (events on the current stream),
# and the backward issues its three kernels as three calls.  Used by the
# benchmark to time each kernel inside a full step; None costs nothing.
PROFILE = None

# Kernel family: 'tc' (tcgen05, tensor memory, TMA; FP16 / BF16, head dimension 64 / 128, layouts
# for which tile lists exist, operands and masks TMA can describe) or 'mma' (mma.sync).  What 'tc'
# does not cover always runs on 'mma'; the library decides per call.
PATH = 'tc'

KERNELS_PER_FWD = 1
KERNELS_PER_BWD = 3


def _timed(name, fn):
    if PROFILE is None:
        return fn()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    out = fn()
    t1.record()
    PROFILE.append((name, t0, t1))
    return out


def fused_supported(q, block):
    return q.dtype in (torch.float16, torch.bfloat16) and q.size(-1) in (64, 128) and block in (16, 32, 64, 128)


def _rows(x):
    """[Z,H,L,D] operand with unit stride on D and 16-byte friendly strides."""
    if x.stride(3) != 1 or x.data_ptr() % 16 or any(s % 8 for s in x.stride()[:3]):
        x = x.contiguous()
    return x


def _mask_args(Z, H, L, dtype, rpe, kpm, am, kp_mode, am_mode):
    """Validates the optional bias / masks and flattens them to C arguments;
    returns (args tuple, tensors to keep alive)."""
    keep = []
    r_ptr, rz, rh, rr = None, 0, 0, 0
    if rpe is not None:
        if rpe.dtype != dtype:
            raise ValueError('relative position embedding must be %s' % dtype)
        if rpe.dim() == 3:
            rpe = rpe.unsqueeze(0)
        if rpe.dim() != 4 or tuple(rpe.shape[1:]) != (H, L, L) or rpe.size(0) not in (1, Z):
            raise ValueError('rpe must be [Z, %d, %d, %d] (got %s)' % (H, L, L, tuple(rpe.shape)))
        if rpe.stride(3) != 1:
            rpe = rpe.contiguous()
        keep.append(rpe)
        r_ptr, rz, rh, rr = rpe.data_ptr(), (0 if rpe.size(0) == 1 else rpe.stride(0)), rpe.stride(1), rpe.stride(2)
    k_ptr, kz = None, 0
    if kpm is not None:
        if kpm.dtype != dtype:
            raise ValueError('Key padding mask must be %s' % dtype)
        if kpm.dim() != 2 or kpm.size(1) != L or kpm.size(0) not in (1, Z):
            raise ValueError('key_padding_mask must be [Z, %d] (got %s)' % (L, tuple(kpm.shape)))
        if kpm.stride(1) != 1:
            kpm = kpm.contiguous()
        keep.append(kpm)
        k_ptr, kz = kpm.data_ptr(), (0 if kpm.size(0) == 1 else kpm.stride(0))
    a_ptr, ar = None, 0
    if am is not None:
        if am.dtype != dtype:
            raise ValueError('Attention mask must be %s' % dtype)
        if am.dim() != 2 or tuple(am.shape) != (L, L):
            raise ValueError('attn_mask must be [%d, %d] (got %s)' % (L, L, tuple(am.shape)))
        if am.stride(1) != 1:
            am = am.contiguous()
        keep.append(am)
        a_ptr, ar = am.data_ptr(), am.stride(0)
    # 'causal' (internal): a 'mul' mask known to be lower triangular; the kernels that can do so
    # derive it from the indices instead of reading it (flag 2), the others read it as 'mul'
    if kp_mode not in ('add', 'mul'):
        raise ValueError("key_padding_mask_mode must be 'add' or 'mul'")
    if am_mode not in ('add', 'mul', 'causal'):
        raise ValueError("attn_mask_mode must be 'add' or 'mul'")
    am_flag = {'add': 0, 'mul': 1, 'causal': 2}[am_mode]
    return (r_ptr, rz, rh, rr, k_ptr, kz, 1 if kp_mode == 'mul' else 0, a_ptr, ar, am_flag), keep


class _fused_attention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, meta, tiles, block, scale, rpe, kpm, am, kp_mode, am_mode, seq_first_out=False):
        _require_cuda(q, k, v)
        Z, H, L, D = q.shape
        q, k, v = _rows(q), _rows(k), _rows(v)
        margs, keep = _mask_args(Z, H, L, q.dtype, rpe, kpm, am, kp_mode, am_mode)
        if seq_first_out:
            # the result in [L, Z, H * D] memory order (what a sequence-first caller reshapes it to
            # anyway), handed to the kernel through its batch / head / row strides: no copy later
            o = torch.empty((L, Z, H, D), dtype=q.dtype, device=q.device).permute(1, 2, 0, 3)
        else:
            o = torch.empty((Z, H, L, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((Z, H, L), dtype=torch.float32, device=q.device)
        _timed('attn_fwd', lambda: _lib.check(_lib.lib().bsp_attn_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
            _dtype_code(q), block, Z, H, L, D,
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
            meta.hdr.data_ptr(), meta.on(q.device).data_ptr(), *_tile_args(tiles, q.device), scale, *margs, _stream(q))))
        ctx.save_for_backward(q, k, v, o, lse, *keep)
        ctx.meta, ctx.tiles, ctx.block, ctx.scale = meta, tiles, block, scale
        ctx.mask_spec = (rpe is not None, kpm is not None, am is not None, kp_mode, am_mode)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors[:5]
        rest = list(ctx.saved_tensors[5:])
        has_rpe, has_kpm, has_am, kp_mode, am_mode = ctx.mask_spec
        rpe = rest.pop(0) if has_rpe else None
        kpm = rest.pop(0) if has_kpm else None
        am = rest.pop(0) if has_am else None
        Z, H, L, D = q.shape
        do = _rows(do)
        margs, _ = _mask_args(Z, H, L, q.dtype, rpe, kpm, am, kp_mode, am_mode)
        dq, dk, dv = (torch.empty((Z, H, L, D), dtype=q.dtype, device=q.device) for _ in range(3))   # the kernels write these densely
        delta = torch.empty((Z, H, L), dtype=torch.float32, device=q.device)
        args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _dtype_code(q), ctx.block, Z, H, L, D,
                q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
                do.stride(0), do.stride(1), do.stride(2),
                ctx.meta.hdr.data_ptr(), ctx.meta.on(q.device).data_ptr(), *_tile_args(ctx.tiles, q.device),
                ctx.scale) + margs
        L_ = _lib.lib()
        if PROFILE is None:
            _lib.check(L_.bsp_attn_bwd(*args, _stream(q)))
        else:
            for name, part in (('attn_bwd_delta', 1), ('attn_bwd_dkdv', 2), ('attn_bwd_dq', 4)):
                _timed(name, lambda part=part: _lib.check(L_.bsp_attn_bwd_parts(*args, part, _stream(q))))
        return (dq, dk, dv) + (None,) * 10


def _tile_args(tiles, device):
    if tiles is None or PATH != 'tc':
        return (None, None)
    return (tiles.hdr.data_ptr(), tiles.on(device).data_ptr())


def device_status():
    """0, or non-zero when a bounded wait inside a tcgen05 kernel expired since the last read
    (synchronises; reading clears the status)."""
    return _lib.device_status()


def fused_attention(q, k, v, meta, block, scale, rpe=None, key_padding_mask=None, attn_mask=None,
                    key_padding_mask_mode='add', attn_mask_mode='mul', tiles=None, seq_first_out=False):
    """O = softmax(scale * Q K^T + rpe + masks, on the layout) V for [Z, H, L, D] operands."""
    if meta.H != q.size(1) or meta.Mb != meta.Nb or meta.Mb * block != q.size(2):
        raise ValueError('layout [%d,%d,%d] with block %d does not fit operands of shape %s'
                         % (meta.H, meta.Mb, meta.Nb, block, tuple(q.shape)))
    return _fused_attention.apply(q, k, v, meta, tiles, block, float(scale), rpe, key_padding_mask, attn_mask,
                                  key_padding_mask_mode, attn_mask_mode, seq_first_out)


class GraphedStep:
    """Forward + backward of the fused attention on fixed buffers, captured once in a CUDA graph
    and replayed with one launch: for steady-state loops whose steps are short enough for the
    launches themselves to matter (a small shard of a problem split over several GPUs).

        step = module.graphed(q, k, v, do)      # q, k, v, do: [Z, H, L, D] device tensors, kept by the caller
        step.replay()                            # reads q, k, v, do as they are now; fills step.o, .dq, .dk, .dv

    No rpe / masks (use the module's forward for those).  The captured work is exactly what
    module(q, k, v) followed by backward(do) launches, the dQ kernel beside the dK / dV kernel
    included; results are bit-identical to that path."""

    def __init__(self, meta, tiles, block, scale, q, k, v, do):
        _require_cuda(q, k, v, do)
        if not fused_supported(q, block):
            raise NotImplementedError('graphed step: FP16 / BF16 operands with head dimension 64 or 128')
        self.q, self.k, self.v, self.do = (_rows(t) for t in (q, k, v, do))
        for a, b in zip((self.q, self.k, self.v, self.do), (q, k, v, do)):
            if a is not b:
                raise ValueError('graphed step: operands need unit stride on the last dimension, 16-byte alignment and '
                                 'strides that are multiples of 8 elements')
        Z, H, L, D = q.shape
        dev = q.device
        self.o, self.dq, self.dk, self.dv = (torch.empty((Z, H, L, D), dtype=q.dtype, device=dev) for _ in range(4))
        self.lse = torch.empty((Z, H, L), dtype=torch.float32, device=dev)
        self.delta = torch.empty((Z, H, L), dtype=torch.float32, device=dev)
        self._keep = (meta, tiles)
        L_ = _lib.lib()
        code = _dtype_code(q)
        st3 = lambda t: (t.stride(0), t.stride(1), t.stride(2))
        none_masks = (None, 0, 0, 0, None, 0, 0, None, 0, 0)
        tile_args = _tile_args(tiles, dev)
        meta_args = (meta.hdr.data_ptr(), meta.on(dev).data_ptr())

        def launch():
            stream = torch.cuda.current_stream(dev).cuda_stream
            _lib.check(L_.bsp_attn_fwd(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.o.data_ptr(), self.lse.data_ptr(),
                code, block, Z, H, L, D, *st3(self.q), *st3(self.k), *st3(self.v), *st3(self.o),
                *meta_args, *tile_args, scale, *none_masks, stream))
            _lib.check(L_.bsp_attn_bwd(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.o.data_ptr(), self.do.data_ptr(),
                self.lse.data_ptr(), self.delta.data_ptr(), self.dq.data_ptr(), self.dk.data_ptr(), self.dv.data_ptr(),
                code, block, Z, H, L, D, *st3(self.q), *st3(self.k), *st3(self.v), *st3(self.o), *st3(self.do),
                *meta_args, *tile_args, scale, *none_masks, stream))

        with torch.cuda.device(dev):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):          # once eagerly: tensor maps, second stream and kernel attributes exist
                launch()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                launch()

    def replay(self):
        self.graph.replay()
        return self.o
