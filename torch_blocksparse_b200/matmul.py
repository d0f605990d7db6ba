"""Block-sparse matrix multiplication with the reference's Python interface.

Mirrors torch_blocksparse/matmul.py:
  MatMul(layout, block, mode, trans_a=False, trans_b=False, bench=False)   (matmul.py:643-659)
  MatMul.__call__(a, b)                                                    (matmul.py:670-690)
  MatMul.make_lut(dtype, device)                                           (matmul.py:611-641)
  _sparse_matmul: autograd function with the mode algebra of the backward  (matmul.py:558-606)

mode 'sdd': sparse = op(a) @ op(b);  'dsd': dense = op(a_sparse) @ op(b);
'dds': dense = op(a) @ op(b_sparse).  Dense tensors are [Z, H, rows, cols],
sparse ones [Z, nnz, block, block] in layout.nonzero() order.

All arithmetic runs in the native CUDA library; there is no other code path.
"""
import math

import torch

from . import _lib, tables

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _dtype_code(t):
    if t.dtype not in _DTYPES:
        raise ValueError('unsupported dtype %s (float32, float16 and bfloat16 are)' % t.dtype)
    return _DTYPES[t.dtype]


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError('torch_blocksparse_b200 runs on CUDA tensors only (got a %s tensor)' % t.device)


def _prep_dense(x):
    """Returns a view/copy of a [Z,H,R,C] operand the kernels can address: one
    unit inner stride, every other stride a multiple of 16 bytes, aligned base."""
    vec = 16 // x.element_size()
    s = list(x.stride())
    for d in range(4):           # strides of size-1 dimensions carry no meaning
        if x.size(d) == 1:
            s[d] = 0 if d < 2 else (1 if d == 3 else x.size(3))
    ok = (s[3] == 1 or s[2] == 1)
    if ok:
        other = s[2] if s[3] == 1 else s[3]
        ok = s[0] % vec == 0 and s[1] % vec == 0 and (other == 1 or other % vec == 0) and x.data_ptr() % 16 == 0
    if not ok:
        x = x.contiguous()
        s = list(x.stride())
    return x, s


def _prep_sparse(x, block):
    if x.stride(3) != 1 or x.stride(2) != block or x.stride(1) != block * block or x.data_ptr() % 16 or \
            (x.size(0) > 1 and x.stride(0) % (16 // x.element_size())):
        x = x.contiguous()
    return x


class _Timer:
    """CUDA-event timing of one launch when bench=True (seconds)."""

    def __init__(self, enabled, ref, slot):
        self.enabled, self.ref, self.slot = enabled, ref, slot

    def __enter__(self):
        if self.enabled:
            self.t0 = torch.cuda.Event(enable_timing=True)
            self.t1 = torch.cuda.Event(enable_timing=True)
            self.t0.record()
        return self

    def __exit__(self, *exc):
        if self.enabled and exc[0] is None:
            self.t1.record()
            self.t1.synchronize()
            self.slot[0] = self.t0.elapsed_time(self.t1) * 1e-3
            _lib.check_device()              # this path synchronises anyway: a bounded wait that expired raises here
        return False


class _sparse_matmul(torch.autograd.Function):

    # ---- table builders, same names and results as the reference's ----------
    @staticmethod
    def make_sdd_lut(layout, block, dtype, device):
        """matmul.py:281-297."""
        return tables.make_sdd_lut(layout, block, device)

    @staticmethod
    def make_dxx_lut(layout, block, step, trans, device, transform=None):
        """matmul.py:372-458 (`transform` other than identity is not supported)."""
        if transform is not None:
            raise NotImplementedError('make_dxx_lut: only the identity transform is supported')
        return tables.make_dxx_lut(layout, block, step, trans, device)

    # ---- the three products ------------------------------------------------
    @staticmethod
    def _sdd_matmul(a, b, trans_a, trans_b, trans_c, spdims, block, meta, bench, time):
        """matmul.py:299-364."""
        if trans_c:
            a, b = b, a
            trans_a, trans_b = not trans_b, not trans_a
        a, sa = _prep_dense(a)
        b, sb = _prep_dense(b)
        K = a.size(2 if trans_a else 3)
        if K % 16 != 0:
            raise ValueError('Reduction size for SDD must be a multiple of 16')
        Z = a.size(0)
        M, N = a.size(3 if trans_a else 2), b.size(2 if trans_b else 3)
        if (b.size(0), b.size(1)) != (Z, a.size(1)) or a.size(1) != spdims[0] or b.size(3 if trans_b else 2) != K \
                or M != spdims[1] * block or N != spdims[2] * block:
            raise ValueError('sdd: operand shapes %s, %s do not match layout %s with block %d'
                             % (tuple(a.shape), tuple(b.shape), tuple(spdims), block))
        a_sm, a_sk = (sa[3], sa[2]) if trans_a else (sa[2], sa[3])
        b_sk, b_sn = (sb[3], sb[2]) if trans_b else (sb[2], sb[3])
        c = torch.empty((Z, meta.nnz, block, block), dtype=a.dtype, device=a.device)
        with _Timer(bench, None, time):
            _lib.check(_lib.lib().bsp_sdd(
                a.data_ptr(), b.data_ptr(), c.data_ptr(), _dtype_code(a), block, Z, a.size(1), K,
                sa[0], sa[1], a_sm, a_sk, sb[0], sb[1], b_sk, b_sn, c.stride(0),
                meta.hdr.data_ptr(), meta.on(a.device).data_ptr(), _stream(a)))
        return c

    @staticmethod
    def _dsd_matmul(a, b, trans_a, trans_b, trans_c, spdims, block, meta, bench, time):
        """matmul.py:507-552."""
        a = _prep_sparse(a, block)
        # the kernels read the dense operand in 16-byte pieces along its free dimension: a width that
        # is not a multiple of 8 (4 for FP32) is padded with zero columns, which are cut off again
        n_dim = 2 if trans_b else 3
        pad = (-b.size(n_dim)) % (4 if b.dtype == torch.float32 else 8)
        if pad:
            b = torch.nn.functional.pad(b, (0, pad) if n_dim == 3 else (0, 0, 0, pad))
        b, sb = _prep_dense(b)
        Z, H = b.size(0), b.size(1)
        M = block * spdims[2 if trans_a else 1]
        N = b.size(2 if trans_b else 3)
        if tuple(a.shape) != (Z, meta.nnz, block, block) or H != spdims[0] \
                or b.size(3 if trans_b else 2) != block * spdims[1 if trans_a else 2]:
            raise ValueError('dsd: operand shapes %s, %s do not match layout %s with block %d'
                             % (tuple(a.shape), tuple(b.shape), tuple(spdims), block))
        b_sk, b_sn = (sb[3], sb[2]) if trans_b else (sb[2], sb[3])
        c = torch.empty((Z, H, N, M) if trans_c else (Z, H, M, N), dtype=a.dtype, device=a.device)
        c_sm, c_sn = (c.stride(3), c.stride(2)) if trans_c else (c.stride(2), c.stride(3))
        with _Timer(bench, None, time):
            _lib.check(_lib.lib().bsp_dsd(
                a.data_ptr(), b.data_ptr(), c.data_ptr(), _dtype_code(a), block, Z, H, N,
                a.stride(0), 1 if trans_a else 0, sb[0], sb[1], b_sk, b_sn,
                c.stride(0), c.stride(1), c_sm, c_sn,
                meta.hdr.data_ptr(), meta.on(b.device).data_ptr(), _stream(b)))
        if pad:
            c = c[:, :, :N - pad] if trans_c else c[:, :, :, :N - pad]
        return c

    @staticmethod
    def _dds_matmul(a, b, trans_a, trans_b, trans_c, spdims, block, meta, bench, time):
        """matmul.py:460-505."""
        m_dim = 3 if trans_a else 2                      # (see _dsd_matmul: zero rows up to a multiple of 8 / 4)
        pad = (-a.size(m_dim)) % (4 if a.dtype == torch.float32 else 8)
        if pad:
            a = torch.nn.functional.pad(a, (0, pad) if m_dim == 3 else (0, 0, 0, pad))
        a, sa = _prep_dense(a)
        b = _prep_sparse(b, block)
        Z, H = a.size(0), a.size(1)
        M = a.size(3 if trans_a else 2)
        N = block * spdims[1 if trans_b else 2]
        if tuple(b.shape) != (Z, meta.nnz, block, block) or H != spdims[0] \
                or a.size(2 if trans_a else 3) != block * spdims[2 if trans_b else 1]:
            raise ValueError('dds: operand shapes %s, %s do not match layout %s with block %d'
                             % (tuple(a.shape), tuple(b.shape), tuple(spdims), block))
        a_sm, a_sk = (sa[3], sa[2]) if trans_a else (sa[2], sa[3])
        c = torch.empty((Z, H, N, M) if trans_c else (Z, H, M, N), dtype=a.dtype, device=a.device)
        c_sm, c_sn = (c.stride(3), c.stride(2)) if trans_c else (c.stride(2), c.stride(3))
        with _Timer(bench, None, time):
            _lib.check(_lib.lib().bsp_dds(
                a.data_ptr(), b.data_ptr(), c.data_ptr(), _dtype_code(a), block, Z, H, M,
                sa[0], sa[1], a_sm, a_sk, b.stride(0), 1 if trans_b else 0,
                c.stride(0), c.stride(1), c_sm, c_sn,
                meta.hdr.data_ptr(), meta.on(a.device).data_ptr(), _stream(a)))
        if pad:
            c = c[:, :, :, :M - pad] if trans_c else c[:, :, :M - pad]
        return c

    fn = {'sdd': _sdd_matmul.__get__(object),
          'dsd': _dsd_matmul.__get__(object),
          'dds': _dds_matmul.__get__(object)}

    @staticmethod
    def forward(ctx, a, b, trans_a, trans_b, trans_c, mode, spdims, block, meta,
                c_bench, c_time, da_bench, da_time, db_bench, db_time):
        _require_cuda(a, b)
        if a.dtype != b.dtype:
            raise ValueError('operands must have the same dtype (got %s and %s)' % (a.dtype, b.dtype))
        c = _sparse_matmul.fn[mode](a, b, trans_a, trans_b, trans_c, spdims, block, meta, c_bench, c_time)
        ctx.save_for_backward(a, b)
        ctx.meta = meta
        ctx.da_bench, ctx.da_time = da_bench, da_time
        ctx.db_bench, ctx.db_time = db_bench, db_time
        ctx.mode, ctx.spdims, ctx.block = mode, spdims, block
        ctx.trans_a, ctx.trans_b = trans_a, trans_b
        return c

    @staticmethod
    def backward(ctx, dc):
        """matmul.py:587-606: da through mode[1]+mode[0]+mode[2], db through
        mode[2]+mode[1]+mode[0]."""
        a, b = ctx.saved_tensors
        mode = ctx.mode
        da = db = None
        if ctx.needs_input_grad[0]:
            mode_da = mode[1] + mode[0] + mode[2]
            da = _sparse_matmul.fn[mode_da](dc, b, False, not ctx.trans_b, ctx.trans_a, ctx.spdims, ctx.block,
                                            ctx.meta, ctx.da_bench, ctx.da_time)
        if ctx.needs_input_grad[1]:
            mode_db = mode[2] + mode[1] + mode[0]
            db = _sparse_matmul.fn[mode_db](a, dc, not ctx.trans_a, False, ctx.trans_b, ctx.spdims, ctx.block,
                                            ctx.meta, ctx.db_bench, ctx.db_time)
        return (da, db) + (None,) * 13


class MatMul:

    def make_lut(self, dtype, device):
        """The reference-format tables for c, da and db (matmul.py:611-641), cached
        per (dtype, device):
        (c_lut, c_num_locks, c_width, c_packs, da_..., db_...)."""
        key = (dtype, device)
        if key in self.lut_cache:
            return self.lut_cache[key]
        layout, block = self.layout, self.block
        step = 8 if dtype == torch.float32 else 16
        sdd = lambda: tables.make_sdd_lut(layout, block, device)
        dxx = lambda trans: tables.make_dxx_lut(layout, block, step, trans, device)
        if self.mode == 'sdd':
            c, da, db = sdd(), dxx(True), dxx(False)
        elif self.mode == 'dsd':
            c, da, db = dxx(not self.trans_a), sdd(), dxx(self.trans_a)
        else:
            c, da, db = dxx(self.trans_b), dxx(not self.trans_b), sdd()
        self.lut_cache[key] = tuple(c) + tuple(da) + tuple(db)
        return self.lut_cache[key]

    def __init__(self, layout, block, mode, trans_a=False, trans_b=False, bench=False):
        if mode not in ['sdd', 'dsd', 'dds']:
            raise NotImplementedError('Supported modes are: sdd, dsd, dds')
        self.lut_cache = dict()
        self.trans_a = trans_a
        self.trans_b = trans_b
        self.mode = mode
        self.spdims = layout.shape
        self.block = block
        self.layout = layout
        self.bench = bench
        self.time_c = None
        self.time_da = None
        self.time_db = None
        self._meta = None

    @property
    def meta(self):
        """Execution metadata of the layout (built on first use)."""
        if self._meta is None:
            self._meta = tables.build_meta(self.layout)
        return self._meta

    @staticmethod
    def _pad_shape(x, is_sparse):
        """matmul.py:663-668."""
        max_dim = 3 if is_sparse else 4
        for _ in range(max_dim - x.dim()):
            x = x.unsqueeze(0)
        return x

    def __call__(self, a, b):
        time_c, time_da, time_db = [None], [None], [None]
        a = MatMul._pad_shape(a, self.mode == 'dsd')
        b = MatMul._pad_shape(b, self.mode == 'dds')
        if self.mode == 'dsd' and a.dim() == 3:
            a = a.unsqueeze(0)
        if self.mode == 'dds' and b.dim() == 3:
            b = b.unsqueeze(0)
        c = _sparse_matmul.apply(a, b, self.trans_a, self.trans_b, False,
                                 self.mode, self.spdims, self.block, self.meta,
                                 self.bench, time_c, self.bench, time_da, self.bench, time_db)
        self.time_c = time_c[0]
        self.time_da = time_da[0]
        self.time_db = time_db[0]
        return c


class Linear(torch.nn.Module):
    """y = x . W with a block-sparse weight (torch_blocksparse/matmul.py:693-709).

    The reference's class cannot be constructed: it calls MatMul with its
    arguments in the wrong order (matmul.py:702).  This is the layer it
    describes: `weight` holds the nonzero blocks of an [in_features,
    out_features] matrix as [nnz, block, block] (Kaiming-uniform, as the
    reference initialises it), `layout` is [in_features / block, out_features /
    block] (a leading singleton head dimension is accepted), and forward is the
    'dds' product.  Inputs of any rank [..., in_features] are flattened to rows.
    There is no bias, as in the reference.
    """

    def __init__(self, in_features, out_features, block, layout, bench=False):
        super().__init__()
        if layout.dim() == 2:
            layout = layout.unsqueeze(0)
        if layout.dim() != 3 or layout.size(0) != 1:
            raise ValueError('Linear: layout must be [in_features / block, out_features / block]')
        if in_features % block or out_features % block:
            raise ValueError('Linear: in_features and out_features must be multiples of block %d' % block)
        if tuple(layout.shape[1:]) != (in_features // block, out_features // block):
            raise ValueError('Linear: layout %s does not fit %d x %d features with block %d'
                             % (tuple(layout.shape[1:]), in_features, out_features, block))
        self.in_features = in_features
        self.out_features = out_features
        self.block = block
        self.weight = torch.nn.Parameter(torch.empty(int(layout.sum()), block, block))
        self.reset_parameters()
        self.matmul = MatMul(layout, block, 'dds', trans_a=False, trans_b=False, bench=bench)

    def reset_parameters(self):
        torch.nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, input):
        if input.size(-1) != self.in_features:
            raise ValueError('Linear: expected %d input features, got %d' % (self.in_features, input.size(-1)))
        lead = input.shape[:-1]
        x = input.reshape(1, 1, -1, self.in_features)
        # rows are the reduction dimension of the weight gradient (an sdd product), which must be
        # a multiple of 16 (matmul.py:318-319); zero rows change nothing
        pad = (-x.size(2)) % 16
        if pad:
            x = torch.nn.functional.pad(x, (0, 0, 0, pad))
        y = self.matmul(x, self.weight.to(x.dtype))
        if pad:
            y = y[:, :, :y.size(2) - pad]
        return y.reshape(*lead, self.out_features)
