"""Layout -> table builders (Python face of the native builders in csrc/lut.cpp).

Every function takes the layout as an integer CPU tensor [H, Mb, Nb] (never
modified) and returns int32 tensors whose contents are bit-identical to what
the reference's builders return:
  make_sdd_lut      torch_blocksparse/matmul.py:281-297 (+ csrc/utils.cpp:11-120)
  make_dxx_lut      torch_blocksparse/matmul.py:372-458 (+ load_balance 221-267)
  make_softmax_lut  torch_blocksparse/softmax.py:201-221
  make_fixed_layout torch_blocksparse/deepspeedsparseselfattention.py:33-65
`build_meta` produces the CSR/CSC execution metadata the kernels read.
"""
import ctypes

import torch

from . import _lib


def _layout_i64(layout):
    if layout.dim() != 3:
        raise ValueError('layout must be a [H, Mb, Nb] tensor')
    lay = layout.detach().to(device='cpu', dtype=torch.int64).contiguous()
    return lay, lay.shape[0], lay.shape[1], lay.shape[2]


def _two_pass(call):
    """Runs a native builder twice: size query, then fill.  `call(ptr, cap, total)`
    returns the status."""
    total = ctypes.c_int64(0)
    _lib.check(call(None, 0, ctypes.byref(total)))
    out = torch.empty(max(total.value, 1), dtype=torch.int32)
    _lib.check(call(out.data_ptr(), out.numel(), ctypes.byref(total)))
    return out[:total.value]


def make_sdd_lut(layout, block, device='cpu'):
    """Returns (luts, None, widths, packs) as the reference does: one int32
    table [h,i,j,b, ...] per pack size, the number of super-blocks of each and
    the pack sizes, in decreasing pack order."""
    lay, H, Mb, Nb = _layout_i64(layout)
    L = _lib.lib()
    packs = (ctypes.c_int32 * _lib.MAX_PACKS)()
    widths = (ctypes.c_int64 * _lib.MAX_PACKS)()
    offsets = (ctypes.c_int64 * _lib.MAX_PACKS)()
    n_packs = ctypes.c_int(0)

    def call(ptr, cap, total):
        return L.bsp_sdd_lut_build(lay.data_ptr(), H, Mb, Nb, block, ptr, cap,
                                   packs, widths, offsets, ctypes.byref(n_packs), total)

    flat = _two_pass(call)
    luts, ws, ps = [], [], []
    for p in range(n_packs.value):
        n = widths[p] * packs[p] * packs[p] * 4
        luts.append(flat[offsets[p]:offsets[p] + n].clone().to(device))
        ws.append(int(widths[p]))
        ps.append(int(packs[p]))
    return luts, None, ws, ps


def make_dxx_lut(layout, block, step, trans, device='cpu'):
    """Returns (lut, num_locks, width, None) as the reference does."""
    lay, H, Mb, Nb = _layout_i64(layout)
    L = _lib.lib()
    num_locks = ctypes.c_int(0)
    width = ctypes.c_int(0)

    def call(ptr, cap, total):
        return L.bsp_dxx_lut_build(lay.data_ptr(), H, Mb, Nb, block, step, 1 if trans else 0,
                                   ptr, cap, total, ctypes.byref(num_locks), ctypes.byref(width))

    lut = _two_pass(call)
    return lut.to(device), int(num_locks.value), int(width.value), None


def make_softmax_lut(layout, device='cpu'):
    """Returns (lut, maxlut) as the reference does."""
    lay, H, Mb, Nb = _layout_i64(layout)
    L = _lib.lib()
    maxlut = ctypes.c_int(0)

    def call(ptr, cap, total):
        return L.bsp_softmax_lut_build(lay.data_ptr(), H, Mb, Nb, ptr, cap, total, ctypes.byref(maxlut))

    lut = _two_pass(call)
    return lut.to(device), int(maxlut.value)


def make_fixed_layout(num_heads, num_blocks, mode, block_stride, attention, numverts, vertsize):
    """'dense' or 'fixed' layout as an int64 tensor [num_heads, num_blocks, num_blocks]."""
    if mode not in ('dense', 'fixed'):
        raise NotImplementedError('only "dense" and "fixed" modes are supported for now')
    if attention not in ('unidirectional', 'bidirectional'):
        raise NotImplementedError('only "uni/bi-directional" attentions are supported for now')
    out = torch.empty((num_heads, num_blocks, num_blocks), dtype=torch.int64)
    _lib.check(_lib.lib().bsp_fixed_layout_build(num_heads, num_blocks, 0 if mode == 'dense' else 1,
                                                 block_stride, 1 if attention == 'unidirectional' else 0,
                                                 numverts, vertsize, out.data_ptr()))
    return out


class Meta:
    """Execution metadata of one layout: host header + device buffer."""

    def __init__(self, host):
        self.host = host                      # int32 CPU tensor (whole buffer)
        self.hdr = host[:_lib.META_HEADER].clone()
        self.H, self.Mb, self.Nb, self.nnz = (int(v) for v in host[1:5])
        self.max_row, self.max_col = int(host[5]), int(host[6])
        self._dev = {}

    def on(self, device):
        key = str(device)
        if key not in self._dev:
            self._dev[key] = self.host.to(device)
        return self._dev[key]


def build_meta(layout):
    lay, H, Mb, Nb = _layout_i64(layout)
    L = _lib.lib()

    def call(ptr, cap, total):
        return L.bsp_meta_build(lay.data_ptr(), H, Mb, Nb, ptr, cap, total)

    return Meta(_two_pass(call).clone())


class AttnTiles:
    """Tile lists of the tcgen05 attention kernels: host header + device buffer."""

    def __init__(self, host):
        self.host = host
        self.hdr = host[:8].clone()
        self._dev = {}

    def on(self, device):
        key = str(device)
        if key not in self._dev:
            self._dev[key] = self.host.to(device)
        return self._dev[key]


def build_attn_tiles(layout, block):
    """Returns the AttnTiles of a square [H, nb, nb] layout, or None when the
    tcgen05 kernels do not cover it (blocks 64 and 128, and blocks 16 / 32 whose count per side is a multiple of 4 / 2, are covered)."""
    lay, H, Mb, Nb = _layout_i64(layout)
    if Mb != Nb or block not in (16, 32, 64, 128) or (block < 64 and Mb % (64 // block)):
        return None
    L = _lib.lib()

    def call(ptr, cap, total):
        return L.bsp_attn_tiles_build(lay.data_ptr(), H, Mb, block, ptr, cap, total)

    return AttnTiles(_two_pass(call).clone())
