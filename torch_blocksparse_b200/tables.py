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
import collections
import ctypes
import hashlib
import os

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


def make_softmax_lut_device(layout, device=None):
    """(lut, maxlut) for a layout that lives in device memory: the table is written by a kernel from
    the metadata built on that device, nothing but the metadata's 8-int header visits the host.
    Bit-identical to make_softmax_lut."""
    meta = build_meta(layout)
    device = layout.device if device is None else torch.device(device)
    dev = meta.on(device)
    L = _lib.lib()
    total, maxlut = ctypes.c_int64(0), ctypes.c_int(0)
    _lib.check(L.bsp_softmax_lut_from_meta(meta.hdr.data_ptr(), dev.data_ptr(), None, 0, ctypes.byref(total),
                                           ctypes.byref(maxlut), None))
    with torch.cuda.device(device):
        out = torch.empty(int(total.value), dtype=torch.int32, device=device)
        _lib.check(L.bsp_softmax_lut_from_meta(meta.hdr.data_ptr(), dev.data_ptr(), out.data_ptr(), out.numel(),
                                               ctypes.byref(total), ctypes.byref(maxlut),
                                               torch.cuda.current_stream(device).cuda_stream))
    return out, int(maxlut.value)


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


# ---------------------------------------------------------------------------------------------
# Process-wide cache of the execution metadata and the attention tile lists, keyed by the
# layout's content: ops built on one layout share one buffer, a changed layout is rebuilt.
# ---------------------------------------------------------------------------------------------
_CACHE = collections.OrderedDict()
_CACHE_ENTRIES = 64
CACHE_STATS = {'hits': 0, 'misses': 0, 'device_builds': 0, 'host_builds': 0}


def layout_key(layout):
    """Content key of a layout: for a host tensor the SHA-1 of its nonzero pattern, for a device
    tensor two 64-bit checksums computed on the device (16 bytes come back to the host)."""
    if layout.dim() != 3:
        raise ValueError('layout must be a [H, Mb, Nb] tensor')
    present = layout != 0
    if layout.is_cuda:
        flat = present.reshape(-1).to(torch.int64)
        idx = torch.arange(flat.numel(), device=layout.device, dtype=torch.int64)
        c1 = (flat * (idx * -7046029254386353131 + 1442695040888963407)).sum()
        c2 = (flat * ((idx ^ (idx >> 7)) * 6364136223846793005 + 1)).sum()
        sums = torch.stack((c1, c2, flat.sum())).tolist()
        return ('cuda', layout.device.index, tuple(layout.shape)) + tuple(sums)
    return ('cpu', tuple(layout.shape), hashlib.sha1(present.contiguous().numpy().tobytes()).hexdigest())


def _cached(kind, layout, extra, build):
    key = (kind,) + layout_key(layout) + tuple(extra)
    hit = _CACHE.get(key)
    if hit is not None:
        _CACHE.move_to_end(key)
        CACHE_STATS['hits'] += 1
        return hit
    CACHE_STATS['misses'] += 1
    obj = build()
    _CACHE[key] = obj
    while len(_CACHE) > _CACHE_ENTRIES:
        _CACHE.popitem(last=False)
    return obj


def clear_cache():
    _CACHE.clear()


DEBUG = os.environ.get('BSP_DEBUG', '') not in ('', '0')


def validate_device_buffer(buf, tiles=False):
    """Checks every table-derived index of a device metadata buffer (or attention tile lists)
    against the buffer's header; raises ValueError naming the failed check.  Run on every
    upload when BSP_DEBUG=1 is set."""
    code, pos = ctypes.c_int(0), ctypes.c_int(0)
    fn = _lib.lib().bsp_attn_tiles_validate if tiles else _lib.lib().bsp_meta_validate
    with torch.cuda.device(buf.device):
        _lib.check(fn(buf.data_ptr(), buf.numel(), ctypes.byref(code), ctypes.byref(pos),
                      torch.cuda.current_stream(buf.device).cuda_stream))


class Meta:
    """Execution metadata of one layout: host header + device buffer(s).  Built on the host
    (host layout) and uploaded once per device, or built on the device the layout lives on."""

    def __init__(self, host=None, hdr=None, dev=None):
        self._host = host                     # int32 CPU tensor (whole buffer), or None when built on a device
        self.hdr = host[:_lib.META_HEADER].clone() if hdr is None else hdr
        self.H, self.Mb, self.Nb, self.nnz = (int(v) for v in self.hdr[1:5])
        self.max_row, self.max_col = int(self.hdr[5]), int(self.hdr[6])
        self._dev = {}
        if dev is not None:
            self._dev[str(dev.device)] = dev

    @property
    def host(self):
        if self._host is None:
            self._host = next(iter(self._dev.values())).cpu()
        return self._host

    def on(self, device):
        key = str(torch.device(device)) if not isinstance(device, str) else device
        if key not in self._dev:
            if self._host is not None:
                self._dev[key] = self._host.to(device)
            else:
                self._dev[key] = next(iter(self._dev.values())).to(device)
            if DEBUG:
                validate_device_buffer(self._dev[key])
        return self._dev[key]


def _meta_total(H, Mb, Nb, nnz):
    return _lib.META_HEADER + (H * Mb + 1) + 3 * nnz + (H * Nb + 1) + 2 * nnz + H * Mb + H * Nb


def build_meta_device(layout):
    """Builds the metadata on the device `layout` lives on (any integer / bool dtype of 1, 4 or 8
    bytes): the layout never travels to the host, only the 8-int header comes back."""
    if not layout.is_cuda or layout.dim() != 3:
        raise ValueError('build_meta_device: a [H, Mb, Nb] CUDA tensor is required')
    lay = layout
    if lay.dtype == torch.bool:
        lay = lay.view(torch.uint8)
    if lay.element_size() not in (1, 4, 8) or lay.is_floating_point():
        lay = (layout != 0).view(torch.uint8)
    lay = lay.contiguous()
    H, Mb, Nb = lay.shape
    L = _lib.lib()
    cap = L.bsp_meta_device_capacity(H, Mb, Nb)
    hdr = torch.zeros(_lib.META_HEADER, dtype=torch.int32)
    with torch.cuda.device(lay.device):
        out = torch.empty(cap, dtype=torch.int32, device=lay.device)
        _lib.check(L.bsp_meta_build_device(lay.data_ptr(), lay.element_size(), H, Mb, Nb, out.data_ptr(), cap,
                                           hdr.data_ptr(), torch.cuda.current_stream(lay.device).cuda_stream))
    total = _meta_total(H, Mb, Nb, int(hdr[4]))
    CACHE_STATS['device_builds'] += 1
    return Meta(hdr=hdr, dev=out[:total])


def build_meta(layout):
    """Execution metadata of `layout`, from the process-wide cache when a layout with the same
    content has been seen.  A layout in device memory is processed there."""
    def build():
        if layout.is_cuda:
            return build_meta_device(layout)
        lay, H, Mb, Nb = _layout_i64(layout)
        L = _lib.lib()

        def call(ptr, cap, total):
            return L.bsp_meta_build(lay.data_ptr(), H, Mb, Nb, ptr, cap, total)

        CACHE_STATS['host_builds'] += 1
        return Meta(_two_pass(call).clone())
    return _cached('meta', layout, (), build)


class AttnTiles:
    """Tile lists of the tcgen05 attention kernels: host header + device buffer(s).  Built on the
    host and uploaded once per device, or built on the device the layout lives on."""

    def __init__(self, host=None, hdr=None, dev=None):
        self._host = host
        self.hdr = host[:8].clone() if hdr is None else hdr
        self._dev = {}
        if dev is not None:
            self._dev[str(dev.device)] = dev

    @property
    def host(self):
        if self._host is None:
            self._host = next(iter(self._dev.values())).cpu()
        return self._host

    def on(self, device):
        key = str(torch.device(device)) if not isinstance(device, str) else device
        if key not in self._dev:
            self._dev[key] = self.host.to(device)
            if DEBUG:
                validate_device_buffer(self._dev[key], tiles=True)
        return self._dev[key]


TILES_DEVICE_MAX_BLOCKS = 512


def build_attn_tiles_device(layout, block):
    """Builds the tile lists on the device `layout` lives on (at most 512 positions of 64, or of
    128 for block 128, per side; blocks 16 and 32 are coarsened there): only the 8-int header comes
    back to the host."""
    if not layout.is_cuda or layout.dim() != 3 or layout.size(1) != layout.size(2):
        raise ValueError('build_attn_tiles_device: a square [H, nb, nb] CUDA tensor is required')
    lay = layout
    if lay.dtype == torch.bool:
        lay = lay.view(torch.uint8)
    if lay.element_size() not in (1, 4, 8) or lay.is_floating_point():
        lay = (layout != 0).view(torch.uint8)
    lay = lay.contiguous()
    H, nb, _ = lay.shape
    L = _lib.lib()
    cap = L.bsp_attn_tiles_device_capacity(H, nb, block)
    hdr = torch.zeros(8, dtype=torch.int32)
    with torch.cuda.device(lay.device):
        out = torch.empty(max(cap, 8), dtype=torch.int32, device=lay.device)
        _lib.check(L.bsp_attn_tiles_build_device(lay.data_ptr(), lay.element_size(), H, nb, block, out.data_ptr(), cap,
                                                 hdr.data_ptr(), torch.cuda.current_stream(lay.device).cuda_stream))
    n = H * int(hdr[4])
    total = 8 + 2 * (4 * n + 1) + 3 * int(hdr[5]) + 3 * int(hdr[6])
    CACHE_STATS['device_builds'] += 1
    return AttnTiles(hdr=hdr, dev=out[:total].clone())


def build_attn_tiles(layout, block):
    """Returns the AttnTiles of a square [H, nb, nb] layout (from the process-wide cache when the
    same content has been seen), or None when the tcgen05 kernels do not cover it (blocks 64 and
    128, and blocks 16 / 32 whose count per side is a multiple of 4 / 2, are covered)."""
    if layout.dim() != 3:
        raise ValueError('layout must be a [H, Mb, Nb] tensor')
    H, Mb, Nb = layout.shape
    if Mb != Nb or block not in (16, 32, 64, 128) or (block < 64 and Mb % (64 // block)):
        return None

    def build():
        if layout.is_cuda and Mb // max(1, 64 // block) <= TILES_DEVICE_MAX_BLOCKS:
            return build_attn_tiles_device(layout, block)
        lay, H, Mb_, Nb_ = _layout_i64(layout)
        L = _lib.lib()

        def call(ptr, cap, total):
            return L.bsp_attn_tiles_build(lay.data_ptr(), H, Mb_, block, ptr, cap, total)

        return AttnTiles(_two_pass(call).clone())
    return _cached('tiles', layout, (block,), build)
