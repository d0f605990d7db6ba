"""CPU restatement of the reference's layout -> look-up-table builders (numpy).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file;
only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may.

Each function restates one reference routine and cites it.  The restatement is
pinned against tables produced by the reference's own builders (imported and
run on CPU, see oracle/build_ref.py and tests/golden/make_golden.py); the
resulting fixtures live in tests/golden/.

Reference routines restated here:
  * sdd_segment / segment_blocks      csrc/utils.cpp:11-120
  * _sparse_matmul.make_sdd_lut       torch_blocksparse/matmul.py:281-297
  * _sparse_matmul.load_balance       torch_blocksparse/matmul.py:221-267
  * _sparse_matmul.make_dxx_lut       torch_blocksparse/matmul.py:372-458
  * _sparse_softmax.make_lut          torch_blocksparse/softmax.py:201-221
  * DeepSpeedSparseSelfAttention._make_layout
                                      torch_blocksparse/deepspeedsparseselfattention.py:33-65
"""
import numpy as np


def _as_layout(layout):
    lay = np.asarray(layout)
    if lay.ndim != 3:
        raise ValueError('layout must be [H, Mb, Nb]')
    return lay.astype(np.int64)


# --------------------------------------------------------------------------
# SDD table
# --------------------------------------------------------------------------
def _segment_pass(lay, idx, w):
    """One greedy packing pass at super-block width `w` (csrc/utils.cpp:11-92).

    `lay` ([H,M,N] int) is consumed in place: every block that is packed into a
    w x w super-block is zeroed so that the next (narrower) pass skips it.
    Returns an int array [n, 4] of (head, row, col, block id) entries.
    """
    H, M, N = lay.shape
    out = []
    for h in range(H):
        tmp = np.zeros((M, N), dtype=np.int64)
        left = [-1] * w                      # last w visited nonzero columns (never reset)
        top = [[-1] * N for _ in range(w)]   # last w nonzero rows seen per column
        L = lay[h]
        for m in range(M):
            row = L[m]
            for n in np.flatnonzero(row):
                n = int(n)
                if row[n] == 0:      # zeroed by an emission earlier in this row
                    continue
                n_left = left[w - 1]
                m_top = top[w - 1][n]
                t = tmp[m_top, n] if m_top >= 0 else 0
                l = tmp[m, n_left] if n_left >= 0 else 0
                tl = tmp[m_top, n_left] if (m_top >= 0 and n_left >= 0) else 0
                width = min(l, t, tl) + 1
                for nn in range(n_left + 1, n):
                    if top[w - 1][nn] > top[w - 1][n]:
                        width = 1
                tmp[m, n] = width
                left.pop(0)
                left.append(n)
                for k in range(w - 1):
                    top[k][n] = top[k + 1][n]
                top[w - 1][n] = m
                if width != w:
                    continue
                for km in range(w):
                    for kn in range(w):
                        mm = top[km][n]
                        nn = left[kn]
                        if mm < 0 or nn < 0:
                            continue
                        L[mm, nn] = 0
                        tmp[mm, nn] = 0
                        out.append((h, mm, nn, int(idx[h, mm, nn])))
    return np.asarray(out, dtype=np.int32).reshape(-1, 4)


def sdd_segment(layout, start_width):
    """csrc/utils.cpp:95-120.  Returns [(width, int32[n,4]), ...] for
    width = start_width, start_width/2, ..., 1 (empty passes omitted)."""
    lay = _as_layout(layout).copy()
    nzmask = lay != 0
    idx = np.zeros_like(lay)
    idx[nzmask] = np.arange(int(nzmask.sum()))
    ret = []
    w = int(start_width)
    while w > 0:
        rows = _segment_pass(lay, idx, w)
        if rows.shape[0] > 0:
            ret.append((w, rows))
        w //= 2
    return ret


def make_sdd_lut(layout, block):
    """matmul.py:281-297.  Returns (luts, widths, packs): per pack size an int32
    vector [h,i,j,b, h,i,j,b, ...], the number of super-blocks and the pack."""
    luts, widths, packs = [], [], []
    for size, rows in sdd_segment(layout, 64 // block):
        luts.append(rows.reshape(-1).astype(np.int32))
        widths.append(rows.shape[0] // (size * size))
        packs.append(size)
    return luts, widths, packs


# --------------------------------------------------------------------------
# DSD / DDS table
# --------------------------------------------------------------------------
def _cdiv(a, b):
    return (a + b - 1) // b


def load_balance(sizes):
    """matmul.py:221-267.  `sizes` = nonzero blocks per output column (or row).
    Returns (segments, column, lockid, maxid, offsets) as int64 arrays."""
    sizes = np.asarray(sizes, dtype=np.int64)
    nz = sizes[sizes != 0]
    if nz.size == 0:
        raise RuntimeError('load_balance: layout slice has no nonzero block')
    seg_max = int(sizes.max())
    seg_min = max(_cdiv(seg_max, 4), 4)
    segments, column, lockid, maxid = [], [], [], []
    nlocks = 0
    for col, s in enumerate(sizes.tolist()):
        d, r = s // seg_max, s % seg_max
        isempty = s < seg_min
        n = d + (1 if r >= seg_min else 0) + (1 if isempty else 0)
        seg = [0] * n
        for k in range(d):
            seg[k] = seg_max
        if r < seg_min and not isempty:
            seg[d - 1] += r
        if r >= seg_min or isempty:
            seg[d] = r
        lk, mx = 0, 0
        if d > 1 or (d == 1 and r >= seg_min):
            nlocks += 1
            lk, mx = nlocks, n
        segments += seg
        column += [col] * n
        lockid += [lk] * n
        maxid += [mx] * n
    segments = np.asarray(segments, dtype=np.int64)
    offsets = np.zeros_like(segments)
    offsets[1:] = np.cumsum(segments[:-1])
    return (segments, np.asarray(column, dtype=np.int64), np.asarray(lockid, dtype=np.int64),
            np.asarray(maxid, dtype=np.int64), offsets)


def make_dxx_lut(layout, block, step, trans):
    """matmul.py:372-458.  Returns (lut int32, num_locks, width)."""
    lay = (_as_layout(layout) != 0).astype(np.int64)
    H = lay.shape[0]
    segs, cols, deps, lks, mxs, offs = [], [], [], [], [], []
    cur_off, cur_max = 0, 0
    for z in range(H):
        sizes = lay[z].sum(1) if trans else lay[z].sum(0)
        s, c, lk, mx, of = load_balance(sizes)
        lk = lk.copy()
        lk[lk > 0] += cur_max
        cur_max = int(lk.max())
        segs.append(s); cols.append(c); deps.append(np.full_like(s, z))
        lks.append(lk); mxs.append(mx); offs.append(cur_off + of)
        cur_off += int(lay[z].sum())
    segments = np.concatenate(segs) * step
    column = np.concatenate(cols)
    depth = np.concatenate(deps)
    lockid = np.concatenate(lks)
    maxid = np.concatenate(mxs)
    offsets = np.concatenate(offs)
    # list of nonzero blocks in traversal order
    if trans:
        nnz = np.argwhere(lay)
    else:
        nnz = np.argwhere(lay.transpose(0, 2, 1))
    num_blocks = nnz.shape[0]
    offsets = np.minimum(offsets, num_blocks - 1)
    idx = nnz[:, 2] * block
    xincs = idx.copy()
    xincs[1:] -= idx[:-1]
    div = block // step
    xincs = np.repeat(xincs[:, None], div, axis=1)
    xincs[:, 1:] = step
    xincs[:, 0] -= (div - 1) * step
    first = offsets[segments > 0]
    xincs[first, 0] = idx[first]
    xincs = xincs.reshape(-1)
    # block-format operand increments
    if trans:
        widx = np.arange(num_blocks, dtype=np.int64)
    else:
        parts, base = [], 0
        for z in range(H):
            lw = lay[z].copy()
            msum = int(lw.sum())
            lw[lw > 0] = 1 + np.arange(msum)
            lt = lw.T
            parts.append(base + lt[lt > 0] - 1)
            base += msum
        widx = np.concatenate(parts) if parts else np.zeros(0, dtype=np.int64)
    wincs = widx * block * block
    wincs[1:] -= widx[:-1] * block * block
    wincs = np.repeat(wincs[:, None], div, axis=1)
    if trans:
        wincs[:, 1:] = step
        wincs[:, 0] -= (div - 1) * step
    else:
        wincs[:, 1:] = step * block
        wincs[:, 0] -= (div - 1) * step * block
    wincs[first, 0] = widx[first]
    wincs = wincs.reshape(-1)
    offsets = offsets * 2 * div
    segments = segments * div
    width = column.shape[0]
    offsets = offsets + 6 * width
    header = np.stack((offsets, segments, column, depth, lockid, maxid), axis=1).reshape(-1)
    incs = np.stack((xincs, wincs), axis=1).reshape(-1)
    incs = np.concatenate((incs, np.zeros(2, dtype=np.int64)))
    lut = np.concatenate((header, incs)).astype(np.int32)
    num_locks = max(1, int(lockid.max()))
    return lut, num_locks, width


# --------------------------------------------------------------------------
# Softmax table
# --------------------------------------------------------------------------
def make_softmax_lut(layout):
    """softmax.py:201-221.  Returns (lut int32, maxlut)."""
    lay = (_as_layout(layout) != 0).astype(np.int64)
    sizes = lay.sum(-1).reshape(-1)
    offsets = np.zeros_like(sizes)
    offsets[1:] = np.cumsum(sizes[:-1])
    nnz = np.argwhere(lay)
    idx = np.arange(nnz.shape[0], dtype=np.int64)
    core = np.stack((idx, nnz[:, 2], nnz[:, 1], nnz[:, 0]), axis=1).reshape(-1)
    offsets = offsets * 4 + 2 * sizes.size
    header = np.stack((sizes, offsets), axis=1).reshape(-1)
    lut = np.concatenate((header, core)).astype(np.int32)
    return lut, int(sizes.max())


# --------------------------------------------------------------------------
# "fixed" sparse-transformer layout
# --------------------------------------------------------------------------
def make_fixed_layout(num_heads, num_blocks, mode, block_stride, attention, numverts, vertsize):
    """deepspeedsparseselfattention.py:33-65 (the Python builder the wrapper uses)."""
    if (block_stride / vertsize) != (block_stride // vertsize):
        raise ValueError('stride window must be dividable by vertical block size')
    if numverts > (block_stride / vertsize):
        raise ValueError('number of layout versions too large')
    lay = np.zeros((num_heads, num_blocks, num_blocks), dtype=np.int64)
    if mode == 'dense':
        lay[:] = 1
        return lay
    uni = attention == 'unidirectional'
    for h in range(num_heads):
        for i in range(0, num_blocks, block_stride):
            for j in range(i, i + block_stride):
                for k in range(i, (j + 1) if uni else (i + block_stride)):
                    lay[h, j, k] = 1
        start = block_stride - (1 + h % numverts) * vertsize
        for i in range(num_blocks):
            end = i if uni else num_blocks
            for j in range(start, end, block_stride):
                for k in range(j, min(j + vertsize, num_blocks)):
                    lay[h, i, k] = 1
    return lay
