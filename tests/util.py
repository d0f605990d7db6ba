"""Helpers shared by the test modules."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')

# Parity gates: FP32 rtol/atol 1e-4; FP16 / BF16 rtol/atol 1e-2.
TOL = {torch.float32: (1e-4, 1e-4), torch.float16: (1e-2, 1e-2), torch.bfloat16: (1e-2, 1e-2)}


def assert_close(got, want, what=''):
    assert got.shape == want.shape, '%s: shape %s vs %s' % (what, tuple(got.shape), tuple(want.shape))
    assert got.dtype == want.dtype, '%s: dtype %s vs %s' % (what, got.dtype, want.dtype)
    rtol, atol = TOL[want.dtype]
    g, w = got.detach().cpu().float(), want.detach().cpu().float()
    ok = torch.isclose(g, w, rtol=rtol, atol=atol, equal_nan=True)
    if not bool(ok.all()):
        bad = (~ok).nonzero()
        i = tuple(bad[0].tolist())
        err = (g - w).abs()
        err[~torch.isfinite(err)] = 0
        raise AssertionError('%s: %d of %d elements differ (first at %s: got %r want %r; max abs err %g)'
                             % (what, bad.shape[0], ok.numel(), i, g[i].item(), w[i].item(), err.max().item()))


def head_blocks(layout, h):
    """Range [b0, b1) of canonical block ids that belong to head h."""
    per = (layout != 0).sum((1, 2))
    b0 = int(per[:h].sum())
    return b0, b0 + int(per[h])


def load_npz(name):
    return np.load(os.path.join(GOLDEN, name))


class Guarded:
    """A tensor in the middle of a larger allocation whose margins are filled with NaN (the idea
    of the reference's unused `mempad`, tests/utils.py:36-40): a kernel that writes outside the
    tensor it was given destroys a NaN, and check() sees it.  Stands in for a device memory
    checker in the small GPU tests."""

    def __init__(self, shape, dtype, device, pad_elems=8192, fill=None):
        n = 1
        for d in shape:
            n *= d
        self.pad = pad_elems
        self.buf = torch.full((n + 2 * pad_elems,), float('nan'), dtype=dtype, device=device)
        self.t = self.buf[pad_elems:pad_elems + n].view(*shape)
        if fill is not None:
            self.t.copy_(fill)

    def check(self, what=''):
        lo, hi = self.buf[:self.pad], self.buf[-self.pad:]
        assert bool(torch.isnan(lo).all()) and bool(torch.isnan(hi).all()), 'write outside %s' % (what or 'the tensor')
