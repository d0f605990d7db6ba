"""Generates the fixtures in this directory from the reference itself (CPU only).

    python tests/golden/make_golden.py

Needs the reference checkout (BSP_REFERENCE_ROOT, see oracle/build_ref.py for the default); the
fixtures it writes are committed so that the tests run without it.

  lut_small.npz       tables produced by the reference's own builders
                      (_sparse_matmul.make_sdd_lut / make_dxx_lut,
                      _sparse_softmax.make_lut, _make_layout) for small layouts,
                      stored in full
  lut_configs.json    SHA-256 + sizes of the same tables for the layouts of the
                      five benchmark configurations (too large to store)
  fixed_layouts.npz   layouts returned by the reference's
                      DeepSpeedSparseSelfAttention._make_layout
                      (deepspeedsparseselfattention.py:51-65) for six argument sets
  dense_masked.npz    inputs and outputs of the reference's dense-masked test
                      oracles (tests/test_matmul.py:run_mm_reference,
                      tests/test_softmax.py:run_softmax_reference, with the
                      helpers of tests/utils.py), executed on CPU tensors
"""
import ast
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402
import workloads  # noqa: E402


def small_layouts():
    """Named small layouts: random densities, the quirk triggers and edge cases."""
    out = {}
    rng = np.random.default_rng(1234)
    for i, (H, Mb, Nb, p) in enumerate([(1, 4, 4, 0.5), (2, 8, 12, 0.5), (3, 16, 16, 0.3), (2, 16, 32, 0.5),
                                        (2, 12, 7, 0.8), (1, 20, 20, 0.95), (4, 6, 9, 0.15), (2, 16, 16, 1.0)]):
        lay = (rng.random((H, Mb, Nb)) < p).astype(np.int64)
        for h in range(H):
            if lay[h].sum() == 0:
                lay[h, 0, 0] = 1
        out['rand%d' % i] = lay
    # reductions shorter than 4 everywhere: the extra zero-length segment of load_balance
    out['tiny_rows'] = np.array([[[1, 0], [1, 1]]], dtype=np.int64)
    # empty rows and columns
    lay = np.zeros((2, 6, 6), dtype=np.int64)
    lay[0, 1, 2] = lay[0, 1, 4] = lay[0, 5, 0] = 1
    lay[1, 0, 0] = lay[1, 3, 3] = 1
    out['holes'] = lay
    # a layout whose 4x4 packing emits entries outside the layout (duplicate block id 0)
    rng = np.random.default_rng(7)
    ref = build_ref.import_reference()
    for _ in range(2000):
        lay = (rng.random((2, 16, 32)) < 0.5).astype(np.int64)
        luts, _, widths, packs = ref.matmul._sparse_matmul.make_sdd_lut(torch.from_numpy(lay).clone(), 16, torch.float16, 'cpu')
        if sum(l.numel() for l in luts) // 4 > lay.sum():
            out['bogus_entries'] = lay
            break
    return out


def tables_of(ref, lay, blocks=(16, 32, 64), steps=(8, 16)):
    RM = ref.matmul._sparse_matmul
    t = torch.from_numpy(lay)
    res = {}
    for block in blocks:
        luts, _, widths, packs = RM.make_sdd_lut(t.clone(), block, torch.float16, 'cpu')
        res['sdd_b%d_packs' % block] = np.asarray(packs, dtype=np.int64)
        res['sdd_b%d_widths' % block] = np.asarray(widths, dtype=np.int64)
        res['sdd_b%d_lut' % block] = (np.concatenate([l.numpy() for l in luts]) if luts else np.zeros(0, np.int32))
        for step in steps:
            for trans in (0, 1):
                lut, nlocks, width, _ = RM.make_dxx_lut(t.clone(), block, step, bool(trans), 'cpu')
                key = 'dxx_b%d_s%d_t%d' % (block, step, trans)
                res[key + '_lut'] = lut.numpy()
                res[key + '_meta'] = np.asarray([int(nlocks), int(width)], dtype=np.int64)
    lut, maxlut = ref.softmax._sparse_softmax.make_lut(t, 16, 'cpu')
    res['softmax_lut'] = lut.numpy()
    res['softmax_maxlut'] = np.asarray([maxlut], dtype=np.int64)
    return res


def config_layouts():
    out = {
        'c1': (workloads.config1()['layout'], 16),
        'c2': (workloads.config2()['layout'], 32),
        'c3': (workloads.config3(small=True)['layout'], 64),   # same family; full-size built below
        'c4_uni': (workloads.config4('unidirectional', small=True)['layout'], 64),
        'c4_bi': (workloads.config4('bidirectional', small=True)['layout'], 64),
        'c5': (workloads.config5(small=True)['layout'], 128),
    }
    from torch_blocksparse_b200 import layouts
    out['c3_full'] = (layouts.causal_band(16, 64, 4, 1), 64)
    out['c4_uni_full'] = (layouts.fixed(16, 128, 4, 'unidirectional'), 64)
    out['c4_bi_full'] = (layouts.fixed(16, 128, 4, 'bidirectional'), 64)
    out['c5_full'] = (layouts.bigbird(16, 128, 3, 3, 2, seed=0), 128)
    return out


FIXED_LAYOUT_ARGS = [(4, 16, 'fixed', 4, 'unidirectional', 1, 1), (4, 16, 'fixed', 4, 'bidirectional', 2, 2),
                     (3, 32, 'fixed', 8, 'unidirectional', 4, 2), (2, 8, 'dense', 4, 'unidirectional', 1, 1),
                     (16, 128, 'fixed', 4, 'bidirectional', 1, 1), (16, 128, 'fixed', 4, 'unidirectional', 1, 1)]


def fixed_layout_cases(ref):
    """The reference's own _make_layout on each argument set; keys are the arguments joined by '_'."""
    make = ref.deepspeedsparseselfattention.DeepSpeedSparseSelfAttention._make_layout
    out = {}
    for args in FIXED_LAYOUT_ARGS:
        out['_'.join(str(a) for a in args)] = make(*args).numpy().astype(np.int8)
    return out


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def load_ref_functions(path, names, ns):
    """Executes the named top-level functions of a reference test file inside
    `ns` without importing the file (it needs nose and runs a GPU bench on import)."""
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            node.decorator_list = []
            exec(compile(ast.Module(body=[node], type_ignores=[]), path, 'exec'), ns)


def dense_masked_cases():
    tdir = os.path.join(build_ref.REFERENCE_ROOT, 'tests')
    ns = {'torch': torch}
    exec(compile(open(os.path.join(tdir, 'utils.py')).read(), 'utils.py', 'exec'), ns)
    load_ref_functions(os.path.join(tdir, 'test_matmul.py'), {'run_mm_reference'}, ns)
    load_ref_functions(os.path.join(tdir, 'test_softmax.py'), {'run_softmax_reference'}, ns)
    out = {}
    g = torch.Generator().manual_seed(11)
    # MatMul: 3 modes x 4 transpose combinations, block 16, FP32 (exact on CPU)
    # values on a 1/8 grid: compressible fixtures and exact FP32 products
    Z, H, M, N, K, block = 1, 2, 32, 48, 32, 16
    grid = lambda shape: torch.randint(0, 8, shape, generator=g).float() / 8
    for mode in ('sdd', 'dsd', 'dds'):
        for ta in (0, 1):
            for tb in (0, 1):
                AS = (K, M) if ta else (M, K)
                BS = (N, K) if tb else (K, N)
                shape = {'sdd': (M, N), 'dsd': AS, 'dds': BS}[mode]
                layout = torch.bernoulli(torch.full((H, shape[0] // block, shape[1] // block), 0.6), generator=g).long()
                layout[:, 0, 0] = 1
                x = grid((Z, H) + AS).requires_grad_()
                w = grid((Z, H) + BS).requires_grad_()
                dy = grid((Z, H, M, N))
                y, dx, dw = ns['run_mm_reference'](x.clone(), w.clone(), mode, bool(ta), bool(tb), layout, block, dy)
                key = 'mm_%s_%d%d' % (mode, ta, tb)
                for nme, t in (('layout', layout), ('x', x), ('w', w), ('dy', dy), ('y', y), ('dx', dx), ('dw', dw)):
                    out[key + '_' + nme] = t.detach().numpy()
    # Softmax: the reference test's own configuration shrunk (block 16, scale 0.4,
    # key-padding mask 'add' with -inf, attention mask 'mul' given as bool to the oracle)
    Z, H, M, N, block, scale = 2, 2, 64, 64, 16, 0.4
    layout = torch.bernoulli(torch.full((H, M // block, N // block), 0.6), generator=g).long()
    layout[:, :, 0] = 1
    x = (torch.randint(0, 64, (Z, H, M, N), generator=g).float() / 8).requires_grad_()
    dx = torch.randint(0, 16, (Z, H, M, N), generator=g).float() / 16
    am = torch.randint(0, 2, (N, N), generator=g, dtype=torch.bool)
    am[:, 0] = True                       # keep one visible column per row: no NaN rows
    kp = torch.randint(0, 2, (Z, N), generator=g).float()
    kp[:, 0] = 0
    kp[kp == 1.] = float('-inf')
    y, gx = ns['run_softmax_reference'](x.clone(), scale, dx, kp, am, layout, block)
    for nme, t in (('layout', layout), ('x', x), ('dy', dx), ('am', am.float()), ('kp', kp), ('y', y), ('dx', gx)):
        out['sm_' + nme] = t.detach().numpy()
    out['sm_scale'] = np.asarray([scale])
    # helpers: dense <-> block format
    w = torch.randint(0, 256, (2, 2, 32, 48), generator=g).float()
    lay = torch.bernoulli(torch.full((2, 2, 3), 0.5), generator=g).long()
    out['fmt_w'] = w.numpy()
    out['fmt_layout'] = lay.numpy()
    out['fmt_sparse'] = ns['dense_to_sparse'](w, lay, 16).numpy()
    out['fmt_dense_ninf'] = ns['sparse_to_dense'](w, lay, 16, float('-inf')).numpy()
    return out


def main():
    ref = build_ref.import_reference()
    if ref is None:
        raise SystemExit('reference checkout not available')
    small = {}
    for name, lay in small_layouts().items():
        small[name + '/layout'] = lay
        for k, v in tables_of(ref, lay).items():
            small[name + '/' + k] = v
    np.savez_compressed(os.path.join(HERE, 'lut_small.npz'), **small)
    cfg = {}
    for name, (layout, block) in config_layouts().items():
        lay = layout.numpy()
        blocks = (block,) if block != 128 else (128,)
        entry = {'layout_sha': sha(lay), 'shape': list(lay.shape), 'block': block, 'nnz': int(lay.sum())}
        for k, v in tables_of(ref, lay, blocks=blocks).items():
            entry[k] = {'sha': sha(v), 'size': int(v.size)}
        cfg[name] = entry
    json.dump(cfg, open(os.path.join(HERE, 'lut_configs.json'), 'w'), indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, 'dense_masked.npz'), **dense_masked_cases())
    np.savez_compressed(os.path.join(HERE, 'fixed_layouts.npz'), **fixed_layout_cases(ref))
    for f in ('lut_small.npz', 'lut_configs.json', 'dense_masked.npz', 'fixed_layouts.npz'):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == '__main__':
    main()
