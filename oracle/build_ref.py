"""Build and import the reference's own layout->table builders (CPU only).

TEST INFRASTRUCTURE ONLY.  Used to pin oracle/lut.py and to generate the
fixtures under tests/golden/.  Nothing in the product package imports this.

The reference's native helper (csrc/utils.cpp: sdd_segment, make_layout) is
compiled from the sources where they lie in the reference checkout, into
oracle/_ref/ (git-ignored).  With that module registered under the name the
reference imports (torch_blocksparse_cpp_utils) the reference's Python package
imports on CPU: its Triton kernels are only touched at launch time, so the
table builders (MatMul.make_lut, _sparse_matmul.make_sdd_lut / make_dxx_lut /
load_balance, _sparse_softmax.make_lut, _make_layout) run without a GPU.

The reference checkout is located through the environment variable
BSP_REFERENCE_ROOT; without it a directory named `reference` beside this
repository is tried.  When neither exists every entry point here returns
None / False; callers then fall back to the committed fixtures.
"""
import importlib
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, '_ref')
REFERENCE_ROOT = os.environ.get('BSP_REFERENCE_ROOT') or os.path.join(os.path.dirname(os.path.dirname(_HERE)), 'reference')
_MOD = 'torch_blocksparse_cpp_utils'


def reference_present():
    return os.path.isfile(os.path.join(REFERENCE_ROOT, 'csrc', 'utils.cpp'))


def _built_so():
    if not os.path.isdir(REF_DIR):
        return None
    for f in sorted(os.listdir(REF_DIR)):
        if f.startswith(_MOD) and f.endswith('.so'):
            return os.path.join(REF_DIR, f)
    return None


def build(verbose=False):
    """Compile csrc/utils.cpp of the reference into oracle/_ref/.  Returns the
    path of the shared object, or None when the reference is not mounted."""
    so = _built_so()
    if so is not None:
        return so
    if not reference_present():
        return None
    os.makedirs(REF_DIR, exist_ok=True)
    # the image's default CXX wrapper cannot link OpenMP; the reference builds
    # without it too (the pragma is guarded by _OPENMP)
    os.environ.setdefault('CXX', '/usr/bin/g++')
    from torch.utils.cpp_extension import load
    load(name=_MOD, sources=[os.path.join(REFERENCE_ROOT, 'csrc', 'utils.cpp')],
         extra_cflags=['-O2'], build_directory=REF_DIR, verbose=verbose)
    return _built_so()


def load_cpp_utils():
    """Import the compiled reference helper module (or None)."""
    if _MOD in sys.modules:
        return sys.modules[_MOD]
    so = build()
    if so is None:
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(_MOD, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[_MOD] = mod
    return mod


def import_reference():
    """Import the reference Python package under the private name
    `_bsp_reference` so that it never shadows (or is shadowed by) a package
    called torch_blocksparse on sys.path.  Returns the module or None."""
    if '_bsp_reference' in sys.modules:
        return sys.modules['_bsp_reference']
    if load_cpp_utils() is None:
        return None
    try:
        import triton  # noqa: F401  (imported by the reference at module scope)
    except Exception:
        return None
    pkg_dir = os.path.join(REFERENCE_ROOT, 'torch_blocksparse')
    # the reference does `import torch_blocksparse` inside its own submodules,
    # so it has to be importable under its real name while it loads
    saved = sys.modules.get('torch_blocksparse')
    spec = importlib.util.spec_from_file_location(
        'torch_blocksparse', os.path.join(pkg_dir, '__init__.py'),
        submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules['torch_blocksparse'] = mod
    try:
        spec.loader.exec_module(mod)
        # the wrapper is not exported by the reference's __init__
        importlib.import_module('torch_blocksparse.deepspeedsparseselfattention')
    finally:
        loaded = {k: v for k, v in sys.modules.items()
                  if k == 'torch_blocksparse' or k.startswith('torch_blocksparse.')}
        for k in loaded:
            del sys.modules[k]
        if saved is not None:
            sys.modules['torch_blocksparse'] = saved
    sys.modules['_bsp_reference'] = mod
    return mod


if __name__ == '__main__':
    print('reference present:', reference_present())
    print('built:', build(verbose=True))
    ref = import_reference()
    print('reference package importable:', ref is not None)
