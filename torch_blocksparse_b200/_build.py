"""Compiles the native library (CUDA kernels + host table builders) in-tree.

    python -m torch_blocksparse_b200._build [--force] [--verbose]

The result is torch_blocksparse_b200/libbsp_b200.so, built with nvcc for
sm_100a only.  Object files are cached under torch_blocksparse_b200/build/ and
recompiled when a source or header is newer.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG_DIR, 'csrc')
OBJ_DIR = os.path.join(PKG_DIR, 'build')
LIB_PATH = os.path.join(PKG_DIR, 'libbsp_b200.so')
INCLUDE_DIR = os.path.join(os.path.dirname(PKG_DIR), 'include')

NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '-Xcompiler', '-fPIC', '-Xcompiler', '-O3',
              '--expt-relaxed-constexpr', '-I', INCLUDE_DIR]


def _nvcc():
    for cand in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if cand and (os.path.isfile(cand) or cand == 'nvcc'):
            return cand
    return 'nvcc'


def _sources():
    return sorted(os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR) if f.endswith(('.cu', '.cpp')))


def _headers():
    hs = [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR) if f.endswith(('.h', '.cuh'))]
    hs += [os.path.join(INCLUDE_DIR, f) for f in os.listdir(INCLUDE_DIR) if f.endswith('.h')]
    return hs


def _mtime(p):
    return os.path.getmtime(p) if os.path.exists(p) else 0.0


def needs_build():
    newest_src = max(_mtime(p) for p in _sources() + _headers())
    return _mtime(LIB_PATH) < newest_src


def build(force=False, verbose=False):
    """Compile every source for sm_100a and link libbsp_b200.so.  Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    newest_hdr = max(_mtime(p) for p in _headers())
    jobs = []
    objs = []
    for src in _sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + '.o')
        objs.append(obj)
        if force or _mtime(obj) < max(_mtime(src), newest_hdr):
            cmd = [nvcc] + NVCC_FLAGS + (['-Xptxas', '-v'] if verbose else []) + ['-x', 'cu', '-c', src, '-o', obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(' '.join(cmd) + '\n' + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError('nvcc failed for ' + cmd[-3])
    link = [nvcc, '-shared', '-o', LIB_PATH] + objs + ['-Xcompiler', '-fPIC', '-lpthread']
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError('link failed')
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
