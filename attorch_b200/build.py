"""
Builds libattorch_b200.so in-tree with nvcc for sm_100a.

Run as ``python -m attorch_b200.build`` (add ``--force`` to rebuild, ``--verbose`` for
``-Xptxas -v`` output).  The library links only against the CUDA runtime; it has no torch or
Python dependency, so the same file serves ctypes (this package) and any other C-ABI binding.
"""

import argparse
import concurrent.futures
import hashlib
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / 'csrc'
INCLUDE = PKG_DIR.parent / 'include'
LIB_PATH = PKG_DIR / 'libattorch_b200.so'
STAMP_PATH = PKG_DIR / '.libattorch_b200.stamp'

OBJ_DIR = PKG_DIR / '_obj'
NVCC_FLAGS = [
    '-std=c++20', '-O3', '-lineinfo',
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-Xcompiler', '-fPIC',
    '--expt-relaxed-constexpr',
]
LINK_FLAGS = ['-shared', '-cudart', 'shared', '-gencode', 'arch=compute_100a,code=sm_100a']


def find_nvcc() -> str:
    """Locates nvcc: $CUDA_HOME/bin, the default toolkit location, then PATH."""
    candidates = []
    if os.environ.get('CUDA_HOME'):
        candidates.append(Path(os.environ['CUDA_HOME']) / 'bin' / 'nvcc')
    candidates.append(Path('/usr/local/cuda/bin/nvcc'))
    for cand in candidates:
        if cand.exists():
            return str(cand)
    found = shutil.which('nvcc')
    if found is None:
        raise RuntimeError('nvcc not found; set CUDA_HOME')
    return found


def source_digest() -> str:
    """Hash of every file the library is built from, plus the flags."""
    h = hashlib.sha256()
    files = sorted(CSRC.glob('*.cu')) + sorted(CSRC.glob('*.cuh')) + sorted(INCLUDE.glob('*.h'))
    for path in files:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(' '.join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return (LIB_PATH.exists() and STAMP_PATH.exists()
            and STAMP_PATH.read_text().strip() == source_digest())


_INCLUDE_RE = re.compile(r'^\s*#\s*include\s*"([^"]+)"', re.MULTILINE)


def _dependencies(src: Path, seen=None) -> set:
    """The source file and every file of this repository it includes, directly or not."""
    seen = set() if seen is None else seen
    if src in seen or not src.exists():
        return seen
    seen.add(src)
    for name in _INCLUDE_RE.findall(src.read_text()):
        for base in (src.parent, CSRC, INCLUDE):
            cand = (base / name).resolve()
            if cand.exists():
                _dependencies(cand, seen)
                break
    return seen


def _unit_digest(src: Path) -> str:
    h = hashlib.sha256()
    for path in sorted(_dependencies(src.resolve())):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(' '.join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(nvcc: str, src: Path, verbose: bool, force: bool = False) -> Path:
    """Compiles one translation unit unless its object is newer than everything it includes."""
    obj = OBJ_DIR / (src.stem + '.o')
    stamp = OBJ_DIR / (src.stem + '.stamp')
    digest = _unit_digest(src)
    if not force and not verbose and obj.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return obj
    cmd = [nvcc, *NVCC_FLAGS, f'-I{INCLUDE}', f'-I{CSRC}']
    if verbose:
        cmd += ['-Xptxas', '-v']
    cmd += ['-c', str(src), '-o', str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f'nvcc failed on {src.name} with exit code {proc.returncode}')
    stamp.write_text(digest + '\n')
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the shared library if it is missing or older than its sources."""
    if not force and is_current():
        return LIB_PATH
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob('*.cu'))
    workers = min(len(sources), os.cpu_count() or 1)
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        objects = list(pool.map(lambda src: _compile(nvcc, src, verbose, force), sources))
    cmd = [nvcc, *LINK_FLAGS, *[str(o) for o in objects], '-o', str(LIB_PATH)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        sys.stderr.write(proc.stderr)
        raise RuntimeError(f'link failed with exit code {proc.returncode}')
    STAMP_PATH.write_text(source_digest() + '\n')
    return LIB_PATH


if __name__ == '__main__':
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument('--force', action='store_true')
    parser.add_argument('--verbose', action='store_true')
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))
