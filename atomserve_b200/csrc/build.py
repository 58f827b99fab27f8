"""Builds the CUDA sources of this folder into one shared library for sm_100a.

`nvcc` compiles each `.cu` to an object (in parallel, a few seconds each: the kernels include
no framework headers) and links `libatomserve_b200.so`. Objects and library live beside the
package (`atomserve_b200/_build/`, `atomserve_b200/_lib/`) when that is writable, so a library
built on one machine travels with the tree; otherwise under the system's temporary folder.
A manifest of source hashes decides whether anything has to be rebuilt, so a fresh checkout
compiles at its first call and later calls only load. Progress goes to stderr, a line per file.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PACKAGE = CSRC.parent
LIB_NAME = "libatomserve_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _log(message: str) -> None:
    print(f"[atomserve_b200 build] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("ATOMSERVE_B200_NVCC"), shutil.which("nvcc")]
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            candidates.append(str(Path(root) / "bin" / "nvcc"))
    for c in candidates:
        if c and Path(c).exists():
            return c
    raise RuntimeError(
        "nvcc not found (looked at ATOMSERVE_B200_NVCC, PATH, CUDA_HOME, /usr/local/cuda): "
        "the CUDA kernels cannot be compiled"
    )


def _writable(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_root() -> Path:
    """Where objects and the library go: $ATOMSERVE_B200_BUILD_DIR, the package, or /tmp."""
    env = os.environ.get("ATOMSERVE_B200_BUILD_DIR")
    if env:
        return Path(env)
    if _writable(PACKAGE / "_lib") and _writable(PACKAGE / "_build"):
        return PACKAGE
    return Path(tempfile.gettempdir()) / f"atomserve_b200_{os.getuid()}"


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for header in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _digest(source: Path, headers: str) -> str:
    return hashlib.sha256(source.read_bytes() + headers.encode()).hexdigest()


def library_path(root: Path | None = None) -> Path:
    return (root or build_root()) / "_lib" / LIB_NAME


def manifest_digest() -> str:
    headers = _headers_digest()
    h = hashlib.sha256()
    for s in sources():
        h.update(s.name.encode())
        h.update(_digest(s, headers).encode())
    return h.hexdigest()


def is_current(root: Path | None = None) -> bool:
    root = root or build_root()
    lib, stamp = library_path(root), root / "_lib" / "manifest.sha256"
    return lib.exists() and stamp.exists() and stamp.read_text().strip() == manifest_digest()


def _compile(nvcc: str, source: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(source), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    start = time.time()
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{done.stdout}\n{done.stderr}")
    _log(f"compiled {source.name} in {time.time() - start:.1f}s")
    return done.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what changed and link the library; returns its path."""
    root = build_root()
    lib = library_path(root)
    if not force and is_current(root):
        return lib
    nvcc = find_nvcc()
    obj_dir = root / "_build"
    obj_dir.mkdir(parents=True, exist_ok=True)
    lib.parent.mkdir(parents=True, exist_ok=True)
    headers = _headers_digest()
    todo, objects = [], []
    for s in sources():
        obj, stamp = obj_dir / (s.stem + ".o"), obj_dir / (s.stem + ".sha256")
        objects.append(obj)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != _digest(s, headers):
            todo.append((s, obj, stamp))
    _log(f"compiling {len(todo)} of {len(objects)} CUDA sources for sm_100a with {nvcc} into {root}")
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        futures = {pool.submit(_compile, nvcc, s, obj, verbose): (s, stamp) for s, obj, stamp in todo}
        for f in concurrent.futures.as_completed(futures):
            s, stamp = futures[f]
            out = f.result()
            if verbose and out:
                print(out, file=sys.stderr)
            stamp.write_text(_digest(s, headers))
    tmp = lib.with_suffix(f".tmp{os.getpid()}")
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objects)]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{done.stdout}\n{done.stderr}")
    os.replace(tmp, lib)
    (lib.parent / "manifest.sha256").write_text(manifest_digest())
    _log(f"linked {lib}")
    return lib


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
