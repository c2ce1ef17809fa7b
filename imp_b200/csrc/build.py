"""Compiles the CUDA sources of this folder into one shared library for sm_100a.

`nvcc -gencode arch=compute_100a,code=sm_100a` on every `.cu` file here, one
object per file (in parallel), linked into `_build/libimp_b200-<hash>.so` next
to the sources; the hash covers the sources, the headers and the flags, so an
edited file rebuilds and an unchanged tree loads at once.  When the source
tree cannot be written (an installed, read-only copy), the library goes to
`$IMP_B200_BUILD_DIR` or a per-user folder under the system's temporary
directory.  Progress goes to stderr, one line per file.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
LINK_FLAGS = ["-shared", "-Xcompiler", "-fPIC"]
# Extra compiler flags for experiments (e.g. "-DIMP_PDL_EARLY=0"); part of the build's hash.
NVCC_FLAGS += os.environ.get("IMP_B200_NVCC_FLAGS", "").split()


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[imp_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    cands.append("/usr/local/cuda/bin/nvcc")
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $CUDA_HOME/bin, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be compiled")


HOST_DIR = os.path.join(CSRC_DIR, "host")
INCLUDE_DIR = os.path.normpath(os.path.join(CSRC_DIR, "..", "..", "include"))
HOST_FLAGS = ["-O2", "-std=c++20", "-Wno-deprecated-gpu-targets", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Xcompiler", "-Wall"]


def sources() -> List[str]:
    """The kernels (*.cu here) and the host (host/*.cpp), as paths relative to this folder."""
    return (sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu")) +
            sorted(os.path.join("host", f) for f in os.listdir(HOST_DIR) if f.endswith(".cpp")))


def kernel_headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def headers() -> List[str]:
    own = kernel_headers()
    host = sorted(os.path.join("host", f) for f in os.listdir(HOST_DIR) if f.endswith((".hpp", ".h")))
    public = sorted(os.path.join(INCLUDE_DIR, "imp_b200", f) for f in os.listdir(os.path.join(INCLUDE_DIR, "imp_b200")))
    return own + host + public


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + HOST_FLAGS + LINK_FLAGS).encode())
    for f in sources() + headers():
        h.update(os.path.basename(f).encode())
        with open(os.path.join(CSRC_DIR, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}-{threading.get_ident()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir_cache = {}


def build_dir() -> str:
    key = os.environ.get("IMP_B200_BUILD_DIR", "")
    if key not in _build_dir_cache:
        _build_dir_cache[key] = _find_build_dir()
    return _build_dir_cache[key]


def _find_build_dir() -> str:
    env = os.environ.get("IMP_B200_BUILD_DIR")
    if env:
        if not _writable_dir(env):
            raise BuildError(f"IMP_B200_BUILD_DIR={env} cannot be written")
        return env
    local = os.path.join(CSRC_DIR, "_build")
    if _writable_dir(local):
        return local
    fallback = os.path.join(tempfile.gettempdir(), f"imp_b200-build-{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"neither {local} nor {fallback} can be written; set IMP_B200_BUILD_DIR")


def library_path(create: bool = True) -> str:
    return os.path.join(build_dir(), f"libimp_b200-{source_hash()}.so")


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> None:
    if src.endswith(".cpp"):
        cmd = [nvcc, *HOST_FLAGS, "-I", CSRC_DIR, "-I", HOST_DIR, "-I", INCLUDE_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
    else:
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
    if verbose and not src.endswith(".cpp"):
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    t0 = time.time()
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{p.stdout}\n{p.stderr}")
    _log(f"compiled {src} in {time.time() - t0:.1f}s")
    if verbose and p.stderr:
        sys.stderr.write(p.stderr)


def _object_hash(src: str) -> str:
    """What one object file depends on: its flags, its source, and the headers of its side."""
    h = hashlib.sha256()
    host = src.endswith(".cpp")
    h.update(" ".join(HOST_FLAGS if host else NVCC_FLAGS).encode())
    deps = [src] + ([f for f in headers()] if host else kernel_headers())
    for f in deps:
        with open(os.path.join(CSRC_DIR, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def build(force: bool = False, verbose: bool = False) -> str:
    """Build (if needed) and return the path of the shared library.  Object files are kept by the hash
    of what they depend on, so an edit recompiles only what it touches."""
    out = library_path()
    if os.path.exists(out) and not force:
        return out
    nvcc = find_nvcc()
    bdir = build_dir()
    objdir = os.path.join(bdir, "obj")
    os.makedirs(objdir, exist_ok=True)
    srcs = sources()
    objs = [os.path.join(objdir, f"{os.path.splitext(s)[0].replace(os.sep, '_')}-{_object_hash(s)}.o") for s in srcs]
    todo = [(s, o) for s, o in zip(srcs, objs) if force or verbose or not os.path.exists(o)]
    if todo:
        _log(f"compiling {len(todo)} of {len(srcs)} source files for sm_100a with {nvcc} (this takes a minute the first time)")

    def compile_to(src, obj):
        tmp = f"{obj}.tmp-{os.getpid()}"
        _compile_one(nvcc, src, tmp, verbose)
        os.replace(tmp, obj)

    with ThreadPoolExecutor(max_workers=min(os.cpu_count() or 8, 16, max(len(todo), 1))) as ex:
        futs = [ex.submit(compile_to, s, o) for s, o in todo]
        for f in futs:
            f.result()
    tmp = out + f".tmp-{os.getpid()}"
    p = subprocess.run([nvcc, *LINK_FLAGS, "-o", tmp, *objs, "-ldl"], capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"link failed:\n{p.stdout}\n{p.stderr}")
    os.replace(tmp, out)  # atomic: concurrent builders race benignly
    _log(f"linked {os.path.basename(out)}")
    # Drop libraries and objects of older source states.
    keep = set(objs)
    for f in os.listdir(objdir):
        if f.endswith(".o") and os.path.join(objdir, f) not in keep:
            try:
                os.remove(os.path.join(objdir, f))
            except OSError:
                pass
    for f in os.listdir(bdir):
        if f.startswith("libimp_b200-") and f.endswith(".so") and os.path.join(bdir, f) != out:
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass
    return out


# ---------------------------------------------------------------------------
# Variant libraries: one source compiled with given macro values (e.g. the attention
# kernels per head size).  Built on first use of that variant, cached like the base library.
# ---------------------------------------------------------------------------
VARIANT_DIR = os.path.join(CSRC_DIR, "variants")


def variant_hash(source: str, defines: dict) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + LINK_FLAGS).encode())
    h.update(repr(sorted(defines.items())).encode())
    # everything that goes into the image: the source, runtime.cu (compiled in), and every header beside them
    variant_headers = sorted(f for f in os.listdir(VARIANT_DIR) if f.endswith((".cuh", ".h")))
    paths = ([os.path.join(VARIANT_DIR, source), os.path.join(CSRC_DIR, "runtime.cu")] +
             [os.path.join(CSRC_DIR, f) for f in kernel_headers()] + [os.path.join(VARIANT_DIR, f) for f in variant_headers])
    for path in paths:
        with open(path, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def build_variant(source: str, defines: dict, force: bool = False, verbose: bool = False) -> str:
    """Compile variants/<source> with -D<key>=<value> into its own shared library; returns its path."""
    tag = "_".join(f"{k.lower()}{v}" for k, v in sorted(defines.items()))
    stem = os.path.splitext(source)[0]
    bdir = build_dir()
    out = os.path.join(bdir, f"libimp_{stem}_{tag}-{variant_hash(source, defines)}.so")
    if os.path.exists(out) and not force:
        return out
    nvcc = find_nvcc()
    _log(f"compiling {source} for {tag} (first use)")
    t0 = time.time()
    tmp = out + f".tmp-{os.getpid()}"
    # error reporting lives in the base library's runtime.cu; a variant carries its own copy
    cmd = [nvcc, *NVCC_FLAGS, *LINK_FLAGS, "-I", CSRC_DIR, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
           os.path.join(VARIANT_DIR, source), os.path.join(CSRC_DIR, "runtime.cu"), "-o", tmp]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {source} ({tag}):\n{p.stdout}\n{p.stderr}")
    os.replace(tmp, out)
    _log(f"built {os.path.basename(out)} in {time.time() - t0:.1f}s")
    if verbose and p.stderr:
        sys.stderr.write(p.stderr)
    prefix = f"libimp_{stem}_{tag}-"
    for f in os.listdir(bdir):
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(bdir, f) != out:
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass
    return out


ATTENTION_HEAD_DIMS = tuple(range(16, 257, 16))
ATTENTION_TC_HEAD_DIMS = (64, 128)     # head sizes of the tensor-memory prefill kernel


def build_all(force: bool = False) -> List[str]:
    """The base library and the attention variant of every supported head size."""
    paths = [build(force)]
    with ThreadPoolExecutor(max_workers=8) as ex:
        futs = [ex.submit(build_variant, "attention_mma.cu", {"IMP_ATTN_DH": dh}, force) for dh in ATTENTION_HEAD_DIMS]
        futs += [ex.submit(build_variant, "attention_tc.cu", {"IMP_ATTN_DH": dh}, force) for dh in ATTENTION_TC_HEAD_DIMS]
        paths += [f.result() for f in futs]
    return paths


if __name__ == "__main__":
    if "--all" in sys.argv:
        print("\n".join(build_all(force="--force" in sys.argv)))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
