"""Builds the native libraries at first use and finds them afterwards.

Two libraries, both kept inside the package tree (``dlm_b200/_lib``) when it can
be written, else under the system temporary folder:

* ``_dlm_host``    : cache manager and scheduler (C++ only, no CUDA needed);
* ``_dlm_kernels`` : the sm_100a kernels and their launchers (nvcc).

A library is rebuilt when the hash of its sources and flags changes.  While the
compilers run, a line is printed to stderr now and then.
"""
from __future__ import annotations

import fcntl
import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcudafe", "--diag_suppress=177"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[dlm_b200 build] {msg}", file=sys.stderr, flush=True)


def lib_dir() -> str:
    """Where built libraries live: in the tree if writable, else a per-user temp folder."""
    override = os.environ.get("DLM_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    d = os.path.join(_PKG, "_lib")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"dlm_b200_lib_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _find(tool: str, env: str, extra: list[str]) -> str:
    cand = os.environ.get(env)
    if cand and os.path.exists(cand):
        return cand
    found = shutil.which(tool)
    if found:
        return found
    for e in extra:
        if os.path.exists(e):
            return e
    raise BuildError(f"{tool} not found (set ${env})")


def _nvcc() -> str:
    return _find("nvcc", "NVCC", ["/usr/local/cuda/bin/nvcc"])


def _cxx() -> str:
    return _find("g++", "CXX", ["/usr/bin/g++", "/usr/bin/c++"])


def _cuda_home() -> str:
    return os.path.dirname(os.path.dirname(os.path.realpath(_nvcc())))


def _sources(sub: str, exts: tuple[str, ...]) -> list[str]:
    d = os.path.join(_CSRC, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def _headers() -> list[str]:
    out = []
    for root, _, files in os.walk(_CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".h", ".hpp", ".cuh"))]
    return sorted(out)


def _hash(files: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(f.replace(_PKG, "<pkg>") for f in flags).encode())
    h.update(sys.version.encode())
    return h.hexdigest()[:20]


def _run(cmd: list[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n$ {' '.join(cmd)}\n{p.stdout}")
    if os.environ.get("DLM_B200_BUILD_VERBOSE") and p.stdout.strip():
        _say(p.stdout.strip())


class _Ticker:
    def __init__(self, what: str):
        self.what, self.stop = what, threading.Event()
        self.t0 = time.time()
        self.th = threading.Thread(target=self._loop, daemon=True)

    def _loop(self):
        while not self.stop.wait(10.0):
            _say(f"still compiling {self.what} ... {time.time() - self.t0:.0f} s")

    def __enter__(self):
        self.th.start()
        return self

    def __exit__(self, *a):
        self.stop.set()


def _py_includes() -> list[str]:
    import pybind11
    return ["-I" + sysconfig.get_paths()["include"], "-I" + pybind11.get_include()]


def _build(name: str, compile_jobs: list[tuple[list[str], str, str]], link_cmd_tail: list[str],
           all_files: list[str], flags: list[str]) -> str:
    """compile_jobs: (command-prefix, source, object).  Returns the path of the library."""
    out_dir = lib_dir()
    tag = _hash(all_files, flags)
    so = os.path.join(out_dir, f"{name}{sysconfig.get_config_var('EXT_SUFFIX')}")
    stamp = os.path.join(out_dir, f"{name}.hash")
    lock_path = os.path.join(out_dir, f"{name}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(so) and os.path.exists(stamp) and open(stamp).read().strip() == tag:
                return so
            obj_dir = os.path.join(out_dir, f"{name}_obj")
            os.makedirs(obj_dir, exist_ok=True)
            t0 = time.time()
            _say(f"compiling {name}: {len(compile_jobs)} files into {out_dir}")
            with _Ticker(name):
                def one(job):
                    prefix, src, obj = job
                    _run(prefix + ["-c", src, "-o", obj], os.path.basename(src))
                    _say(f"  compiled {os.path.basename(src)} ({time.time() - t0:.0f} s)")
                    return obj
                jobs = [(p, s, os.path.join(obj_dir, os.path.basename(s) + ".o")) for p, s, _ in compile_jobs]
                with ThreadPoolExecutor(max_workers=min(8, max(1, os.cpu_count() or 1))) as ex:
                    objs = list(ex.map(one, jobs))
                tmp_so = so + f".tmp{os.getpid()}"
                _run([_cxx(), "-shared", "-o", tmp_so] + objs + link_cmd_tail, name)
                os.replace(tmp_so, so)
            with open(stamp, "w") as f:
                f.write(tag)
            _say(f"built {name} in {time.time() - t0:.0f} s")
            return so
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def build_host() -> str:
    srcs = _sources("host", (".cpp",))
    flags = CXX_FLAGS + _py_includes()
    prefix = [_cxx()] + flags + ["-I" + os.path.join(_CSRC, "host")]
    return _build("_dlm_host", [(prefix, s, "") for s in srcs], [], srcs + _headers(), flags)


def build_kernels() -> str:
    cu = _sources("kernels", (".cu",))
    cpp = _sources("kernels", (".cpp",))
    inc = ["-I" + os.path.join(_CSRC, "kernels")]
    nv_flags = NVCC_ARCH + NVCC_FLAGS + inc
    cx_flags = CXX_FLAGS + _py_includes() + inc + ["-I" + os.path.join(_cuda_home(), "include")]
    jobs = [([_nvcc()] + nv_flags, s, "") for s in cu] + [([_cxx()] + cx_flags, s, "") for s in cpp]
    lib64 = os.path.join(_cuda_home(), "lib64")
    tail = ["-L" + lib64, "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    return _build("_dlm_kernels", jobs, tail, cu + cpp + _headers(), nv_flags + cx_flags)


def _load(name: str, path: str):
    spec = importlib.util.spec_from_file_location(name, path)
    if spec is None or spec.loader is None:
        raise BuildError(f"cannot load {path}")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[name] = mod
    return mod


_loaded: dict[str, object] = {}


def load_host():
    """The host runtime module (built on first use)."""
    if "_dlm_host" not in _loaded:
        _loaded["_dlm_host"] = _load("_dlm_host", build_host())
    return _loaded["_dlm_host"]


def load_kernels():
    """The kernel module (built on first use).  There is no fallback: a failure to build
    or load it is an error for every caller."""
    if "_dlm_kernels" not in _loaded:
        _loaded["_dlm_kernels"] = _load("_dlm_kernels", build_kernels())
    return _loaded["_dlm_kernels"]


def kernels_library_path() -> str:
    """Path of the built kernel library (for callers that bind its C symbols)."""
    return build_kernels()


if __name__ == "__main__":
    build_host()
    build_kernels()
