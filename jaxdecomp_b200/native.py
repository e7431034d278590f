"""Build and load the native core (``_jdb200``: CUDA kernels for sm_100a plus
the C++ runtime around them).

The shared object is built in-tree, next to this file, with explicit ``nvcc``
commands (``-gencode arch=compute_100a,code=sm_100a``), so that it travels with
the source tree to machines that have a GPU.  A content hash of the sources is
stored beside it; the library is rebuilt only when the sources changed.  The
reference builds its native module with CMake/scikit-build against cuDecomp
(``CMakeLists.txt:1-123``); this build has no third-party dependency besides
the CUDA toolkit and pybind11.

Two variants of the library exist.  The normal one, and a checked one
(``_jdb200_bounds``: same sources compiled with ``-DJD_BOUNDS_CHECK=1``) in
which every store of every tile pass and halo kernel is compared with the size
of its destination buffer first; a store that would leave the buffer is
skipped and reported as ``BOUNDS`` through the status block.  Setting
``JD_B200_BOUNDS=1`` before the package is imported selects the checked
variant (several times slower; for debugging new plans and for the tests).
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
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Optional

from .utils.errors import NativeExtensionError

_HERE = Path(__file__).resolve().parent
_CSRC = _HERE / "csrc"
_EXT = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
BOUNDS = os.environ.get("JD_B200_BOUNDS", "0") not in ("", "0")


def _variant_paths(bounds: bool):
    stem = "_jdb200_bounds" if bounds else "_jdb200"
    return _HERE / (stem + _EXT), _HERE / (stem + ".hash"), _CSRC / ("build_bounds" if bounds else "build")


_SO, _HASH, _OBJ = _variant_paths(BOUNDS)

SOURCES = [
    "bindings.cpp",
    "runtime.cpp",
    "arena.cpp",
    "tables.cpp",
    "trace.cpp",
    "cpu_ref.cpp",
    "fft_pass.cu",
    "copy_fast.cu",
    "fft_fast.cu", "fft_mixed.cu", "fft_mixed_sa.cu", "fft_mixed_sb.cu", "fft_mixed_sc.cu",
    "signal.cu",
    "halo.cu",
    "cic.cu",
    "kspace.cu",
    "no_alloc.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]

_module = None
_load_error: Optional[str] = None


def _nvcc() -> Optional[str]:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def _existing_sources():
    return [s for s in SOURCES if (_CSRC / s).exists()]


def _source_hash() -> str:
    h = hashlib.sha256()
    files = sorted(p for p in _CSRC.iterdir() if p.suffix in (".cu", ".cpp", ".h", ".cuh"))
    for p in files:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_built(bounds: Optional[bool] = None) -> bool:
    so, hsh, _ = _variant_paths(BOUNDS if bounds is None else bounds)
    return so.exists() and hsh.exists() and hsh.read_text().strip() == _source_hash()


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, bounds: Optional[bool] = None) -> Path:
    """Compile every source for sm_100a and link ``_jdb200`` (or, with ``bounds=True``, the checked
    variant ``_jdb200_bounds``; default: the variant this process uses).  Safe to call from several
    processes at once (file lock); a no-op when the library is current."""
    nvcc = _nvcc()
    if nvcc is None:
        raise NativeExtensionError("nvcc not found; cannot build the native core")
    bounds = BOUNDS if bounds is None else bool(bounds)
    _SO, _HASH, _OBJ = _variant_paths(bounds)
    _OBJ.mkdir(parents=True, exist_ok=True)
    lock_path = _OBJ / ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if is_built(bounds) and not force:
                return _SO
            import pybind11

            inc = ["-I", sysconfig.get_paths()["include"], "-I", pybind11.get_include(), "-I", str(_CSRC)]
            flags = list(NVCC_FLAGS)
            if bounds:
                flags += ["-DJD_BOUNDS_CHECK=1"]
            if ptxas_info:
                flags += ["-Xptxas", "-v"]

            def compile_one(src: str):
                obj = _OBJ / (src + ".o")
                cmd = [nvcc, *flags, *inc, "-c", str(_CSRC / src), "-o", str(obj)]
                r = subprocess.run(cmd, capture_output=True, text=True)
                if r.returncode != 0:
                    raise NativeExtensionError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
                if verbose or ptxas_info:
                    sys.stderr.write(r.stderr)
                return obj

            with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
                objs = list(ex.map(compile_one, _existing_sources()))
            tmp = _SO.with_suffix(".tmp")
            cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs], "-ldl", "-lpthread",
                   "-gencode", "arch=compute_100a,code=sm_100a"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise NativeExtensionError(f"link failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, _SO)
            _HASH.write_text(_source_hash())
            return _SO
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


HOST_SELFTEST_SOURCES = ["host_selftest.cpp", "cpu_ref.cpp", "tables.cpp"]


_SAN_FLAGS = ["-fsanitize=address,undefined", "-fno-sanitize-recover=all"]
_sanitizer_cxx: Optional[str] = None


def sanitizer_compiler() -> Optional[str]:
    """A C++ compiler that can link a program with the AddressSanitizer and UndefinedBehaviorSanitizer
    run-times (``$CXX`` first, then ``g++`` on the path), or ``None``."""
    global _sanitizer_cxx
    if _sanitizer_cxx is not None:
        return _sanitizer_cxx or None
    import tempfile

    cands = [c for c in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++") if c]
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "probe.cpp"
        src.write_text("int main() { return 0; }\n")
        for cxx in dict.fromkeys(cands):
            try:
                r = subprocess.run([cxx, *_SAN_FLAGS, str(src), "-o", str(Path(tmp) / "probe")], capture_output=True)
            except OSError:
                continue
            if r.returncode == 0:
                _sanitizer_cxx = cxx
                return cxx
    _sanitizer_cxx = ""
    return None


def build_host_selftest(force: bool = False) -> Path:
    """Compile the host side of the core (CPU emulation of the tile pass, table construction) together
    with ``csrc/host_selftest.cpp`` into a stand-alone program under AddressSanitizer and
    UndefinedBehaviorSanitizer (``g++ -fsanitize=address,undefined``, reports abort the program).  The
    program replays pass descriptors written by the planner; ``tests/test_sanitizer_cpu.py`` drives it.
    Needs g++ with the sanitizer run-times and the CUDA headers and run-time library (``tables.cpp`` also
    holds the device-table path, which this program never takes); no GPU."""
    cxx = sanitizer_compiler()
    nvcc = _nvcc()
    if cxx is None or nvcc is None:
        raise NativeExtensionError("no C++ compiler with the sanitizer run-times, or no CUDA toolkit: cannot build "
                                   "the sanitizer self-test")
    cuda_root = Path(nvcc).resolve().parent.parent
    out_dir = _CSRC / "build_sanitize"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe, stamp = out_dir / "host_selftest", out_dir / "host_selftest.hash"
    with open(out_dir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if exe.exists() and stamp.exists() and stamp.read_text().strip() == _source_hash() and not force:
                return exe
            libdir = next((d for d in (cuda_root / "lib64", cuda_root / "targets" / "x86_64-linux" / "lib")
                           if (d / "libcudart.so").exists()), cuda_root / "lib64")
            cmd = [cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *_SAN_FLAGS, "-I", str(cuda_root / "include"), "-I", str(_CSRC),
                   *[str(_CSRC / s) for s in HOST_SELFTEST_SOURCES], "-o", str(exe),
                   "-L", str(libdir), f"-Wl,-rpath,{libdir}", "-lcudart", "-lpthread", "-ldl"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise NativeExtensionError(f"sanitizer self-test failed to build:\n{r.stdout}\n{r.stderr}")
            stamp.write_text(_source_hash())
            return exe
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def load(build_if_needed: bool = True):
    """Import the native module, building it first if it is missing or stale."""
    global _module, _load_error
    if _module is not None:
        return _module
    try:
        if not is_built():
            if not build_if_needed:
                raise NativeExtensionError("native core is not built; run `python -m jaxdecomp_b200.native`")
            build()
        spec = importlib.util.spec_from_file_location("jaxdecomp_b200._jdb200", str(_SO))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules["jaxdecomp_b200._jdb200"] = mod
        _module = mod
        return mod
    except Exception as e:  # noqa: BLE001
        _load_error = f"{type(e).__name__}: {e}"
        raise


def available() -> bool:
    """True when the native module can be imported (it also works, for the CPU
    emulation and the host-side utilities, on a machine without a GPU)."""
    try:
        load()
        return True
    except Exception:  # noqa: BLE001
        return False


def require():
    """Return the native module or raise a loud, explicit error."""
    try:
        return load()
    except Exception as e:  # noqa: BLE001
        raise NativeExtensionError(
            "the native sm_100a core of jaxdecomp_b200 could not be built or loaded "
            f"({_load_error or e}); refusing to fall back to library kernels on a CUDA tensor"
        ) from e


def so_path() -> Path:
    return _SO


if __name__ == "__main__":
    # python -m jaxdecomp_b200.native [--force] [--ptxas] [--bounds] | --selftest
    if "--selftest" in sys.argv:
        print(build_host_selftest(force="--force" in sys.argv))
    else:
        print(build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv,
                    bounds=True if "--bounds" in sys.argv else None))
