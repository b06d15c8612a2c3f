"""Builds the two shared libraries of the package with nvcc, in-tree.

  diopi_b200/lib/libdiopi_impl.so  the backend: exported DIOPI ops + sm_100a kernels
  diopi_b200/lib/libdiopi_rt.so    the consumer-side test run time (tensor/context handles)

The backend leaves the diopirt accessors (diopiGetTensorData, diopiGetStream, ...)
undefined, as a DIOPI backend does (impl/CMakeLists.txt:45-46 builds one
libdiopi_impl.so that resolves them from its consumer); everything except the
exported C symbols has hidden visibility. Run as ``python -m diopi_b200.build``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = ROOT / "build" / "obj"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = [
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    f"-I{ROOT / 'include'}", f"-I{CSRC}",
]

IMPL_SOURCES = [
    "abi/common.cpp",
    "abi/exports.cpp",
    "abi/tp_group.cpp",
    "kernels/dest_index_copy.cu",
    "kernels/token_decode.cu",
    "kernels/token_decode_gqa.cu",
    "kernels/rms_norm.cu",
    "kernels/rms_norm_backward.cu",
    "kernels/rotary.cu",
    "kernels/apply_penalty.cu",
    "kernels/context_attention.cu",
    "kernels/context_attention_sm100.cu",
    "kernels/matmul_allreduce.cu",
]
RT_SOURCES = ["rt/testrt.cpp"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build diopi_b200")
    return exe


def _headers_stamp() -> str:
    h = hashlib.sha1()
    for p in sorted(list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.cuh")) + list((ROOT / "include").glob("*.h"))):
        h.update(p.read_bytes())
    h.update(" ".join(COMMON + ARCH).encode())
    return h.hexdigest()[:16]


def _compile(src: str, stamp: str, verbose: bool) -> Path:
    s = CSRC / src
    o = OBJ / (src.replace("/", "_") + f".{stamp}.o")
    if o.exists() and o.stat().st_mtime >= s.stat().st_mtime:
        return o
    for old in OBJ.glob(src.replace("/", "_") + ".*.o"):
        old.unlink()
    cmd = [nvcc(), "-x", "cu", *ARCH, *COMMON, "-c", str(s), "-o", str(o)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if verbose or r.stderr.strip():
        sys.stderr.write(r.stderr)
    return o


def _link(objs: list[Path], out: Path, extra: list[str]) -> None:
    cmd = [nvcc(), *ARCH, "-shared", "-cudart", "static", "-o", str(out), *map(str, objs), *extra]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link of {out.name} failed:\n{r.stdout}\n{r.stderr}")


def _sources_stamp() -> str:
    h = hashlib.sha1(_headers_stamp().encode())
    for src in IMPL_SOURCES + RT_SOURCES:
        h.update((CSRC / src).read_bytes())
    return h.hexdigest()


def build(verbose: bool = False, jobs: int | None = None) -> dict[str, Path]:
    """Compiles what is out of date and returns the paths of the two libraries.

    lib/build_stamp.txt holds a hash of every source, header and flag the libraries were built from;
    when it matches, nothing is compiled (file times do not survive a copy of the tree, hashes do)."""
    LIB.mkdir(parents=True, exist_ok=True)
    impl = LIB / "libdiopi_impl.so"
    rt = LIB / "libdiopi_rt.so"
    stamp_file = LIB / "build_stamp.txt"
    full = _sources_stamp()
    if not verbose and impl.exists() and rt.exists() and stamp_file.exists() and stamp_file.read_text().strip() == full:
        return {"impl": impl, "rt": rt}
    OBJ.mkdir(parents=True, exist_ok=True)
    stamp = _headers_stamp()
    jobs = jobs or min(8, os.cpu_count() or 1)
    with ThreadPoolExecutor(jobs) as ex:
        impl_objs = list(ex.map(lambda s: _compile(s, stamp, verbose), IMPL_SOURCES))
        rt_objs = list(ex.map(lambda s: _compile(s, stamp, verbose), RT_SOURCES))
    _link(impl_objs, impl, [])
    _link(rt_objs, rt, [])
    stamp_file.write_text(full + "\n")
    return {"impl": impl, "rt": rt}


if __name__ == "__main__":
    paths = build(verbose="-v" in sys.argv)
    for k, v in paths.items():
        print(f"{k}: {v}")
