"""In-tree build of libk44wavec.so with nvcc for sm_100a (no JIT cache: the built library travels
with the source tree). Run as `python -m snntome_b200.build` or through `__graft_entry__.build()`."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libk44wavec.so"
SOURCES = ["k44_kernels.cu", "k44_stream_n64.cu", "k44_stream_n128.cu", "k44_stream_n256.cu", "k44_pair_kernel.cu", "k44_shift_kernel.cu", "k44_shift_ws_kernel.cu", "k44_mma_kernel.cu", "k44_valu.cu", "k44_image.cu", "k44_exec.cu", "k44_capi.cu", "k44_static.cu", "k44_peer.cu"]
HEADERS = ["k44_host.hpp", "k44_tcff.hpp", "k44_graph.hpp", "k44_kernels.cuh", "k44_epilogue.cuh", "k44_ptx.cuh", "k44_stream_kernel.cuh", "k44_exec.hpp"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return cand


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [PKG.parent / "include" / "k44b.h", PKG.parent / "include" / "k44wavec.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    obj_dir = PKG / "build"
    obj_dir.mkdir(exist_ok=True)
    common = [nvcc, "-std=c++17", "-O3", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC,-Wall", "-ccbin", "g++"]
    if verbose:
        common += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for s in SOURCES:
        o = obj_dir / (s.rsplit(".", 1)[0] + ".o")
        objs.append(str(o))
        procs.append((s, subprocess.Popen(common + ["-c", str(CSRC / s), "-o", str(o)], stdout=subprocess.PIPE,
                                          stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(f"--- {s}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, "-shared", *ARCH, "-o", str(LIB), *objs, "-cudart", "static", "-ccbin", "g++"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
