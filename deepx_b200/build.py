"""Build recipe for the native libraries (sm_100a only).

``python -m deepx_b200.build`` compiles every ``csrc/kernels/*.cu`` into
``deepx_b200/libdeepx_b200.so`` (the C ABI declared in ``include/dx_kernels.h``)
and every ``csrc/host/*.cpp`` + ``csrc/host/*.cu`` into ``deepx_b200/libdeepx_exec.so``
and the executables ``deepx_b200/deepx-op-b200`` (the executor) and ``deepx_b200/deepx-heapmem``
(the heap-tensor service).  nvcc cross-compiles
without a GPU.  Objects are cached under ``build/`` by source mtime.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = ROOT / "build"
INCLUDE = ROOT / "include"

NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", f"-I{INCLUDE}",
          f"-I{CSRC / 'kernels'}", f"-I{CSRC / 'host'}"]

KERNEL_LIB = PKG / "libdeepx_b200.so"
EXEC_LIB = PKG / "libdeepx_exec.so"
EXEC_BIN = PKG / "deepx-op-b200"
HEAP_BIN = PKG / "deepx-heapmem"
# one executable per csrc/host/*_main.cpp
MAIN_BINARIES = {"host_udp_main.o": EXEC_BIN, "host_heapmem_main.o": HEAP_BIN}


def _newest_header() -> float:
    hs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, extra: list[str], hdr_mtime: float, verbose: bool) -> Path:
    obj = OBJ / (src.parent.name + "_" + src.stem + ".o")
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return obj
    cmd = [NVCC, *ARCH, *COMMON, *extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, flush=True)
    return obj


def _link(objs: list[Path], out: Path, shared: bool, libs: list[str], verbose: bool) -> None:
    if out.exists() and all(out.stat().st_mtime > o.stat().st_mtime for o in objs):
        return
    cmd = [NVCC, *ARCH, "-o", str(out), *map(str, objs), "-cudart", "static", *libs]
    if shared:
        cmd.insert(1, "-shared")
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed for {out.name}:\n{r.stdout}\n{r.stderr}")


def build(verbose: bool = False, ptxas_info: bool = False) -> dict[str, Path]:
    """Compile and link everything; returns the artefact paths."""
    OBJ.mkdir(exist_ok=True)
    hdr = _newest_header()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    ksrcs = sorted((CSRC / "kernels").glob("*.cu"))
    hsrcs = sorted(list((CSRC / "host").glob("*.cpp")) + list((CSRC / "host").glob("*.cu"))) if (CSRC / "host").exists() else []
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        kfut = [ex.submit(_compile, s, extra, hdr, verbose) for s in ksrcs]
        hfut = [ex.submit(_compile, s, ["-x", "cu"] + extra, hdr, verbose) for s in hsrcs]
        kobjs = [f.result() for f in kfut]
        hobjs = [f.result() for f in hfut]
    _link(kobjs, KERNEL_LIB, True, [], verbose)
    out = {"kernels": KERNEL_LIB}
    if hobjs:
        lib_objs = [o for o in hobjs if not o.name.endswith("_main.o")]
        main_objs = [o for o in hobjs if o.name.endswith("_main.o")]
        _link(lib_objs + kobjs, EXEC_LIB, True, ["-lpthread"], verbose)
        out["exec"] = EXEC_LIB
        for m in main_objs:
            target = MAIN_BINARIES.get(m.name)
            if target is None:
                raise RuntimeError(f"no executable name for {m.name}: add it to MAIN_BINARIES")
            _link([m] + lib_objs + kobjs, target, False, ["-lpthread"], verbose)
            out["bin" if target == EXEC_BIN else target.name] = target
    return out


if __name__ == "__main__":
    arts = build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    for k, v in arts.items():
        print(f"{k}: {v}")
