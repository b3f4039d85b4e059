"""Builds the native parts of the package in-tree.

  neoml_b200/lib/libneoml_b200.so      CUDA kernels + C ABI (include/neoml_b200.h), sm_100a only
  neoml_b200/lib/libNeoMathEngineB200.so  C++ IMathEngine implementation over that C ABI; compiled against the
                                       NeoMathEngine headers of a NeoML checkout ($NEOML_REFERENCE_DIR), so it is
                                       only (re)built where such a checkout exists

Run as `python -m neoml_b200.build`.  nvcc cross-compiles for sm_100a without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build"
INCLUDE = ROOT.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--ftz=true", "-Xptxas", "-v",
]


def _newer(src: Path, dst: Path, deps: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def build_kernels(verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    objs = []

    def compile_one(src: Path) -> tuple[Path, str]:
        obj = OBJ / (src.stem + ".o")
        log = ""
        if _newer(src, obj, headers):
            cmd = ["nvcc", *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            log = r.stdout + r.stderr
            (OBJ / (src.stem + ".ptxas.log")).write_text(log)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src.name}:\n{log}")
        return obj, log

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for obj, log in ex.map(compile_one, sources):
            objs.append(obj)
            if verbose and log:
                print(log)
    out = LIB / "libneoml_b200.so"
    if not out.exists() or any(o.stat().st_mtime > out.stat().st_mtime for o in objs):
        cmd = ["nvcc", "-shared", "-o", str(out), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return out


def reference_dir() -> Path:
    return Path(os.environ.get("NEOML_REFERENCE_DIR", "/root/reference"))


def build_hosted(verbose: bool = False) -> Path | None:
    """make -C neoml_b200/host: NeoML (unmodified) + a libNeoMathEngine.so with this repository's factory and engine +
    the CDnn harness, into neoml_b200/lib/host.  Needs a NeoML checkout; where there is none the prebuilt files stay."""
    out = LIB / "host" / "libcdnn_host.so"
    if not (reference_dir() / "NeoML" / "src").exists():
        return out if out.exists() else None
    r = subprocess.run(["make", "-C", str(ROOT / "host"), f"-j{min(8, os.cpu_count() or 1)}", f"REF={reference_dir()}",
                        f"PYTHON={sys.executable}"], capture_output=True, text=True)
    if verbose:
        print(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"hosted build failed:\n{r.stdout[-3000:]}{r.stderr[-3000:]}")
    return out


def build_engine(verbose: bool = False) -> Path | None:
    """g++ build of the IMathEngine implementation.  The class is generated/compiled against the NeoMathEngine headers
    of a NeoML checkout; the base-class symbols (IMathEngine's key functions, the exception handler, CBlobDesc) stay
    undefined in this library and bind at load time to the libNeoMathEngine.so of the hosting NeoML process."""
    ref = reference_dir()
    eng = ROOT / "engine"
    out = LIB / "libNeoMathEngineB200.so"
    sources = sorted(eng.glob("*.cpp"))
    header = ref / "NeoMathEngine" / "include" / "NeoMathEngine" / "NeoMathEngine.h"
    if not sources:
        return None
    if not header.exists():
        return out if out.exists() else None
    LIB.mkdir(exist_ok=True)
    gen = OBJ / "engine_gen"
    deps = sorted(eng.glob("*.h")) + sorted(eng.glob("*.py")) + sorted(INCLUDE.glob("*.h")) + [header]
    if out.exists() and not any(_newer(s, out, deps) for s in sources):
        return out
    r = subprocess.run([sys.executable, str(eng / "gen_stubs.py"), str(header), str(gen)], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"stub generation failed:\n{r.stdout}{r.stderr}")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-D_LINUX", "-w",
           f"-I{ref}/NeoMathEngine/include", f"-I{INCLUDE}", f"-I{eng}", f"-I{gen}", "-I/usr/local/cuda/include",
           *map(str, sources), str(gen / "B200MathEngineStubs.cpp"), "-o", str(out),
           f"-L{LIB}", "-lneoml_b200", "-L/usr/local/cuda/lib64", "-lcudart_static", "-ldl", "-lrt", "-lpthread",
           "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        print(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"engine build failed:\n{r.stdout}{r.stderr}")
    return out


def main() -> None:
    verbose = "-v" in sys.argv
    print(build_kernels(verbose))
    print(build_engine(verbose))
    print(build_hosted(verbose))


if __name__ == "__main__":
    main()
