"""Builds lib/libcml_b200.so: every csrc/*.cu with nvcc for sm_100a, every csrc/*.c and
host/*.c with gcc -std=c11, linked into one shared library that exports the cmlb200 C-ABI
and the C-ML-compatible host API -- exactly the functions and variables the two public headers
declare (a linker version script generated from include/*.h hides everything else).
Incremental (mtime based). No GPU is needed to build."""
import os
import re
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libcml_b200.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
CC_FLAGS = ["-std=c11", "-O2", "-fPIC", "-Wall", "-Wextra", "-D_POSIX_C_SOURCE=200809L"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the CUDA extension cannot be built")


def _headers():
    return list((ROOT / "include").glob("*.h")) + list((PKG / "csrc").glob("*.cuh")) + list((PKG / "host").glob("*.h"))


def _stale(out: Path, deps) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _compile(src: Path, verbose: bool):
    obj = OBJ / (src.parent.name + "_" + src.stem + ".o")
    if not _stale(obj, [src] + _headers()):
        return obj, None
    inc = ["-I", str(ROOT / "include"), "-I", str(PKG / "csrc"), "-I", str(PKG / "host")]
    if src.suffix == ".cu":
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + inc + ["-c", str(src), "-o", str(obj)]
    else:
        cmd = [os.environ.get("CC", "gcc")] + CC_FLAGS + inc + ["-I", "/usr/local/cuda/include", "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return obj, (r.stdout + r.stderr)


def public_symbols():
    """Names the public headers declare: every function prototype and every `extern` variable."""
    names = set()
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}()]*(?:\([^()]*\)[^;{}()]*)*\)\s*;", text):
            if m.group(1) not in ("defined", "sizeof", "__attribute__"):
                names.add(m.group(1))
        for m in re.finditer(r"\bextern\s+(?!\"C\")[^;()]*?\b([A-Za-z_][A-Za-z0-9_]*)\s*(?:\[[^\]]*\])?\s*;", text):
            names.add(m.group(1))
    return sorted(names)


def _version_script() -> Path:
    path = OBJ / "exports.map"
    body = "{\n  global:\n" + "".join(f"    {n};\n" for n in public_symbols()) + "  local: *;\n};\n"
    if not path.exists() or path.read_text() != body:
        path.write_text(body)
    return path


def build(verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted((PKG / "csrc").glob("*.cu")) + sorted((PKG / "csrc").glob("*.c")) + sorted((PKG / "host").glob("*.c"))
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    vs = _version_script()
    if _stale(LIB, objs + [vs]):
        cmd = [_nvcc(), "-shared", "-o", str(LIB)] + [str(o) for o in objs] + ["-Xlinker", "-Bsymbolic", "-Xlinker", f"--version-script={vs}",
                                                                             "-lcudart_static", "-ldl", "-lpthread", "-lrt", "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
