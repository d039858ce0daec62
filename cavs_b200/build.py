"""In-tree build of libcavs_b200.so (host C++ + sm_100a CUDA kernels behind the C ABI).

    python -m cavs_b200.build [--force] [--verbose]

Every .cc/.cu under cavs_b200/csrc is compiled with nvcc for sm_100a only
(-gencode arch=compute_100a,code=sm_100a) and linked into one shared library next
to this file.  Objects are cached under cavs_b200/build/ and rebuilt when the
source or any header is newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libcavs_b200.so"

NVCC = os.environ.get("CAVS_NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", f"-I{ROOT / 'include'}", f"-I{CSRC}", "-Xcompiler", "-fPIC,-Wall,-fvisibility=hidden"]
CUFLAGS = ["--expt-relaxed-constexpr", "-Xptxas", "-v" if os.environ.get("CAVS_PTXAS_V") else "-O3"]


def _sources():
    return sorted(list(CSRC.rglob("*.cc")) + list(CSRC.rglob("*.cu")))


def _headers_mtime() -> float:
    hs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [NVCC, *ARCH, *COMMON]
    if src.suffix == ".cu":
        cmd += CUFLAGS
    else:
        cmd += ["-x", "cu"] if False else []
    cmd += ["-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    out = (r.stdout + r.stderr).strip()
    if verbose and out:
        return f"--- {src.name}\n{out}"
    return ""


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    hdr_m = _headers_mtime()
    jobs, objs = [], []
    for src in _sources():
        obj = OBJ / (str(src.relative_to(CSRC)).replace("/", "__") + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            for msg in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
                if msg:
                    print(msg)
    stale = [o for o in OBJ.glob("*.o") if o not in objs]
    for o in stale:
        o.unlink()
    if jobs or force or not LIB.exists():
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-ldl", "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return LIB


HOST_LIB = PKG / "libcavs_host.so"
HOST_SRC = PKG / "cavs"
CPP_TESTS = ROOT / "tests" / "cpp"
CXX = os.environ.get("CAVS_CXX", "g++")
CUDA_HOME = Path(NVCC).resolve().parent.parent


def build_host(force: bool = False) -> Path:
    """libcavs_host.so: the C++ mirror of the reference's operator interface (cavs/backend, cavs/midend)
    on top of the C ABI.  Plain g++; links libcavs_b200.so and the CUDA runtime."""
    srcs = sorted(HOST_SRC.rglob("*.cc"))
    hdrs = list(HOST_SRC.rglob("*.h")) + list((ROOT / "include").glob("*.h"))
    newest = max(p.stat().st_mtime for p in srcs + hdrs + [LIB])
    if force or not HOST_LIB.exists() or HOST_LIB.stat().st_mtime < newest:
        cmd = [CXX, "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", f"-I{ROOT / 'include'}", f"-I{PKG}", f"-I{CUDA_HOME / 'include'}",
               *map(str, srcs), "-o", str(HOST_LIB), f"-L{PKG}", "-lcavs_b200", f"-L{CUDA_HOME / 'lib64'}", "-lcudart", "-ldl",
               "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"host library failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return HOST_LIB


def build_cpp_tests(force: bool = False) -> list[Path]:
    """tests/cpp/*.cc -> tests/cpp/bin/<name>; they link the host library and the test oracle."""
    out_dir = CPP_TESTS / "bin"
    out_dir.mkdir(exist_ok=True)
    oracle_dir = ROOT / "oracle"
    built = []
    for src in sorted(CPP_TESTS.glob("*.cc")):
        exe = out_dir / src.stem
        built.append(exe)
        deps = [src, HOST_LIB, oracle_dir / "libcavs_oracle.so"]
        if not force and exe.exists() and all(exe.stat().st_mtime >= d.stat().st_mtime for d in deps if d.exists()):
            continue
        cmd = [CXX, "-std=c++17", "-O1", "-Wall", f"-I{ROOT / 'include'}", f"-I{PKG}", f"-I{CUDA_HOME / 'include'}", str(src), "-o", str(exe),
               f"-L{PKG}", "-lcavs_host", "-lcavs_b200", f"-L{oracle_dir}", "-lcavs_oracle", f"-L{CUDA_HOME / 'lib64'}", "-lcudart",
               f"-Wl,-rpath,{PKG}", f"-Wl,-rpath,{oracle_dir}", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"C++ test failed to build: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return built


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
    print(build_host(force="--force" in sys.argv))
