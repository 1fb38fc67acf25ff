"""In-tree native build: every CUDA source is compiled for sm_100a into
``ksanallm_b200/lib/libksana_kernels.so`` (plain C ABI, loaded with ctypes) and the C++
host runtime into the pybind11 module ``ksanallm_b200/lib/_ksana_engine*.so``.

Run ``python -m ksanallm_b200.build`` (add ``--force`` to rebuild everything). The build
needs nvcc and g++ but no GPU; objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wno-unused-function",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall", "-Wno-sign-compare"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")
    return r.stdout + r.stderr


def kernels_lib_path() -> Path:
    return LIB / "libksana_kernels.so"


def engine_lib_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return LIB / f"_ksana_engine{suffix}"


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    kdir = CSRC / "kernels"
    srcs = sorted(kdir.glob("*.cu"))
    hdrs = sorted(kdir.glob("*.cuh")) + sorted(kdir.glob("*.h"))
    objs = []
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if force or _newer(o, [s, *hdrs]):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(kdir), "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            outs = list(ex.map(_run, jobs))
        if verbose:
            print("\n".join(outs))
    out = kernels_lib_path()
    if force or jobs or not out.exists():
        _run([_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    return out


def build_engine(force: bool = False) -> Path:
    import pybind11

    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    edir = CSRC / "engine"
    srcs = sorted(edir.glob("*.cpp"))
    hdrs = sorted(edir.glob("*.h"))
    inc = ["-I", str(edir), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    objs, jobs = [], []
    for s in srcs:
        o = OBJ / ("eng_" + s.stem + ".o")
        objs.append(o)
        if force or _newer(o, [s, *hdrs]):
            jobs.append(["g++", *CXX_FLAGS, *inc, "-c", str(s), "-o", str(o)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    out = engine_lib_path()
    if force or jobs or not out.exists():
        _run(["g++", "-shared", "-pthread", "-o", str(out), *map(str, objs), "-ldl"])
    return out


def build_host_stress(sanitizer: str = "thread") -> Path:
    """Stand-alone stress driver of the scheduler / cache manager / control plane (csrc/engine/host_stress.cpp)
    compiled with -fsanitize=<thread|address|undefined>; run the returned binary, it exits 0 when clean."""
    OBJ.mkdir(exist_ok=True)
    edir = CSRC / "engine"
    srcs = [edir / n for n in ("host_stress.cpp", "scheduler.cpp", "cache_manager.cpp", "control_channel.cpp", "logger.cpp", "batch_loop.cpp",
                                 "otlp_export.cpp")]
    out = OBJ / f"host_stress_{sanitizer}"
    if _newer(out, [*srcs, *sorted(edir.glob("*.h"))]):
        _run(["g++", "-O1", "-g", "-std=c++17", "-pthread", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer",
              "-DKSANA_NO_PYBIND", "-I", str(edir), *map(str, srcs), "-o", str(out)])
    return out


def build_client() -> Path:
    """The stand-alone C++ /forward client (csrc/client/serving_forward_client.cpp) -> lib/serving_forward_client."""
    LIB.mkdir(exist_ok=True)
    src = CSRC / "client" / "serving_forward_client.cpp"
    codec = CSRC / "engine" / "request_packer.cpp"
    out = LIB / "serving_forward_client"
    if _newer(out, [src, codec, CSRC / "engine" / "request_packer.h"]):
        _run(["g++", "-O2", "-std=c++17", "-Wall", "-DKSANA_NO_PYBIND", str(src), str(codec), "-o", str(out)])
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_engine(force)


if __name__ == "__main__":
    if "--client" in sys.argv:
        print(build_client())
        sys.exit(0)
    if "--sanitizer" in sys.argv:
        print(build_host_stress(sys.argv[sys.argv.index("--sanitizer") + 1]))
        sys.exit(0)
    k, e = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(k)
    print(e)
