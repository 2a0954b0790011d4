"""In-tree native build: compiles the C++ runtime and the sm_100a kernels into
shared objects that sit next to the Python packages that load them.

    python -m dataflow_b200.build            # build what is out of date
    python -m dataflow_b200.build --force    # rebuild everything

Nothing is installed outside the source tree and nothing is compiled at import
time: a fresh GPU machine that receives the tree with the built ``.so`` files
can import and run immediately.  CUDA code is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``).
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def _pybind_includes() -> list[str]:
    import pybind11
    return [f"-I{sysconfig.get_paths()['include']}", f"-I{pybind11.get_include()}"]


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce
    inc = [f"-I{p}" for p in ce.include_paths()]
    lib = Path(torch.__file__).parent / "lib"
    return inc, lib


def _cutlass_include() -> list[str]:
    """CUTLASS / CuTe headers vendored inside site-packages (header-only use)."""
    import site
    for sp in site.getsitepackages():
        for rel in ("flashinfer/data/cutlass/include", "tilelang/3rdparty/cutlass/include"):
            p = Path(sp) / rel
            if (p / "cute" / "tensor.hpp").exists():
                return [f"-I{p}"]
    return []


def _stale(out: Path, deps: list[Path], cmd_sig: str) -> bool:
    sig = out.with_suffix(out.suffix + ".sig")
    if not out.exists() or not sig.exists() or sig.read_text() != cmd_sig:
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} ... {cmd[-1]}")
    if r.stderr.strip() and os.environ.get("DFB_BUILD_VERBOSE"):
        sys.stderr.write(r.stderr)


def _compile_objects(jobs: list[tuple[list[str], Path, list[Path]]], force: bool) -> bool:
    """jobs: (command, output, deps).  Returns True if anything was rebuilt."""
    todo = []
    for cmd, out, deps in jobs:
        sig = hashlib.sha256(" ".join(cmd).encode()).hexdigest()
        if force or _stale(out, deps, sig):
            todo.append((cmd, out, sig))
    if not todo:
        return False
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
        list(ex.map(lambda j: _run(j[0]), todo))
    for _, out, sig in todo:
        out.with_suffix(out.suffix + ".sig").write_text(sig)
    return True


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    src = ROOT / "runtime" / "csrc"
    obj = ROOT / "runtime" / "csrc" / "build"
    obj.mkdir(exist_ok=True)
    hdrs = list(src.glob("*.hpp"))
    inc = _pybind_includes() + [f"-I{CUDA_HOME}/include", f"-I{src}"]
    cxx = ["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-DDFB_WITH_CUDA", "-Wall", "-Wno-sign-compare"]
    jobs = []
    for f in ("engine.cpp", "backends_host.cpp", "backend_cuda.cpp", "vmm.cpp", "bindings.cpp"):
        o = obj / (f + ".o")
        jobs.append((cxx + inc + ["-c", str(src / f), "-o", str(o)], o, [src / f] + hdrs))
    o = obj / "spin.cu.o"
    jobs.append(([NVCC, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-lineinfo"] + ARCH_FLAGS +
                 ["-c", str(src / "spin.cu"), "-o", str(o)], o, [src / "spin.cu"]))
    changed = _compile_objects(jobs, force)
    out = ROOT / "runtime" / ("_runtime" + EXT_SUFFIX)
    if changed or not out.exists():
        _run(["g++", "-shared", "-o", str(out)] + [str(j[1]) for j in jobs] +
             [f"-L{CUDA_HOME}/lib64", "-lcudart", f"-Wl,-rpath,{CUDA_HOME}/lib64", "-lpthread", "-ldl"])
    return out


def ops_sources() -> list[Path]:
    return sorted((ROOT / "ops" / "csrc").glob("*.cu")) + sorted((ROOT / "ops" / "csrc").glob("*.cpp"))


def build_ops(force: bool = False, verbose: bool = False) -> Path:
    src = ROOT / "ops" / "csrc"
    obj = src / "build"
    obj.mkdir(exist_ok=True)
    tinc, tlib = _torch_paths()
    hdrs = list(src.glob("*.cuh")) + list(src.glob("*.h")) + list(src.glob("*.hpp"))
    inc = tinc + [f"-I{sysconfig.get_paths()['include']}", f"-I{src}"] + _cutlass_include()
    common = ["-O3", "-std=c++17", "-DTORCH_EXTENSION_NAME=_ops", "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=1"]
    nv = [NVCC] + common + ["-Xcompiler", "-fPIC", "-lineinfo", "--expt-relaxed-constexpr",
                            "--expt-extended-lambda", "-Xptxas", "-v" if verbose else "-O3",
                            "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                            "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"] + ARCH_FLAGS
    cxx = ["g++"] + common + ["-fPIC", "-Wno-unused-variable"]
    jobs = []
    for f in ops_sources():
        o = obj / (f.name + ".o")
        if f.suffix == ".cu":
            jobs.append((nv + inc + ["-c", str(f), "-o", str(o)], o, [f] + hdrs))
        else:
            jobs.append((cxx + inc + [f"-I{CUDA_HOME}/include", "-c", str(f), "-o", str(o)], o, [f] + hdrs))
    changed = _compile_objects(jobs, force)
    out = ROOT / "ops" / ("_ops" + EXT_SUFFIX)
    if changed or not out.exists():
        _run(["g++", "-shared", "-o", str(out)] + [str(j[1]) for j in jobs] +
             [f"-L{tlib}", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
              f"-L{CUDA_HOME}/lib64", "-lcudart", "-ldl",
              f"-Wl,-rpath,{tlib}", f"-Wl,-rpath,{CUDA_HOME}/lib64"])
    return out


def build_all(force: bool = False, verbose: bool = False) -> list[Path]:
    outs = [build_runtime(force, verbose)]
    if ops_sources():
        outs.append(build_ops(force, verbose))
    return outs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v (register / spill / smem report)")
    ap.add_argument("--only", choices=["runtime", "ops"])
    a = ap.parse_args(argv)
    if a.verbose:
        os.environ["DFB_BUILD_VERBOSE"] = "1"
    if a.only == "runtime":
        outs = [build_runtime(a.force, a.verbose)]
    elif a.only == "ops":
        outs = [build_ops(a.force, a.verbose)]
    else:
        outs = build_all(a.force, a.verbose)
    for o in outs:
        print(f"built {o.relative_to(ROOT.parent)}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
