"""Builds libtilejax_b200.so (the CUDA kernels and their C ABI) in-tree with nvcc, for sm_100a only.

    python -m tilejax_b200.csrc.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The CUDA runtime is linked statically and the driver API is reached
through cudaGetDriverEntryPoint, so the library has no load-time dependency on libcuda and also loads (for
symbol checks) on a machine without a driver.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PACKAGE = CSRC.parent
LIBRARY = PACKAGE / "libtilejax_b200.so"
SOURCES = ["tjx_host.cu", "tjx_steps.cu", "tjx_gemm.cu", "tjx_rmsnorm.cu", "tjx_block.cu", "tjx_decode.cu", "tjx_mla.cu", "tjx_attention.cu"]
HEADERS = ["tjx_host.cuh", "tjx_ptx.cuh", "../../include/tilejax_b200.h"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return found


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    built = target.stat().st_mtime
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (), output: Path | None = None) -> Path:
    """Compile every source that changed and link the shared library; returns its path. `defines` (-D macros: the
    kernels' tuning constants) and `output` build a variant beside the default library, in its own object folder."""
    library = LIBRARY if output is None else Path(output).resolve()
    objdir = CSRC / "build" if output is None else library.parent / (library.stem + "_obj")
    objdir.mkdir(parents=True, exist_ok=True)
    headers = [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__).resolve()]
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    objects = []
    jobs = []
    for src in sources:
        obj = objdir / (src.stem + ".o")
        objects.append(obj)
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, *[f"-D{d}" for d in defines], "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, proc in jobs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed.append(f"{src.name}:\n{out}")
        elif verbose or out.strip():
            print(f"--- {src.name}\n{out}", file=sys.stderr)
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
    if force or jobs or _stale(library, objects):
        # Link beside the target and rename over it: a reader never sees a half-written library.
        fresh = library.with_suffix(".so.new")
        cmd = [nvcc(), *ARCH_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-o", str(fresh), *map(str, objects)]
        subprocess.run(cmd, check=True)
        os.replace(fresh, library)
    return library


def ffi_include_dir() -> str | None:
    """Where jaxlib keeps the XLA FFI headers, or None where JAX is not installed."""
    try:
        import jax

        return jax.ffi.include_dir()
    except Exception:
        return None


def build_ffi(verbose: bool = False) -> Path | None:
    """Compile tjx_xla_ffi.cc (the jax.ffi handlers over the C ABI) into libtilejax_b200_ffi.so beside the library, if
    jaxlib's FFI headers are there; returns None (and builds nothing) otherwise."""
    include = ffi_include_dir()
    if include is None:
        return None
    build()
    target = PACKAGE / "libtilejax_b200_ffi.so"
    source = CSRC / "tjx_xla_ffi.cc"
    if _stale(target, [source, LIBRARY]):
        cmd = [nvcc(), *ARCH_FLAGS, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", f"-I{include}", str(source),
               "-o", str(target), f"-L{PACKAGE}", "-ltilejax_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
    return target


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true", help="print ptxas resource usage (registers, spills, smem)")
    parser.add_argument("-D", dest="defines", action="append", default=[], help="a macro for every source, e.g. TJX_DEC_STAGES=3")
    parser.add_argument("--output", default=None, help="write a variant library here instead of the package's own")
    parser.add_argument("--ffi", action="store_true", help="also build the jax.ffi handler library (needs jaxlib's headers)")
    args = parser.parse_args()
    output = Path(args.output).resolve() if args.output else None
    os.chdir(CSRC)
    print(build(args.force, args.verbose, tuple(args.defines), output))
    if args.ffi:
        print(build_ffi(args.verbose) or "jax.ffi.include_dir() is not available: the handler library was not built")
