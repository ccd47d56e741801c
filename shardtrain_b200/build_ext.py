"""In-tree build of the sm_100a extension: `python -m shardtrain_b200.build_ext`.

nvcc compiles each kernel file for `compute_100a/sm_100a` (no torch headers, so it takes seconds),
g++ compiles the torch bindings, and the result is linked into `shardtrain_b200/_C.so`, next to
the sources, so the library travels with the tree.  Rebuilds only what is older than its sources.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_C.so"
OBJ = ROOT / "csrc" / "build"

CUDA_SOURCES = ["gemm_sm100.cu", "gemm_allgather_sm100.cu", "elementwise.cu", "peer.cu",
                "attention_sm100.cu", "noalloc.cu"]
CPP_SOURCES = ["bindings.cpp", "layer_executor.cpp"]
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(d.stat().st_mtime > stamp for d in deps)


def _run(cmd: list[str], log: Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))


def build(verbose: bool = False) -> Path:
    from torch.utils import cpp_extension

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = str(Path(cuda_home) / "bin" / "nvcc")
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    objects = []
    for name in CUDA_SOURCES:
        src = CSRC / name
        if not src.exists():
            continue
        obj = OBJ / (name + ".o")
        if _newer(obj, [src, *headers]):
            if verbose:
                print("nvcc", name, flush=True)
            _run([nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)], OBJ / (name + ".ptxas.log"))
        objects.append(obj)
    includes = [f"-I{p}" for p in cpp_extension.include_paths(device_type="cuda")]
    defines = ["-D_GLIBCXX_USE_CXX11_ABI=1"]
    if (CSRC / "attention_sm100.cu").exists():
        defines.append("-DSTB_WITH_ATTENTION")
    for name in CPP_SOURCES:
        src = CSRC / name
        if not src.exists():
            continue
        obj = OBJ / (name + ".o")
        if _newer(obj, [src, *headers]):
            if verbose:
                print("g++", name, flush=True)
            _run(["g++", "-O2", "-std=c++17", "-fPIC", *defines, *includes, "-c", str(src), "-o", str(obj)])
        objects.append(obj)
    if _newer(OUT, objects):
        libdirs = cpp_extension.library_paths(device_type="cuda")
        # link beside the target and rename: a reader never sees a half-written library
        staged = OUT.with_name(OUT.name + ".link")
        link = ["g++", "-shared", "-o", str(staged), *map(str, objects)]
        for d in libdirs:
            link += [f"-L{d}", f"-Wl,-rpath,{d}"]
        link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"]
        if verbose:
            print("link", OUT.name, flush=True)
        _run(link)
        os.replace(staged, OUT)
    return OUT


def main() -> int:
    print(build(verbose=True))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
