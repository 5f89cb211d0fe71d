"""Builds libllmcp_b200.so in-tree with nvcc for sm_100a.

    python -m llmcp_b200.build [--force]

Objects go to build/ at the repository root; the shared library is written next to this
file so that it travels with the source tree.  nvcc cross-compiles without a GPU.
"""
import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

PACKAGE = pathlib.Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libllmcp_b200.so"

SOURCES = ["q8_linear.cu", "gemv_rows.cu", "gemv_cols.cu", "gemm_tc.cu", "gemm_tma.cu", "norms.cu", "mixers.cu", "attn_decode.cu", "attn_prefill.cu", "bf16_linear.cu", "engine.cu", "api.cu", "tp_comm.cu", "noalloc.cu", "format.cpp", "checkpoint.cpp", "text.cpp", "text_regex.cpp"]
TOOLS = {"llmcp-benchmark": ["tools/llmcp_benchmark.cpp"], "llmcp-pack": ["tools/llmcp_pack.cpp"],
         "llmcp-run": ["tools/llmcp_run.cpp", "text.cpp", "text_regex.cpp"]}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # Every f32 multiply/add stays a separate IEEE operation; fused multiply-adds are
    # written explicitly where the reference has them.
    "-fmad=false",
    "-Xcompiler", "-fPIC,-fopenmp,-ffp-contract=off,-Wall",
]


def nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found")
    return path


def _newer(target, sources):
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(pathlib.Path(s).stat().st_mtime > stamp for s in sources)


def _headers():
    return [str(p) for p in list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [ROOT / "include" / "llmcp_b200.h"]]


def build(force=False, verbose=False):
    objdir = ROOT / "build" / "llmcp_b200"
    objdir.mkdir(parents=True, exist_ok=True)
    headers = _headers()
    env = dict(os.environ)
    env.pop("CXX", None)
    env.pop("CC", None)

    def compile_one(name):
        src = CSRC / name
        obj = objdir / (name.replace("/", "_") + ".o")
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc(), *NVCC_FLAGS, "-ccbin", "/usr/bin/g++", "-c", str(src), "-o", str(obj)]
            if verbose:
                print(" ".join(cmd), flush=True)
            subprocess.run(cmd, check=True, env=env)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        objects = list(pool.map(compile_one, SOURCES))
    if force or _newer(LIBRARY, objects):
        cmd = [nvcc(), "-shared", "-ccbin", "/usr/bin/g++", "-o", str(LIBRARY), *map(str, objects),
               "-Xcompiler", "-fopenmp", "-lgomp", "-ldl", "-Wno-deprecated-gpu-targets"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True, env=env)
    for tool, sources in TOOLS.items():
        paths = [CSRC / s for s in sources]
        if not all(p.exists() for p in paths):
            continue
        target = PACKAGE / "bin" / tool
        target.parent.mkdir(exist_ok=True)
        if force or _newer(target, [*paths, *headers, CSRC / "format.cpp", CSRC / "checkpoint.cpp"]):
            cmd = ["/usr/bin/g++", "-O2", "-std=c++17", "-fopenmp", "-ffp-contract=off", "-o", str(target),
                   *map(str, paths), str(CSRC / "format.cpp"), str(CSRC / "checkpoint.cpp"), "-ldl"]
            if verbose:
                print(" ".join(cmd), flush=True)
            subprocess.run(cmd, check=True, env=env)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
