"""Builds libtensorbridge_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python atc26-tensorbridge_b200/build.py [--force] [--verbose]
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBRARY = os.path.join(HERE, "libtensorbridge_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
SOURCES = ["tb_api.cu", "tb_ep.cu", "tb_inst_w8_t1.cu", "tb_inst_w8_t2.cu", "tb_inst_w16_t4.cu"]
HEADERS = ["tb_ptx.cuh", "tb_bridge.cuh", "tb_gemm.cuh", "tb_aux.cuh", "tb_launch.cuh", "tb_launch_impl.cuh", "tb_ep.cuh", os.path.join("..", "..", "include", "tensorbridge_b200.h")]


def nvcc_path() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def is_stale() -> bool:
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    return any(os.path.getmtime(os.path.join(CSRC, name)) > built for name in SOURCES + HEADERS)


def _compile(source: str, verbose: bool) -> tuple[str, subprocess.CompletedProcess]:
    obj = os.path.join(OBJ_DIR, os.path.splitext(source)[0] + ".o")
    command = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
               "-Xcompiler", "-fPIC", "-c", "-o", obj] + (["-Xptxas", "-v"] if verbose else []) + [os.path.join(CSRC, source)]
    return obj, subprocess.run(command, capture_output=True, text=True)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path.  The translation units are
    compiled in parallel (one per kernel variant) and linked with `nvcc -shared`."""
    if not force and not is_stale():
        return LIBRARY
    os.makedirs(OBJ_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(lambda src: _compile(src, verbose), SOURCES))
    for _, result in results:
        if verbose or result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
    if any(result.returncode != 0 for _, result in results):
        raise RuntimeError("nvcc failed building libtensorbridge_b200.so")
    link = subprocess.run([nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIBRARY]
                          + [obj for obj, _ in results], capture_output=True, text=True)
    if link.returncode != 0:
        sys.stderr.write(link.stdout + link.stderr)
        raise RuntimeError("nvcc failed linking libtensorbridge_b200.so")
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
