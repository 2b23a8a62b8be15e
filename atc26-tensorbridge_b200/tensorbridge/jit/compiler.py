"""NVRTC compilation of generated kernel sources to sm_100a cubins, with a disk cache.

The counterpart of the reference's `tensorbridge/jit/compiler.py:91-189` (`get_cache_dir`, `get_flags`, `cache_key`,
`compile_program`, `build`): same cache layout idea (one directory per key holding the source, the compile log, the
cubin and a `meta.json` written last), same key ingredients (NVRTC version, flags, entry point, source and the bytes
of every kernel header).  No Triton, no process pool: a translation unit here is one template point and compiles in
about ten seconds.
"""
from __future__ import annotations

import dataclasses
import glob
import hashlib
import json
import os
import re
import threading
from pathlib import Path

from tensorbridge.jit.codegen import KernelSource

CSRC_DIR = Path(__file__).resolve().parent.parent.parent / "csrc"
_lock = threading.Lock()


@dataclasses.dataclass(frozen=True)
class PtxasStats:
    registers: int = 0
    spill_stores: int = 0
    spill_loads: int = 0

    @classmethod
    def parse(cls, log: str) -> "PtxasStats":
        regs = re.search(r"Used (\d+) registers", log)
        spills = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", log)
        return cls(int(regs.group(1)) if regs else 0, int(spills.group(1)) if spills else 0, int(spills.group(2)) if spills else 0)


@dataclasses.dataclass(frozen=True)
class CompiledKernel:
    cubin_path: str
    entry: str
    stats: PtxasStats
    cached: bool


def get_cache_dir() -> Path:
    return Path(os.environ.get("TENSORBRIDGE_CACHE_DIR", Path.home() / ".tensorbridge_b200" / "cache"))


def cuda_include_dirs() -> list[str]:
    """Directories that hold `cuda_bf16.h` (the one toolkit header the kernels include under NVRTC)."""
    candidates = [os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"]
    found = [str(Path(c) / "include") for c in candidates if c and (Path(c) / "include" / "cuda_bf16.h").exists()]
    if not found:
        raise RuntimeError("no CUDA toolkit headers found (set CUDA_HOME): the JIT needs cuda_bf16.h")
    return found[:1]


def get_flags(include_root: Path = CSRC_DIR) -> list[str]:
    return ["--gpu-architecture=sm_100a", "-std=c++17", "--generate-line-info", "--ptxas-options=-v", "-default-device",
            f"-I{include_root}", *(f"-I{path}" for path in cuda_include_dirs())]


def cache_key(source: str, entry: str, flags: list[str], include_root: Path = CSRC_DIR) -> str:
    from cuda.bindings import nvrtc  # noqa: PLC0415

    hasher = hashlib.sha256()
    _, major, minor = nvrtc.nvrtcVersion()
    hasher.update(json.dumps([major, minor, flags, entry, source]).encode())
    for header in sorted(glob.glob(f"{include_root}/*.cuh")):  # the headers are part of the program
        hasher.update(Path(header).read_bytes())
    return hasher.hexdigest()[:16]


def _check(result, what: str) -> None:
    from cuda.bindings import nvrtc  # noqa: PLC0415

    if result != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        raise RuntimeError(f"{what} failed: {result}")


def compile_program(source: str, entry: str, flags: list[str], out_dir: Path) -> None:
    """Compile `source` to `out_dir/kernel.cubin`; the compile log (ptxas register and spill statistics included) goes
    to `out_dir/compile.log`, and `meta.json`, written last, marks the directory as complete."""
    from cuda.bindings import nvrtc  # noqa: PLC0415

    result, program = nvrtc.nvrtcCreateProgram(source.encode(), b"kernel.cu", 0, [], [])
    _check(result, "nvrtcCreateProgram")
    try:
        options = [flag.encode() for flag in flags]
        result = nvrtc.nvrtcCompileProgram(program, len(options), options)[0]
        _, log_size = nvrtc.nvrtcGetProgramLogSize(program)
        log = b"\0" * log_size
        nvrtc.nvrtcGetProgramLog(program, log)
        log_text = log.decode(errors="replace").rstrip("\0")
        (out_dir / "compile.log").write_text(log_text)
        if result != nvrtc.nvrtcResult.NVRTC_SUCCESS:
            raise RuntimeError(f"NVRTC failed, see {out_dir / 'compile.log'}:\n{log_text}")
        _, size = nvrtc.nvrtcGetCUBINSize(program)
        cubin = b"\0" * size
        _check(nvrtc.nvrtcGetCUBIN(program, cubin)[0], "nvrtcGetCUBIN")
    finally:
        nvrtc.nvrtcDestroyProgram(program)
    (out_dir / "kernel.cubin").write_bytes(cubin)
    (out_dir / "meta.json").write_text(json.dumps({"entry": entry}))


def build(kernel: KernelSource, include_root: Path = CSRC_DIR) -> CompiledKernel:
    """The cubin of `kernel`, from the disk cache when a complete entry with the same key exists."""
    flags = get_flags(include_root)
    out_dir = get_cache_dir() / cache_key(kernel.source, kernel.name, flags, include_root)
    out_dir.mkdir(parents=True, exist_ok=True)
    with _lock:
        cached = (out_dir / "meta.json").exists()
        if not cached:
            (out_dir / "kernel.cu").write_text(kernel.source)
            compile_program(kernel.source, kernel.name, flags, out_dir)
    stats = PtxasStats.parse((out_dir / "compile.log").read_text())
    return CompiledKernel(str(out_dir / "kernel.cubin"), kernel.name, stats, cached)
