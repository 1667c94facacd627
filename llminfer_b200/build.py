"""Builds the CUDA library and the C++ shim for sm_100a with nvcc, in tree.

``python -m llminfer_b200.build`` compiles
  llminfer_b200/lib/libgqa_b200.so        the kernels and the C ABI
  llminfer_b200/lib/libllminfer_shim.so   the C++ operator shim (reference signatures)
  llminfer_b200/lib/shim_driver           a small executable that drives the shim in tests
nvcc cross-compiles without a GPU. Sources are only rebuilt when newer than the output.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
LIB_DIR = ROOT / "lib"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

KERNEL_SOURCES = [
    "csrc/decode_bf16.cu",
    "csrc/decode_f32.cu",
    "csrc/front_stage.cu",
    "csrc/gqa_api.cu",
    "csrc/session.cu",
    "csrc/static_scratch.cu",
    "csrc/kv_pool.cpp",
    "csrc/shard_comm.cu",
    "csrc/proj.cu",
]
KERNEL_HEADERS = ["csrc/ptx.cuh", "csrc/work_map.cuh", "csrc/decode_kernels.cuh",
                  "csrc/peer_window.cuh", "csrc/front_math.cuh"]


def _stale(output: Path, inputs: list[Path]) -> bool:
    if not output.exists():
        return True
    out_time = output.stat().st_mtime
    return any(p.stat().st_mtime > out_time for p in inputs if p.exists())


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, cwd=REPO, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    out = LIB_DIR / "libgqa_b200.so"
    srcs = [ROOT / s for s in KERNEL_SOURCES]
    deps = srcs + [ROOT / h for h in KERNEL_HEADERS] + [REPO / "include" / "gqa_b200.h"]
    if force or _stale(out, deps):
        LIB_DIR.mkdir(exist_ok=True)
        cmd = [NVCC, "-std=c++17", "-O3", *ARCH, "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", str(out), *map(str, srcs), "-ldl"]
        _run(cmd)
    return out


def build_shim(force: bool = False) -> Path | None:
    shim_dir = ROOT / "shim"
    if not shim_dir.exists():
        return None
    out = LIB_DIR / "libllminfer_shim.so"
    srcs = sorted(shim_dir.glob("src/*.cpp"))
    deps = srcs + sorted(shim_dir.glob("include/**/*.h")) + [REPO / "include" / "gqa_b200.h"]
    if force or _stale(out, deps):
        LIB_DIR.mkdir(exist_ok=True)
        _run([NVCC, "-std=c++17", "-O2", "--shared", "-Xcompiler", "-fPIC",
              "-I", str(shim_dir / "include"), "-I", str(REPO / "include"),
              "-o", str(out), *map(str, srcs),
              "-L", str(LIB_DIR), "-lgqa_b200", "-Xlinker", "-rpath=$ORIGIN"])
    driver_src = shim_dir / "driver" / "shim_driver.cpp"
    driver = LIB_DIR / "shim_driver"
    if driver_src.exists() and (force or _stale(driver, [driver_src, out])):
        _run([NVCC, "-std=c++17", "-O2", "-I", str(shim_dir / "include"),
              "-I", str(REPO / "include"), "-o", str(driver), str(driver_src),
              "-L", str(LIB_DIR), "-lllminfer_shim", "-lgqa_b200", "-Xlinker", "-rpath=$ORIGIN"])
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_shim(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print("built", LIB_DIR)
