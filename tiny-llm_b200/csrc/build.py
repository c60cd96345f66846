"""Build libtiny_llm_b200.so (sm_100a only) in-tree with nvcc.

The reference drives CMake through mlx.extension.CMakeBuild
(/root/reference/src/extensions_ref/build.py:11-24, CMakeLists.txt:32-84) to
produce a metallib plus a nanobind module; here one nvcc invocation per
translation unit produces objects that are linked into a C-ABI shared library
loaded with ctypes.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ROOT = CSRC.parent.parent
OUT_DIR = CSRC.parent / "extensions_b200" / "tiny_llm_ext_b200"
# Experiment builds: TL_DEFINES="-DS4_DEPTH_SMALL=3 ..." TL_LIB_SUFFIX=_d3 python build.py
# -> libtiny_llm_b200_d3.so next to the product library (tools/kbench.py --lib selects it).
SUFFIX = os.environ.get("TL_LIB_SUFFIX", "")
LIB = OUT_DIR / f"libtiny_llm_b200{SUFFIX}.so"
BUILD = CSRC / f"build{SUFFIX}"

SOURCES = [
    "c_abi.cu",
    "elementwise.cu",
    "w4a16_matvec.cu",
    "w4a16_gemm.cu",
    "w4a16_gemm2.cu",
    "w4a16_skinny.cu",
    "attention_decode.cu",
    "attention_prefill.cu",
    "attention_prefill_tc.cu",
    "decode_attention_fused.cu",
]

# The second library: building blocks for models with unquantised weights (include/tiny_llm_b200_blocks.h).  It links
# on its own, so a process that runs only such a model compiles these few files and nothing of the W4A16 path.
BLOCKS_LIB = OUT_DIR / f"libtiny_llm_b200_blocks{SUFFIX}.so"
BLOCKS_SOURCES = [
    "blocks/blocks_rows.cu",
    "blocks/blocks_latent_attention.cu",
    "blocks/blocks_latent_attention_mma.cu",
    "blocks/blocks_moe.cu",
    "blocks/blocks_paged_attention.cu",
    "blocks/blocks_paged_attention_mma.cu",
    "blocks/blocks_linear_attention.cu",
    "blocks/blocks_delta_rule.cu",
    "blocks/blocks_streams.cu",
]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-I", str(ROOT / "include"),
    *os.environ.get("TL_DEFINES", "").split(),
]


def _digest(path: Path) -> str:
    h = hashlib.sha256()
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT / "include").glob("*.h"))
    if path.parent != CSRC:
        headers += list(path.parent.glob("*.cuh"))
    for dep in sorted(headers + [path]):
        h.update(dep.read_bytes())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


def _compile(src: str, verbose: bool) -> Path:
    path = CSRC / src
    obj = BUILD / (path.stem + ".o")
    stamp = BUILD / (path.stem + ".sha")
    want = _digest(path)
    if obj.exists() and stamp.exists() and stamp.read_text() == want:
        return obj
    part = obj.with_name(f".{obj.name}.{os.getpid()}")
    cmd = [NVCC, *FLAGS, "-c", str(path), "-o", str(part)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"nvcc failed on {src}")
    if verbose:
        sys.stderr.write(proc.stderr)
    os.replace(part, obj)
    stamp.write_text(want)
    return obj


def _link(lib: Path, sources: list, verbose: bool) -> Path:
    BUILD.mkdir(exist_ok=True)
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources))
    newest = max(o.stat().st_mtime for o in objs)
    if not lib.exists() or lib.stat().st_mtime < newest:
        # link beside the target and rename: another process may be loading or building the same library
        part = lib.with_name(f".{lib.name}.{os.getpid()}")
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
               "-o", str(part), *map(str, objs), "-lcuda"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("link failed")
        os.replace(part, lib)
    return lib


def build_blocks(verbose: bool = False) -> Path:
    """libtiny_llm_b200_blocks.so alone (seconds)."""
    return _link(BLOCKS_LIB, BLOCKS_SOURCES, verbose)


def build(verbose: bool = False) -> Path:
    """Both libraries; returns the W4A16 one."""
    build_blocks(verbose)
    return _link(LIB, SOURCES, verbose)


if __name__ == "__main__":
    print((build_blocks if "--blocks" in sys.argv else build)(verbose="-v" in sys.argv))
