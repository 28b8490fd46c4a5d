"""In-tree build of libjllama_b200.so (nvcc, sm_100a only) and its location.

The library is plain CUDA C++ behind a C ABI (include/jllama_b200.h): no torch headers, so a full
rebuild is seconds and the artefact can be called from C, C++ or ctypes alike.  It is built into the
package directory so that it travels with the source tree to the GPU box.
"""
from __future__ import annotations

import hashlib
import logging
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional

logger = logging.getLogger(__name__)

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
INCLUDE = ROOT / "include"
OUT_DIR = Path(__file__).resolve().parent / "_C"
LIB_PATH = OUT_DIR / "libjllama_b200.so"
STAMP = OUT_DIR / "build.stamp"

# Sources whose arithmetic has to be exact float32 (true division, expf, tanhf, sqrtf): built without --use_fast_math.
PRECISE_SOURCES = {"seq_norm.cu", "seq_linear.cu", "attn_generic.cu", "gla_scan.cu", "moe.cu", "seq_mix.cu", "delta_scan.cu", "seq_token.cu"}

# Named subsets of the library: a model family that needs only some kernels gets a small library of its own at the
# first use in a fresh tree (seconds instead of the minutes of the whole-step decode kernels).  The full library
# contains every subset; `ops/_lib.py` prefers it when it is already built.
SUBSETS = {
    "hybrid": ["error.cu", "seq_norm.cu", "seq_linear.cu", "attn_generic.cu", "gla_scan.cu", "moe.cu", "seq_mix.cu", "delta_scan.cu", "seq_token.cu", "sample_full.cu",
               "gemm_tcgen05.cu", "gemm_2cta.cu", "tensormap.cu", "flash_prefill.cu", "prefill_attn_mma.cu", "decode_attn.cu"],
    # the members of the hybrid family whose only mixer is softmax attention: no recurrent scans, no one-token kernel of the
    # fixed head sizes
    "hybrid_attention": ["error.cu", "seq_norm.cu", "seq_linear.cu", "attn_generic.cu", "moe.cu", "seq_mix.cu", "seq_token.cu",
                         "sample_full.cu", "gemm_tcgen05.cu", "gemm_2cta.cu", "tensormap.cu", "flash_prefill.cu",
                         "prefill_attn_mma.cu"],
}


def subset_path(name: str) -> Path:
    return OUT_DIR / f"libjllama_b200_{name}.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _flags_for(src: Path) -> List[str]:
    if src.name in PRECISE_SOURCES:
        return [f for f in NVCC_FLAGS if f != "--use_fast_math"]
    return list(NVCC_FLAGS)


def _source_hash(src: Path, headers: str) -> str:
    h = hashlib.sha256()
    h.update(headers.encode())
    h.update(src.name.encode())
    h.update(src.read_bytes())
    h.update(" ".join(_flags_for(src)).encode())
    return h.hexdigest()


def _fingerprint(srcs: Optional[List[Path]] = None) -> str:
    headers = _headers_hash()
    h = hashlib.sha256()
    for f in (sources() if srcs is None else srcs):
        h.update(_source_hash(f, headers).encode())
    return h.hexdigest()


def _stamp_of(lib: Path) -> Path:
    return lib.with_suffix(".stamp") if lib != LIB_PATH else STAMP


def is_fresh(subset: Optional[str] = None) -> bool:
    lib, srcs = (LIB_PATH, None) if subset is None else (subset_path(subset), [CSRC / n for n in SUBSETS[subset]])
    stamp = _stamp_of(lib)
    return lib.exists() and stamp.exists() and stamp.read_text().strip() == _fingerprint(srcs)


def build_library(force: bool = False, verbose: bool = False, subset: Optional[str] = None) -> Path:
    """Compile csrc/*.cu (or the sources of a named subset) for sm_100a and link the shared library.  Objects are
    cached per source (keyed by the source, the headers and the flags), so subsets and the full library share
    them and an edit recompiles one file.  Returns the library's path."""
    lib = LIB_PATH if subset is None else subset_path(subset)
    srcs = sources() if subset is None else [CSRC / n for n in SUBSETS[subset]]
    if not force and is_fresh(subset):
        return lib
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = ROOT / "build" / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    cc = nvcc()
    headers = _headers_hash()

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        tag = obj_dir / (src.stem + ".hash")
        want = _source_hash(src, headers)
        if not force and obj.exists() and tag.exists() and tag.read_text().strip() == want:
            return obj
        cmd = [cc, *_flags_for(src), f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        tag.write_text(want + "\n")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = lib.with_suffix(f".tmp{os.getpid()}.so")            # link beside the target, then rename: no half-written library
    link = [cc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    _stamp_of(lib).write_text(_fingerprint(None if subset is None else srcs) + "\n")
    logger.info("built %s", lib)
    return lib


if __name__ == "__main__":
    logging.basicConfig(level=logging.INFO)
    names = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--subset=")]
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, subset=names[0] if names else None))
