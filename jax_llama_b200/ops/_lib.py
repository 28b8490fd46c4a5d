"""ctypes binding of libjllama_b200.so (the C ABI in include/jllama_b200.h).

Loading is lazy and *loud*: on a machine with a CUDA device, a missing or stale library is an error,
never a silent fall back to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

from .build import LIB_PATH, build_library

_lib: Optional[C.CDLL] = None

vp, ip, fp = C.c_void_p, C.c_void_p, C.c_void_p   # all pointers travel as integers from tensor.data_ptr()
i32, f32, u64, sz, i64 = C.c_int, C.c_float, C.c_ulonglong, C.c_size_t, C.c_longlong

_SIGNATURES = {
    "jl_last_error": (C.c_char_p, []),
    "jl_version": (i32, []),
    "jl_launch_count": (u64, []),
    "jl_embed": (i32, [ip, vp, vp, i32, i32, i32, vp]),
    "jl_rmsnorm": (i32, [vp, vp, vp, vp, vp, i32, i32, f32, vp]),
    "jl_rope_kv_write": (i32, [vp, vp, vp, vp, fp, fp, ip, ip, ip, i32, i32, i32, i32, i32, i32, i32, vp]),
    "jl_swiglu": (i32, [vp, vp, i32, i32, i32, vp]),
    "jl_gemv": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, f32, i32, i32, i32, vp]),
    "jl_gemv_tma": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, f32, i32, i32, i32, vp]),
    "jl_gemm": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]),
    "jl_gemm_2cta": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]),
    "jl_gemm_set_workspace": (i32, [vp, sz, vp, i32]),
    "jl_gemm_set_trace": (None, [vp]),
    "jl_decode_attn_scratch_bytes": (sz, [i32, i32, i32, i32]),
    "jl_decode_attn_splits": (i32, [i32, i32, i32, i32]),
    "jl_decode_attn": (i32, [vp, vp, vp, ip, ip, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32, i32, vp]),
    "jl_decode_attn_fused_scratch_bytes": (sz, [i32, i32, i32, i32, i32]),
    "jl_decode_attn_fused_splits": (i32, [i32, i32, i32, i32]),
    "jl_decode_attn_fused": (i32, [vp, vp, vp, fp, fp, ip, ip, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32, vp]),
    "jl_decode_attn_fused_set_variant": (i32, [i32]),
    "jl_decode_mega_scratch_bytes": (sz, [i32, i32, i32, i32, i32, i32]),
    "jl_decode_mega_cand_offset": (sz, [i32, i32, i32, i32, i32, i32]),
    "jl_decode_mega_peer_bytes": (sz, [i32, i32, i32, i32, vp]),
    "jl_nvls_bcast_f32": (i32, [fp, fp, i32, i32, i32, i32, i32, i32, i32, vp, i32, i32, ip, ip, vp]),
    "jl_sample_full": (i32, [fp, i32, i32, i32, f32, i32, f32, u64, ip, ip, vp, vp, i32, i32, i32, i32, ip, ip, ip, ip,
                             i32, i32, i32, ip, ip, ip, ip, vp]),
    "jl_decode_mega": (i32, [vp] * 9 + [ip, fp, i32, i32, i32, vp, vp, fp, fp, ip, ip, vp, vp] + [i32] * 11 +
                       [f32, f32, i32, i32, i32, vp, vp, vp, vp, vp]),
    "jl_mega_select": (i32, [vp, vp] + [i32] * 5 + [ip] * 4 + [i32] * 3 + [ip] * 4 + [vp]),
    "jl_nvls_selftest": (i32, [vp, vp, vp, i32, i32, C.c_uint, vp]),
    "jl_argmax": (i32, [fp, i32, i32, i32, i32, fp, ip, vp]),
    "jl_topk": (i32, [fp, i32, i32, i32, i32, i32, fp, ip, vp]),
    "jl_sample": (i32, [fp, ip, i32, i32, sz, i32, i32, f32, f32, u64, ip, ip, vp]),
    "jl_decode_advance": (i32, [ip, ip, ip, ip, i32, i32, i32, i32, ip, ip, ip, ip, vp]),
}

# kernels of the hybrid decoder family (csrc/seq_*.cu, attn_generic.cu, gla_scan.cu, delta_scan.cu, moe.cu)
_HYBRID = {
    "jl_embed_f32": (i32, [ip, vp, fp, i32, i32, i32, i32, vp]),
    "jl_norm_f32": (i32, [fp, vp, vp, i32, i32, f32, f32, i32, vp]),
    "jl_postnorm_add": (i32, [fp, i32, vp, fp, vp, vp, i32, i32, f32, f32, i32, vp]),
    "jl_headnorm_gate": (i32, [fp, vp, fp, i32, vp, i32, i32, i32, f32, i32, i32, vp]),
    "jl_act_cast": (i32, [fp, i32, vp, i32, i32, i32, i32, f32, f32, i32, vp]),
    "jl_act_inplace": (i32, [vp, i32, i32, i32, i32, f32, f32, i32, vp]),
    "jl_linear_any": (i32, [vp, i32, vp, vp, i32, i32, i32, i32, i32, f32, f32, i32, i32, vp]),
    "jl_attn_prep": (i32, [fp, i32, i32, i32, i32, vp, vp, vp, fp, fp, i32, i32, i32, f32, ip, ip] + [i32] * 7 + [fp, i32, i32, i32, vp]),
    "jl_attn_generic": (i32, [vp, vp, vp, vp, fp, i32, ip, ip] + [i32] * 7 + [f32, fp, i32, i32, vp]),
    "jl_attn_generic_splits": (i32, [i32, i32, i32, i32]),
    "jl_head_gate": (i32, [vp, fp, i32, i32, i32, i32, i32, vp]),
    "jl_gla_scan": (i32, [fp, i32, i32, i32, i32, i32, vp, vp, fp, fp, ip, ip] + [i32] * 6 + [f32, f32, fp, i32, vp]),
    "jl_gla_scan_ws_floats": (sz, [i32, i32, i32, i32, i32]),
    "jl_retention_scan": (i32, [fp, i32, i32, i32, i32, fp, fp, fp, i32, i32, i32, f32, f32, fp, fp, ip, ip] + [i32] * 5 + [fp, vp]),
    "jl_branch_add_norm": (i32, [fp, i32, fp, i32, f32, fp, vp, vp, vp, vp, i32, i32, f32, i32, vp]),
    "jl_linear_tile_rows": (i32, []),
    "jl_linear_grouped": (i32, [vp, i32, i64, vp, i64, vp, i32, i64, i32, i32, i32, i32, i32, i32, f32, f32, ip, ip, ip, i32, i32,
                                vp]),
    "jl_attn_windowed": (i32, [vp, vp, vp, vp, ip, ip] + [i32] * 9 + [i64] * 4 + [i32, f32, fp, i32, i32, fp, i32, vp]),
    "jl_latent_prep": (i32, [fp] + [i32] * 8 + [vp, vp, vp, vp, fp, fp, i32, f32, ip, ip, i32, i32, i32, vp, vp, i32, vp]),
    "jl_rotary_slice": (i32, [vp, i32, i32, i32, vp, i32, i32, i32, i32, i32, i32, i32, fp, fp, i32, ip, ip, i32, i32, i32, vp]),
    "jl_moe_route": (i32, [fp] + [i32] * 9 + [f32, fp, ip, fp, vp]),
    "jl_moe_sorted_rows": (i32, [i32, i32, i32]),
    "jl_moe_sort": (i32, [ip] + [i32] * 5 + [ip, ip, ip, ip, vp]),
    "jl_moe_gather": (i32, [vp, i32, ip, vp, i32, i32, i32, vp]),
    "jl_gemm_grouped": (i32, [vp, vp, vp, i32, i32, i32, i32, ip, ip, i32, i32, vp]),
    "jl_moe_combine": (i32, [fp, i32, ip, fp, i32, fp, i32, fp, i32, fp, i32, i32, vp]),
    "jl_embed_pair_norm": (i32, [ip, vp, vp, vp, fp, ip, ip, ip] + [i32] * 5 + [i64, i64, f32, i32, vp]),
    "jl_causal_conv": (i32, [fp, i32, i32, i32, vp, vp, fp, fp, i32, ip, ip] + [i32] * 5 + [vp]),
    "jl_norm_mean2": (i32, [fp, i32, vp, fp, i32, vp, f32, fp, i32, i32, f32, i32, vp]),
    "jl_gated_groupnorm": (i32, [fp, fp, i32, vp, i32, fp, i32, vp, vp, i32, i32, i32, f32, i32, i32, vp]),
    "jl_glu_act": (i32, [fp, i32, i32, i32, vp, i32, i32, i32, i32, i32, f32, f32, ip, i32, i32, vp]),
    "jl_talk_mix": (i32, [fp, vp, vp] + [i32] * 7 + [vp]),
    "jl_ssd_gates": (i32, [fp, i32, i32, vp, vp, fp, i32, i32, i32, vp]),
    "jl_ssd_scan": (i32, [fp, i32, i32, i32, i32, i32, fp, fp, fp, ip, ip] + [i32] * 5 + [fp, vp]),
    "jl_delta_scan_ws_floats": (sz, [i32] * 5),
    "jl_embed_pos": (i32, [ip, vp, vp, fp, ip, ip] + [i32] * 6 + [vp]),
    "jl_side_gate": (i32, [fp, i32, ip, vp, i32, i32, vp, i32, i32, i32, i32, i32, vp]),
    "jl_branch_add_cast": (i32, [fp, i32, fp, i32, f32, fp, vp, i32, i32, i32, vp]),
    "jl_side_gate_rows": (i32, [fp, i32, ip, vp, i32, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp]),
    "jl_attn_prep_ex": (i32, [fp, i32, i32, i32, i32, vp, vp, vp, fp, fp, i32, i32, i32, i32, vp, vp, f32, fp, fp, i32, i32, ip, ip]
                        + [i32] * 7 + [fp, i32, i32, i32, vp]),
    "jl_attn_masked": (i32, [vp, vp, vp, vp, fp, i32, ip, ip] + [i32] * 9 + [i64] * 4 + [i32, i32, f32, fp, i32, i32, fp, fp, fp,
                                                                                      i32, i32, fp, i32, vp]),
    "jl_moe_route_ex": (i32, [fp] + [i32] * 9 + [f32, fp, fp, i32, fp, ip, fp, vp]),
    "jl_moe_combine_ex": (i32, [fp, i32, ip, fp, i32, fp, i32, fp, i32, fp, i32, i32, ip, fp, vp, i32, i32, vp]),
    "jl_delta_scan": (i32, [fp, i32, i32, i32, i32, i32, fp, i32, i32, i32, vp, vp, vp, fp, fp, ip, ip] + [i32] * 6 + [fp, i32, vp]),
}

_OPTIONAL = {
    "jl_flash_prefill_occupancy": (i32, [i32]),
    "jl_decode_mega_stages": (i32, [i32, i32, i32, i32, i32, i32]),
    "jl_flash_prefill": (i32, [vp, vp, vp, ip, ip, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp]),
    "jl_flash_prefill_masked": (i32, [vp, vp, vp, ip, vp] + [i32] * 7 + [f32, i32, i32, fp, fp, i32, fp, fp, i32, vp]),
    "jl_prefill_attn_mma": (i32, [vp, vp, vp, ip, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp]),
}


class NativeLibraryError(RuntimeError):
    pass


_subset: Optional[str] = None


def use_subset(name: str) -> None:
    """Declare, before the first kernel call, that this process needs only the kernels of the named subset
    (`ops/build.py` SUBSETS).  If the full library is already built and fresh it is used as always; otherwise the
    subset's small library is built and loaded instead of the full one.  Entry points outside the subset are then
    absent and calling them is an AttributeError, not a silent fallback."""
    global _subset
    if _lib is None:
        _subset = name


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    from .build import is_fresh
    path = LIB_PATH
    partial = False
    if os.environ.get("JLLAMA_LIB"):           # A/B of two builds on one box (scripts/sweep_env.sh JLLAMA_LIB "a.so b.so")
        from pathlib import Path
        path = Path(os.environ["JLLAMA_LIB"])
    elif _subset is not None and not is_fresh():
        path, partial = build_library(subset=_subset), True
    if not path.exists() or (path == LIB_PATH and not partial and not is_fresh()
                             and not os.environ.get("JLLAMA_NO_AUTOBUILD")):
        if os.environ.get("JLLAMA_NO_AUTOBUILD"):
            raise NativeLibraryError(f"{path} is missing: run `python -m jax_llama_b200.ops.build`")
        build_library()
    try:
        handle = C.CDLL(str(path))
    except OSError as e:
        raise NativeLibraryError(f"cannot load {path}: {e}") from e
    for name, (res, args) in {**_SIGNATURES, **_HYBRID, **_OPTIONAL}.items():
        try:
            fn = getattr(handle, name)
        except AttributeError:
            if name in _OPTIONAL or partial:
                continue
            raise NativeLibraryError(f"{path} is stale: symbol {name} missing; rebuild with "
                                     "`python -m jax_llama_b200.ops.build --force`")
        fn.restype, fn.argtypes = res, args
    _lib = handle
    return handle


def has(symbol: str) -> bool:
    return hasattr(lib(), symbol)


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {lib().jl_last_error().decode()}")


def launch_count() -> int:
    return int(lib().jl_launch_count())
