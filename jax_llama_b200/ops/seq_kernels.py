"""Python front-ends of the kernels of the hybrid decoder family (csrc/seq_norm.cu, seq_linear.cu, attn_generic.cu,
gla_scan.cu): fp32 residual stream, operands in bfloat16 or true float32, softmax attention with arbitrary head sizes
and linear-recurrence mixers.

CUDA tensors only: these ops are the product path and have no PyTorch stand-in (the numerical oracles live with the
tests).  Every call runs on the current stream and is legal under CUDA-graph capture when the caller passes `out`
buffers (otherwise outputs come from the caching allocator, which a torch graph capture also handles).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib
from .kernels import _p, _stream, ensure_gemm_workspace, num_sms

ACT_NONE, ACT_RELU2, ACT_GELU_TANH, ACT_SILU, ACT_SCALE_SOFTCAP, ACT_SIGMOID, ACT_XIELU = 0, 1, 2, 3, 4, 5, 6
DELTA_FUSED_MAX_TOKENS = 8    # the same for the delta-rule scan (csrc/delta_scan.cu DS_FUSED_MAX_TOKENS)
GLA_FUSED_MAX_TOKENS = 8      # up to this many tokens per row the gated-linear-attention scan stays one fused launch
ACTIVATIONS = {"none": ACT_NONE, "relu2": ACT_RELU2, "gelu_tanh": ACT_GELU_TANH, "silu": ACT_SILU, "sigmoid": ACT_SIGMOID,
               "xielu": ACT_XIELU}         # xielu takes two numbers (p0, p1): z > 0: p0 z^2 + z/2, else p1 (e^z - 1 - z) + z/2
GLU_PRODUCT, GLU_CLAMPED = 0, 1         # act(gate) * up;  g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, ±limit)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return 0
    if dtype == torch.float32:
        return 1
    raise ValueError(f"the hybrid kernels run in bfloat16 or float32, not {dtype}")


def _need(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name}: the hybrid kernels take CUDA tensors only")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


def tensor_cores_enabled() -> bool:
    """JLLAMA_HYBRID_TC=0 keeps every linear layer on the exact SIMT kernels (A/B and debugging)."""
    return os.environ.get("JLLAMA_HYBRID_TC", "1") != "0"


def embed_f32(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    ids32 = ids.to(torch.int32).contiguous().view(-1)
    V, W = table.shape
    if out is None:
        out = torch.empty((ids32.numel(), W), dtype=torch.float32, device=table.device)
    _lib.check(_lib.lib().jl_embed_f32(ids32.data_ptr(), table.data_ptr(), out.data_ptr(), ids32.numel(), W, V,
                                       dtype_code(table.dtype), _stream()), "jl_embed_f32")
    return out


def norm_f32(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float, out: Optional[torch.Tensor] = None
             ) -> torch.Tensor:
    """x fp32 [M, W] → x / rms(x) * (offset + w) in w's dtype."""
    _need(x, torch.float32, "x")
    M, W = x.shape
    if out is None:
        out = torch.empty((M, W), dtype=w.dtype, device=x.device)
    _lib.check(_lib.lib().jl_norm_f32(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, W, float(eps), float(offset),
                                      dtype_code(w.dtype), _stream()), "jl_norm_f32")
    return out


def postnorm_add(y: torch.Tensor, w_post: torch.Tensor, x: torch.Tensor, eps: float, offset: float,
                 w_next: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x += norm(y) · (offset + w_post), in place; with `w_next` also returns norm(x) · (offset + w_next)."""
    _need(y, torch.float32, "y")
    _need(x, torch.float32, "x")
    M, W = x.shape
    if w_next is not None and h_out is None:
        h_out = torch.empty((M, W), dtype=w_next.dtype, device=x.device)
    _lib.check(_lib.lib().jl_postnorm_add(y.data_ptr(), y.stride(0), w_post.data_ptr(), x.data_ptr(), _p(w_next),
                                          _p(h_out) if w_next is not None else 0, M, W, float(eps), float(offset),
                                          dtype_code(w_post.dtype), _stream()), "jl_postnorm_add")
    return h_out if w_next is not None else None


def headnorm_gate(o: torch.Tensor, w: Optional[torch.Tensor], gate: torch.Tensor, H: int, V: int, eps: float,
                  gate_act: int = ACT_SILU, out: Optional[torch.Tensor] = None, dtype: Optional[torch.dtype] = None
                  ) -> torch.Tensor:
    """o fp32 [M, H·V]; gate: fp32 view [M, H·V] (any row pitch) → norm over V per head · w · act(gate), in w's dtype
    (w None: no weight, the result in `dtype`)."""
    _need(o, torch.float32, "o")
    _need(gate, torch.float32, "gate")
    M = o.shape[0]
    odt = w.dtype if w is not None else dtype
    if out is None:
        out = torch.empty((M, H * V), dtype=odt, device=o.device)
    _lib.check(_lib.lib().jl_headnorm_gate(o.data_ptr(), _p(w), gate.data_ptr(), gate.stride(0), out.data_ptr(),
                                           M, H, V, float(eps), gate_act, dtype_code(odt), _stream()),
               "jl_headnorm_gate")
    return out


def act_cast(y: torch.Tensor, out_dtype: torch.dtype, act: int = ACT_NONE, p0: float = 0.0, p1: float = 0.0,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(y) for an fp32 [M, N] view into `out_dtype` (in place when out is y itself)."""
    _need(y, torch.float32, "y")
    M, N = y.shape
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=y.device)
    _lib.check(_lib.lib().jl_act_cast(y.data_ptr(), y.stride(0), out.data_ptr(), out.stride(0), M, N, act, float(p0),
                                      float(p1), dtype_code(out_dtype), _stream()), "jl_act_cast")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, *, act: int = ACT_NONE, p0: float = 0.0, p1: float = 0.0,
           out_f32: bool = True, out: Optional[torch.Tensor] = None, tensor_cores: Optional[bool] = None) -> torch.Tensor:
    """act(x Wᵀ): x [M, K] and W [N, K] of one dtype (bf16 or fp32) → fp32 (or the operand dtype) [M, N].

    bfloat16 with more than 8 rows and 16-byte pitches runs the tcgen05 GEMM (fp32 accumulate; the activation is
    then an in-place pass over the stored result); 8 rows or fewer the weight-streaming kernel; everything else — true
    float32 in particular — the exact tiled SIMT kernel."""
    if not x.is_cuda:
        raise ValueError("linear: CUDA tensors only")
    _need(w, x.dtype, "w")
    N, K = w.shape
    M = x.numel() // K
    x = x.view(M, K) if x.is_contiguous() else x
    odt = torch.float32 if out_f32 else x.dtype
    if out is None:
        out = torch.empty((M, N), dtype=odt, device=x.device)
    L = _lib.lib()
    use_tc = tensor_cores_enabled() if tensor_cores is None else tensor_cores
    if (use_tc and x.dtype == torch.bfloat16 and M > 8 and K % 8 == 0 and N % 8 == 0 and x.is_contiguous()
            and w.is_contiguous() and out.is_contiguous() and out.shape[1] == N):
        if M <= 128:
            ensure_gemm_workspace(x.device)
        f32 = out.dtype == torch.float32
        _lib.check(L.jl_gemm(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), M, N, K, 0, int(f32), num_sms(x.device),
                             _stream()), "jl_gemm")
        if act != ACT_NONE:
            # the activation runs on the stored result (bf16 results: on the rounded value), in place
            _lib.check(L.jl_act_inplace(out.data_ptr(), out.stride(0), M, N, act, float(p0), float(p1),
                                        dtype_code(out.dtype), _stream()), "jl_act_inplace")
        return out
    _lib.check(L.jl_linear_any(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), M, N, K, act,
                               float(p0), float(p1), dtype_code(x.dtype), int(out.dtype == torch.float32), _stream()),
               "jl_linear_any")
    return out


def attn_prep(y: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor,
              k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
              rot: int, unit_norm: bool, eps: float, cache_len: torch.Tensor, pad_left: Optional[torch.Tensor],
              B: int, S: int, H: int, G: int, D: int, Dv: int, bias: Optional[torch.Tensor] = None, v_unit_norm: bool = False,
              v_token_major: bool = False, layout: int = 0, q_norm_w: Optional[torch.Tensor] = None,
              k_norm_w: Optional[torch.Tensor] = None, v_cos: Optional[torch.Tensor] = None, v_sin: Optional[torch.Tensor] = None
              ) -> None:
    """Rotate / normalise q (and k), append k, v to the caches [B, G, T, D] / [B, G, T, Dv].  k_off < 0: queries only.
    bias: fp32 over the columns of y, added first; v_unit_norm: values scaled to unit RMS per head before they are cached;
    v_token_major: the value cache is [B, T, G·Dv].  layout: pairing of the rotated channels (ROT_INTERLEAVED / ROT_HALF);
    q_norm_w / k_norm_w [D]: an RMS norm with a weight on every head BEFORE the rotation; v_cos / v_sin fp32 [positions, Dv/2]:
    values are rotated at their own position over all their channels (same pairing) before they are cached."""
    _need(y, torch.float32, "y")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    T_cap = k_cache.shape[2] if k_cache is not None else 0
    if layout or q_norm_w is not None or v_cos is not None:
        _lib.check(_lib.lib().jl_attn_prep_ex(
            y.data_ptr(), y.stride(0), q_off, k_off, v_off, q_out.data_ptr(), _p(k_cache), _p(v_cache), cos.data_ptr(),
            sin.data_ptr(), cos.shape[0], rot, int(layout), int(unit_norm), _p(q_norm_w), _p(k_norm_w), float(eps), _p(v_cos),
            _p(v_sin), v_cos.shape[0] if v_cos is not None else 0, int(layout), _p(cache_len), _p(pad_left), B, S, H, G, D, Dv,
            T_cap, _p(bias), int(v_unit_norm), int(v_token_major), dtype_code(q_out.dtype), _stream()), "jl_attn_prep_ex")
        return
    _lib.check(_lib.lib().jl_attn_prep(
        y.data_ptr(), y.stride(0), q_off, k_off, v_off, q_out.data_ptr(), _p(k_cache), _p(v_cache), cos.data_ptr(),
        sin.data_ptr(), cos.shape[0], rot, int(unit_norm), float(eps), _p(cache_len), _p(pad_left), B, S, H, G, D, Dv,
        T_cap, _p(bias), int(v_unit_norm), int(v_token_major), dtype_code(q_out.dtype), _stream()), "jl_attn_prep")


def attn_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, gate: Optional[torch.Tensor],
                 cache_len: torch.Tensor, pad_left: Optional[torch.Tensor], B: int, S: int, H: int, scale: float,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of S new tokens per row against the (already appended) caches; gate: fp32 view [M, H]."""
    G, T_cap, D = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    Dv = v_cache.shape[3]
    if out is None:
        out = torch.empty((B * S, H * Dv), dtype=q.dtype, device=q.device)
    L = _lib.lib()
    splits, scratch = 0, None
    if S == 1:                     # one new token: keys split over CTAs, partial results meet in scratch
        splits = int(L.jl_attn_generic_splits(B, H, G, T_cap))
        if splits:
            scratch = torch.empty(B * H * splits * (Dv + 2), dtype=torch.float32, device=q.device)
    _lib.check(L.jl_attn_generic(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(gate),
        gate.stride(0) if gate is not None else 0, _p(cache_len), _p(pad_left), B, S, H, G, D, Dv, T_cap, float(scale),
        _p(scratch), splits, dtype_code(q.dtype), _stream()), "jl_attn_generic")
    return out


def head_gate(out: torch.Tensor, gate: torch.Tensor, H: int, Dv: int) -> torch.Tensor:
    M = out.shape[0]
    _lib.check(_lib.lib().jl_head_gate(out.data_ptr(), gate.data_ptr(), gate.stride(0), M, H, Dv, dtype_code(out.dtype),
                                       _stream()), "jl_head_gate")
    return out


def gla_scan(y: torch.Tensor, q_off: int, k_off: int, v_off: int, a_off: int, a2: torch.Tensor, a2_bias: torch.Tensor,
             state: torch.Tensor, cache_len: Optional[torch.Tensor], pad_left: Optional[torch.Tensor], B: int, S: int,
             H: int, D: int, Dv: int, q_scale: float, tau: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Advance the fp32 state [B, H, D, Dv] over S tokens per row; returns the raw read-outs o fp32 [B·S, H·Dv]."""
    _need(y, torch.float32, "y")
    _need(state, torch.float32, "state")
    R = a2.shape[1]
    if out is None:
        out = torch.empty((B * S, H * Dv), dtype=torch.float32, device=y.device)
    L = _lib.lib()
    ws = None
    if S > GLA_FUSED_MAX_TOKENS:          # prompts: token-parallel preparation + pipelined scan (two launches)
        ws = torch.empty(int(L.jl_gla_scan_ws_floats(B, S, H, D, Dv)), dtype=torch.float32, device=y.device)
    _lib.check(L.jl_gla_scan(
        y.data_ptr(), y.stride(0), q_off, k_off, v_off, a_off, a2.data_ptr(), a2_bias.data_ptr(), state.data_ptr(),
        out.data_ptr(), _p(cache_len), _p(pad_left), B, S, H, D, Dv, R, float(q_scale), float(tau), _p(ws),
        dtype_code(a2.dtype), _stream()), "jl_gla_scan")
    return out


# --------------------------------------------------------------------------- parallel blocks, latent attention, retention, experts
ROT_INTERLEAVED, ROT_HALF = 0, 1        # channel 2i with 2i+1 / channel i with i + dims/2
ROT_LAYOUTS = {"interleaved": ROT_INTERLEAVED, "half": ROT_HALF}
SCORE_SIGMOID, SCORE_SOFTMAX = 0, 1
SCORES = {"sigmoid": SCORE_SIGMOID, "softmax": SCORE_SOFTMAX}
MOE_PAIR_ROWS = 16                      # up to this many token rows every (token, choice) pair streams its own expert


def branch_add_norm(x: torch.Tensor, y1: Optional[torch.Tensor], y2: Optional[torch.Tensor], mult: float,
                    w1: Optional[torch.Tensor], w2: Optional[torch.Tensor], eps: float
                    ) -> "tuple[Optional[torch.Tensor], Optional[torch.Tensor]]":
    """x += mult · (y1 + y2) in place (fp32; either branch may be None), then h1 = norm(x) · w1 and h2 = norm(x) · w2
    for the weights given (plain weights, the weights' dtype)."""
    _need(x, torch.float32, "x")
    M, W = x.shape
    for y in (y1, y2):
        if y is not None:
            _need(y, torch.float32, "y")
    h1 = torch.empty((M, W), dtype=w1.dtype, device=x.device) if w1 is not None else None
    h2 = torch.empty((M, W), dtype=w2.dtype, device=x.device) if w2 is not None else None
    if y1 is None and y2 is None and w1 is None and w2 is None:
        return None, None
    dt = w1.dtype if w1 is not None else (w2.dtype if w2 is not None else torch.float32)
    _lib.check(_lib.lib().jl_branch_add_norm(_p(y1), y1.stride(0) if y1 is not None else 0, _p(y2),
                                             y2.stride(0) if y2 is not None else 0, float(mult), x.data_ptr(), _p(w1), _p(h1),
                                             _p(w2), _p(h2), M, W, float(eps), dtype_code(dt), _stream()), "jl_branch_add_norm")
    return h1, h2


def linear_batched(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, nbatch: int, rows: int, x_bs: int, o_bs: int,
                   x_div: int = 1, w_index: Optional[torch.Tensor] = None, act: int = ACT_NONE) -> torch.Tensor:
    """`nbatch` products act(x_z W_zᵀ) of `rows` rows each: x_z starts (z // x_div) · x_bs elements into x (row pitch
    x.stride(0)), W_z = w[w_index[z]] or w[z] (w [n, N, K]), the result goes o_bs · z elements into out (row pitch
    out.stride(0); fp32 or the operand type)."""
    _need(w, x.dtype, "w")
    _, N, K = w.shape
    _lib.check(_lib.lib().jl_linear_grouped(
        x.data_ptr(), x.stride(0), int(x_bs), w.data_ptr(), N * K, out.data_ptr(), out.stride(0), int(o_bs), int(nbatch),
        int(x_div), int(rows), N, K, act, 0.0, 0.0, _p(w_index), 0, 0, dtype_code(x.dtype), int(out.dtype == torch.float32),
        _stream()), "jl_linear_grouped")
    return out


def linear_sorted(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor,
                  row_src: Optional[torch.Tensor], act: int = ACT_NONE) -> torch.Tensor:
    """Rows sorted by weight matrix: out[p] = act(W_g x[row_src[p]]) with g = tile_group[p // tile] (w [n, N, K])."""
    _need(w, x.dtype, "w")
    _, N, K = w.shape
    _lib.check(_lib.lib().jl_linear_grouped(
        x.data_ptr(), x.stride(0), 0, w.data_ptr(), N * K, out.data_ptr(), out.stride(0), 0, 1, 1, out.shape[0], N, K, act,
        0.0, 0.0, 0, tile_group.data_ptr(), _p(row_src), dtype_code(x.dtype), int(out.dtype == torch.float32), _stream()),
        "jl_linear_grouped")
    return out


def latent_prep(y: torch.Tensor, q_off: int, q_rank: int, kv_off: int, kv_rank: int, rot_dim: int, rot: int, layout: int,
                wq_norm: Optional[torch.Tensor], wkv_norm: torch.Tensor, cache: torch.Tensor, cos: torch.Tensor,
                sin: torch.Tensor, eps: float, cache_len: torch.Tensor, pad_left: Optional[torch.Tensor], B: int, S: int,
                token_major: bool = False) -> "tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]":
    """Norm both latents, rotate the shared key part, append [latent | key part] to cache [B, T, kv_rank + rot_dim].
    Returns (normed query latent [B·S, q_rank] or None when q_rank == 0, and with `token_major` contiguous copies of
    the appended latents [B·S, kv_rank] and key parts [B·S, rot_dim], else None, None)."""
    _need(y, torch.float32, "y")
    M = B * S
    cq = torch.empty((M, q_rank), dtype=cache.dtype, device=y.device) if q_rank else None
    c_out = torch.empty((M, kv_rank), dtype=cache.dtype, device=y.device) if token_major else None
    kr_out = torch.empty((M, max(rot_dim, 1)), dtype=cache.dtype, device=y.device) if token_major else None
    _lib.check(_lib.lib().jl_latent_prep(
        y.data_ptr(), y.stride(0), q_off, q_rank, kv_off, kv_rank, rot_dim, rot, layout, _p(wq_norm), wkv_norm.data_ptr(),
        _p(cq), cache.data_ptr(), cos.data_ptr(), sin.data_ptr(), cos.shape[0], float(eps), _p(cache_len), _p(pad_left), B, S,
        cache.shape[1], _p(c_out), _p(kr_out), dtype_code(cache.dtype), _stream()), "jl_latent_prep")
    return cq, c_out, kr_out


def rotary_slice(src: torch.Tensor, in_hs: int, in_off: int, out: torch.Tensor, out_hs: int, out_off: int, H: int, n: int,
                 rot: int, layout: int, cos: torch.Tensor, sin: torch.Tensor, cache_len: torch.Tensor,
                 pad_left: Optional[torch.Tensor], B: int, S: int) -> torch.Tensor:
    _need(out, src.dtype, "out")
    _lib.check(_lib.lib().jl_rotary_slice(
        src.data_ptr(), src.stride(0), in_hs, in_off, out.data_ptr(), out.stride(0), out_hs, out_off, H, n, rot, layout,
        cos.data_ptr(), sin.data_ptr(), cos.shape[0], _p(cache_len), _p(pad_left), B, S, dtype_code(src.dtype), _stream()),
        "jl_rotary_slice")
    return out


def attn_windowed(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cache_len: torch.Tensor,
                  pad_left: Optional[torch.Tensor], B: int, S: int, H: int, G: int, D: int, Dv: int, T_cap: int, ldk: int,
                  ldv: int, window: int, scale: float, out: Optional[torch.Tensor] = None,
                  strides: "tuple[int, int, int, int]" = (0, 0, 0, 0), sink: bool = False, out_f32: bool = False
                  ) -> torch.Tensor:
    """Causal attention of S new tokens per row over key / value rows of pitch ldk / ldv (keys and values may be
    columns of one cached row); window > 0 keeps the last `window` slots up to the query's own.  `strides`: elements
    between batch rows and between key/value heads for keys and for values — all zero: caches [B, G, T_cap, ·];
    token-major projections [B·T, G, d] have (T·G·d, d) and a row pitch of G·d.  sink: one more term exp(0) in the softmax
    denominator (a key with score 0 and no value); out_f32: the result in fp32 whatever the operand type."""
    if out is None:
        out = torch.empty((B * S, H * Dv), dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
    f32_out = out.dtype == torch.float32 and q.dtype != torch.float32
    L = _lib.lib()
    splits, scratch = 0, None
    if S == 1:
        splits = int(L.jl_attn_generic_splits(B, H, G, min(T_cap, window) if window > 0 else T_cap))
        if splits:
            scratch = torch.empty(B * H * splits * (Dv + 2), dtype=torch.float32, device=q.device)
    _lib.check(L.jl_attn_windowed(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), 0 if f32_out else out.data_ptr(), _p(cache_len), _p(pad_left),
        B, S, H, G, D, Dv, T_cap, ldk, ldv, *(int(v) for v in strides), int(window), float(scale), _p(scratch), splits,
        int(sink), out.data_ptr() if f32_out else 0, dtype_code(q.dtype), _stream()), "jl_attn_windowed")
    return out


def attn_masked(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cache_len: torch.Tensor,
                pad_left: Optional[torch.Tensor], B: int, S: int, H: int, G: int, D: int, Dv: int, scale: float, *,
                gate: Optional[torch.Tensor] = None, window: int = 0, chunk: int = 0, sink: bool = False,
                sink_logit: Optional[torch.Tensor] = None, v_cos: Optional[torch.Tensor] = None,
                v_sin: Optional[torch.Tensor] = None, v_layout: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of S new tokens per row over caches [B, G, T, D] / [B, G, T, Dv] with everything the kernels take:
    gate fp32 view [M, H] (sigmoid per head on the output); window; chunk > 0: positions form blocks of `chunk` and a query sees
    the keys of its own block only; sink with an optional learned logit per head (fp32 [H]); v_cos / v_sin fp32
    [positions, Dv/2]: the values were cached rotated at their own positions and every head's sum is rotated back by the
    query's position, before the gate."""
    T_cap = k_cache.shape[2]
    if out is None:
        out = torch.empty((B * S, H * Dv), dtype=q.dtype, device=q.device)
    if sink_logit is not None:
        _need(sink_logit, torch.float32, "sink_logit")
    L = _lib.lib()
    splits, scratch = 0, None
    if S == 1:
        reach = min([T_cap] + [int(v) for v in (window, chunk) if v > 0])
        splits = int(L.jl_attn_generic_splits(B, H, G, reach))
        if splits:
            scratch = torch.empty(B * H * splits * (Dv + 2), dtype=torch.float32, device=q.device)
    _lib.check(L.jl_attn_masked(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(gate), gate.stride(0) if gate is not None else 0,
        _p(cache_len), _p(pad_left), B, S, H, G, D, Dv, T_cap, D, Dv, 0, 0, 0, 0, int(window), int(chunk), float(scale), _p(scratch),
        splits, int(sink), _p(sink_logit), _p(v_cos), _p(v_sin), v_cos.shape[0] if v_cos is not None else 0, int(v_layout), 0,
        dtype_code(q.dtype), _stream()), "jl_attn_masked")
    return out


def retention_scan(y: torch.Tensor, q_off: int, k_off: int, v_off: int, head_decay: torch.Tensor, cos: torch.Tensor,
                   sin: torch.Tensor, rot: int, layout: int, k_scale: float, state: torch.Tensor,
                   cache_len: Optional[torch.Tensor], pad_left: Optional[torch.Tensor], B: int, S: int, H: int, D: int,
                   Dv: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Advance the fp32 state [B, H, D, Dv] over S tokens per row with one fixed decay per head (fp32 [H]), q and k
    rotated at the token's position, k scaled after the rotation; returns the raw read-outs fp32 [B·S, H·Dv]."""
    _need(y, torch.float32, "y")
    _need(state, torch.float32, "state")
    _need(head_decay, torch.float32, "head_decay")
    if out is None:
        out = torch.empty((B * S, H * Dv), dtype=torch.float32, device=y.device)
    L = _lib.lib()
    ws = None
    if S > GLA_FUSED_MAX_TOKENS:
        ws = torch.empty(int(L.jl_gla_scan_ws_floats(B, S, H, D, Dv)), dtype=torch.float32, device=y.device)
    _lib.check(L.jl_retention_scan(
        y.data_ptr(), y.stride(0), q_off, k_off, v_off, head_decay.data_ptr(), cos.data_ptr(), sin.data_ptr(), cos.shape[0],
        rot, layout, 1.0, float(k_scale), state.data_ptr(), out.data_ptr(), _p(cache_len), _p(pad_left), B, S, H, D, Dv,
        _p(ws), _stream()), "jl_retention_scan")
    return out


def moe_route(z: torch.Tensor, E: int, top: int, groups: int, keep: int, group_top: int, score: int, normalise: bool,
              scale: float, bias: Optional[torch.Tensor] = None, choice_bias: Optional[torch.Tensor] = None, n_real: Optional[int] = None,
              ident_w: Optional[torch.Tensor] = None) -> "tuple[torch.Tensor, torch.Tensor]":
    """fp32 router logits (columns 0..E-1 of z, plus the fp32 `bias` [E]) → (experts int32 [M, top], weights fp32 [M, top]).
    choice_bias fp32 [E]: added to the scores for the choice (group scores and top) only.  n_real < E: the router outputs from
    n_real on are identity experts; a chosen one is reported as expert -1 and its weight is added to ident_w fp32 [M]."""
    _need(z, torch.float32, "z")
    M = z.shape[0]
    idx = torch.empty((M, top), dtype=torch.int32, device=z.device)
    wt = torch.empty((M, top), dtype=torch.float32, device=z.device)
    if choice_bias is not None or (n_real is not None and n_real != E):
        _lib.check(_lib.lib().jl_moe_route_ex(z.data_ptr(), z.stride(0), M, E, top, groups, keep, group_top, score, int(normalise),
                                              float(scale), _p(bias), _p(choice_bias), E if n_real is None else int(n_real),
                                              _p(ident_w), idx.data_ptr(), wt.data_ptr(), _stream()), "jl_moe_route_ex")
        return idx, wt
    _lib.check(_lib.lib().jl_moe_route(z.data_ptr(), z.stride(0), M, E, top, groups, keep, group_top, score, int(normalise),
                                       float(scale), _p(bias), idx.data_ptr(), wt.data_ptr(), _stream()), "jl_moe_route")
    return idx, wt


def moe_sort(idx: torch.Tensor, E: int, tile: Optional[int] = None
             ) -> "tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]":
    """(pos int32 [M·top], row_src int32 [rows], tile_group int32 [rows / tile], tiles_used int32 [1]) of the pairs
    ordered by expert, every expert's segment rounded up to `tile` rows (default: the row tile of the SIMT grouped
    linear); tiles_used counts the leading tiles that belong to an expert."""
    L = _lib.lib()
    M, top = idx.shape
    tile = int(L.jl_linear_tile_rows()) if tile is None else int(tile)
    cap = int(L.jl_moe_sorted_rows(M * top, E, tile))
    pos = torch.empty(M * top, dtype=torch.int32, device=idx.device)
    row_src = torch.empty(cap, dtype=torch.int32, device=idx.device)
    tile_group = torch.empty(cap // tile, dtype=torch.int32, device=idx.device)
    used = torch.empty(1, dtype=torch.int32, device=idx.device)
    _lib.check(L.jl_moe_sort(idx.data_ptr(), M, top, E, tile, cap, pos.data_ptr(), row_src.data_ptr(), tile_group.data_ptr(),
                             used.data_ptr(), _stream()), "jl_moe_sort")
    return pos, row_src, tile_group, used


GEMM_TILE_ROWS = 128                    # row tile of the tcgen05 GEMM: the segment size of the grouped form


def moe_gather(x: torch.Tensor, row_src: torch.Tensor) -> torch.Tensor:
    """xs[p] = x[row_src[p]] (zeros where row_src[p] < 0)."""
    W = x.shape[1]
    xs = torch.empty((row_src.shape[0], W), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().jl_moe_gather(x.data_ptr(), x.stride(0), row_src.data_ptr(), xs.data_ptr(), row_src.shape[0], W,
                                        dtype_code(x.dtype), _stream()), "jl_moe_gather")
    return xs


def gemm_grouped(x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, *, act: int = ACT_NONE, out_f32: bool = True,
                 tiles_used: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tcgen05 GEMM over sorted rows: x bf16 [rows, K] (rows a multiple of 128, contiguous), w bf16 [n, N, K]; 128-row
    tile t runs against w[tile_group[t]]; with `tiles_used` (device int) only that many leading tiles are computed
    (the rows after them are left as they are).  The activation is an in-place pass over the stored result."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    n, N, K = w.shape
    rows = x.shape[0]
    out = torch.empty((rows, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    L = _lib.lib()
    _lib.check(L.jl_gemm_grouped(x.data_ptr(), w.data_ptr(), out.data_ptr(), rows, N, K, n, tile_group.data_ptr(), _p(tiles_used),
                                 int(out_f32), num_sms(x.device), _stream()), "jl_gemm_grouped")
    if act != ACT_NONE:
        _lib.check(L.jl_act_inplace(out.data_ptr(), out.stride(0), rows, N, act, 0.0, 0.0, dtype_code(out.dtype), _stream()),
                   "jl_act_inplace")
    return out


def moe_combine(z: torch.Tensor, pos: Optional[torch.Tensor], wt: torch.Tensor, shared: Optional[torch.Tensor],
                gate: Optional[torch.Tensor], W: int, idx: Optional[torch.Tensor] = None, ident_w: Optional[torch.Tensor] = None,
                x: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Σ_k wt[m, k] · z[pos[m, k]] (+ sigmoid(gate[m]) · shared[m]) → fp32 [M, W]; gate: fp32 view [M, 1] (any pitch).
    With `idx` the pairs whose expert is < 0 are skipped, and ident_w[m] · x[m] (identity experts) is added."""
    M, top = wt.shape
    out = torch.empty((M, W), dtype=torch.float32, device=z.device)
    if idx is not None:
        _lib.check(_lib.lib().jl_moe_combine_ex(z.data_ptr(), z.stride(0), _p(pos), wt.data_ptr(), top, _p(shared),
                                                shared.stride(0) if shared is not None else 0, _p(gate),
                                                gate.stride(0) if gate is not None else 0, out.data_ptr(), M, W, idx.data_ptr(),
                                                _p(ident_w), _p(x), x.stride(0) if x is not None else 0,
                                                dtype_code(x.dtype) if x is not None else 1, _stream()), "jl_moe_combine_ex")
        return out
    _lib.check(_lib.lib().jl_moe_combine(z.data_ptr(), z.stride(0), _p(pos), wt.data_ptr(), top, _p(shared),
                                         shared.stride(0) if shared is not None else 0, _p(gate),
                                         gate.stride(0) if gate is not None else 0, out.data_ptr(), M, W, _stream()),
               "jl_moe_combine")
    return out


# --------------------------------------------------------------------------- pair-hash embedding, short convolutions, delta rule, state space
def embed_pair_norm(ids: torch.Tensor, table: torch.Tensor, pair: torch.Tensor, norm_w: Optional[torch.Tensor],
                    prev_tok: torch.Tensor, cache_len: Optional[torch.Tensor], pad_left: Optional[torch.Tensor], B: int, S: int,
                    buckets: int, mul_prev: int, mul_cur: int, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """norm(table[id] + pair[(prev · mul_prev + id · mul_cur) mod buckets]) · norm_w as fp32 [B·S, W]; a sequence's first token
    takes row `buckets`; prev_tok int32 [B] carries the last token from call to call."""
    ids32 = ids.to(torch.int32).contiguous().view(-1)
    V, W = table.shape
    if out is None:
        out = torch.empty((B * S, W), dtype=torch.float32, device=table.device)
    _lib.check(_lib.lib().jl_embed_pair_norm(ids32.data_ptr(), table.data_ptr(), pair.data_ptr(), _p(norm_w), out.data_ptr(),
                                             prev_tok.data_ptr(), _p(cache_len), _p(pad_left), B, S, W, V, int(buckets),
                                             int(mul_prev), int(mul_cur), float(eps), dtype_code(table.dtype), _stream()),
               "jl_embed_pair_norm")
    return out


def causal_conv(y: torch.Tensor, col0: int, w: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor],
                cache_len: Optional[torch.Tensor], pad_left: Optional[torch.Tensor], B: int, S: int, act: int = ACT_SILU,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(causal convolution over time) of the C = w.shape[0] columns of y (fp32) from col0; w [C, taps], the last tap on the
    current token; state fp32 [B, taps-1, C]: the inputs before this call, replaced by this call's last."""
    _need(y, torch.float32, "y")
    C, taps = w.shape
    if out is None:
        out = torch.empty((B * S, C), dtype=torch.float32, device=y.device)
    _lib.check(_lib.lib().jl_causal_conv(y.data_ptr(), y.stride(0), int(col0), C, w.data_ptr(), _p(bias), _p(state), out.data_ptr(),
                                         out.stride(0), _p(cache_len), _p(pad_left), B, S, taps, act, dtype_code(w.dtype), _stream()),
               "jl_causal_conv")
    return out


def norm_mean2(a: torch.Tensor, wa: torch.Tensor, b: Optional[torch.Tensor], wb: Optional[torch.Tensor], c: float, eps: float
               ) -> torch.Tensor:
    """c · (norm(a) · wa + norm(b) · wb), fp32 [M, W]."""
    _need(a, torch.float32, "a")
    M, W = a.shape
    out = torch.empty((M, W), dtype=torch.float32, device=a.device)
    _lib.check(_lib.lib().jl_norm_mean2(a.data_ptr(), a.stride(0), wa.data_ptr(), _p(b), b.stride(0) if b is not None else 0,
                                        _p(wb), float(c), out.data_ptr(), M, W, float(eps), dtype_code(wa.dtype), _stream()),
               "jl_norm_mean2")
    return out


def gated_groupnorm(o: torch.Tensor, x: Optional[torch.Tensor], skip: Optional[torch.Tensor], P: int, z: torch.Tensor,
                    w: torch.Tensor, groups: int, eps: float, gate_act: int = ACT_SILU) -> torch.Tensor:
    """((o + skip[head] · x) · act(z)) normed over each of `groups` equal parts of a row, times w; o fp32 [M, N]; x, z fp32 views."""
    _need(o, torch.float32, "o")
    M, N = o.shape
    out = torch.empty((M, N), dtype=w.dtype, device=o.device)
    _lib.check(_lib.lib().jl_gated_groupnorm(o.data_ptr(), _p(x), x.stride(0) if x is not None else 0, _p(skip), int(P),
                                             z.data_ptr(), z.stride(0), w.data_ptr(), out.data_ptr(), M, N, int(groups),
                                             float(eps), gate_act, dtype_code(w.dtype), _stream()), "jl_gated_groupnorm")
    return out


def glu_act(y: torch.Tensor, g_off: int, u_off: int, F: int, out_dtype: torch.dtype, *, kind: int = GLU_PRODUCT,
            act: int = ACT_GELU_TANH, limit: float = 0.0, alpha: float = 1.0, rows_used: Optional[torch.Tensor] = None,
            rows_mult: int = 1, zero: bool = False) -> torch.Tensor:
    """Gated activation of the fp32 product y [M, gate | up] → [M, F] in `out_dtype`.  rows_used (device int): only the leading
    rows_used · rows_mult rows are computed (`zero`: the rest reads as zero)."""
    _need(y, torch.float32, "y")
    M = y.shape[0]
    out = (torch.zeros if zero else torch.empty)((M, F), dtype=out_dtype, device=y.device)
    _lib.check(_lib.lib().jl_glu_act(y.data_ptr(), y.stride(0), int(g_off), int(u_off), out.data_ptr(), out.stride(0), M, F, kind,
                                     act, float(limit), float(alpha), _p(rows_used), int(rows_mult), dtype_code(out_dtype), _stream()),
               "jl_glu_act")
    return out


def talk_mix(o: torch.Tensor, mix: torch.Tensor, out: torch.Tensor, H: int, G: int, Gc: int, c0: int, Dv: int) -> torch.Tensor:
    """out[m, h] = Σ_g mix[h, g] · o[m, g, kv(h) − c0] for the heads whose key/value head lies in [c0, c0 + Gc); o fp32."""
    _need(o, torch.float32, "o")
    _lib.check(_lib.lib().jl_talk_mix(o.data_ptr(), mix.data_ptr(), out.data_ptr(), out.shape[0], H, G, Gc, c0, Dv,
                                      dtype_code(mix.dtype), _stream()), "jl_talk_mix")
    return out


def ssd_scan(y: torch.Tensor, dt_off: int, dt_bias: torch.Tensor, a_log: torch.Tensor, u: torch.Tensor, q_off: int, k_off: int,
             v_off: int, G: int, state: torch.Tensor, cache_len: Optional[torch.Tensor], pad_left: Optional[torch.Tensor], B: int,
             S: int, H: int, D: int, Dv: int) -> torch.Tensor:
    """Selective state space scan: dt = softplus(y[:, dt_off + h] + dt_bias), S_t = exp(−exp(a_log) dt) S_(t−1) + dt k_t v_tᵀ,
    o_t = S_tᵀ q_t with q / k (G groups of D, columns of u) shared by the heads of a group; state fp32 [B, H, D, Dv]."""
    _need(y, torch.float32, "y")
    _need(u, torch.float32, "u")
    _need(state, torch.float32, "state")
    M = B * S
    L = _lib.lib()
    aux = torch.empty((M, 2 * H), dtype=torch.float32, device=y.device)
    _lib.check(L.jl_ssd_gates(y.data_ptr(), y.stride(0), int(dt_off), dt_bias.data_ptr(), a_log.data_ptr(), aux.data_ptr(), M, H,
                              dtype_code(a_log.dtype), _stream()), "jl_ssd_gates")
    out = torch.empty((M, H * Dv), dtype=torch.float32, device=y.device)
    ws = None
    if S > GLA_FUSED_MAX_TOKENS:
        ws = torch.empty(int(L.jl_gla_scan_ws_floats(B, S, H, D, Dv)), dtype=torch.float32, device=y.device)
    _lib.check(L.jl_ssd_scan(u.data_ptr(), u.stride(0), q_off, k_off, v_off, G, aux.data_ptr(), state.data_ptr(), out.data_ptr(),
                             _p(cache_len), _p(pad_left), B, S, H, D, Dv, _p(ws), _stream()), "jl_ssd_scan")
    return out


def delta_scan(u: torch.Tensor, q_off: int, k_off: int, v_off: int, G: int, y: torch.Tensor, b_off: int, a_off: int,
               a2: torch.Tensor, a_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor,
               cache_len: Optional[torch.Tensor], pad_left: Optional[torch.Tensor], B: int, S: int, H: int, D: int, Dv: int
               ) -> torch.Tensor:
    """Gated delta rule over S tokens per row (see csrc/delta_scan.cu); returns the raw read-outs fp32 [B·S, H·Dv]."""
    _need(u, torch.float32, "u")
    _need(y, torch.float32, "y")
    _need(state, torch.float32, "state")
    L = _lib.lib()
    R = a2.shape[1]
    out = torch.empty((B * S, H * Dv), dtype=torch.float32, device=y.device)
    ws = None
    if S > DELTA_FUSED_MAX_TOKENS:        # prompts: token-parallel records + pipelined scan; fewer tokens: one fused launch
        ws = torch.empty(int(L.jl_delta_scan_ws_floats(B, S, H, D, Dv)), dtype=torch.float32, device=y.device)
    _lib.check(L.jl_delta_scan(u.data_ptr(), u.stride(0), q_off, k_off, v_off, G, y.data_ptr(), y.stride(0), b_off, a_off,
                               a2.data_ptr(), a_bias.data_ptr(), a_log.data_ptr(), state.data_ptr(), out.data_ptr(),
                               _p(cache_len), _p(pad_left), B, S, H, D, Dv, R, _p(ws), dtype_code(a2.dtype), _stream()),
               "jl_delta_scan")
    return out


# --------------------------------------------------------------------------- learned positions, per-layer token input
def embed_pos(ids: torch.Tensor, table: torch.Tensor, pos_table: torch.Tensor, cache_len: Optional[torch.Tensor],
              pad_left: Optional[torch.Tensor], B: int, S: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """table[id] + pos_table[position] as fp32 [B·S, W]; token (b, s) is at position *cache_len + s − pad_left[b]."""
    ids32 = ids if ids.dtype == torch.int32 and ids.is_contiguous() else ids.to(torch.int32).contiguous()
    V, W = table.shape
    if out is None:
        out = torch.empty((B * S, W), dtype=torch.float32, device=table.device)
    _lib.check(_lib.lib().jl_embed_pos(ids32.data_ptr(), table.data_ptr(), pos_table.data_ptr(), out.data_ptr(), _p(cache_len),
                                       _p(pad_left), B, S, W, V, pos_table.shape[0], dtype_code(table.dtype), _stream()),
               "jl_embed_pos")
    return out


def side_gate(t: torch.Tensor, ids: torch.Tensor, side: torch.Tensor, col0: int, n: int, out_dtype: torch.dtype) -> torch.Tensor:
    """gelu_tanh(t[m, c]) · side[ids[m], col0 + c] for c < n; t fp32 [M, ≥ n]; ids int32 [M]; the result in `out_dtype`."""
    _need(t, torch.float32, "t")
    _need(ids, torch.int32, "ids")
    M = t.shape[0]
    out = torch.empty((M, n), dtype=out_dtype, device=t.device)
    _lib.check(_lib.lib().jl_side_gate(t.data_ptr(), t.stride(0), ids.data_ptr(), side.data_ptr(), side.stride(0), int(col0),
                                       out.data_ptr(), out.stride(0), M, int(n), side.shape[0], dtype_code(out_dtype), _stream()),
               "jl_side_gate")
    return out


def side_gate_rows(x: torch.Tensor, ids: torch.Tensor, side: torch.Tensor, col0: int, w_gate: torch.Tensor) -> torch.Tensor:
    """gelu_tanh(w_gate x[m]) · side[ids[m], col0 : col0 + n] for up to 8 rows in one launch; x fp32 [M, W] is read as it is
    (not rounded to the weights' type); the result in the weights' dtype."""
    _need(x, torch.float32, "x")
    _need(ids, torch.int32, "ids")
    M, W = x.shape
    n = w_gate.shape[0]
    out = torch.empty((M, n), dtype=w_gate.dtype, device=x.device)
    _lib.check(_lib.lib().jl_side_gate_rows(x.data_ptr(), x.stride(0), ids.data_ptr(), side.data_ptr(), side.stride(0), int(col0),
                                            w_gate.data_ptr(), out.data_ptr(), out.stride(0), M, W, n, side.shape[0],
                                            dtype_code(w_gate.dtype), _stream()), "jl_side_gate_rows")
    return out


def branch_add_cast(x: torch.Tensor, y1: Optional[torch.Tensor], y2: Optional[torch.Tensor], mult: float, dtype: torch.dtype
                    ) -> torch.Tensor:
    """x += mult · (y1 + y2) in place (fp32; either branch may be None); returns the updated rows in `dtype`."""
    _need(x, torch.float32, "x")
    M, W = x.shape
    xc = torch.empty((M, W), dtype=dtype, device=x.device)
    _lib.check(_lib.lib().jl_branch_add_cast(_p(y1), y1.stride(0) if y1 is not None else 0, _p(y2),
                                             y2.stride(0) if y2 is not None else 0, float(mult), x.data_ptr(), xc.data_ptr(), M, W,
                                             dtype_code(dtype), _stream()), "jl_branch_add_cast")
    return xc
