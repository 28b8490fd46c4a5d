"""Side-by-side throughput of a newer design and the closest existing model of equal width, depth and head counts, with
random weights, plus the time of each kernel of the new design beside the like kernel of the other path:

* ``bench.py --compare folirax`` — Folirax beside LLaMA (`run`),
* ``bench.py --compare nikonex`` — Nikonex beside Folirax (`run_nikonex`),
* ``bench.py --compare bazulorn`` — Bazulorn beside Nikonex (`run_bazulorn`),
* ``bench.py --compare datozen`` — Datozen beside Bazulorn (`run_datozen`).

Everything is timed with CUDA events on the launching stream after warm-up; per-kernel timings flush L2 (a 256 MB write)
between iterations, whole-model timings stream more weight bytes than L2 holds.  Fractions are of the measured peaks in
MEASURED_PEAKS.json (HBM copy bandwidth, cuBLAS bf16 burst).
"""
from __future__ import annotations

import json
import os
import statistics
from typing import Any, Callable, Dict, List

import torch

SIZES: Dict[str, Dict[str, int]] = {
    # width, heads x 128 attention (kv heads), ff, layers, vocab
    "w2048": dict(width=2048, heads=16, kv_heads=4, ff=8192, layers=8, vocab=32000),
    "w4096": dict(width=4096, heads=32, kv_heads=8, ff=14336, layers=4, vocab=32000),
}


def folirax_config(s: Dict[str, int]) -> Any:
    from ..config import FoliraxConfig

    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
           "rot": {"dims": 64, "base": 10000.0}}
    gla = {"heads": s["heads"], "dim": 64, "vdim": 128, "tau": 16.0}
    mlp = {"kind": "dense", "ff": s["ff"]}
    block = [{"type": "gla", "mixer": gla, "mlp": None}, {"type": "attention", "mixer": att, "mlp": mlp},
             {"type": "attention", "mixer": dict(att, kv_from=None), "mlp": mlp}, {"type": "gla", "mixer": gla, "mlp": mlp}]
    layers: List[Dict[str, Any]] = []
    for i in range(s["layers"]):
        l = json.loads(json.dumps(block[i % 4]))
        if i % 4 == 2:
            l["mixer"]["kv_from"] = i - 1
        layers.append(l)
    return FoliraxConfig.from_dict({"architecture": "Folirax", "vocab": s["vocab"], "width": s["width"],
                                    "norm": {"eps": 1e-5}, "logit_scale": 0.5, "logit_softcap": 30.0, "layers": layers})


def llama_config(s: Dict[str, int]) -> Any:
    from ..config import LLaMAConfig

    return LLaMAConfig(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"],
                       num_hidden_layers=s["layers"], num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"],
                       max_sequence_length=4096, rms_norm_eps=1e-5)


class Timer:
    def __init__(self, device: torch.device):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def kernel(self, fn: Callable[[], Any], reps: int = 10) -> float:
        """Median ms of one call of fn with a cold L2."""
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)


def _model_times(eng: Any, vocab: int, prompt_len: int, batches: List[int], steps: int, warmup: int) -> Dict[str, Any]:
    dev = eng.device
    out: Dict[str, Any] = {}
    g = torch.Generator().manual_seed(7)
    for B in batches:
        ids = torch.randint(1, vocab, (B, prompt_len), generator=g).to(dev)
        max_len = prompt_len + warmup + steps + 8
        st = eng._decode_state(B, max_len)
        pre = []
        for i in range(4):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.prepare(st, ids, None, 0)
            e1.record()
            torch.cuda.synchronize()
            if i:
                pre.append(e0.elapsed_time(e1))
        stream = eng.begin_stream(ids, None, max_length=max_len, eos_token_id=-1)
        for _ in range(warmup):
            stream.graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            stream.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[f"batch{B}"] = {"prefill_ms": round(min(pre), 3), "prefill_tokens_per_sec": round(B * prompt_len / min(pre) * 1e3, 1),
                            "decode_ms_per_step": round(ms, 4), "decode_tokens_per_sec": round(B / ms * 1e3, 1),
                            "launches_per_decode_step": eng.launches_per_step(st)}
        stream.close()
    out["weight_bytes_per_step"] = eng.weight_bytes_per_step()
    return out


def _kernel_table(s: Dict[str, int], dev: torch.device, peaks: Dict[str, float], prompt_len: int) -> List[Dict[str, Any]]:
    """Each kernel of the new design at this size beside the like kernel of the LLaMA path: ms, achieved rate, and the
    fraction of the measured roofline (HBM copy peak for memory-bound kernels, cuBLAS bf16 burst for GEMM-shaped ones)."""
    from ..models.mixers import rotary_table
    from ..models.reference import rope_cos_sin
    from ..ops import _lib as L
    from ..ops import kernels as K
    from ..ops import seq_kernels as SK

    t = Timer(dev)
    hbm, tf = peaks["hbm_gbs"], peaks["bf16_tflops"]
    W, H, G, F = s["width"], s["heads"], s["kv_heads"], s["ff"]
    D = Dv = 128
    gd, gv, R = 64, 128, 16
    bf = dict(dtype=torch.bfloat16, device=dev)
    rows: List[Dict[str, Any]] = []

    def add(name: str, ms: float, like: str, like_ms: float, nbytes: float = 0.0, flops: float = 0.0, note: str = "",
            like_nbytes: float = 0.0) -> None:
        r: Dict[str, Any] = {"kernel": name, "ms": round(ms, 4), "like": like, "like_ms": round(like_ms, 4) if like_ms else None}
        if nbytes:
            r["gbs"] = round(nbytes / ms / 1e6, 1)
            r["frac_hbm_of_measured"] = round(nbytes / ms / 1e6 / hbm, 3)
            if like_ms:
                r["like_frac"] = round((like_nbytes or nbytes) / like_ms / 1e6 / hbm, 3)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["frac_bf16_of_measured"] = round(flops / ms / 1e9 / tf, 3)
            if like_ms:
                r["like_frac"] = round(flops / like_ms / 1e9 / tf, 3)
        if note:
            r["note"] = note
        rows.append(r)

    # ---- decode, one row: stacked input projection of a recurrent layer / fused qkv of LLaMA (weight streaming)
    n_in = 2 * H * gd + 2 * H * gv + R
    n_in += (-n_in) % 8
    w = torch.randn(n_in, W, **bf) * 0.02
    x = torch.randn(1, W, **bf)
    add("linear_rows (stacked projection, M=1)", t.kernel(lambda: SK.linear(x, w)), "gemv_kernel",
        t.kernel(lambda: K.linear(x, w, out_f32=True)), nbytes=w.numel() * 2)
    wd = torch.randn(W, F, **bf) * 0.02
    xf = torch.randn(1, F, **bf)
    add("linear_rows (ff down, M=1)", t.kernel(lambda: SK.linear(xf, wd)), "gemv_kernel",
        t.kernel(lambda: K.linear(xf, wd, out_f32=True)), nbytes=wd.numel() * 2)
    x8 = torch.randn(8, W, **bf)
    add("linear_rows (stacked projection, M=8)", t.kernel(lambda: SK.linear(x8, w)), "gemv_kernel (M=8)",
        t.kernel(lambda: K.linear(x8, w, out_f32=True, force="gemv")), nbytes=w.numel() * 2)

    # ---- prefill GEMM: the same tcgen05 kernel, fp32 result + activation pass vs bf16 result
    xp = torch.randn(prompt_len, W, **bf)
    wu = torch.randn(F, W, **bf) * 0.02
    fl = 2.0 * prompt_len * F * W
    add("tcgen05 GEMM bf16 out + in-place relu^2 pass (ff up)", t.kernel(lambda: SK.linear(xp, wu, act=SK.ACT_RELU2, out_f32=False)),
        "tcgen05 GEMM bf16 out (same N, K)", t.kernel(lambda: K.linear(xp, wu)), flops=fl)

    # ---- norms
    xr = torch.randn(prompt_len, W, device=dev)
    yr = torch.randn(prompt_len, W, device=dev)
    wn = torch.zeros(W, **bf)
    xb, db = xr.to(torch.bfloat16), yr.to(torch.bfloat16)
    add("postnorm_add (+ next norm), fp32 stream", t.kernel(lambda: SK.postnorm_add(yr, wn, xr, 1e-5, 1.0, w_next=wn)),
        "rmsnorm_kernel (+ residual), bf16 stream", t.kernel(lambda: K.rmsnorm(xb, wn, 1e-5, delta=db)),
        nbytes=prompt_len * W * (4 + 4 + 4 + 2), like_nbytes=prompt_len * W * 8,
        note="like kernel moves 8 B per element, this one 14 B (fp32 residual)")

    # ---- attention, prompt and one token at a 2k context
    T = prompt_len + 8
    cos, sin = rotary_table(64, 10000.0, T, dev)
    y = torch.randn(prompt_len, (H + 2 * G) * D + 8, device=dev)
    q = torch.empty(prompt_len, H * D, **bf)
    kc, vc = torch.zeros(1, G, T, D, **bf), torch.zeros(1, G, T, Dv, **bf)
    zero, pad = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    prep = lambda: SK.attn_prep(y, 0, H * D, (H + G) * D, q, kc, vc, cos, sin, 64, True, 1e-5, zero, pad, 1, prompt_len,  # noqa: E731
                                H, G, D, Dv)
    prep()
    lc, ls = (c.to(dev) for c in rope_cos_sin(D, T, 10000.0))
    qkv = torch.randn(prompt_len, (H + 2 * G) * D, **bf)
    q2 = torch.empty(prompt_len, H * D, **bf)
    add("attn_prep (rotary + unit norm + append), prompt", t.kernel(prep), "rope_kv_kernel",
        t.kernel(lambda: K.rope_kv_write(qkv, kc, vc, lc, ls, 1, prompt_len, H, G, D, cache_len=zero, pad_left=pad, q_out=q2)),
        nbytes=prompt_len * (H + 2 * G) * D * (4 + 2), like_nbytes=prompt_len * (H + 2 * G) * D * (2 + 2),
        note="reads the fp32 projection (4 B) where the like kernel reads bf16")
    causal = 4.0 * prompt_len * prompt_len / 2 * D * H
    out = torch.empty(prompt_len, H * Dv, **bf)
    flash = lambda: L.check(L.lib().jl_flash_prefill(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), zero.data_ptr(), pad.data_ptr(),  # noqa: E731
                                                     out.data_ptr(), 1, prompt_len, H, G, D, T, 0, D ** -0.5, K._stream()), "flash")
    ms_flash = t.kernel(flash)
    gate = y[:, :H]
    add("flash_prefill_kernel + head_gate pass", ms_flash + t.kernel(lambda: SK.head_gate(out, gate, H, Dv)),
        "flash_prefill_kernel", ms_flash, flops=causal)
    add("attn_rows_kernel (exact SIMT, any head size)", t.kernel(lambda: SK.attn_generic(q, kc, vc, gate, zero, pad, 1, prompt_len, H, D ** -0.5), reps=3),
        "flash_prefill_kernel", ms_flash, flops=causal, note="fall-back for head sizes other than 64 / 128 and for float32")
    ctx = torch.full((1,), prompt_len, dtype=torch.int32, device=dev)
    q1 = torch.randn(1, H * D, **bf)
    kv_bytes = 2.0 * G * prompt_len * D * 2
    splits, scratch = K.decode_attn_plan(1, H, G, D, T, dev)
    o1 = torch.empty(1, H * Dv, **bf)
    dec = lambda: L.check(L.lib().jl_decode_attn(q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(), pad.data_ptr(),  # noqa: E731
                                                 K._p(scratch), o1.data_ptr(), 1, H, G, D, T, 1, D ** -0.5, splits, 0, K._stream()), "dec")
    ms_dec = t.kernel(dec)
    add("decode_attn_kernel (shared) + head_gate", ms_dec + t.kernel(lambda: SK.head_gate(o1, gate[:1], H, Dv)),
        "decode_attn_kernel", ms_dec, nbytes=kv_bytes)
    add("attn_decode_kernel (exact SIMT, any head size)", t.kernel(lambda: SK.attn_generic(q1, kc, vc, gate[:1], ctx, pad, 1, 1, H, D ** -0.5)),
        "decode_attn_kernel", ms_dec, nbytes=kv_bytes, note="one CTA per (row, head): fall-back shapes only")

    # ---- gated linear attention: no like kernel in the LLaMA path
    n_y = 2 * H * gd + 2 * H * gv + R
    yg = torch.randn(prompt_len, n_y, device=dev) * 0.3
    a2 = torch.randn(H * gd, R, **bf) * 0.1
    a2b = torch.full((H * gd,), 3.0, **bf)
    state = torch.zeros(1, H, gd, gv, device=dev)
    scan = lambda S: SK.gla_scan(yg[:S], 0, H * gd, 2 * H * gd, 2 * H * gd + 2 * H * gv, a2, a2b, state, zero, pad, 1, S, H, gd, gv,  # noqa: E731
                                 gd ** -0.5, 16.0)
    ms = t.kernel(lambda: scan(prompt_len), reps=5)
    add("gla_scan_kernel, prompt", ms, "(none)", 0.0, flops=0.0,
        note=f"{3.0 * prompt_len * H * gd * gv / ms / 1e9:.2f} fp32 TFLOP/s of recurrence (3 ops per state element and token); "
             "sequential in time, parallel over heads and value columns")
    state8 = torch.zeros(8, H, gd, gv, device=dev)
    yg8 = yg[:8].contiguous()
    ms1 = t.kernel(lambda: SK.gla_scan(yg8, 0, H * gd, 2 * H * gd, 2 * H * gd + 2 * H * gv, a2, a2b, state8, zero,
                                       torch.zeros(8, dtype=torch.int32, device=dev), 8, 1, H, gd, gv, gd ** -0.5, 16.0))
    add("gla_scan_kernel, one token, batch 8", ms1, "(none)", 0.0, nbytes=2.0 * state8.numel() * 4,
        note="reads and writes the fp32 state once")
    o = torch.randn(prompt_len, H * gv, device=dev)
    add("headnorm_gate_kernel", t.kernel(lambda: SK.headnorm_gate(o, torch.ones(gv, **bf), yg[:, :H * gv], H, gv, 1e-5)),
        "swiglu_kernel", t.kernel(lambda: K.swiglu(torch.randn(prompt_len, 2 * H * gv, **bf))), nbytes=prompt_len * H * gv * (4 + 4 + 2))
    return rows


def run(sizes: List[str], prompt_len: int = 2048, steps: int = 64, warmup: int = 8, batches: List[int] = (1, 8),
        kernels: bool = True) -> Dict[str, Any]:
    from ..models.engine import B200Engine
    from ..models.hybrid_engine import HybridEngine

    dev = torch.device("cuda", torch.cuda.current_device())
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        peaks = {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        pass
    result: Dict[str, Any] = {"metric": "folirax_vs_llama_equal_size", "data": "synthetic", "dtype": "bf16", "peaks": peaks,
                              "prompt_len": prompt_len, "steps": steps, "warmup": warmup, "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        entry: Dict[str, Any] = {"shape": s}
        fcfg = folirax_config(s)
        eng = HybridEngine.random_init(fcfg, dev, seed=0)
        entry["folirax"] = _model_times(eng, s["vocab"], prompt_len, list(batches), steps, warmup)
        del eng
        torch.cuda.empty_cache()
        leng = B200Engine.random_init(llama_config(s), dev, seed=0)
        entry["llama"] = _model_times(leng, s["vocab"], prompt_len, list(batches), steps, warmup)
        del leng
        torch.cuda.empty_cache()
        if kernels:
            entry["kernels"] = _kernel_table(s, dev, peaks, prompt_len)
        result["sizes"][name] = entry
    return result


# --------------------------------------------------------------------------- Nikonex beside Folirax
# width, heads, dense ff of the Folirax model; the Nikonex model of equal size has top x expert_ff + shared_ff = ff active
# feed-forward columns per token, the same head counts and recurrent head sizes, and latent attention with 128 + 64
# wide heads over a latent of 512
NIKONEX_SIZES: Dict[str, Dict[str, int]] = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, ff=8192, layers=8, vocab=32000, experts=32, top=4, expert_ff=1536,
                  shared_ff=2048, q_rank=768, kv_rank=512, window=1024),
    "w4096": dict(width=4096, heads=32, kv_heads=8, ff=14336, layers=4, vocab=32000, experts=32, top=4, expert_ff=2560,
                  shared_ff=4096, q_rank=1536, kv_rank=512, window=1024),
}


def nikonex_config(s: Dict[str, int]) -> Any:
    from ..config import NikonexConfig

    H = s["heads"]
    lat = {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": s["q_rank"], "kv_rank": s["kv_rank"],
           "scale": 192 ** -0.5, "mask": {"size": s["window"]},
           "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}
    ret = {"heads": H, "dim": 64, "vdim": 128, "decay": [1.0 - 0.05 * 0.1 ** (h / max(H - 1, 1)) for h in range(H)],
           "rot": {"dims": 64, "base": 10000.0}}
    mlp = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]},
           "router": {"experts": s["experts"], "top": s["top"], "scale": 2.0, "groups": {"count": 4, "keep": 2}}}
    block = [("retention", ret, None), ("latent_attention", lat, mlp), ("latent_attention", lat, mlp), ("retention", ret, mlp)]
    layers = [{"type": block[i % 4][0], "mixer": block[i % 4][1], "mlp": block[i % 4][2]} for i in range(s["layers"])]
    return NikonexConfig.from_dict({"architecture": "Nikonex", "vocab": s["vocab"], "width": s["width"],
                                    "norm": {"eps": 1e-5}, "residual_mult": 0.5, "layers": layers})


def _nikonex_kernel_table(s: Dict[str, int], dev: torch.device, peaks: Dict[str, float], prompt_len: int) -> List[Dict[str, Any]]:
    """Each kernel that Nikonex adds, at this size, beside the like kernel of the Folirax path: ms, achieved rate and the
    fraction of the measured roofline, and how much farther from it the new kernel is (`distance_ratio`)."""
    from ..config import MoeMlpSpec
    from ..models.feedforward import MoeFeedForward
    from ..models.mixers import rotary_table
    from ..ops import seq_kernels as SK

    t = Timer(dev)
    hbm, tf = peaks["hbm_gbs"], peaks["bf16_tflops"]
    W, H, F = s["width"], s["heads"], s["ff"]
    E, top, ef, sf = s["experts"], s["top"], s["expert_ff"], s["shared_ff"]
    rank, qr, win = s["kv_rank"], s["q_rank"], s["window"]
    D, R, Dv, gd, gv = 128, 64, 128, 64, 128
    P = prompt_len
    bf = dict(dtype=torch.bfloat16, device=dev)
    rows: List[Dict[str, Any]] = []

    def add(name: str, ms: float, like: str, like_ms: float, nbytes: float = 0.0, flops: float = 0.0, like_nbytes: float = 0.0,
            like_flops: float = 0.0, note: str = "") -> None:
        r: Dict[str, Any] = {"kernel": name, "ms": round(ms, 4), "like": like, "like_ms": round(like_ms, 4) if like_ms else None}
        frac = like_frac = None
        if nbytes:
            r["gbs"] = round(nbytes / ms / 1e6, 1)
            frac = nbytes / ms / 1e6 / hbm
            r["frac_hbm_of_measured"] = round(frac, 3)
            if like_ms:
                like_frac = (like_nbytes or nbytes) / like_ms / 1e6 / hbm
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            frac = flops / ms / 1e9 / tf
            r["frac_bf16_of_measured"] = round(frac, 4)
            if like_ms:
                like_frac = (like_flops or flops) / like_ms / 1e9 / tf
        if like_frac is not None:
            r["like_frac"] = round(like_frac, 4)
            r["distance_ratio"] = round(like_frac / frac, 2)
        if note:
            r["note"] = note
        rows.append(r)

    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pad = torch.zeros(1, dtype=torch.int32, device=dev)
    ctx_len = torch.full((1,), P, dtype=torch.int32, device=dev)

    # ---- residual step: both branches + two norms in one kernel / one branch + post-norm + next norm
    x, y1, y2 = (torch.randn(P, W, device=dev) for _ in range(3))
    w1, w2 = torch.ones(W, **bf), torch.ones(W, **bf)
    add("branch_add_norm (two branches, two norms)", t.kernel(lambda: SK.branch_add_norm(x, y1, y2, 0.5, w1, w2, 1e-5)),
        "postnorm_add (+ next norm)", t.kernel(lambda: SK.postnorm_add(y1, w1, x, 1e-5, 1.0, w_next=w2)),
        nbytes=P * W * 20.0, like_nbytes=P * W * 14.0)

    # ---- latent attention: preparation, windowed attention over the cached latents (prompt, one token)
    T = P + 8
    cos, sin = rotary_table(R, 10000.0, T, dev)
    n_in = qr + rank + R
    y = torch.randn(P, n_in, device=dev)
    wqn, wkn = torch.ones(qr, **bf), torch.ones(rank, **bf)
    cache = torch.zeros(1, T, rank + R, **bf)
    prep = lambda: SK.latent_prep(y, 0, qr, qr, rank, R, R, 0, wqn, wkn, cache, cos, sin, 1e-5, zero, pad, 1, P)   # noqa: E731
    prep()
    yq = torch.randn(P, (H + 2 * H // 4) * D + 8, device=dev)
    qo = torch.empty(P, H * D, **bf)
    kc, vc = torch.zeros(1, H // 4, T, D, **bf), torch.zeros(1, H // 4, T, Dv, **bf)
    add("latent_prep (two norms, rotation, append)", t.kernel(prep), "attn_prep (rotation, unit norm, append)",
        t.kernel(lambda: SK.attn_prep(yq, 0, H * D, (H + H // 4) * D, qo, kc, vc, cos, sin, 64, True, 1e-5, zero, pad, 1, P, H,
                                      H // 4, D, Dv)),
        nbytes=P * n_in * 4.0 + P * (qr + rank + R) * 2.0, like_nbytes=P * (H + 2 * H // 4) * D * 6.0)
    row = rank + R
    qd = D + R
    win_keys = sum(min(i + 1, win) for i in range(P))
    qf = torch.randn(P, H * qd, **bf) * 0.05
    kf = torch.randn(P, H * qd, **bf) * 0.05
    vf = torch.randn(P, H * Dv, **bf)
    q128 = torch.randn(P, H * D, **bf) * 0.05
    kg, vg = torch.randn(1, H // 4, T, D, **bf), torch.randn(1, H // 4, T, Dv, **bf)
    full_keys = P * (P + 1) / 2
    add("attn_rows_kernel, windowed, projected per-head keys (prompt)",
        t.kernel(lambda: SK.attn_windowed(qf, kf, vf, zero, pad, 1, P, H, H, qd, Dv, P, H * qd, H * Dv, win, 192 ** -0.5,
                                          strides=(P * H * qd, qd, P * H * Dv, Dv)), reps=3),
        "attn_rows_kernel (prompt)", t.kernel(lambda: SK.attn_generic(q128, kg, vg, None, zero, pad, 1, P, H, D ** -0.5), reps=3),
        flops=2.0 * H * win_keys * (qd + Dv), like_flops=2.0 * H * full_keys * (D + Dv),
        note="the same exact SIMT kernel (heads of 192 / 128 channels fit no tensor-core attention kernel of the framework); "
             "fractions are of the tensor-core peak")
    cl = torch.randn(P, rank, **bf)
    wkv = torch.randn(H * (D + Dv), rank, **bf) * 0.04
    wqkv = torch.randn(H * (D + Dv), W, **bf) * 0.02
    xw = torch.randn(P, W, **bf)
    add("tcgen05 GEMM (latents up to per-head keys and values, prompt)", t.kernel(lambda: SK.linear(cl, wkv, out_f32=False)),
        "tcgen05 GEMM (projection from the stream, same N)", t.kernel(lambda: SK.linear(xw, wqkv, out_f32=False)),
        flops=2.0 * P * H * (D + Dv) * rank, like_flops=2.0 * P * H * (D + Dv) * W, note="the same kernel at K = latent size")
    q1 = torch.randn(1, H * row, **bf) * 0.05
    q1g = torch.randn(1, H * D, **bf) * 0.05
    add("attn_split_kernel, windowed, shared latent rows (one token)",
        t.kernel(lambda: SK.attn_windowed(q1, cache, cache, ctx_len, pad, 1, 1, H, 1, row, rank, T, row, row, win, 192 ** -0.5)),
        "attn_split_kernel (one token)", t.kernel(lambda: SK.attn_generic(q1g, kg, vg, None, ctx_len, pad, 1, 1, H, D ** -0.5)),
        nbytes=min(win, P) * row * 2.0, like_nbytes=2.0 * (H // 4) * P * D * 2.0,
        note="reads one shared latent row per key for all heads")
    # per-head products into and out of the latent (one token; prompts use the GEMM above)
    ukt = torch.randn(H, rank, D, **bf) * 0.05
    wd = torch.randn(H * D, W, **bf) * 0.02
    q1h = torch.randn(1, H * (D + R), **bf)
    q1abs = torch.empty(1, H * row, **bf)
    x1 = torch.randn(1, W, **bf)
    add("linear_batched (per-head map into the latent, one token)",
        t.kernel(lambda: SK.linear_batched(q1h, ukt, q1abs, nbatch=H, rows=1, x_bs=D + R, o_bs=row)),
        "linear_rows (q projection, one token)", t.kernel(lambda: SK.linear(x1, wd)),
        nbytes=ukt.numel() * 2.0, like_nbytes=wd.numel() * 2.0)

    # ---- retention beside gated linear attention
    n_y = 2 * H * gd + 2 * H * gv + 16
    yg = torch.randn(P, n_y, device=dev) * 0.3
    a2 = torch.randn(H * gd, 16, **bf) * 0.1
    a2b = torch.full((H * gd,), 3.0, **bf)
    state = torch.zeros(1, H, gd, gv, device=dev)
    decay = torch.linspace(0.97, 0.999, H, device=dev)
    rc, rs = rotary_table(gd, 10000.0, T, dev)
    rec = 3.0 * P * H * gd * gv
    ms_r = t.kernel(lambda: SK.retention_scan(yg, 0, H * gd, 2 * H * gd, decay, rc, rs, gd, SK.ROT_HALF, gd ** -0.5, state, zero, pad,
                                              1, P, H, gd, gv), reps=5)
    ms_g = t.kernel(lambda: SK.gla_scan(yg, 0, H * gd, 2 * H * gd, 2 * H * gd + 2 * H * gv, a2, a2b, state, zero, pad, 1, P, H, gd,
                                        gv, gd ** -0.5, 16.0), reps=5)
    rows.append({"kernel": "retention scan (prompt)", "ms": round(ms_r, 4), "like": "gla scan (prompt)", "like_ms": round(ms_g, 4),
                 "recurrence_tflops_fp32": round(rec / ms_r / 1e9, 2), "like_recurrence_tflops_fp32": round(rec / ms_g / 1e9, 2),
                 "distance_ratio": round(ms_r / ms_g, 2), "note": "the same kernels; the decay is a constant per head"})
    state8 = torch.zeros(8, H, gd, gv, device=dev)
    yg8 = yg[:8].contiguous()
    pad8 = torch.zeros(8, dtype=torch.int32, device=dev)
    add("retention scan (one token, batch 8)",
        t.kernel(lambda: SK.retention_scan(yg8, 0, H * gd, 2 * H * gd, decay, rc, rs, gd, SK.ROT_HALF, gd ** -0.5, state8, ctx_len,
                                           pad8, 8, 1, H, gd, gv)),
        "gla scan (one token, batch 8)",
        t.kernel(lambda: SK.gla_scan(yg8, 0, H * gd, 2 * H * gd, 2 * H * gd + 2 * H * gv, a2, a2b, state8, ctx_len, pad8, 8, 1, H, gd,
                                     gv, gd ** -0.5, 16.0)), nbytes=2.0 * state8.numel() * 4)

    # ---- mixture of experts beside the dense feed-forward of equal active size
    spec = MoeMlpSpec(experts=E, top=top, ff=ef, groups=4, keep=2, scale=2.0, shared_ff=0)
    g = torch.Generator(device=dev).manual_seed(3)
    wts = {n: (torch.randn(sh, device=dev, generator=g) / sh[1] ** 0.5).to(torch.bfloat16)
           for n, sh in MoeFeedForward.shapes(spec, W).items()}
    moe = MoeFeedForward(spec, wts)
    del wts
    hp = torch.randn(P, W, device=dev, generator=g).to(torch.bfloat16)
    z = SK.linear(hp, moe.w_route)
    route = lambda: SK.moe_route(z, E, top, 4, 2, 2, SK.SCORE_SIGMOID, True, 2.0)      # noqa: E731
    idx, wt = route()
    rows.append({"kernel": "moe_route (prompt)", "ms": round(t.kernel(route), 4), "like": "(none)", "like_ms": None,
                 "note": "one warp per token over the fp32 logits"})
    sort = lambda: SK.moe_sort(idx, E, tile=SK.GEMM_TILE_ROWS)                            # noqa: E731
    pos, row_src, tile_group, used = sort()
    rows.append({"kernel": "moe_sort (prompt)", "ms": round(t.kernel(sort), 4), "like": "(none)", "like_ms": None,
                 "note": "one CTA orders the (token, choice) pairs by expert"})
    nrows = row_src.shape[0]
    xs = SK.moe_gather(hp, row_src)
    add("moe_gather (rows in sorted order)", t.kernel(lambda: SK.moe_gather(hp, row_src)), "(none)", 0.0, nbytes=nrows * W * 4.0)
    wu = torch.randn(top * ef, W, **bf) * 0.02
    fl_up = 2.0 * P * top * ef * W
    add("grouped tcgen05 GEMM + relu^2 pass (experts up)",
        t.kernel(lambda: SK.gemm_grouped(xs, moe.up, tile_group, act=SK.ACT_RELU2, out_f32=False, tiles_used=used)),
        "tcgen05 GEMM + relu^2 pass (dense up, equal active size)",
        t.kernel(lambda: SK.linear(hp, wu, act=SK.ACT_RELU2, out_f32=False)), flops=fl_up,
        note=f"{int(used.item()) * 128} sorted rows for {P * top} pairs (segments rounded up to 128)")
    tmid = torch.randn(nrows, ef, **bf) * 0.1
    tdense = torch.randn(P, top * ef, **bf) * 0.1
    wdn = torch.randn(W, top * ef, **bf) * 0.02
    add("grouped tcgen05 GEMM, fp32 out (experts down)", t.kernel(lambda: SK.gemm_grouped(tmid, moe.down, tile_group, tiles_used=used)),
        "tcgen05 GEMM, fp32 out (dense down, equal active size)", t.kernel(lambda: SK.linear(tdense, wdn)), flops=fl_up)
    yexp = torch.randn(nrows, W, device=dev)
    sh = torch.randn(P, W, device=dev)
    add("moe_combine (weighted sum + gated shared expert)", t.kernel(lambda: SK.moe_combine(yexp, pos, wt, sh, z[:, E:E + 1], W)),
        "(none)", 0.0, nbytes=P * W * 4.0 * (top + 2))
    h1 = hp[:1].contiguous()
    ms_moe1 = t.kernel(lambda: moe.run(h1))
    wu1 = torch.randn(top * ef, W, **bf) * 0.02
    wd1 = torch.randn(W, top * ef, **bf) * 0.02
    t1 = torch.randn(1, top * ef, **bf)
    ms_dense1 = t.kernel(lambda: SK.linear(t1, wd1)) + t.kernel(lambda: SK.linear(h1, wu1, act=SK.ACT_RELU2, out_f32=False))
    add("experts, one token (router, choice, two batched weight streams, combine)", ms_moe1,
        "dense feed-forward of equal active size, one token (two weight streams)", ms_dense1,
        nbytes=2.0 * top * ef * W * 2 + moe.w_route.numel() * 2.0, like_nbytes=2.0 * top * ef * W * 2,
        note="five launches against two")
    return rows


def run_nikonex(sizes: List[str], prompt_len: int = 2048, steps: int = 64, warmup: int = 8, batches: List[int] = (1, 8),
                kernels: bool = True) -> Dict[str, Any]:
    """Nikonex beside the closest existing design, Folirax, at equal width, depth, head counts and active feed-forward size."""
    from ..models.hybrid_engine import HybridEngine

    dev = torch.device("cuda", torch.cuda.current_device())
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        peaks = {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        pass
    result: Dict[str, Any] = {"metric": "nikonex_vs_folirax_equal_size", "data": "synthetic", "dtype": "bf16", "peaks": peaks,
                              "prompt_len": prompt_len, "steps": steps, "warmup": warmup, "sizes": {}}
    for name in sizes:
        s = NIKONEX_SIZES[name]
        entry: Dict[str, Any] = {"shape": s}
        for label, cfg in (("nikonex", nikonex_config(s)), ("folirax", folirax_config(s))):
            eng = HybridEngine.random_init(cfg, dev, seed=0)
            entry[label] = _model_times(eng, s["vocab"], prompt_len, list(batches), steps, warmup)
            del eng
            torch.cuda.empty_cache()
        if kernels:
            entry["kernels"] = _nikonex_kernel_table(s, dev, peaks, prompt_len)
        result["sizes"][name] = entry
    return result


# --------------------------------------------------------------------------------------------- Bazulorn beside Nikonex
def bazulorn_config(s: Dict[str, int]) -> Any:
    """[delta, parallel + experts, parallel + experts, delta + experts] × n at the head counts of the Nikonex shape: the
    delta rule in place of retention (same 64 × 128 heads), windowed attention with 128-wide heads in place of latent
    attention, a state space layer beside it, gated experts whose three matrices hold what Nikonex's two hold."""
    from ..config import BazulornConfig

    H = s["heads"]
    dl = {"heads": H, "kv_heads": H, "dim": 64, "vdim": 128, "conv": 4}
    pm = {"left": {"heads": H, "kv_heads": s["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                   "mask": {"size": s["window"]}},
          "right": {"heads": H, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}}
    ef, sf = s["expert_ff"] * 2 // 3 // 8 * 8, s["shared_ff"] * 2 // 3 // 8 * 8
    mlp = {"kind": "moe", "expert": {"ff": ef, "limit": 7.0}, "shared": {"ff": sf, "limit": 7.0},
           "router": {"experts": s["experts"], "top": s["top"]}}
    block = [("channel_delta", dl, None), ("parallel", pm, mlp), ("parallel", pm, mlp), ("channel_delta", dl, mlp)]
    layers = [{"type": block[i % 4][0], "mixer": block[i % 4][1], "mlp": block[i % 4][2]} for i in range(s["layers"])]
    return BazulornConfig.from_dict({"architecture": "Bazulorn", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
                                     "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 7919}},
                                     "layers": layers})


def _bazulorn_kernel_table(s: Dict[str, int], dev: torch.device, peaks: Dict[str, float], prompt_len: int) -> List[Dict[str, Any]]:
    """Each kernel that Bazulorn adds, at this size, beside the like kernel of the Nikonex path: ms, achieved rate, the
    fraction of the measured roofline, and how much farther from it the new kernel is (`distance_ratio`)."""
    from ..config import MoeMlpSpec
    from ..models.feedforward import MoeFeedForward
    from ..models.mixers import rotary_table
    from ..ops import seq_kernels as SK

    t = Timer(dev)
    hbm, tf = peaks["hbm_gbs"], peaks["bf16_tflops"]
    W, H, G = s["width"], s["heads"], s["kv_heads"]
    E, top = s["experts"], s["top"]
    ef, nef = s["expert_ff"] * 2 // 3 // 8 * 8, s["expert_ff"]
    win, P = s["window"], prompt_len
    D = Dv = 128
    gd, gv, N, sv, R = 64, 128, 128, 64, 16
    bf = dict(dtype=torch.bfloat16, device=dev)
    rows: List[Dict[str, Any]] = []

    def add(name: str, ms: float, like: str, like_ms: float, nbytes: float = 0.0, flops: float = 0.0, like_nbytes: float = 0.0,
            like_flops: float = 0.0, note: str = "") -> None:
        r: Dict[str, Any] = {"kernel": name, "ms": round(ms, 4), "like": like, "like_ms": round(like_ms, 4) if like_ms else None}
        frac = like_frac = None
        if nbytes:
            r["gbs"] = round(nbytes / ms / 1e6, 1)
            frac = nbytes / ms / 1e6 / hbm
            r["frac_hbm_of_measured"] = round(frac, 4)
            if like_ms:
                like_frac = (like_nbytes or nbytes) / like_ms / 1e6 / hbm
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
            frac = flops / ms / 1e9 / tf
            r["frac_bf16_of_measured"] = round(frac, 5)
            if like_ms:
                like_frac = (like_flops or flops) / like_ms / 1e9 / tf
        if like_frac is not None:
            r["like_frac"] = round(like_frac, 5)
            r["distance_ratio"] = round(like_frac / frac, 2)
        if note:
            r["note"] = note
        rows.append(r)

    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pad = torch.zeros(1, dtype=torch.int32, device=dev)
    pad8 = torch.zeros(8, dtype=torch.int32, device=dev)
    ctx_len = torch.full((1,), P, dtype=torch.int32, device=dev)
    T = P + 8

    # ---- embedding: token row + hashed pair row + norm, beside the plain lookup
    V = s["vocab"]
    emb, pair, wn = torch.randn(V, W, **bf), torch.randn(65522, W, **bf), torch.ones(W, **bf)
    ids = torch.randint(0, V, (P,), dtype=torch.int32, device=dev)
    prev = torch.zeros(1, dtype=torch.int32, device=dev)
    add("embed_pair_norm (two table rows, norm)",
        t.kernel(lambda: SK.embed_pair_norm(ids, emb, pair, wn, prev, zero, pad, 1, P, 65521, 1000003, 7919, 1e-5)),
        "embed_f32 (one table row)", t.kernel(lambda: SK.embed_f32(ids, emb)), nbytes=P * W * 8.0, like_nbytes=P * W * 6.0)

    # ---- the norms around two mixers side by side, beside the block's residual step
    x, y1, y2 = (torch.randn(P, W, device=dev) for _ in range(3))
    w1, w2 = torch.ones(W, **bf), torch.ones(W, **bf)
    add("norm_mean2 (two branch norms, half their sum)", t.kernel(lambda: SK.norm_mean2(y1, w1, y2, w2, 0.5, 1e-5)),
        "branch_add_norm (two branches, two norms)", t.kernel(lambda: SK.branch_add_norm(x, y1, y2, 0.5, w1, w2, 1e-5)),
        nbytes=P * W * 12.0, like_nbytes=P * W * 20.0)

    # ---- short convolutions (prompt and one token x 8 rows), beside the preparation kernel of latent attention
    C = 2 * H * gd + H * gv
    yc = torch.randn(P, C + H + 2 * R + 8, device=dev)
    cw = torch.randn(C, 4, **bf)
    cst = torch.zeros(1, 3, C, device=dev)
    qr, rank, Rr = s["q_rank"], s["kv_rank"], 64
    cos, sin = rotary_table(Rr, 10000.0, T, dev)
    yl = torch.randn(P, qr + rank + Rr, device=dev)
    wqn, wkn = torch.ones(qr, **bf), torch.ones(rank, **bf)
    lcache = torch.zeros(1, T, rank + Rr, **bf)
    add("causal_conv + silu (q | k | v of the delta rule, prompt)", t.kernel(lambda: SK.causal_conv(yc, 0, cw, None, cst, zero, pad, 1, P)),
        "latent_prep (two norms, rotation, append)",
        t.kernel(lambda: SK.latent_prep(yl, 0, qr, qr, rank, Rr, Rr, 0, wqn, wkn, lcache, cos, sin, 1e-5, zero, pad, 1, P)),
        nbytes=P * C * 8.0, like_nbytes=P * (qr + rank + Rr) * 6.0)

    # ---- recurrences: delta rule and state space scan beside retention (prompt; one token x 8 rows)
    u = torch.randn(P, C, device=dev) * 0.3
    yb = torch.randn(P, H + R + 8, device=dev) * 0.3
    a2 = torch.randn(H * gd, R, **bf) * 0.1
    ab = torch.full((H * gd,), 0.5, **bf)
    al = torch.full((H,), -3.0, **bf)
    dstate = torch.zeros(1, H, gd, gv, device=dev)
    yr = torch.randn(P, 2 * H * gd + 2 * H * gv, device=dev) * 0.3
    rstate = torch.zeros(1, H, gd, gv, device=dev)
    decay = torch.linspace(0.97, 0.999, H, device=dev)
    rc, rs = rotary_table(gd, 10000.0, T, dev)
    ms_ret = t.kernel(lambda: SK.retention_scan(yr, 0, H * gd, 2 * H * gd, decay, rc, rs, gd, 1, gd ** -0.5, rstate, zero, pad, 1, P,
                                                H, gd, gv), reps=5)
    state_fl = 4.0 * P * H * gd * gv
    add("delta rule scan (prompt: token-parallel preparation + sequential scan)",
        t.kernel(lambda: SK.delta_scan(u, 0, H * gd, 2 * H * gd, H, yb, 0, H, a2, ab, al, dstate, zero, pad, 1, P, H, gd, gv), reps=5),
        "retention scan (prompt, time chunks)", ms_ret, flops=1.5 * state_fl, like_flops=state_fl,
        note="the correction multiplies the state by (I - beta k k^T): no chunk-parallel two-pass form; fractions are of the "
             "tensor-core peak and only rank the two")
    inner, gn = H * sv, N
    us = torch.randn(P, inner + 2 * gn, device=dev) * 0.3
    ys = torch.randn(P, 2 * inner + 2 * gn + H, device=dev) * 0.3
    dtb, sal = torch.zeros(H, **bf), torch.full((H,), -3.0, **bf)
    sstate = torch.zeros(1, H, N, sv, device=dev)
    add("state space scan (prompt; the gated-linear-attention kernels with per-token decays)",
        t.kernel(lambda: SK.ssd_scan(ys, 2 * inner + 2 * gn, dtb, sal, us, inner + gn, inner, 0, 1, sstate, zero, pad, 1, P, H, N, sv),
                 reps=5),
        "retention scan (prompt, time chunks)", ms_ret, flops=4.0 * P * H * N * sv, like_flops=state_fl)
    u8, yb8 = u[:8].contiguous(), yb[:8].contiguous()
    d8 = torch.zeros(8, H, gd, gv, device=dev)
    r8 = torch.zeros(8, H, gd, gv, device=dev)
    yr8 = yr[:8].contiguous()
    add("delta rule scan, one token x 8 rows (one fused launch)",
        t.kernel(lambda: SK.delta_scan(u8, 0, H * gd, 2 * H * gd, H, yb8, 0, H, a2, ab, al, d8, ctx_len, pad8, 8, 1, H, gd, gv)),
        "retention scan, one token x 8 rows (one launch)",
        t.kernel(lambda: SK.retention_scan(yr8, 0, H * gd, 2 * H * gd, decay, rc, rs, gd, 1, gd ** -0.5, r8, ctx_len, pad8, 8, 1, H,
                                           gd, gv)),
        nbytes=8.0 * H * gd * gv * 8.0)

    # ---- attention: preparation, prompt and one token with mixed head weights, beside Nikonex's windowed attention
    n_qkv = (H + 2 * G) * D
    yq = torch.randn(P, n_qkv + 8, device=dev) * 0.3
    bias = torch.zeros(n_qkv + 8, device=dev)
    qo = torch.empty(P, H * D, **bf)
    kc, vtm = torch.zeros(1, G, T, D, **bf), torch.zeros(1, T, G * Dv, **bf)
    kc2, vc2 = torch.zeros(1, G, T, D, **bf), torch.zeros(1, G, T, Dv, **bf)
    one = torch.ones(1, 1, device=dev)
    add("attn_prep (biases, unit-RMS values, append; no rotation)",
        t.kernel(lambda: SK.attn_prep(yq, 0, H * D, (H + G) * D, qo, kc, vtm, one, one, 0, False, 1e-5, zero, pad, 1, P, H, G, D, Dv,
                                      bias=bias, v_unit_norm=True, v_token_major=True)),
        "attn_prep (rotation, unit norm, append)",
        t.kernel(lambda: SK.attn_prep(yq, 0, H * D, (H + G) * D, qo, kc2, vc2, cos, sin, 64, True, 1e-5, zero, pad, 1, P, H, G, D, Dv)),
        nbytes=P * n_qkv * 6.0)
    kc.normal_()
    vtm.normal_()
    qf = torch.randn(P, H * D, **bf) * 0.05
    win_keys = sum(min(i + 1, win) for i in range(P))
    qd = D + 64
    qn = torch.randn(P, H * qd, **bf) * 0.05
    kn = torch.randn(P, H * qd, **bf) * 0.05
    vn = torch.randn(P, H * Dv, **bf)
    talk = torch.randn(H, H, **bf) * 0.1
    mixed = torch.empty(P, H * Dv, **bf)

    def attend(S: int, q: torch.Tensor, length: torch.Tensor, out: torch.Tensor) -> None:
        per = max(1, 512 // Dv)
        for c0 in range(0, G, per):
            gc = min(per, G - c0)
            o = SK.attn_windowed(q, kc, vtm[:, :, c0 * Dv:], length, pad, 1, S, H, G, D, gc * Dv, T, D, G * Dv, win, D ** -0.5,
                                 strides=(G * T * D, T * D, T * G * Dv, 0), sink=True, out_f32=True)
            SK.talk_mix(o, talk, out, H, G, gc, c0, Dv)

    add("attention with mixed head weights (prompt): attn_rows over all value heads + talk_mix",
        t.kernel(lambda: attend(P, qf, zero, mixed), reps=3),
        "attn_rows_kernel, windowed, per-head keys (prompt, Nikonex)",
        t.kernel(lambda: SK.attn_windowed(qn, kn, vn, zero, pad, 1, P, H, H, qd, Dv, P, H * qd, H * Dv, win, 192 ** -0.5,
                                          strides=(P * H * qd, qd, P * H * Dv, Dv)), reps=3),
        flops=2.0 * H * win_keys * (D + G * Dv), like_flops=2.0 * H * win_keys * (qd + Dv),
        note="every query head weighs the values of all key/value heads, so that the mix across heads is a small product "
             "afterwards; the same exact SIMT kernel on both sides")
    q1 = qf[:1].contiguous()
    m1 = torch.empty(1, H * Dv, **bf)
    row = rank + Rr
    q1l = torch.randn(1, H * row, **bf) * 0.05
    add("attention with mixed head weights (one token): attn_split + attn_merge + talk_mix",
        t.kernel(lambda: attend(1, q1, ctx_len, m1)), "attn_split + attn_merge, windowed latent rows (one token, Nikonex)",
        t.kernel(lambda: SK.attn_windowed(q1l, lcache, lcache, ctx_len, pad, 1, 1, H, 1, row, rank, T, row, row, win, 192 ** -0.5)),
        nbytes=min(win, P) * G * (D + Dv) * 2.0, like_nbytes=min(win, P) * row * 2.0)

    # ---- gated read-outs
    o = torch.randn(P, H * gv, device=dev)
    gate = torch.randn(P, H * gv, device=dev)
    wv = torch.ones(gv, **bf)
    wfull = torch.ones(H * gv, **bf)
    skip = torch.ones(H, **bf)
    add("gated_groupnorm ((o + D x) silu(z), norm, weight)",
        t.kernel(lambda: SK.gated_groupnorm(o, gate, skip, gv, gate, wfull, 1, 1e-5)),
        "headnorm_gate (norm per head, silu gate)", t.kernel(lambda: SK.headnorm_gate(o, wv, gate, H, gv, 1e-5, SK.ACT_SILU)),
        nbytes=P * H * gv * 14.0, like_nbytes=P * H * gv * 10.0)

    # ---- experts: prompt and one token, beside Nikonex's experts of equal parameter count
    hp = torch.randn(P, W, **bf)
    torch.manual_seed(0)

    def make(gated: bool) -> MoeFeedForward:
        f = ef if gated else nef
        spec = MoeMlpSpec(experts=E, top=top, ff=f, act="glu_clamped" if gated else "relu2", score="softmax" if gated else "sigmoid",
                          shared_ff=0, shared_gate=False, gated=gated, limit=7.0, router_bias=gated)
        w = {"router": torch.randn(E, W, **bf) * 0.02}
        if gated:
            w["router.b"] = torch.zeros(E, **bf)
        for e in range(E):
            w[f"e{e}.up"], w[f"e{e}.down"] = torch.randn(f, W, **bf) * 0.02, torch.randn(W, f, **bf) * 0.02
            if gated:
                w[f"e{e}.gate"] = torch.randn(f, W, **bf) * 0.02
        return MoeFeedForward(spec, w)

    new, old = make(True), make(False)
    fl_new, fl_old = 2.0 * P * top * 3 * ef * W, 2.0 * P * top * 2 * nef * W
    add("gated experts, prompt (router, sort, gather, grouped tcgen05 GEMM, gated activation, grouped GEMM, combine)",
        t.kernel(lambda: new.run(hp), reps=5), "experts, prompt (Nikonex: the same chain with relu² in place)",
        t.kernel(lambda: old.run(hp), reps=5), flops=fl_new, like_flops=fl_old)
    h1 = hp[:1].contiguous()
    add("gated experts, one token (router, choice, gate | up stream, gated activation, down stream, combine)",
        t.kernel(lambda: new.run(h1)), "experts, one token (Nikonex)", t.kernel(lambda: old.run(h1)),
        nbytes=top * 3.0 * ef * W * 2, like_nbytes=top * 2.0 * nef * W * 2, note="six launches against five")
    return rows


def run_bazulorn(sizes: List[str], prompt_len: int = 2048, steps: int = 64, warmup: int = 8, batches: List[int] = (1, 8),
                 kernels: bool = True) -> Dict[str, Any]:
    """Bazulorn beside the closest existing design, Nikonex, at equal width, depth, head counts and expert parameters."""
    from ..models.hybrid_engine import HybridEngine

    dev = torch.device("cuda", torch.cuda.current_device())
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        peaks = {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        pass
    result: Dict[str, Any] = {"metric": "bazulorn_vs_nikonex_equal_size", "data": "synthetic", "dtype": "bf16", "peaks": peaks,
                              "prompt_len": prompt_len, "steps": steps, "warmup": warmup, "sizes": {}}
    for name in sizes:
        s = NIKONEX_SIZES[name]
        entry: Dict[str, Any] = {"shape": s}
        for label, cfg in (("bazulorn", bazulorn_config(s)), ("nikonex", nikonex_config(s))):
            eng = HybridEngine.random_init(cfg, dev, seed=0)
            entry[label] = _model_times(eng, s["vocab"], prompt_len, list(batches), steps, warmup)
            del eng
            torch.cuda.empty_cache()
        if kernels:
            entry["kernels"] = _bazulorn_kernel_table(s, dev, peaks, prompt_len)
        result["sizes"][name] = entry
    return result


# --------------------------------------------------------------------------------------------- Datozen beside Bazulorn
def datozen_config(s: Dict[str, int], positions: int = 4096) -> Any:
    """Attention layers with 128-wide heads at the head counts of the Nikonex shape, blocks of `window` positions, the same
    gated experts as the Bazulorn shape (two of the router's outputs are identity experts) behind a dense layer; a quarter of
    the layer runs come from a stretch that runs twice, so that the number of runs equals the other model's depth."""
    from ..config import DatozenConfig

    H = s["heads"]
    att = {"heads": H, "kv_heads": s["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": s["window"]},
           "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}
    ef, sf = s["expert_ff"] * 2 // 3 // 8 * 8, s["shared_ff"] * 2 // 3 // 8 * 8
    moe = {"kind": "moe", "expert": {"ff": ef}, "shared": {"ff": sf},
           "router": {"experts": s["experts"] - 2, "identity": 2, "top": s["top"], "groups": {"count": 4, "keep": 2}}}
    dense = {"kind": "dense", "ff": s["shared_ff"]}
    k = max(1, s["layers"] // 4)
    n = s["layers"] - k
    layers = [{"type": "attention", "mixer": att, "mlp": dense if i % 4 == 0 else moe} for i in range(n)]
    return DatozenConfig.from_dict({"architecture": "Datozen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
                                    "max_positions": positions, "token_side": {"dim": 256},
                                    "loop": {"start": n - k, "stop": n, "times": 2}, "layers": layers})


def _datozen_kernel_table(s: Dict[str, int], dev: torch.device, peaks: Dict[str, float], prompt_len: int) -> List[Dict[str, Any]]:
    """Each kernel that Datozen adds or extends, at this size, beside the like kernel of the Bazulorn path: ms, achieved rate,
    the fraction of the measured roofline, and how much farther from it the new kernel is (`distance_ratio`)."""
    from ..config import DenseMlpSpec, MoeMlpSpec
    from ..models.feedforward import DenseFeedForward, MoeFeedForward
    from ..models.hybrid_engine import TokenSide
    from ..models.mixers import rotary_table
    from ..ops import seq_kernels as SK

    t = Timer(dev)
    hbm, tf = peaks["hbm_gbs"], peaks["bf16_tflops"]
    W, H, G, V = s["width"], s["heads"], s["kv_heads"], s["vocab"]
    E, top = s["experts"], s["top"]
    ef = s["expert_ff"] * 2 // 3 // 8 * 8
    chunk, P = s["window"], prompt_len
    D = Dv = 128
    T = P + 8
    bf = dict(dtype=torch.bfloat16, device=dev)
    rows: List[Dict[str, Any]] = []

    def add(name: str, ms: float, like: str, like_ms: float, nbytes: float = 0.0, flops: float = 0.0, like_nbytes: float = 0.0,
            like_flops: float = 0.0, note: str = "") -> None:
        r: Dict[str, Any] = {"kernel": name, "ms": round(ms, 4), "like": like, "like_ms": round(like_ms, 4) if like_ms else None}
        frac = like_frac = None
        if nbytes:
            r["gbs"] = round(nbytes / ms / 1e6, 1)
            frac = nbytes / ms / 1e6 / hbm
            r["frac_hbm_of_measured"] = round(frac, 4)
            if like_ms:
                like_frac = (like_nbytes or nbytes) / like_ms / 1e6 / hbm
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
            frac = flops / ms / 1e9 / tf
            r["frac_bf16_of_measured"] = round(frac, 5)
            if like_ms:
                like_frac = (like_flops or flops) / like_ms / 1e9 / tf
        if like_frac is not None:
            r["like_frac"] = round(like_frac, 5)
            r["distance_ratio"] = round(like_frac / frac, 2)
        if note:
            r["note"] = note
        rows.append(r)

    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pad = torch.zeros(1, dtype=torch.int32, device=dev)
    pad8 = torch.zeros(8, dtype=torch.int32, device=dev)
    ctx_len = torch.full((1,), P, dtype=torch.int32, device=dev)

    # ---- embedding: token row + position row, beside token row + hashed pair row + norm
    emb, pair, wn, post = torch.randn(V, W, **bf), torch.randn(65522, W, **bf), torch.ones(W, **bf), torch.randn(T, W, **bf)
    ids = torch.randint(0, V, (P,), dtype=torch.int32, device=dev)
    prev = torch.zeros(1, dtype=torch.int32, device=dev)
    add("embed_pos (token row + position row)", t.kernel(lambda: SK.embed_pos(ids, emb, post, zero, pad, 1, P)),
        "embed_pair_norm (two table rows, norm; Bazulorn)",
        t.kernel(lambda: SK.embed_pair_norm(ids, emb, pair, wn, prev, zero, pad, 1, P, 65521, 1000003, 7919, 1e-5)), nbytes=P * W * 8.0)

    # ---- attention, preparation: weighted q / k norms before a half-split rotation, rotated values, append
    n_qkv = (H + 2 * G) * D
    yq = torch.randn(P, n_qkv + 8, device=dev) * 0.3
    bias = torch.zeros(n_qkv + 8, device=dev)
    qo = torch.empty(P, H * D, **bf)
    kc, vc = torch.zeros(1, G, T, D, **bf), torch.zeros(1, G, T, Dv, **bf)
    kc2, vtm = torch.zeros(1, G, T, D, **bf), torch.zeros(1, T, G * Dv, **bf)
    cos, sin = rotary_table(64, 10000.0, T, dev)
    vcos, vsin = rotary_table(Dv, 10000.0, T, dev)
    qw, kw = torch.ones(D, **bf), torch.ones(D, **bf)
    one = torch.ones(1, 1, device=dev)
    add("attn_prep (weighted q / k norms, half-split rotation, rotated values, append)",
        t.kernel(lambda: SK.attn_prep(yq, 0, H * D, (H + G) * D, qo, kc, vc, cos, sin, 64, False, 1e-5, zero, pad, 1, P, H, G, D, Dv,
                                      layout=SK.ROT_HALF, q_norm_w=qw, k_norm_w=kw, v_cos=vcos, v_sin=vsin)),
        "attn_prep (biases, unit-RMS values, append; Bazulorn)",
        t.kernel(lambda: SK.attn_prep(yq, 0, H * D, (H + G) * D, qo, kc2, vtm, one, one, 0, False, 1e-5, zero, pad, 1, P, H, G, D, Dv,
                                      bias=bias, v_unit_norm=True, v_token_major=True)), nbytes=P * n_qkv * 6.0)

    # ---- attention proper: prompt and one token
    kc.normal_()
    vc.normal_()
    kc2.normal_()
    vtm.normal_()
    qf = torch.randn(P, H * D, **bf) * 0.05
    gate = torch.randn(P, H, device=dev)
    sink = torch.zeros(H, device=dev)
    talk = torch.randn(H, H, **bf) * 0.1
    mixed = torch.empty(P, H * Dv, **bf)
    blk_keys = sum(i % chunk + 1 for i in range(P))
    win_keys = sum(min(i + 1, chunk) for i in range(P))

    def attend_mixed(S: int, q: torch.Tensor, length: torch.Tensor, out: torch.Tensor) -> None:
        per = max(1, 512 // Dv)
        for c0 in range(0, G, per):
            gc = min(per, G - c0)
            o = SK.attn_windowed(q, kc2, vtm[:, :, c0 * Dv:], length, pad, 1, S, H, G, D, gc * Dv, T, D, G * Dv, chunk, D ** -0.5,
                                 strides=(G * T * D, T * D, T * G * Dv, 0), sink=True, out_f32=True)
            SK.talk_mix(o, talk, out, H, G, gc, c0, Dv)

    def attend(S: int, q: torch.Tensor, g: torch.Tensor, length: torch.Tensor) -> torch.Tensor:
        return SK.attn_masked(q, kc, vc, length, pad, 1, S, H, G, D, Dv, D ** -0.5, gate=g, chunk=chunk, sink=True, sink_logit=sink,
                              v_cos=vcos, v_sin=vsin, v_layout=SK.ROT_HALF)

    add("attention in blocks of positions, learned sink, sums turned back, gate (prompt): attn_rows",
        t.kernel(lambda: attend(P, qf, gate, zero), reps=3),
        "attention with a window and mixed head weights (prompt, Bazulorn): attn_rows over all value heads + talk_mix",
        t.kernel(lambda: attend_mixed(P, qf, zero, mixed), reps=3),
        flops=2.0 * H * blk_keys * (D + Dv), like_flops=2.0 * H * win_keys * (D + G * Dv),
        note="the same exact SIMT kernel on both sides; a block hides on average half of what a window of the same size shows")
    from ..ops import _lib as L
    from ..ops import kernels as K
    fo = torch.empty(P, H * Dv, **bf)

    def flash(masked: bool) -> None:
        if masked:
            L.check(L.lib().jl_flash_prefill_masked(qf.data_ptr(), kc.data_ptr(), vc.data_ptr(), pad.data_ptr(), fo.data_ptr(), 1, P, H, G,
                                                    D, T, 0, D ** -0.5, chunk, 1, sink.data_ptr(), gate.data_ptr(), gate.stride(0),
                                                    vcos.data_ptr(), vsin.data_ptr(), vcos.shape[0], K._stream()), "flash masked")
        else:
            L.check(L.lib().jl_flash_prefill(qf.data_ptr(), kc.data_ptr(), vc.data_ptr(), zero.data_ptr(), pad.data_ptr(), fo.data_ptr(),
                                             1, P, H, G, D, T, 0, D ** -0.5, K._stream()), "flash")

    add("attention in blocks, prompt, bfloat16 and 128-wide heads: the tcgen05 kernel with block bound, sink, gate and turn back",
        t.kernel(lambda: flash(True)), "the same kernel, plain causal attention (LLaMA path)", t.kernel(lambda: flash(False)),
        flops=2.0 * H * blk_keys * (D + Dv), like_flops=2.0 * H * (P * (P + 1) / 2) * (D + Dv),
        note="what Datozen's bfloat16 prompts run at these head sizes; key tiles are 64 wide, so short blocks leave tiles partly masked")
    q1, g1 = qf[:1].contiguous(), gate[:1].contiguous()
    m1 = torch.empty(1, H * Dv, **bf)
    last = torch.full((1,), P - 1, dtype=torch.int32, device=dev)               # the new token closes a block when chunk divides P
    seen1 = (P - 1) % chunk + 1
    add("attention in blocks (one token): attn_split + attn_merge with the turn back and the gate",
        t.kernel(lambda: attend(1, q1, g1, last)),
        "attention with a window and mixed head weights (one token, Bazulorn): attn_split + attn_merge + talk_mix",
        t.kernel(lambda: attend_mixed(1, q1, last, m1)),
        nbytes=seen1 * G * (D + Dv) * 2.0, like_nbytes=min(chunk, P) * G * (D + Dv) * 2.0,
        note=f"the new token is position {P - 1}: its block shows {seen1} keys, the window {min(chunk, P)}; both are launch-bound at this length")

    # ---- per-layer token input: prompt (two GEMMs around a gate kernel, fused norm / add / next norm) and 8 rows (one launch)
    n_side = 256
    side = TokenSide(torch.randn(V, 4 * n_side, **bf), n_side, {"gate": torch.randn(n_side, W, **bf) * 0.02,
                                                                 "proj": torch.randn(W, n_side, **bf) * 0.02, "norm": torch.ones(W, **bf)})
    x = torch.randn(P, W, device=dev)
    y1, y2 = torch.randn(P, W, device=dev), torch.randn(P, W, device=dev)
    w1 = torch.ones(W, **bf)
    def block_end() -> None:
        side.run(x, ids, w1, 1e-5, x_cast=SK.branch_add_cast(x, y1, y2, 1.0, torch.bfloat16))

    add("residual step + token input, prompt (add + cast, gate GEMM, gate kernel, up GEMM, norm + add + next norm)",
        t.kernel(block_end, reps=5), "branch_add_norm (two branches, two norms; the residual step of every block)",
        t.kernel(lambda: SK.branch_add_norm(x, y1, y2, 0.5, w1, w1, 1e-5)),
        nbytes=P * W * (18 + 2 + 4 + 14.0) + P * n_side * 8.0, like_nbytes=P * W * 20.0,
        note="bytes of the five passes (the residual step among them); its two products add 4 P W n flops")
    x8, ids8 = x[:8].contiguous(), ids[:8].contiguous()
    wl = torch.randn(2 * n_side, W, **bf) * 0.02
    h8 = torch.randn(8, W, **bf)
    add("token input, 8 rows (gate kernel with the small projection inside, weight-streaming up projection, norm + add + next norm)",
        t.kernel(lambda: side.run(x8, ids8, w1, 1e-5)),
        "weight-streaming linear of the same weight bytes, 8 rows (one launch)", t.kernel(lambda: SK.linear(h8, wl)),
        nbytes=2.0 * n_side * W * 2, note="three dependent launches of a few microseconds against one")

    # ---- dense feed-forward with the two-parameter activation, beside Bazulorn's gated layer of equal parameters
    F = s["shared_ff"]
    hp = torch.randn(P, W, **bf)
    dn = DenseFeedForward(DenseMlpSpec(ff=F, act="xielu", gated=False),
                          {"up": torch.randn(F, W, **bf) * 0.02, "down": torch.randn(W, F, **bf) * 0.02, "act": torch.zeros(2, **bf)})
    Fg = F * 2 // 3 // 8 * 8
    dg = DenseFeedForward(DenseMlpSpec(ff=Fg, act="gelu_tanh", gated=True),
                          {"up": torch.randn(Fg, W, **bf) * 0.02, "gate": torch.randn(Fg, W, **bf) * 0.02, "down": torch.randn(W, Fg, **bf) * 0.02})
    add("dense layer, two-parameter activation (prompt: GEMM, activation in place, GEMM)", t.kernel(lambda: dn.run(hp), reps=5),
        "gated dense layer (prompt, Bazulorn: GEMM, gated activation, GEMM)", t.kernel(lambda: dg.run(hp), reps=5),
        flops=4.0 * P * F * W, like_flops=6.0 * P * Fg * W)
    h1 = hp[:1].contiguous()
    add("dense layer, one token", t.kernel(lambda: dn.run(h1)), "gated dense layer, one token (Bazulorn)", t.kernel(lambda: dg.run(h1)),
        nbytes=2.0 * F * W * 2, like_nbytes=3.0 * Fg * W * 2)

    # ---- experts with a choice bias, groups by their best member and identity experts, beside Bazulorn's experts
    torch.manual_seed(0)

    def make(new: bool) -> MoeFeedForward:
        n_real = E - 2 if new else E
        spec = MoeMlpSpec(experts=n_real, top=top, ff=ef, act="silu" if new else "glu_clamped", score="softmax", groups=4 if new else 1,
                          keep=2 if new else 1, group_top=1, normalise=not new, shared_ff=0, shared_gate=False, gated=True, limit=7.0,
                          router_bias=not new, identity=2 if new else 0, choice_bias=new)
        w = {"router": torch.randn(E, W, **bf) * 0.02}
        w["correction" if new else "router.b"] = torch.zeros(E, **bf)
        for e in range(n_real):
            w[f"e{e}.up"], w[f"e{e}.down"] = torch.randn(ef, W, **bf) * 0.02, torch.randn(W, ef, **bf) * 0.02
            w[f"e{e}.gate"] = torch.randn(ef, W, **bf) * 0.02
        return MoeFeedForward(spec, w)

    new, old = make(True), make(False)
    fl = 2.0 * P * top * 3 * ef * W
    add("experts with identity experts, prompt (router, choice, sort, gather, grouped tcgen05 GEMM, silu gate, grouped GEMM, combine)",
        t.kernel(lambda: new.run(hp), reps=5), "gated experts, prompt (Bazulorn: the same chain)", t.kernel(lambda: old.run(hp), reps=5),
        flops=fl * (E - 2) / E, like_flops=fl, note="one pair in sixteen chooses an identity expert and runs no product")
    add("experts with identity experts, one token", t.kernel(lambda: new.run(h1)), "gated experts, one token (Bazulorn)",
        t.kernel(lambda: old.run(h1)), nbytes=top * 3.0 * ef * W * 2, note="seven launches against six (the identity weights)")
    return rows


def run_datozen(sizes: List[str], prompt_len: int = 2048, steps: int = 64, warmup: int = 8, batches: List[int] = (1, 8),
                kernels: bool = True) -> Dict[str, Any]:
    """Datozen beside the closest existing design, Bazulorn, at equal width, layer runs, head counts and expert sizes."""
    from ..models.hybrid_engine import HybridEngine

    dev = torch.device("cuda", torch.cuda.current_device())
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        peaks = {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        pass
    result: Dict[str, Any] = {"metric": "datozen_vs_bazulorn_equal_size", "data": "synthetic", "dtype": "bf16", "peaks": peaks,
                              "prompt_len": prompt_len, "steps": steps, "warmup": warmup, "sizes": {}}
    for name in sizes:
        s = NIKONEX_SIZES[name]
        entry: Dict[str, Any] = {"shape": s}
        for label, cfg in (("datozen", datozen_config(s, positions=prompt_len + steps + warmup + 64)), ("bazulorn", bazulorn_config(s))):
            eng = HybridEngine.random_init(cfg, dev, seed=0)
            entry[label] = _model_times(eng, s["vocab"], prompt_len, list(batches), steps, warmup)
            entry[label]["layer_runs"] = len(eng.runs)
            del eng
            torch.cuda.empty_cache()
        if kernels:
            entry["kernels"] = _datozen_kernel_table(s, dev, peaks, prompt_len)
        result["sizes"][name] = entry
    return result
