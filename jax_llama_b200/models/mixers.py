"""Sequence mixers of the hybrid decoder family, each a small class over the kernels of `ops/seq_kernels.py`.

A mixer owns its projection weights in kernel layout (projections that read the same input are stacked into one
matrix, so a layer issues one GEMM for them), knows what it keeps between tokens (a key / value cache, a recurrent
state, or nothing of its own when it reads another layer's cache) and turns the normalised input ``h [B·S, width]``
into the input of the output projection.  Constants of a mechanism (rotary share and base, score scale, decay
temperature, which norms and gates are on) are parameters of its spec (`config.py`), not of the code.

The output projection, the norms around the sublayer and the residual sum belong to the layer stack
(`models/hybrid_engine.py`), which is the same for every mixer.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from ..config import (AttentionMixerSpec, DeltaMixerSpec, GlaMixerSpec, LatentAttentionMixerSpec, ParallelMixerSpec,
                      RetentionMixerSpec, RotaryScaling, RotarySpec, StateSpaceMixerSpec)
from ..ops import _lib
from ..ops import kernels as K
from ..ops import seq_kernels as SK


def _stack_rows(parts: List[torch.Tensor], multiple: int = 8) -> Tuple[torch.Tensor, List[int]]:
    """Concatenate weight matrices [n_i, K] on the output axis, zero-padded to a multiple of `multiple` rows (the
    tensor-core GEMM wants N % 8 == 0).  Returns the matrix and the first row of every part."""
    offs, n = [], 0
    for p in parts:
        offs.append(n)
        n += p.shape[0]
    pad = (-n) % multiple
    if pad:
        parts = parts + [torch.zeros((pad, parts[0].shape[1]), dtype=parts[0].dtype, device=parts[0].device)]
    return torch.cat(parts, 0).contiguous(), offs


def rotary_frequencies(dims: int, base: float, scaling: Optional[RotaryScaling] = None) -> Tuple[torch.Tensor, float]:
    """float64 frequencies base^(-2i/dims), i < dims/2, and the factor on cos / sin.  With `scaling`: the channel index
    at which `original` positions make t turns is n(t) = dims · ln(original / (2π t)) / (2 ln base); channels below
    floor(n(fast)) keep their frequency, channels above ceil(n(slow)) are divided by `factor`, linear ramp between."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if scaling is None:
        return freq, 1.0

    def channel_of(turns: float) -> float:
        return dims * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(channel_of(scaling.fast)), 0)
    hi = min(math.ceil(channel_of(scaling.slow)), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / scaling.factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(scaling.factor) + 1.0


def rotary_table(dims: int, base: float, length: int, device: torch.device, scaling: Optional[RotaryScaling] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin of position · frequency for the dims/2 channel pairs, as fp32 [length, dims/2] (angles formed in
    float64; the scaling's factor on cos / sin is in the table)."""
    freq, mult = rotary_frequencies(dims, base, scaling)
    ang = torch.arange(length, dtype=torch.float64)[:, None] * freq[None, :]
    return ((torch.cos(ang) * mult).float().to(device).contiguous(),
            (torch.sin(ang) * mult).float().to(device).contiguous())


class Mixer:
    """What the layer stack asks of a mixer.  `run` gives the input of the output projection `wo`; `forward` the mixer's
    fp32 contribution [M, width] (a mixer made of several overrides it).  `shapes(spec, W, rank_of)` lists the checkpoint
    tensors under the mixer's prefix; `rank_of(name, default)` is the first dimension the checkpoint gives a tensor whose
    inner size no configuration key fixes."""

    def forward(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Optional[Tuple] = None
                ) -> torch.Tensor:
        return SK.linear(self.run(h, B, S, cache, layer, rope), self.wo)


class _CacheView:
    """The cache as one of several mixers of a layer sees it: the shared fill level and left-pad counts, and that mixer's
    own entries under the layer's index."""

    def __init__(self, cache: "object", layer: int, side: int):
        self._cache = cache
        self.ks = {layer: cache.ks[layer][side] if cache.ks[layer] is not None else None}
        self.vs = {layer: cache.vs[layer][side] if cache.vs[layer] is not None else None}
        self.states = {layer: cache.states[layer][side] if cache.states[layer] is not None else None}

    def __getattr__(self, name: str) -> "object":
        return getattr(self._cache, name)


class AttentionMixer(Mixer):
    """Softmax attention: grouped key / value heads, query / key size `dim` and value size `vdim` (they may differ),
    rotary embedding on the first `rot.dims` channels, optional unit-RMS q / k, optional sigmoid gate per head,
    optional reuse of another layer's cache (`kv_from`); optional q / k / v biases, unit-RMS values, sliding window, a
    sink in the softmax denominator and mixing of the heads' weights by a [heads, heads] matrix.

    With mixed weights head h's output is Σ_j (Σ_g T[h, g] p_g(j)) v_c(j) = Σ_g T[h, g] (Σ_j p_g(j) v_c(j)), c its own
    key/value head: the attention kernel forms, per query head g, the weighted sums over the values of ALL key/value heads
    (the value cache is token-major, one row [kv_heads · vdim] per token, read as one wide value head) in fp32, and a
    second small kernel mixes them.  The sink's share is not mixed: it has no values.

    Further options, all parameters of the spec: an RMS norm with a weight on every q / k head before the rotation (`qk_norm`),
    either pairing of the rotated channels (`rot.layout`), values rotated at their own position and the head's sum rotated back
    at the query's (`v_rot`: the value cache holds rotated values, so a cached value never has to be touched again and the
    weighted sum depends on relative positions only), blocks of `chunk` positions instead of (or besides) a window, and a
    learned sink logit per head.  These run the masked form of the generic attention kernels."""

    kind = "attention"

    def __init__(self, spec: AttentionMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        self.shares_kv = spec.kv_from is not None
        parts = [w["q"]] + ([] if self.shares_kv else [w["k"], w["v"]]) + ([w["g"]] if spec.head_gate else [])
        self.w_in, offs = _stack_rows(parts)
        self.q_off = offs[0]
        self.k_off, self.v_off = (-1, -1) if self.shares_kv else (offs[1], offs[2])
        self.g_off = offs[-1] if spec.head_gate else -1
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype
        self._decode_plans: Dict[Tuple[int, int], Tuple[int, Optional[torch.Tensor]]] = {}
        self.bias: Optional[torch.Tensor] = None
        if spec.bias:                                      # fp32 over the columns of the stacked projection
            self.bias = torch.zeros(self.w_in.shape[0], dtype=torch.float32, device=self.wo.device)
            for name, off in (("q", self.q_off), ("k", self.k_off), ("v", self.v_off)):
                if off >= 0:
                    self.bias[off:off + w[name].shape[0]] = w[name + ".b"].float()
        self.talk = w["talk"].contiguous() if spec.talking_heads else None
        if spec.talking_heads and (self.shares_kv or spec.head_gate):
            raise ValueError("mixed attention weights go with a layer's own keys / values and no head gate")
        self.plain = not (spec.bias or spec.v_unit_norm or spec.window or spec.sink or spec.talking_heads or spec.qk_norm
                          or spec.chunk or spec.v_rot or (spec.rot is not None and spec.rot.layout != "interleaved"))
        self.q_norm = w["q.norm"].contiguous() if spec.qk_norm else None
        self.k_norm = w["k.norm"].contiguous() if spec.qk_norm and not self.shares_kv else None
        self.sink_logit = w["sink"].float().contiguous() if spec.sink_learned else None
        if spec.sink_learned and not spec.sink:
            raise ValueError("a learned sink logit needs the sink")
        if spec.v_rot and (spec.rot is None or spec.vdim % 2 or spec.talking_heads or spec.v_unit_norm or self.shares_kv):
            raise ValueError("rotated values need a rotary spec, an even vdim and a layer's own head-major value cache")
        # the rotation of the values: all vdim channels, the base and pairing of the q / k rotation, no interpolation
        self.value_rot = RotarySpec(spec.vdim, spec.rot.base, spec.rot.layout, None) if spec.v_rot else None

    @staticmethod
    def shapes(spec: AttentionMixerSpec, W: int, rank_of: "object" = None) -> Dict[str, Tuple[int, ...]]:
        out: Dict[str, Tuple[int, ...]] = {"q": (spec.heads * spec.dim, W), "o": (W, spec.heads * spec.vdim)}
        if spec.kv_from is None:
            out["k"], out["v"] = (spec.kv_heads * spec.dim, W), (spec.kv_heads * spec.vdim, W)
        if spec.head_gate:
            out["g"] = (spec.heads, W)
        if spec.bias:
            for n in ("q", "k", "v"):
                if n in out:
                    out[n + ".b"] = (out[n][0],)
        if spec.talking_heads:
            out["talk"] = (spec.heads, spec.heads)
        if spec.qk_norm:
            out["q.norm"] = (spec.dim,)
            if spec.kv_from is None:
                out["k.norm"] = (spec.dim,)
        if spec.sink_learned:
            out["sink"] = (spec.heads,)
        return out

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.wo] + [t for t in (self.talk, self.q_norm, self.k_norm, self.sink_logit) if t is not None]

    def new_cache(self, batch: int, length: int, device: torch.device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        if self.shares_kv:
            return None
        s = self.spec
        if s.talking_heads:                                # values token-major: every query head reads all value heads
            return (torch.zeros((batch, s.kv_heads, length, s.dim), dtype=self.dtype, device=device),
                    torch.zeros((batch, length, s.kv_heads * s.vdim), dtype=self.dtype, device=device))
        return (torch.zeros((batch, s.kv_heads, length, s.dim), dtype=self.dtype, device=device),
                torch.zeros((batch, s.kv_heads, length, s.vdim), dtype=self.dtype, device=device))

    def new_state(self, batch: int, device: torch.device) -> Optional[torch.Tensor]:
        return None

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Tuple[torch.Tensor, torch.Tensor]
            ) -> torch.Tensor:
        s = self.spec
        y = SK.linear(h, self.w_in)                                   # fp32 [M, q | k | v | gate]
        q = torch.empty((B * S, s.heads * s.dim), dtype=self.dtype, device=h.device)
        src = layer if not self.shares_kv else s.kv_from
        kc, vc = cache.ks[src], cache.vs[src]
        rot = s.rot.dims if s.rot is not None else 0
        layout = SK.ROT_LAYOUTS[s.rot.layout] if s.rot is not None else 0
        v_cos, v_sin = (rope[2], rope[3]) if s.v_rot else (None, None)      # the engine appends the tables of `value_rot`
        SK.attn_prep(y, self.q_off, self.k_off, self.v_off, q, None if self.shares_kv else kc,
                     None if self.shares_kv else vc, rope[0], rope[1], rot, s.qk_unit_norm, self.eps, cache.len_dev,
                     cache.pad_left, B, S, s.heads, s.kv_heads, s.dim, s.vdim, bias=self.bias, v_unit_norm=s.v_unit_norm,
                     v_token_major=s.talking_heads, layout=layout, q_norm_w=self.q_norm,
                     k_norm_w=self.k_norm if self.k_norm is not None else self.q_norm, v_cos=v_cos, v_sin=v_sin)
        if s.talking_heads:
            return self._attend_mixed(q, kc, vc, cache, B, S)
        gate = y[:, self.g_off:self.g_off + s.heads] if s.head_gate else None
        if not self.plain and (gate is not None or s.chunk or s.sink_learned or s.v_rot):
            if S > 1 and self._flash_masked_shape():
                # prompts of 128-wide heads in bfloat16: the tcgen05 kernel with the block bound, the sink, the gate and the turn
                # back in its softmax and epilogue
                out = torch.empty((B * S, s.heads * s.vdim), dtype=self.dtype, device=q.device)
                _lib.check(_lib.lib().jl_flash_prefill_masked(
                    q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cache.pad_left.data_ptr(), out.data_ptr(), B, S, s.heads,
                    s.kv_heads, s.dim, kc.shape[2], int(cache.index), float(s.scale), int(s.chunk), int(s.sink),
                    K._p(self.sink_logit), K._p(gate), gate.stride(0) if gate is not None else 0, K._p(v_cos), K._p(v_sin),
                    v_cos.shape[0] if v_cos is not None else 0, K._stream()), "jl_flash_prefill_masked")
                return out
            return SK.attn_masked(q, kc, vc, cache.len_dev, cache.pad_left, B, S, s.heads, s.kv_heads, s.dim, s.vdim, s.scale,
                                  gate=gate, window=s.window, chunk=s.chunk, sink=s.sink, sink_logit=self.sink_logit,
                                  v_cos=v_cos, v_sin=v_sin, v_layout=layout)
        if not self.plain:
            T = kc.shape[2]
            return SK.attn_windowed(q, kc, vc, cache.len_dev, cache.pad_left, B, S, s.heads, s.kv_heads, s.dim, s.vdim, T,
                                    s.dim, s.vdim, s.window, s.scale, sink=s.sink)
        if self._library_shape():
            # 64- / 128-wide heads in bfloat16 are the shapes the LLaMA kernels are built for: the tcgen05 flash kernel
            # for prompts, the split-KV kernel for one new token; both take the score scale as an argument
            out = self._attend_shared_kernels(q, kc, vc, cache, B, S)
            if gate is not None:
                SK.head_gate(out, gate, s.heads, s.vdim)
            return out
        return SK.attn_generic(q, kc, vc, gate, cache.len_dev, cache.pad_left, B, S, s.heads, s.scale)

    MAX_VALUE_ROW = 512            # widest value row the attention kernels take in one call

    def _attend_mixed(self, q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, cache: "object", B: int, S: int
                      ) -> torch.Tensor:
        """Weighted sums of every query head over all value heads (fp32), then the mix across heads.  Value heads are
        taken `MAX_VALUE_ROW // vdim` at a time."""
        s = self.spec
        M, H, G, T = B * S, s.heads, s.kv_heads, kc.shape[2]
        out = torch.empty((M, H * s.vdim), dtype=self.dtype, device=q.device)
        per = max(1, min(G, self.MAX_VALUE_ROW // s.vdim))
        row = G * s.vdim
        for c0 in range(0, G, per):
            gc = min(per, G - c0)
            v = vc[:, :, c0 * s.vdim:]                                # same row pitch, first column of this group of heads
            o = SK.attn_windowed(q, kc, v, cache.len_dev, cache.pad_left, B, S, H, G, s.dim, gc * s.vdim, T, s.dim, row,
                                 s.window, s.scale, strides=(G * T * s.dim, T * s.dim, T * row, 0), sink=s.sink, out_f32=True)
            SK.talk_mix(o, self.talk, out, H, G, gc, c0, s.vdim)
        return out

    def _flash_masked_shape(self) -> bool:
        """Whether prompts can run the tcgen05 kernel in its masked form: bfloat16, 128-wide keys and values, a layer's own
        head-major caches, no window, values rotated in the half-split pairing (or not at all)."""
        s = self.spec
        return (SK.tensor_cores_enabled() and self.dtype == torch.bfloat16 and s.dim == s.vdim == 128 and not self.shares_kv
                and s.heads // s.kv_heads in (1, 2, 4, 8, 16) and not (s.window or s.bias or s.v_unit_norm or s.talking_heads)
                and (not s.v_rot or s.rot.layout == "half") and _lib.has("jl_flash_prefill_masked"))

    def _library_shape(self) -> bool:
        s = self.spec
        return (SK.tensor_cores_enabled() and self.dtype == torch.bfloat16 and s.dim == s.vdim and s.dim in (64, 128)
                and s.heads // s.kv_heads in (1, 2, 4, 8))

    def _attend_shared_kernels(self, q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, cache: "object", B: int, S: int
                               ) -> torch.Tensor:
        s = self.spec
        L = _lib.lib()
        out = torch.empty((B * S, s.heads * s.vdim), dtype=self.dtype, device=q.device)
        T = kc.shape[2]
        if S > 1:
            _lib.check(L.jl_flash_prefill(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cache.len_dev.data_ptr(),
                                          cache.pad_left.data_ptr(), out.data_ptr(), B, S, s.heads, s.kv_heads, s.dim, T,
                                          int(cache.index), float(s.scale), K._stream()), "jl_flash_prefill")
            return out
        key = (B, T)
        if key not in self._decode_plans:
            self._decode_plans[key] = K.decode_attn_plan(B, s.heads, s.kv_heads, s.dim, T, q.device)
        splits, scratch = self._decode_plans[key]
        _lib.check(L.jl_decode_attn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cache.len_dev.data_ptr(),
                                    cache.pad_left.data_ptr(), K._p(scratch), out.data_ptr(), B, s.heads, s.kv_heads, s.dim,
                                    T, 1, float(s.scale), splits, 0, K._stream()), "jl_decode_attn")
        return out


class GlaMixer(Mixer):
    """Gated linear attention: S_t = diag(alpha_t) S_(t-1) + k_t v_tᵀ, o_t = S_tᵀ q_t per head, alpha from a low-rank
    projection through sigmoid(·)^(1/tau); read-out normalised per head (plain weight shared by the heads), gated by
    silu of a projection of the input.  The state is fp32 and is what the layer keeps between tokens."""

    kind = "gla"

    def __init__(self, spec: GlaMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        self.w_in, offs = _stack_rows([w["q"], w["k"], w["v"], w["g"], w["a1"]])
        self.q_off, self.k_off, self.v_off, self.g_off, self.a_off = offs
        self.a2 = w["a2"].contiguous()
        self.a2_bias = w["a2.b"].contiguous()
        self.norm = w["norm"].contiguous()
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.a2, self.a2_bias, self.norm, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> None:
        return None

    def new_state(self, batch: int, device: torch.device) -> torch.Tensor:
        s = self.spec
        return torch.zeros((batch, s.heads, s.dim, s.vdim), dtype=torch.float32, device=device)

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Optional[Tuple] = None
            ) -> torch.Tensor:
        s = self.spec
        y = SK.linear(h, self.w_in)                                   # fp32 [M, q | k | v | gate | low-rank decay input]
        o = SK.gla_scan(y, self.q_off, self.k_off, self.v_off, self.a_off, self.a2, self.a2_bias, cache.states[layer],
                        cache.len_dev, cache.pad_left, B, S, s.heads, s.dim, s.vdim, s.dim ** -0.5, s.tau)
        gate = y[:, self.g_off:self.g_off + s.heads * s.vdim]
        return SK.headnorm_gate(o, self.norm, gate, s.heads, s.vdim, self.eps, SK.ACT_SILU)


class LatentAttentionMixer(Mixer):
    """Softmax attention through low-rank latents.  Per token the layer keeps one row [normed key/value latent | rotated
    key part shared by the heads]; nothing per head.

    One token at a time (and prompt portions that continue a cache) the keys' and values' up-projections are applied on
    the query side: with q_h = [r_h | a_h] (rotated | unrotated) the score a_h · (U_h c) + r_h · k_rot equals
    (U_hᵀ a_h) · c + r_h · k_rot, and Σ p_j (V_h c_j) = V_h (Σ p_j c_j) — so the attention runs over the cached rows with
    one shared key/value head of width kv_rank + rot_dim (keys) and kv_rank (values), and two per-head batched products
    map into and out of the latent: every cached row is read once for all heads.

    A prompt that starts a sequence projects its latents up instead (two tensor-core GEMMs for all heads) and attends
    with per-head keys [k_rot | U_h c] and values V_h c in token-major layout, which costs a third of the arithmetic of
    the latent-space form at these head sizes.  Both forms run the windowed generic attention kernel.

    Internally a query head is laid out [rot_dim rotated | dim unrotated] (the rows of the query up-projection are
    permuted once at load), so that the rotation applies to the leading channels of a head as in the other mixers."""

    kind = "latent_attention"

    def __init__(self, spec: LatentAttentionMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        s = spec
        self.w_in, offs = _stack_rows([w["dq"], w["dkv"]])
        self.q_off, self.kv_off = offs
        self.q_norm, self.kv_norm = w["dq.norm"].contiguous(), w["dkv.norm"].contiguous()
        uq = w["uq"].view(s.heads, s.dim + s.rot_dim, s.q_rank)                 # stored [dim unrotated | rot_dim rotated]
        self.uq = torch.cat([uq[:, s.dim:], uq[:, :s.dim]], 1).reshape(s.heads * (s.dim + s.rot_dim), s.q_rank).contiguous()
        self.uk_t = w["uk"].view(s.heads, s.dim, s.kv_rank).transpose(1, 2).contiguous()    # [H, kv_rank, dim]
        self.uv = w["uv"].view(s.heads, s.vdim, s.kv_rank).contiguous()          # [H, vdim, kv_rank]
        self.w_kv, kv_offs = _stack_rows([w["uk"], w["uv"]])                     # [H·dim | H·vdim, kv_rank]: prompts
        self.v_col = kv_offs[1]
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype
        self.row = s.kv_rank + s.rot_dim

    def weights(self) -> List[torch.Tensor]:
        """What a decode step streams (the stacked up-projection of prompts holds the same values once more)."""
        return [self.w_in, self.q_norm, self.kv_norm, self.uq, self.uk_t, self.uv, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> Tuple[torch.Tensor, None]:
        return torch.zeros((batch, length, self.row), dtype=self.dtype, device=device), None

    def new_state(self, batch: int, device: torch.device) -> Optional[torch.Tensor]:
        return None

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Tuple[torch.Tensor, torch.Tensor]
            ) -> torch.Tensor:
        s = self.spec
        M, H, qd = B * S, s.heads, s.dim + s.rot_dim
        rot = s.rot.dims if s.rot is not None else 0
        layout = SK.ROT_LAYOUTS[s.rot.layout] if s.rot is not None else 0
        kc = cache.ks[layer]                                                   # [B, T, kv_rank + rot_dim]
        starts = S > 1 and int(cache.index) == 0                               # a prompt from an empty cache
        y = SK.linear(h, self.w_in)                                            # fp32 [M, query latent | kv latent | key part]
        cq, c_new, kr_new = SK.latent_prep(y, self.q_off, s.q_rank, self.kv_off, s.kv_rank, s.rot_dim, rot, layout,
                                           self.q_norm, self.kv_norm, kc, rope[0], rope[1], self.eps, cache.len_dev,
                                           cache.pad_left, B, S, token_major=starts)
        q = SK.linear(cq, self.uq, out_f32=False)                              # [M, H·(rot_dim + dim)]
        if starts:
            return self._attend_projected(q, c_new, kr_new, cache, B, S, rot, layout, rope)
        qa = torch.empty((M, H * self.row), dtype=self.dtype, device=h.device)
        a = q[:, s.rot_dim:] if s.rot_dim else q                               # head h's unrotated part starts at h·qd
        SK.linear_batched(a, self.uk_t, qa, nbatch=H, rows=M, x_bs=qd, o_bs=self.row)      # U_hᵀ a_h
        if s.rot_dim:
            SK.rotary_slice(q, qd, 0, qa, self.row, s.kv_rank, H, s.rot_dim, rot, layout, rope[0], rope[1],
                            cache.len_dev, cache.pad_left, B, S)
        ctx = SK.attn_windowed(qa, kc, kc, cache.len_dev, cache.pad_left, B, S, H, 1, self.row, s.kv_rank, kc.shape[1],
                               self.row, self.row, s.window, s.scale)         # [M, H·kv_rank]
        out = torch.empty((M, H * s.vdim), dtype=self.dtype, device=h.device)
        SK.linear_batched(ctx, self.uv, out, nbatch=H, rows=M, x_bs=s.kv_rank, o_bs=s.vdim)
        return out

    def _attend_projected(self, q: torch.Tensor, c_new: torch.Tensor, kr_new: torch.Tensor, cache: "object", B: int, S: int,
                          rot: int, layout: int, rope: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
        """Per-head keys and values of the S new tokens of every row, token-major; slot == index within the prompt."""
        s = self.spec
        M, H, qd = B * S, s.heads, s.dim + s.rot_dim
        kv = SK.linear(c_new, self.w_kv, out_f32=False)                        # [M, H·dim | H·vdim (| padding)]
        qf = torch.empty_like(q)
        SK.rotary_slice(q, qd, 0, qf, qd, 0, H, qd, rot, layout, rope[0], rope[1], cache.len_dev, cache.pad_left, B, S)
        kf = torch.empty((M, H * qd), dtype=self.dtype, device=q.device)       # [M, H, rot_dim | dim]
        if s.rot_dim:
            SK.rotary_slice(kr_new, 0, 0, kf, qd, 0, H, s.rot_dim, 0, 0, rope[0], rope[1], cache.len_dev, cache.pad_left, B, S)
        SK.rotary_slice(kv, s.dim, 0, kf, qd, s.rot_dim, H, s.dim, 0, 0, rope[0], rope[1], cache.len_dev, cache.pad_left, B, S)
        v = kv[:, self.v_col:]
        ldv = kv.stride(0)
        return SK.attn_windowed(qf, kf, v, cache.len_dev, cache.pad_left, B, S, H, H, qd, s.vdim, S, H * qd, ldv, s.window,
                                s.scale, strides=(S * H * qd, qd, S * ldv, s.vdim))


class RetentionMixer(Mixer):
    """Retention: linear attention with one fixed decay per head, S_t = decay_h S_(t-1) + k_t v_tᵀ, o_t = S_tᵀ q_t, rotary
    q / k, k scaled by dim^(-1/2) after the rotation; every head's read-out divided by its RMS (no weight) and gated by
    silu of a projection of the input.  The fp32 state is what the layer keeps between tokens."""

    kind = "retention"

    def __init__(self, spec: RetentionMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        self.w_in, offs = _stack_rows([w["q"], w["k"], w["v"], w["g"]])
        self.q_off, self.k_off, self.v_off, self.g_off = offs
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype
        self.decay = torch.tensor([float(a) for a in spec.decay], dtype=torch.float64).to(torch.float32).to(self.wo.device)

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> None:
        return None

    def new_state(self, batch: int, device: torch.device) -> torch.Tensor:
        s = self.spec
        return torch.zeros((batch, s.heads, s.dim, s.vdim), dtype=torch.float32, device=device)

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Tuple[torch.Tensor, torch.Tensor]
            ) -> torch.Tensor:
        s = self.spec
        rot = s.rot.dims if s.rot is not None else 0
        layout = SK.ROT_LAYOUTS[s.rot.layout] if s.rot is not None else 0
        y = SK.linear(h, self.w_in)                                   # fp32 [M, q | k | v | gate]
        o = SK.retention_scan(y, self.q_off, self.k_off, self.v_off, self.decay, rope[0], rope[1], rot, layout,
                              s.dim ** -0.5, cache.states[layer], cache.len_dev, cache.pad_left, B, S, s.heads, s.dim,
                              s.vdim)
        gate = y[:, self.g_off:self.g_off + s.heads * s.vdim]
        return SK.headnorm_gate(o, None, gate, s.heads, s.vdim, self.eps, SK.ACT_SILU, dtype=self.dtype)


class StateSpaceMixer(Mixer):
    """Selective state space layer.  One stacked projection [z | x | B | C | dt]; x, B, C through a causal convolution
    (state: its last taps − 1 inputs) and silu; dt = softplus(dt + bias); per head S_t = exp(−exp(A_log) dt) S_(t−1) +
    dt B_t x_tᵀ, y_t = S_tᵀ C_t + D x_t — the scan kernels of gated linear attention with keys B, queries C (shared by the
    heads of a group), values dt · x and one decay per (token, head); then y · silu(z), an RMS norm over each of
    `norm_groups` parts of the row, the weight, and the output projection.  Step size, decay, state and norm are fp32."""

    kind = "state_space"

    def __init__(self, spec: StateSpaceMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        s = spec
        self.inner = s.heads * s.vdim
        self.gn = s.groups * s.state
        self.w_in, _ = _stack_rows([w["in"]])
        self.z_off, self.x_off = 0, self.inner
        self.dt_off = 2 * self.inner + 2 * self.gn
        self.conv_w, self.conv_b = w["conv"].contiguous(), w["conv.b"].contiguous()
        self.dt_bias, self.a_log, self.skip = w["dt_bias"].contiguous(), w["A_log"].contiguous(), w["D"].contiguous()
        self.norm = w["norm"].contiguous()
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype

    @staticmethod
    def shapes(spec: StateSpaceMixerSpec, W: int, rank_of: "object" = None) -> Dict[str, Tuple[int, ...]]:
        inner, gn = spec.heads * spec.vdim, spec.groups * spec.state
        return {"in": (2 * inner + 2 * gn + spec.heads, W), "conv": (inner + 2 * gn, spec.conv), "conv.b": (inner + 2 * gn,),
                "dt_bias": (spec.heads,), "A_log": (spec.heads,), "D": (spec.heads,), "norm": (inner,), "o": (W, inner)}

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.skip, self.norm, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> None:
        return None

    def new_state(self, batch: int, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
        s = self.spec
        return (torch.zeros((batch, s.heads, s.state, s.vdim), dtype=torch.float32, device=device),
                torch.zeros((batch, max(s.conv - 1, 1), self.inner + 2 * self.gn), dtype=torch.float32, device=device))

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Optional[Tuple] = None
            ) -> torch.Tensor:
        s = self.spec
        state, conv_state = cache.states[layer]
        y = SK.linear(h, self.w_in)                                   # fp32 [M, z | x | B | C | dt]
        u = SK.causal_conv(y, self.x_off, self.conv_w, self.conv_b, conv_state, cache.len_dev, cache.pad_left, B, S,
                           act=SK.ACT_SILU)                           # fp32 [M, x | B | C]
        o = SK.ssd_scan(y, self.dt_off, self.dt_bias, self.a_log, u, self.inner + self.gn, self.inner, 0, s.groups, state,
                        cache.len_dev, cache.pad_left, B, S, s.heads, s.state, s.vdim)
        return SK.gated_groupnorm(o, u[:, :self.inner], self.skip, s.vdim, y[:, self.z_off:self.z_off + self.inner], self.norm,
                                  s.norm_groups, self.eps, SK.ACT_SILU)


class DeltaRuleMixer(Mixer):
    """Gated delta rule with one decay per key channel (see `DeltaMixerSpec`).  One stacked projection
    [q | k | v | beta | decay rank | gate rank]; q, k, v through ONE causal convolution call (their filters stacked; state:
    the last taps − 1 inputs) and silu; the scan kernels normalise q / k, form beta and the decays
    exp(−exp(A_log) softplus(A2 · + bias)) and advance the fp32 state; the read-out is normed per head (weight shared by
    the heads) and gated by sigmoid of the low-rank gate."""

    kind = "channel_delta"

    def __init__(self, spec: DeltaMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        s = spec
        self.w_in, offs = _stack_rows([w["q"], w["k"], w["v"], w["b"], w["a1"], w["g1"]])
        self.q_off, self.k_off, self.v_off, self.b_off, self.a_off, self.g_off = offs
        self.nq, self.nv = s.kv_heads * s.dim, s.heads * s.vdim
        self.conv_w = torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0).contiguous()
        self.a2, self.a_bias, self.a_log = w["a2"].contiguous(), w["dt_bias"].contiguous(), w["A_log"].contiguous()
        self.g2 = w["g2"].contiguous()
        self.gate_rank = w["g1"].shape[0]
        self.norm = w["norm"].contiguous()
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype

    @staticmethod
    def shapes(spec: DeltaMixerSpec, W: int, rank_of: "object" = None) -> Dict[str, Tuple[int, ...]]:
        rank_of = rank_of or (lambda name, default: default)
        nq, nv, nd = spec.kv_heads * spec.dim, spec.heads * spec.vdim, spec.heads * spec.dim
        ra, rg = rank_of("a1", 16), rank_of("g1", 16)
        return {"q": (nq, W), "q.conv": (nq, spec.conv), "k": (nq, W), "k.conv": (nq, spec.conv), "v": (nv, W),
                "v.conv": (nv, spec.conv), "b": (spec.heads, W), "A_log": (spec.heads,), "norm": (spec.vdim,), "a1": (ra, W),
                "a2": (nd, ra), "dt_bias": (nd,), "g1": (rg, W), "g2": (nv, rg), "o": (W, nv)}

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.conv_w, self.a2, self.a_bias, self.a_log, self.g2, self.norm, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> None:
        return None

    def new_state(self, batch: int, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
        s = self.spec
        return (torch.zeros((batch, s.heads, s.dim, s.vdim), dtype=torch.float32, device=device),
                torch.zeros((batch, max(s.conv - 1, 1), 2 * self.nq + self.nv), dtype=torch.float32, device=device))

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Optional[Tuple] = None
            ) -> torch.Tensor:
        s = self.spec
        state, conv_state = cache.states[layer]
        y = SK.linear(h, self.w_in)                                   # fp32 [M, q | k | v | beta | decay rank | gate rank]
        u = SK.causal_conv(y, self.q_off, self.conv_w, None, conv_state, cache.len_dev, cache.pad_left, B, S, act=SK.ACT_SILU)
        o = SK.delta_scan(u, 0, self.nq, 2 * self.nq, s.kv_heads, y, self.b_off, self.a_off, self.a2, self.a_bias,
                          self.a_log, state, cache.len_dev, cache.pad_left, B, S, s.heads, s.dim, s.vdim)
        g_in = SK.act_cast(y[:, self.g_off:self.g_off + self.gate_rank], self.dtype)
        gate = SK.linear(g_in, self.g2)                               # fp32 [M, heads · vdim]
        return SK.headnorm_gate(o, self.norm, gate, s.heads, s.vdim, self.eps, SK.ACT_SIGMOID)


class ParallelMixer(Mixer):
    """Two mixers side by side on the same input: scale · (norm(left(h)) · w_left + norm(right(h)) · w_right), the norms
    over the model width.  Each side keeps its own cache / state; the layer's cache entries are pairs."""

    kind = "parallel"

    def __init__(self, spec: ParallelMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        self.sides = []
        for side, sub in (("left", spec.left), ("right", spec.right)):
            sw = {k[len(side) + 1:]: v for k, v in w.items() if k.startswith(side + ".") and k != side + ".out"}
            self.sides.append(MIXERS[sub.kind](sub, sw, eps))
        self.out_norms = [w["left.out"].contiguous(), w["right.out"].contiguous()]
        self.dtype = self.out_norms[0].dtype

    @staticmethod
    def shapes(spec: ParallelMixerSpec, W: int, rank_of: "object" = None) -> Dict[str, Tuple[int, ...]]:
        out: Dict[str, Tuple[int, ...]] = {}
        for side, sub in (("left", spec.left), ("right", spec.right)):
            sub_rank = (lambda name, default, side=side: rank_of(side + "." + name, default)) if rank_of else None
            for name, shape in MIXERS[sub.kind].shapes(sub, W, sub_rank).items():
                out[f"{side}.{name}"] = shape
            out[f"{side}.out"] = (W,)
        return out

    def weights(self) -> List[torch.Tensor]:
        return [t for m in self.sides for t in m.weights()] + self.out_norms

    def new_cache(self, batch: int, length: int, device: torch.device) -> Optional[Tuple]:
        got = [m.new_cache(batch, length, device) for m in self.sides]
        if all(g is None for g in got):
            return None
        return (tuple(g[0] if g is not None else None for g in got), tuple(g[1] if g is not None else None for g in got))

    def new_state(self, batch: int, device: torch.device) -> Optional[Tuple]:
        got = [m.new_state(batch, device) for m in self.sides]
        return None if all(g is None for g in got) else tuple(got)

    OVERLAP_ROWS = 8               # up to this many rows the two sides run on two streams

    def forward(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Optional[Tuple] = None
                ) -> torch.Tensor:
        """With a few rows (decoding) neither side fills the GPU and each is a chain of short dependent kernels, so the right
        side runs on a second stream beside the left one (inside a graph capture the fork and join become edges of the
        captured graph).  Prompts stay on one stream: their tensor-core GEMMs share one split-K workspace."""
        views = [_CacheView(cache, layer, i) for i in range(2)]
        if B * S <= self.OVERLAP_ROWS:
            main = torch.cuda.current_stream()
            if getattr(self, "_side", None) is None:
                self._side, self._fork, self._join = torch.cuda.Stream(device=h.device), torch.cuda.Event(), torch.cuda.Event()
            self._fork.record(main)
            self._side.wait_event(self._fork)
            with torch.cuda.stream(self._side):
                right = self.sides[1].forward(h, B, S, views[1], layer, rope)
                self._join.record(self._side)
            left = self.sides[0].forward(h, B, S, views[0], layer, rope)
            main.wait_event(self._join)
        else:
            left = self.sides[0].forward(h, B, S, views[0], layer, rope)
            right = self.sides[1].forward(h, B, S, views[1], layer, rope)
        return SK.norm_mean2(left, self.out_norms[0], right, self.out_norms[1], self.spec.scale, self.eps)


MIXERS = {"attention": AttentionMixer, "gla": GlaMixer, "latent_attention": LatentAttentionMixer,
          "retention": RetentionMixer, "state_space": StateSpaceMixer, "channel_delta": DeltaRuleMixer,
          "parallel": ParallelMixer}

