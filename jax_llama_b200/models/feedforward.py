"""Feed-forward sublayers of the hybrid decoder family, each a small class over the kernels of `ops/seq_kernels.py`.

A feed-forward owns its weights in kernel layout and turns the normalised input ``h [M, width]`` into an fp32
``[M, width]`` branch output; norms and the residual sum belong to the layer stack (`models/hybrid_engine.py`).
Constants (activation, score function, group limits, weight scale, shared expert) are parameters of the spec
(`config.py`).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..config import DenseMlpSpec, MoeMlpSpec
from ..ops import seq_kernels as SK
from .mixers import _stack_rows


GLU_ALPHA = 1.702          # slope inside the sigmoid of the clamped gated activation


def _gated_act(y: torch.Tensor, u_off: int, F: int, act: str, limit: float, dtype: torch.dtype, **kw) -> torch.Tensor:
    """The gated activation of a fused gate | up product y fp32 [rows, gate (F) | up at u_off]."""
    if act == "glu_clamped":
        return SK.glu_act(y, 0, u_off, F, dtype, kind=SK.GLU_CLAMPED, limit=limit, alpha=GLU_ALPHA, **kw)
    return SK.glu_act(y, 0, u_off, F, dtype, kind=SK.GLU_PRODUCT, act=SK.ACTIVATIONS[act], **kw)


def _softplus(z: float) -> float:
    return z if z > 30.0 else math.log1p(math.exp(z))


class DenseFeedForward:
    """down(act(up h)); gated: down(act(gate h) · (up h)) with gate and up stacked into one product.  The "xielu" activation
    has two numbers (p, q) per layer in the tensor `act`: its coefficients softplus(p) and 1/2 + softplus(q) are formed once,
    when the weights are loaded."""

    kind = "dense"

    def __init__(self, spec: DenseMlpSpec, w: Dict[str, torch.Tensor]):
        if spec.act not in SK.ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.act!r}")
        self.spec, self.act = spec, SK.ACTIVATIONS[spec.act]
        if spec.gated:
            self.up, offs = _stack_rows([w["gate"], w["up"]])
            self.u_off = offs[1]
        else:
            self.up = w["up"].contiguous()
        self.down = w["down"].contiguous()
        self.p0 = self.p1 = 0.0
        if spec.act == "xielu":
            if spec.gated:
                raise ValueError("the xielu activation goes with an ungated layer")
            p, q = (float(v) for v in w["act"].double().cpu())
            self.p0, self.p1 = float(np.float32(_softplus(p))), float(np.float32(0.5 + _softplus(q)))

    @staticmethod
    def shapes(spec: DenseMlpSpec, W: int) -> Dict[str, Tuple[int, ...]]:
        out = {"up": (spec.ff, W), "down": (W, spec.ff)}
        if spec.gated:
            out["gate"] = (spec.ff, W)
        if spec.act == "xielu":
            out["act"] = (2,)
        return out

    def weights(self) -> List[torch.Tensor]:
        return [self.up, self.down]

    def streamed_weights(self, rows: int) -> List[torch.Tensor]:
        return self.weights()

    def run(self, h: torch.Tensor) -> torch.Tensor:
        if self.spec.gated:
            t = _gated_act(SK.linear(h, self.up), self.u_off, self.spec.ff, self.spec.act, 0.0, h.dtype)
        else:
            t = SK.linear(h, self.up, act=self.act, p0=self.p0, p1=self.p1, out_f32=False)
        return SK.linear(t, self.down)


class MoeFeedForward:
    """Mixture of experts.  The router (and the shared expert's gate) is one fp32-accumulated product; a warp per
    token chooses the experts.  Few rows (decoding): every (token, choice) pair streams its expert's two matrices in
    one batched launch each.  Many rows (prompts): the pairs are ordered by expert into whole row tiles and each tile
    runs against its expert's matrices — in bfloat16 on the grouped tcgen05 GEMM over rows gathered once, otherwise
    (true float32, sizes the tensor-core kernel does not take) on the exact tiled kernel, which gathers as it reads.
    The weighted sum, the shared expert and its gate meet in one combine pass.  Identity experts (router outputs beyond the
    experts with matrices) are chosen like the others; their pairs run no product and their share, weight · input, is added in the
    combine pass."""

    kind = "moe"

    def __init__(self, spec: MoeMlpSpec, w: Dict[str, torch.Tensor]):
        if (spec.act not in SK.ACTIVATIONS and not spec.gated) or spec.score not in SK.SCORES:
            raise ValueError(f"unknown activation {spec.act!r} or score function {spec.score!r}")
        if spec.gated and spec.act != "glu_clamped" and spec.act not in SK.ACTIVATIONS:
            raise ValueError(f"unknown gated activation {spec.act!r}")
        self.spec, self.act, self.score = spec, SK.ACTIVATIONS.get(spec.act, SK.ACT_NONE), SK.SCORES[spec.score]
        E = spec.experts
        self.n_route = E + spec.identity                   # router outputs: experts, then identity experts (no matrices)
        self.choice_bias = w["correction"].float().contiguous() if spec.choice_bias else None
        self.u_off = self.shared_u_off = 0
        if spec.gated:                                                                  # [E, gate | up (padded to 8 rows), W]
            pairs = [_stack_rows([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]
            self.up, self.u_off = torch.stack([p[0] for p in pairs]).contiguous(), pairs[0][1][1]
        else:
            self.up = torch.stack([w[f"e{e}.up"] for e in range(E)]).contiguous()      # [E, ff, W]
        self.down = torch.stack([w[f"e{e}.down"] for e in range(E)]).contiguous()      # [E, W, ff]
        self.router_bias = w["router.b"].float().contiguous() if spec.router_bias else None
        self.has_shared = spec.shared_ff > 0
        gated = self.has_shared and spec.shared_gate
        self.w_route, offs = _stack_rows([w["router"]] + ([w["shared.sg"]] if gated else []))
        self.gate_off = offs[1] if gated else -1
        self.shared_up = w["shared.up"].contiguous() if self.has_shared else None
        if self.has_shared and spec.gated:
            self.shared_up, offs = _stack_rows([w["shared.gate"], w["shared.up"]])
            self.shared_u_off = offs[1]
        self.shared_down = w["shared.down"].contiguous() if self.has_shared else None

    @staticmethod
    def shapes(spec: MoeMlpSpec, W: int) -> Dict[str, Tuple[int, ...]]:
        out: Dict[str, Tuple[int, ...]] = {"router": (spec.experts + spec.identity, W)}
        if spec.router_bias:
            out["router.b"] = (spec.experts + spec.identity,)
        if spec.choice_bias:
            out["correction"] = (spec.experts + spec.identity,)
        for e in range(spec.experts):
            out[f"e{e}.up"], out[f"e{e}.down"] = (spec.ff, W), (W, spec.ff)
            if spec.gated:
                out[f"e{e}.gate"] = (spec.ff, W)
        if spec.shared_ff > 0:
            out["shared.up"], out["shared.down"] = (spec.shared_ff, W), (W, spec.shared_ff)
            if spec.gated:
                out["shared.gate"] = (spec.shared_ff, W)
            if spec.shared_gate:
                out["shared.sg"] = (1, W)
        return out

    def weights(self) -> List[torch.Tensor]:
        return [t for t in (self.up, self.down, self.w_route, self.shared_up, self.shared_down) if t is not None]

    def streamed_weights(self, rows: int) -> List[torch.Tensor]:
        """What a step of `rows` tokens reads at least: at most rows · top experts are touched."""
        s = self.spec
        frac = min(1.0, rows * s.top / s.experts)
        n = max(1, int(round(frac * s.experts)))
        return [self.up[:n], self.down[:n]] + [t for t in (self.w_route, self.shared_up, self.shared_down) if t is not None]

    def run(self, h: torch.Tensor) -> torch.Tensor:
        s = self.spec
        M, W = h.shape
        z = SK.linear(h, self.w_route)                                             # fp32 [M, router logits | gate logit]
        ident_w = torch.empty(M, dtype=torch.float32, device=h.device) if s.identity else None
        idx, wt = SK.moe_route(z, self.n_route, s.top, s.groups, s.keep, s.group_top, self.score, s.normalise, s.scale,
                               bias=self.router_bias, choice_bias=self.choice_bias, n_real=s.experts, ident_w=ident_w)
        n_up = self.up.shape[1]                                                    # ff, or gate | up rows of a gated expert
        if M <= SK.MOE_PAIR_ROWS:
            n = M * s.top
            flat = idx.view(-1)
            if s.gated:
                gu = torch.empty((n, n_up), dtype=torch.float32, device=h.device)
                SK.linear_batched(h, self.up, gu, nbatch=n, rows=1, x_bs=h.stride(0), o_bs=n_up, x_div=s.top, w_index=flat)
                t = _gated_act(gu, self.u_off, s.ff, s.act, s.limit, h.dtype)
            else:
                t = torch.empty((n, s.ff), dtype=h.dtype, device=h.device)
                SK.linear_batched(h, self.up, t, nbatch=n, rows=1, x_bs=h.stride(0), o_bs=s.ff, x_div=s.top, w_index=flat,
                                  act=self.act)
            y = torch.empty((n, W), dtype=torch.float32, device=h.device)
            SK.linear_batched(t, self.down, y, nbatch=n, rows=1, x_bs=s.ff, o_bs=W, w_index=flat)
            pos = None
        elif SK.tensor_cores_enabled() and h.dtype == torch.bfloat16 and W % 8 == 0 and s.ff % 8 == 0 and h.is_contiguous():
            # sorted rows in 128-row segments, gathered once, then the grouped tcgen05 GEMM twice
            pos, row_src, tile_group, used = SK.moe_sort(idx, s.experts, tile=SK.GEMM_TILE_ROWS)
            xs = SK.moe_gather(h, row_src)
            if s.gated:
                gu = SK.gemm_grouped(xs, self.up, tile_group, tiles_used=used)
                t = _gated_act(gu, self.u_off, s.ff, s.act, s.limit, h.dtype, rows_used=used, rows_mult=SK.GEMM_TILE_ROWS,
                               zero=True)
            else:
                t = SK.gemm_grouped(xs, self.up, tile_group, act=self.act, out_f32=False, tiles_used=used)
            y = SK.gemm_grouped(t, self.down, tile_group, tiles_used=used)
        else:
            pos, row_src, tile_group, _ = SK.moe_sort(idx, s.experts)
            rows = row_src.shape[0]
            if s.gated:
                gu = torch.empty((rows, n_up), dtype=torch.float32, device=h.device)
                SK.linear_sorted(h, self.up, gu, tile_group, row_src)
                t = _gated_act(gu, self.u_off, s.ff, s.act, s.limit, h.dtype)
            else:
                t = torch.empty((rows, s.ff), dtype=h.dtype, device=h.device)
                SK.linear_sorted(h, self.up, t, tile_group, row_src, act=self.act)
            y = torch.empty((rows, W), dtype=torch.float32, device=h.device)
            SK.linear_sorted(t, self.down, y, tile_group, None)
        shared: Optional[torch.Tensor] = None
        gate = None
        if self.has_shared:
            if s.gated:
                u = _gated_act(SK.linear(h, self.shared_up), self.shared_u_off, s.shared_ff, s.act, s.shared_limit, h.dtype)
            else:
                u = SK.linear(h, self.shared_up, act=self.act, out_f32=False)
            shared = SK.linear(u, self.shared_down)
            if self.gate_off >= 0:
                gate = z[:, self.gate_off:self.gate_off + 1]
        if s.identity:                                     # pairs that chose an identity expert ran nothing: weight · input instead
            return SK.moe_combine(y, pos, wt, shared, gate, W, idx=idx, ident_w=ident_w, x=h)
        return SK.moe_combine(y, pos, wt, shared, gate, W)


FEED_FORWARDS = {"dense": DenseFeedForward, "moe": MoeFeedForward}
