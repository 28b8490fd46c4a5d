"""Engine of the hybrid decoder family: layers that mix softmax attention and linear-recurrence mixers over an fp32
residual stream, each sublayer between two RMS norms.

It is the B200 engine (`models/engine.py`) with another layer stack: the request batching (left-padded static batch),
the decode state, on-device selection and bookkeeping, CUDA-graph replay of the decode step, `generate` and the
token-at-a-time stream are inherited; what changes is

* the weights (per-layer mixers from `models/mixers.py`, feed-forwards from `models/feedforward.py`; norm weights
  stored around zero or plain, as the configuration says),
* the block form: sublayers one after the other, each between two norms ("sandwich"), or mixer and feed-forward
  side by side on two norms of the same stream, their scaled sum added to it ("parallel"),
* the cache: per attention layer a key / value cache with that layer's head sizes (none for a layer that reads another
  layer's), per recurrent layer an fp32 state, all advanced by the same device-side fill level and left-pad counts; a
  stretch of layers that runs several times over with the same weights (`config.loop`) has one cache entry per layer RUN,
* the ends of a layer: a learned position row added to the token embedding, and a per-layer token input after the
  feed-forward (a second embedding table, gated by a projection of the stream, projected up, normed and added),
* the numerics: norms, softmax, recurrences and the residual sum in fp32; matrix operands in bfloat16, or everything in
  true float32 (`dtype=torch.float32`), which the kernels of this family are built for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..ops import _lib
from ..ops import kernels as K
from ..ops import seq_kernels as SK
from .engine import B200Engine, DecodeState, DeviceKVCache
from .feedforward import FEED_FORWARDS
from .mixers import MIXERS, rotary_table


BRANCH_OVERLAP_ROWS = 8        # up to this many rows the two branches of a parallel block run on two streams


@dataclass
class HybridCache(DeviceKVCache):
    """Per-layer caches of unequal shapes plus recurrent states.  `k` / `v` of the base class point at the first
    attention layer's tensors (identity of the cache for graph keys)."""

    ks: List[Any] = field(default_factory=list)          # per layer: a tensor, None, or a tuple (a layer of several mixers)
    vs: List[Any] = field(default_factory=list)
    states: List[Any] = field(default_factory=list)      # per layer: fp32 tensor(s) carried from token to token
    length: int = 0
    prev_tok: Optional[torch.Tensor] = None              # int32 [B]: every row's last token (embeddings that hash token pairs)
    step_ids: Optional[torch.Tensor] = None              # int32 [B·S]: the tokens of the step in flight (per-layer token inputs)

    @property
    def capacity(self) -> int:
        return self.length

    def set_index(self, value: int) -> None:
        super().set_index(value)
        if int(value) == 0:                       # a new request batch starts from an empty state
            for s in _tensors(self.states):
                s.zero_()

    def mutable_state(self) -> List[torch.Tensor]:
        return [self.len_dev] + _tensors(self.states) + ([self.prev_tok] if self.prev_tok is not None else [])


def _tensors(obj: Any) -> List[torch.Tensor]:
    """The tensors of a nest of lists / tuples (None entries skipped)."""
    if obj is None:
        return []
    if isinstance(obj, torch.Tensor):
        return [obj]
    return [t for o in obj for t in _tensors(o)]


@dataclass
class HybridLayer:
    mixer: Any
    norm1: torch.Tensor
    norm1b: Optional[torch.Tensor] = None          # norms after the sublayers: sandwich blocks only
    norm2: Optional[torch.Tensor] = None
    norm2b: Optional[torch.Tensor] = None
    ff: Any = None
    side: Any = None                               # per-layer token input (`TokenSide`)


class TokenSide:
    """Per-layer token input: y = proj (gelu_tanh(gate x) · Es[token, col0 : col0 + dim]);  x += y / rms(y) · w.  `table` is the
    second embedding table [vocab, layers · dim], shared by the layers; every layer reads its own slice of a row (the same
    slice on every pass of a looped layer).  Many rows: two GEMMs around a small gate kernel, then the fused "norm, add, next
    norm" step; a few rows (decoding): the gate kernel does the small projection itself on the fp32 stream rows, the up
    projection streams its weights once for all rows."""

    ROWS_KERNEL = 8

    def __init__(self, table: torch.Tensor, col0: int, w: Dict[str, torch.Tensor]):
        self.table, self.col0 = table, int(col0)
        self.gate, self.proj, self.norm = w["gate"].contiguous(), w["proj"].contiguous(), w["norm"].contiguous()
        self.dim = self.gate.shape[0]

    def weights(self) -> List[torch.Tensor]:
        return [self.gate, self.proj, self.norm]

    def wants_cast(self, rows: int) -> bool:
        """Whether `run` reads a copy of the stream in the operand type (the caller's residual step can write it on the way)."""
        return rows > self.ROWS_KERNEL and self.gate.dtype != torch.float32

    def run(self, x: torch.Tensor, ids: torch.Tensor, w_next: Optional[torch.Tensor], eps: float,
            x_cast: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Adds the token input to x (fp32, in place); returns norm(x) · w_next when w_next is given.  x_cast: x in the operand
        type, when the caller has it."""
        if x.shape[0] <= self.ROWS_KERNEL:
            g = SK.side_gate_rows(x, ids, self.table, self.col0, self.gate)
        else:
            xc = x_cast if x_cast is not None else (x if self.gate.dtype == torch.float32 else SK.act_cast(x, self.gate.dtype))
            t = SK.linear(xc, self.gate)                                      # fp32 [M, dim]
            g = SK.side_gate(t, ids, self.table, self.col0, self.dim, self.gate.dtype)
        y = SK.linear(g, self.proj)                                           # fp32 [M, width]
        return SK.postnorm_add(y, self.norm, x, eps, 0.0, w_next=w_next)


def tensor_shapes(config: Any, decay_rank: int = 16, present: Optional[Dict[str, Tuple[int, ...]]] = None
                  ) -> Dict[str, Tuple[int, ...]]:
    """Checkpoint tensor names → shapes for a config of this family (what a loader expects, what random_init draws).
    The ranks of low-rank projections are not config keys: a checkpoint fixes them by the shapes of its tensors
    (`present`: name → shape of what the checkpoint holds; absent: `decay_rank`)."""
    W = config.hidden_size
    sandwich = config.block == "sandwich"
    out: Dict[str, Tuple[int, ...]] = {"embed": (config.vocab_size, W), "final.norm": (W,)}
    if not config.tied_head:
        out["head"] = (config.vocab_size, W)
    if config.embed_norm:
        out["embed.norm"] = (W,)
    if config.pair_embedding is not None:
        out["bigram"] = (config.pair_embedding.buckets + 1, W)
    if config.learned_positions:                       # the table's own length wins over the configuration's
        out["pos"] = (int(present["pos"][0]) if present and "pos" in present else config.max_positions, W)
    side = config.token_side_dim
    if side:
        out["side.embed"] = (config.vocab_size, len(config.layers) * side)
    for i, l in enumerate(config.layers):
        p, m = f"l{i}.", l.mixer
        out[p + "norm1"] = (W,)
        if side:
            out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = (side, W), (W, side), (W,)
        if sandwich:
            out[p + "norm1b"] = (W,)
        if hasattr(MIXERS[m.kind], "shapes"):

            def rank_of(name: str, default: int, prefix: str = p + "mix.") -> int:
                return int(present[prefix + name][0]) if present and prefix + name in present else int(decay_rank)

            for name, shape in MIXERS[m.kind].shapes(m, W, rank_of).items():
                out[p + "mix." + name] = shape
        elif m.kind == "gla":
            out.update({p + "mix.q": (m.heads * m.dim, W), p + "mix.k": (m.heads * m.dim, W),
                        p + "mix.v": (m.heads * m.vdim, W), p + "mix.g": (m.heads * m.vdim, W),
                        p + "mix.o": (W, m.heads * m.vdim), p + "mix.norm": (m.vdim,), p + "mix.a1": (decay_rank, W),
                        p + "mix.a2": (m.heads * m.dim, decay_rank), p + "mix.a2.b": (m.heads * m.dim,)})
        elif m.kind == "retention":
            out.update({p + "mix.q": (m.heads * m.dim, W), p + "mix.k": (m.heads * m.dim, W),
                        p + "mix.v": (m.heads * m.vdim, W), p + "mix.g": (m.heads * m.vdim, W),
                        p + "mix.o": (W, m.heads * m.vdim)})
        elif m.kind == "latent_attention":
            out.update({p + "mix.dq": (m.q_rank, W), p + "mix.dq.norm": (m.q_rank,),
                        p + "mix.uq": (m.heads * (m.dim + m.rot_dim), m.q_rank),
                        p + "mix.dkv": (m.kv_rank + m.rot_dim, W), p + "mix.dkv.norm": (m.kv_rank,),
                        p + "mix.uk": (m.heads * m.dim, m.kv_rank), p + "mix.uv": (m.heads * m.vdim, m.kv_rank),
                        p + "mix.o": (W, m.heads * m.vdim)})
        else:
            out[p + "mix.q"] = (m.heads * m.dim, W)
            if m.kv_from is None:
                out[p + "mix.k"], out[p + "mix.v"] = (m.kv_heads * m.dim, W), (m.kv_heads * m.vdim, W)
            if m.head_gate:
                out[p + "mix.g"] = (m.heads, W)
            out[p + "mix.o"] = (W, m.heads * m.vdim)
        if l.mlp is not None:
            if config.block != "parallel_shared":
                out[p + "norm2"] = (W,)
            if sandwich:
                out[p + "norm2b"] = (W,)
            for name, shape in FEED_FORWARDS[l.mlp.kind].shapes(l.mlp, W).items():
                out[p + "mlp." + name] = shape
    return out


class HybridEngine(B200Engine):

    def __init__(self, config: Any, tensors: Dict[str, torch.Tensor], *, dtype: torch.dtype = torch.bfloat16,
                 device: Any = "cuda", use_cuda_graph: bool = True):
        """`tensors`: checkpoint names → tensors (any float dtype, any device); they are cast to `dtype` and moved."""
        self.config = config
        self.dtype = dtype
        SK.dtype_code(dtype)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("HybridEngine needs a CUDA device (there is no CPU path for this family)")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        _lib.lib()
        self.tp, self.rank, self.comm = 1, 0, None
        self.use_cuda_graph = use_cuda_graph
        self.use_megakernel = False
        self.mega_write_logits = False
        self.mega_max_batch = 0
        self.eps = float(config.rms_norm_eps)
        self.norm_offset = float(config.norm_offset)          # 1: norm weights are stored around zero
        if config.block not in ("sandwich", "parallel", "parallel_shared"):
            raise ValueError(f"unknown block form {config.block!r}")
        self.parallel = config.block in ("parallel", "parallel_shared")
        self.shared_norm = config.block == "parallel_shared"      # one norm per block, read by both sublayers
        if self.parallel and self.norm_offset != 0.0:
            raise ValueError("parallel blocks take plain norm weights")
        present = {name: tuple(t.shape) for name, t in tensors.items()}
        rank = next((int(t.shape[0]) for name, t in tensors.items() if name.endswith("mix.a1")), 16)
        want = tensor_shapes(config, decay_rank=rank, present=present)
        missing = sorted(set(want) - set(tensors))
        if missing:
            raise ValueError(f"checkpoint lacks tensors: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
        for name, shape in want.items():
            if tuple(tensors[name].shape) != tuple(shape):
                raise ValueError(f"tensor {name}: shape {tuple(tensors[name].shape)}, config wants {tuple(shape)}")

        def get(name: str) -> torch.Tensor:
            return tensors[name].to(device=self.device, dtype=dtype).contiguous()

        self.embedding = get("embed")
        self.final_norm = get("final.norm")
        self.lm_head = self.embedding if config.tied_head else get("head")
        self.embed_norm = get("embed.norm") if config.embed_norm else None
        self.pair_table = get("bigram") if config.pair_embedding is not None else None
        self.pair_spec = config.pair_embedding
        self.pos_table = get("pos") if config.learned_positions else None
        self.side_table = get("side.embed") if config.token_side_dim else None
        if (self.pos_table is not None or self.side_table is not None) and (self.pair_table is not None or config.embed_norm):
            raise ValueError("learned positions and token inputs do not combine with a pair-hash or normed embedding")
        if self.side_table is not None and not self.parallel:
            raise ValueError("per-layer token inputs go with parallel blocks")
        if self.pair_table is None and self.embed_norm is not None:
            # a normed embedding without a pair table runs the same kernel over a table of zeros
            from ..config import PairEmbeddingSpec
            self.pair_table = torch.zeros((2, config.hidden_size), dtype=dtype, device=self.device)
            self.pair_spec = PairEmbeddingSpec(buckets=1, mul_prev=0, mul_cur=0)
        self.v_local = config.vocab_size
        self.layers: List[HybridLayer] = []
        for i, l in enumerate(config.layers):
            p = f"l{i}."
            w = {k[len(p) + 4:]: get(k) for k in want if k.startswith(p + "mix.")}
            layer = HybridLayer(mixer=MIXERS[l.mixer.kind](l.mixer, w, self.eps), norm1=get(p + "norm1"))
            if not self.parallel:
                layer.norm1b = get(p + "norm1b")
            if l.mlp is not None:
                if not self.shared_norm:
                    layer.norm2 = get(p + "norm2")
                if not self.parallel:
                    layer.norm2b = get(p + "norm2b")
                fw = {k[len(p) + 4:]: get(k) for k in want if k.startswith(p + "mlp.")}
                try:
                    layer.ff = FEED_FORWARDS[l.mlp.kind](l.mlp, fw)
                except ValueError as e:
                    raise ValueError(f"layer {i}: {e}") from None
            if self.side_table is not None:
                sw = {k[len(p) + 5:]: get(k) for k in want if k.startswith(p + "side.")}
                layer.side = TokenSide(self.side_table, i * config.token_side_dim, sw)
            self.layers.append(layer)
        # layer runs: the layer of every step through the stack (a looped stretch appears `times` times); caches and states
        # are per run, weights per layer
        self.runs: List[int] = list(config.layer_runs())
        self._rope: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._decode_states: Dict[Tuple[int, int], DecodeState] = {}
        self._mega_gen = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._mega_fit_cache: Dict[int, bool] = {}
        self.capture_streams: Optional[List[torch.Tensor]] = None      # debugging: residual stream after every layer
        if dtype == torch.bfloat16:
            K.ensure_gemm_workspace(self.device)

    # ------------------------------------------------------------------ construction
    @classmethod
    def random_init(cls, config: Any, device: Any = "cuda", seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                    decay_rank: int = 16, **kw: Any) -> "HybridEngine":
        """Random weights in checkpoint layout, drawn on the device (benchmarks and tests)."""
        return cls(config, random_tensors(config, device, seed, decay_rank), dtype=dtype, device=device, **kw)

    def _mega_fits(self, batch: int) -> bool:
        return False

    def weight_bytes_per_step(self, rows: int = 1) -> int:
        """Bytes of weights a decode step of `rows` tokens streams (a mixture of experts: the experts it can touch)."""
        ws = [self.lm_head, self.final_norm] + [t for t in (self.embed_norm,) if t is not None]
        for l in (self.layers[i] for i in self.runs):
            ws += l.mixer.weights() + [t for t in (l.norm1, l.norm1b, l.norm2, l.norm2b) if t is not None]
            if l.side is not None:
                ws += l.side.weights()
            if l.ff is not None:
                ws += l.ff.streamed_weights(rows)
        return sum(t.numel() * t.element_size() for t in ws)

    # ------------------------------------------------------------------ rotary tables
    def _rope_for(self, rot: Any, length: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos / sin tables of a rotary spec (None: a one-row table that nothing reads), at least `length` positions."""
        if rot is None:
            key: Tuple = (2, 1.0, None)
        else:
            sc = rot.scaling
            key = (int(rot.dims), float(rot.base), None if sc is None else (sc.factor, sc.original, sc.fast, sc.slow))
        have = self._rope.get(key)
        if have is None or (rot is not None and have[0].shape[0] < length):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("rotary table too short for a captured step: size it before the capture")
            self._rope[key] = have = rotary_table(key[0], key[1], max(length, 256) if rot is not None else 1, self.device,
                                                  rot.scaling if rot is not None else None)
        return have

    def _ropes(self, mixer: Any, length: int) -> Tuple[torch.Tensor, ...]:
        """The tables a mixer's `forward` gets: cos / sin of its q / k rotation, then those of its value rotation if it has one."""
        rope = self._rope_for(getattr(mixer.spec, "rot", None), length)
        vrot = getattr(mixer, "value_rot", None)
        return rope if vrot is None else rope + self._rope_for(vrot, length)

    @property
    def position_limit(self) -> Optional[int]:
        """The most positions a sequence can have (a learned position table has that many rows), None when nothing bounds it."""
        return int(self.pos_table.shape[0]) if self.pos_table is not None else None

    def _check_max_length(self, max_length: int) -> None:
        # a sequence of max_length tokens feeds max_length - 1 of them to the model: the last one is only ever an output
        if self.pos_table is not None and max_length - 1 > self.pos_table.shape[0]:
            raise ValueError(f"max_length {max_length} exceeds the {self.pos_table.shape[0]} learned positions")
        for l in self.layers:
            if getattr(l.mixer.spec, "rot", None) is not None:
                self._ropes(l.mixer, max_length)

    # ------------------------------------------------------------------ cache
    def new_cache(self, batch: int, max_length: int) -> HybridCache:
        ks: List[Optional[torch.Tensor]] = []
        vs: List[Optional[torch.Tensor]] = []
        states: List[Optional[torch.Tensor]] = []
        for l in (self.layers[i] for i in self.runs):
            kv = l.mixer.new_cache(batch, max_length, self.device)
            ks.append(kv[0] if kv is not None else None)
            vs.append(kv[1] if kv is not None else None)
            states.append(l.mixer.new_state(batch, self.device))
        first = next(iter(_tensors(ks)), None)
        ident = first if first is not None else torch.zeros(1, dtype=self.dtype, device=self.device)
        self._check_max_length(max_length)
        prev = torch.zeros(batch, dtype=torch.int32, device=self.device) if self.pair_table is not None else None
        return HybridCache(k=ident, v=ident, index=0,
                           pad_left=torch.zeros(batch, dtype=torch.int32, device=self.device),
                           len_dev=torch.zeros(1, dtype=torch.int32, device=self.device),
                           ks=ks, vs=vs, states=states, length=int(max_length), prev_tok=prev)

    def _step_ids(self, ids: torch.Tensor, cache: Optional[HybridCache]) -> torch.Tensor:
        """The step's tokens as int32 [M]; kept with the cache for the layers that take the token itself as an input."""
        ids32 = ids if ids.dtype == torch.int32 and ids.is_contiguous() else ids.to(torch.int32).contiguous()
        ids32 = ids32.view(-1)
        if cache is not None:
            cache.step_ids = ids32
        return ids32

    # ------------------------------------------------------------------ layer stack
    def _embed(self, ids: torch.Tensor, out: Optional[torch.Tensor] = None, cache: Optional[HybridCache] = None,
               B: int = 0, S: int = 0) -> torch.Tensor:
        if self.pair_table is not None:
            pe = self.pair_spec
            if cache is None or cache.prev_tok is None:
                raise ValueError("an embedding that hashes token pairs needs the cache of the request batch")
            return SK.embed_pair_norm(ids, self.embedding, self.pair_table, self.embed_norm, cache.prev_tok, cache.len_dev,
                                      cache.pad_left, B, S, pe.buckets, pe.mul_prev, pe.mul_cur, self.eps, out=out)
        if self.pos_table is not None or self.side_table is not None:
            if cache is None:
                raise ValueError("learned positions and token inputs need the cache of the request batch")
            ids = self._step_ids(ids, cache)
        if self.pos_table is not None:
            return SK.embed_pos(ids, self.embedding, self.pos_table, cache.len_dev, cache.pad_left, B, S, out=out)
        return SK.embed_f32(ids, self.embedding, out=out)

    def _head(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        c = self.config
        h = SK.norm_f32(x, self.final_norm, self.eps, self.norm_offset)
        if c.logit_scale == 1.0 and c.logit_softcap == 0.0:
            return SK.linear(h, self.lm_head, out=out)
        return SK.linear(h, self.lm_head, act=SK.ACT_SCALE_SOFTCAP, p0=c.logit_scale, p1=c.logit_softcap, out=out)

    def _layers(self, x: torch.Tensor, B: int, S: int, cache: HybridCache, positions: Optional[torch.Tensor],
                ws: Optional[DecodeState] = None) -> torch.Tensor:
        """x fp32 [B·S, width], updated in place through all layers.  Appends S slots at cache.len_dev and advances
        the recurrent states by the S tokens (padding tokens excluded); does not advance the fill level."""
        if positions is not None:
            raise NotImplementedError("explicit position_ids are not supported by the hybrid engine (left padding is)")
        if self.parallel:
            return self._layers_parallel(x, B, S, cache)
        eps, off = self.eps, self.norm_offset
        stack = [self.layers[i] for i in self.runs]
        n = len(stack)
        h = SK.norm_f32(x, stack[0].norm1, eps, off)
        for i, l in enumerate(stack):                    # i: the run, which is also the index of its cache entries
            rope = self._ropes(l.mixer, cache.capacity)
            z = l.mixer.forward(h, B, S, cache, i, rope)
            nxt = l.norm2 if l.ff is not None else (stack[i + 1].norm1 if i + 1 < n else None)
            h = SK.postnorm_add(z, l.norm1b, x, eps, off, w_next=nxt)
            if l.ff is not None:
                z = l.ff.run(h)
                nxt = stack[i + 1].norm1 if i + 1 < n else None
                h = SK.postnorm_add(z, l.norm2b, x, eps, off, w_next=nxt)
            if self.capture_streams is not None:
                self.capture_streams.append(x.clone())
        return x

    def _layers_parallel(self, x: torch.Tensor, B: int, S: int, cache: HybridCache) -> torch.Tensor:
        """Parallel blocks: x += m · (mixer(norm1 x) + ff(norm2 x)).  One kernel per layer adds both branches to the
        stream and forms the two norms the next layer reads.

        With at most `BRANCH_OVERLAP_ROWS` rows (decoding) the two branches of a layer run on two streams: neither
        fills the GPU alone and a step is a chain of short dependent kernels, so the feed-forward's chain hides behind
        the mixer's.  Inside a graph capture the fork and join become edges of the captured graph.  Wider steps stay on
        one stream (their tensor-core GEMMs share one split-K workspace)."""
        eps, mult = self.eps, float(self.config.residual_mult)
        stack = [self.layers[i] for i in self.runs]
        n = len(stack)
        overlap = B * S <= BRANCH_OVERLAP_ROWS
        main = torch.cuda.current_stream()
        first = stack[0]
        h1, h2 = SK.branch_add_norm(x, None, None, mult, first.norm1, first.norm2 if first.ff is not None else None, eps)
        for i, l in enumerate(stack):                    # i: the run, which is also the index of its cache entries
            if self.shared_norm:
                h2 = h1
            rope = self._ropes(l.mixer, cache.capacity)
            y2 = None
            forked = overlap and l.ff is not None
            if forked:
                side, fork, join = self._branch_sync(i)
                fork.record(main)
                side.wait_event(fork)                      # h2 is ready
                with torch.cuda.stream(side):
                    y2 = l.ff.run(h2)
                    join.record(side)
            y1 = l.mixer.forward(h1, B, S, cache, i, rope)
            if forked:
                main.wait_event(join)
            elif l.ff is not None:
                y2 = l.ff.run(h2)
            nxt = stack[i + 1] if i + 1 < n else None
            w1 = nxt.norm1 if nxt is not None else None
            w2 = nxt.norm2 if nxt is not None and nxt.ff is not None else None
            if l.side is None:
                h1, h2 = SK.branch_add_norm(x, y1, y2, mult, w1, w2, eps)
            else:
                # the token input reads the stream after both branches were added, and forms the next block's norm itself
                xc = None
                if l.side.wants_cast(B * S):
                    xc = SK.branch_add_cast(x, y1, y2, mult, self.dtype)
                else:
                    SK.branch_add_norm(x, y1, y2, mult, None, None, eps)
                h1 = l.side.run(x, cache.step_ids, w1 if self.shared_norm else None, eps, x_cast=xc)
                if not self.shared_norm and nxt is not None:
                    h1, h2 = SK.branch_add_norm(x, None, None, mult, w1, w2, eps)
            if self.capture_streams is not None:
                self.capture_streams.append(x.clone())
        return x

    def _branch_sync(self, layer: int) -> Tuple[Any, Any, Any]:
        """The second stream and the layer's fork / join events (made once; events without timing can be captured)."""
        if getattr(self, "_branch_stream", None) is None:
            self._branch_stream = torch.cuda.Stream(device=self.device)
            self._branch_events: Dict[int, Tuple[Any, Any]] = {}
        if layer not in self._branch_events:
            self._branch_events[layer] = (torch.cuda.Event(), torch.cuda.Event())
        return (self._branch_stream, *self._branch_events[layer])

    # ------------------------------------------------------------------ decode state
    def _decode_state(self, B: int, max_len: int) -> DecodeState:
        key = (B, max_len)
        if key in self._decode_states:
            return self._decode_states[key]
        c, dev = self.config, self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self._check_max_length(max_len)
        empty = torch.zeros(1, dtype=self.dtype, device=dev)
        st = DecodeState(
            B=B, max_len=max_len, ids=torch.zeros(B, **i32),
            x=torch.zeros(B, c.hidden_size, dtype=torch.float32, device=dev), qkv=empty, attn=empty, mlp=empty,
            logits=torch.zeros(B, c.vocab_size, dtype=torch.float32, device=dev), tok=torch.zeros(B, **i32),
            finished=torch.zeros(B, **i32), sequences=torch.zeros(B, max_len, **i32),
            cur_len=torch.zeros(1, **i32), step=torch.zeros(1, **i32), n_unfinished=torch.zeros(1, **i32),
            splits=1, scratch=None)
        self._decode_states[key] = st
        return st


def random_tensors(config: Any, device: Any = "cuda", seed: int = 0, decay_rank: int = 16) -> Dict[str, torch.Tensor]:
    """Random bfloat16 weights under checkpoint names: projections ~ N(0, 1/fan_in), norm weights small around zero
    (the head norm around one), decay biases spread so that fast and slow channels both occur."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}

    def randn(shape: Tuple[int, ...]) -> torch.Tensor:
        return torch.randn(shape, generator=g, device=dev, dtype=torch.float32)

    for name, shape in tensor_shapes(config, decay_rank).items():
        if name.endswith("mix.norm") or (config.norm_offset == 0.0 and len(shape) == 1 and "norm" in name):
            t = 1.0 + 0.1 * randn(shape)
        elif name.endswith("mix.a2.b"):
            t = 2.0 + 2.0 * randn(shape)
        elif len(shape) == 1:
            t = 0.1 * randn(shape)
        elif name == "embed":
            t = randn(shape)
        else:
            t = randn(shape) / (shape[1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out
