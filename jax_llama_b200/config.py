"""Model configuration.

`LLaMAConfig` keeps the field names, defaults and JSON schema of the reference's HF-style config
(/root/reference/jax_llama/config.py:72-116) but is a free-standing class: it does not depend on
`transformers`, so it loads in every process of a torchrun job without importing HF.

`ModelArgs` / `config_from_params` mirror Meta's ``params.json`` schema and the SwiGLU width formula
(/root/reference/jax_llama/convert_weights.py:13-50).  Unlike the reference, unknown ``params.json``
keys (e.g. LLaMA-3.1's ``use_scaled_rope``) are tolerated and reported instead of raising.
"""
from __future__ import annotations

import copy
import dataclasses
import json
import logging
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

logger = logging.getLogger(__name__)

CONFIG_NAME = "config.json"


class LLaMAConfig:
    """LLaMA-1/2/3 architecture description (same keys as the reference's config.json)."""

    model_type = "llama"

    def __init__(
        self,
        vocab_size: int = 32000,
        hidden_size: int = 4096,
        intermediate_size: int = 11008,
        num_hidden_layers: int = 32,
        num_attention_heads: int = 32,
        num_key_value_heads: Optional[int] = None,
        max_sequence_length: int = 2048,
        rms_norm_eps: float = 1e-6,
        initializer_range: float = 0.02,
        use_cache: bool = True,
        pad_token_id: int = -1,
        bos_token_id: int = 1,
        eos_token_id: int = 2,
        resid_pdrop: float = 0.0,
        embd_pdrop: float = 0.0,
        attn_pdrop: float = 0.0,
        tie_word_embeddings: bool = False,
        gradient_checkpointing: bool = False,
        rope_theta: float = 10000.0,
        **kwargs: Any,
    ):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.num_hidden_layers = int(num_hidden_layers)
        self.num_attention_heads = int(num_attention_heads)
        if num_key_value_heads is None:
            num_key_value_heads = num_attention_heads
        self.num_key_value_heads = int(num_key_value_heads)
        self.max_sequence_length = int(max_sequence_length)
        self.rms_norm_eps = float(rms_norm_eps)
        self.initializer_range = float(initializer_range)
        self.use_cache = bool(use_cache)
        self.pad_token_id = pad_token_id
        self.bos_token_id = bos_token_id
        self.eos_token_id = eos_token_id
        self.resid_pdrop = float(resid_pdrop)
        self.embd_pdrop = float(embd_pdrop)
        self.attn_pdrop = float(attn_pdrop)
        self.tie_word_embeddings = bool(tie_word_embeddings)
        # accepted for schema parity; inference-only framework ignores it (SURVEY §2.4 "remat")
        self.gradient_checkpointing = bool(gradient_checkpointing)
        self.rope_theta = float(rope_theta)
        kwargs.pop("model_type", None)
        # unknown keys are preserved so a config.json written by HF round-trips
        self.extra: Dict[str, Any] = dict(kwargs)
        self.validate()

    # ------------------------------------------------------------------ derived
    @property
    def head_dim(self) -> int:
        """hidden_size // num_attention_heads as in the reference (model.py:115), unless the config carries an
        explicit ``head_dim`` key (newer HF Llama configs do): then q/o project to ``num_attention_heads * head_dim``
        columns, which need not equal hidden_size — e.g. the per-rank slice of a tensor-parallel model as a model."""
        hd = self.extra.get("head_dim") if hasattr(self, "extra") else None
        return int(hd) if hd else self.hidden_size // self.num_attention_heads

    @property
    def n_rep(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def validate(self) -> None:
        if not self.extra.get("head_dim") and self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for rotary embeddings")

    def num_params(self) -> int:
        h, f, v, l = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        kv = self.num_key_value_heads * self.head_dim
        per_layer = h * self.num_attention_heads * self.head_dim * 2 + 2 * h * kv + 3 * h * f + 2 * h
        head = 0 if self.tie_word_embeddings else v * h
        return v * h + l * per_layer + h + head

    # ------------------------------------------------------------------ (de)serialisation
    def to_dict(self) -> Dict[str, Any]:
        d = {k: copy.deepcopy(v) for k, v in self.__dict__.items() if k != "extra"}
        d.update(copy.deepcopy(self.extra))
        d["model_type"] = self.model_type
        return d

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LLaMAConfig":
        return cls(**dict(d))

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def to_json_file(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_json_string())

    @classmethod
    def from_json_file(cls, path: str) -> "LLaMAConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def save_pretrained(self, save_directory: str) -> None:
        os.makedirs(save_directory, exist_ok=True)
        self.to_json_file(os.path.join(save_directory, CONFIG_NAME))

    @classmethod
    def from_pretrained(cls, path: str, **overrides: Any) -> "LLaMAConfig":
        if os.path.isdir(path):
            path = os.path.join(path, CONFIG_NAME)
        cfg = cls.from_json_file(path)
        for k, v in overrides.items():
            setattr(cfg, k, v)
        cfg.validate()
        return cfg

    def __eq__(self, other: object) -> bool:
        return isinstance(other, LLaMAConfig) and self.to_dict() == other.to_dict()

    def __repr__(self) -> str:
        return f"LLaMAConfig {self.to_json_string()}"


@dataclass
class ModelArgs:
    """Meta ``params.json`` schema (/root/reference/jax_llama/convert_weights.py:13-26)."""

    dim: int = 512
    n_layers: int = 8
    n_heads: int = 8
    n_kv_heads: Optional[int] = None
    vocab_size: int = -1
    multiple_of: int = 256
    ffn_dim_multiplier: Optional[float] = None
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_batch_size: int = 32
    max_seq_len: int = 2048

    @classmethod
    def from_params_json(cls, params: Dict[str, Any]) -> "ModelArgs":
        known = {f.name for f in dataclasses.fields(cls)}
        unknown = sorted(set(params) - known)
        if unknown:
            logger.warning("params.json keys ignored (not part of the LLaMA-1/2/3 schema): %s", unknown)
        return cls(**{k: v for k, v in params.items() if k in known})


def swiglu_intermediate_size(dim: int, ffn_dim_multiplier: Optional[float], multiple_of: int) -> int:
    """Meta's FFN width rule: 2/3·4·dim, optional multiplier, rounded up to `multiple_of`."""
    width = int(2 * (dim * 4) / 3)
    if ffn_dim_multiplier is not None:
        width = int(ffn_dim_multiplier * width)
    return multiple_of * ((width + multiple_of - 1) // multiple_of)


def config_from_params(args: ModelArgs) -> LLaMAConfig:
    return LLaMAConfig(
        vocab_size=args.vocab_size,
        hidden_size=args.dim,
        intermediate_size=swiglu_intermediate_size(args.dim, args.ffn_dim_multiplier, args.multiple_of),
        num_hidden_layers=args.n_layers,
        num_attention_heads=args.n_heads,
        num_key_value_heads=args.n_kv_heads,
        max_sequence_length=args.max_seq_len,
        rms_norm_eps=args.norm_eps,
        rope_theta=args.rope_theta,
    )


# Architecture presets for the configurations BASELINE.json names (random-init benchmarking).
PRESETS: Dict[str, Dict[str, Any]] = {
    "tiny": dict(vocab_size=32000, hidden_size=256, intermediate_size=768, num_hidden_layers=2,
                 num_attention_heads=4, num_key_value_heads=4, rms_norm_eps=1e-5),
    "tiny-gqa": dict(vocab_size=1024, hidden_size=512, intermediate_size=1536, num_hidden_layers=2,
                     num_attention_heads=8, num_key_value_heads=2, rms_norm_eps=1e-5),
    "llama1-7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                      num_attention_heads=32, rms_norm_eps=1e-6),
    "llama2-7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                      num_attention_heads=32, rms_norm_eps=1e-5, max_sequence_length=4096),
    "llama2-13b": dict(vocab_size=32000, hidden_size=5120, intermediate_size=13824, num_hidden_layers=40,
                       num_attention_heads=40, rms_norm_eps=1e-5, max_sequence_length=4096),
    "llama1-33b": dict(vocab_size=32000, hidden_size=6656, intermediate_size=17920, num_hidden_layers=60,
                       num_attention_heads=52, rms_norm_eps=1e-6),
    "llama1-65b": dict(vocab_size=32000, hidden_size=8192, intermediate_size=22016, num_hidden_layers=80,
                       num_attention_heads=64, rms_norm_eps=1e-5),
    "llama2-70b": dict(vocab_size=32000, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                       num_attention_heads=64, num_key_value_heads=8, rms_norm_eps=1e-5,
                       max_sequence_length=4096),
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5,
                      rope_theta=500000.0, max_sequence_length=8192, bos_token_id=128000,
                      eos_token_id=128001),
    # 1B-class LLaMA-architecture shape with 64-wide heads and tied embeddings (the architecture of Llama-3.2-1B; its
    # "llama3" RoPE frequency scaling is not applied — the reference has no RoPE scaling either)
    "llama3.2-1b": dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                        num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                        max_sequence_length=8192, bos_token_id=128000, eos_token_id=128001,
                        tie_word_embeddings=True),
    "llama3-70b": dict(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                       num_attention_heads=64, num_key_value_heads=8, rms_norm_eps=1e-5,
                       rope_theta=500000.0, max_sequence_length=8192, bos_token_id=128000,
                       eos_token_id=128001),
}


def preset(name: str, **overrides: Any) -> LLaMAConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; choose from {sorted(PRESETS)}")
    kw = dict(PRESETS[name])
    kw.update(overrides)
    return LLaMAConfig(**kw)


# --------------------------------------------------------------------------- hybrid decoder family
@dataclass
class RotaryScaling:
    """Frequency interpolation for contexts longer than `original` positions: channels that make fewer than `slow`
    turns over `original` positions are slowed by `factor`, channels that make more than `fast` turns are kept, with a
    linear ramp over the channel index in between; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass
class RotarySpec:
    """Rotary embedding on the first `dims` channels of each head, frequencies base^(-2i/dims).  layout "interleaved"
    pairs channel 2i with 2i+1, "half" pairs channel i with i + dims/2."""
    dims: int
    base: float
    layout: str = "interleaved"
    scaling: Optional[RotaryScaling] = None

    @staticmethod
    def parse(rot: Optional[Dict[str, Any]], layout: str = "interleaved") -> Optional["RotarySpec"]:
        if not rot:
            return None
        sc = rot.get("scaling")
        scaling = None
        if sc:
            scaling = RotaryScaling(factor=float(sc["factor"]), original=float(sc["original"]), fast=float(sc["fast"]),
                                    slow=float(sc["slow"]))
        return RotarySpec(int(rot["dims"]), float(rot["base"]), layout, scaling)


@dataclass
class AttentionMixerSpec:
    """Softmax attention mixer.  `kv_from` names the layer whose cached keys / values this layer reads instead of
    projecting its own.  qk_unit_norm: weight-free unit-RMS scaling of q and k per head after the rotation;
    head_gate: one sigmoid gate per head on the output."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotarySpec] = None
    kv_from: Optional[int] = None
    qk_unit_norm: bool = True
    head_gate: bool = True
    bias: bool = False              # q / k / v projections have biases (`<name>.b`)
    v_unit_norm: bool = False       # every head's value scaled to unit RMS (no weight) before it is cached
    window: int = 0                 # > 0: a query sees itself and the window - 1 tokens before it
    sink: bool = False              # one more unit in the softmax denominator: a key with score 0 that carries no value
    talking_heads: bool = False     # the heads' weights are mixed by `talk` [heads, heads] after the softmax
    qk_norm: bool = False           # RMS norm of every q / k head with the weights `q.norm` / `k.norm` [dim] BEFORE the rotation
    chunk: int = 0                  # > 0: positions form blocks of `chunk`; a query sees the keys of its own block only
    sink_learned: bool = False      # the sink's logit is `sink` [heads] instead of 0 (needs sink)
    v_rot: bool = False             # values are rotated at their own position over all vdim channels (frequencies rot.base^(-2m/vdim),
                                    # the pairing of rot.layout, no interpolation), every head's sum is rotated back at the query's
    kind: str = "attention"


@dataclass
class GlaMixerSpec:
    """Gated linear attention mixer: per-head matrix state [dim x vdim], per-key-channel decay sigmoid(z)^(1/tau)."""
    heads: int
    dim: int
    vdim: int
    tau: float
    kind: str = "gla"


@dataclass
class LatentAttentionMixerSpec:
    """Softmax attention through low-rank latents: queries from a normed latent of size q_rank, keys and values from a
    normed latent of size kv_rank (what the layer caches, with one rotated key part of rot_dim channels shared by the
    heads).  A head's query / key is `dim` unrotated channels followed by `rot_dim` rotated ones; `window` > 0 limits a
    query to the last `window` positions up to its own."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Optional[RotarySpec] = None
    window: int = 0
    kind: str = "latent_attention"


@dataclass
class RetentionMixerSpec:
    """Linear attention with one fixed decay per head: S_t = decay_h S_(t-1) + k_t v_tᵀ, o_t = S_tᵀ q_t, no softmax and
    no denominator; rotary q / k, k scaled by dim^(-1/2); read-out divided by its RMS per head, gated by silu."""
    heads: int
    dim: int
    vdim: int
    decay: List[float] = field(default_factory=list)
    rot: Optional[RotarySpec] = None
    kind: str = "retention"


@dataclass
class StateSpaceMixerSpec:
    """Selective state space layer (state space duality form): per head a state [state x vdim] with one scalar decay per
    token, S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_tᵀ, y_t = S_tᵀ C_t + D x_t; B and C shared by the heads of a
    group; x, B, C through a causal convolution of `conv` taps and silu; the read-out gated by silu(z), then RMS-normed in
    `norm_groups` equal parts."""
    heads: int
    vdim: int
    state: int
    groups: int = 1
    conv: int = 4
    norm_groups: int = 1
    kind: str = "state_space"


@dataclass
class DeltaMixerSpec:
    """Gated delta rule with one decay per key channel: S <- diag(a) S; e = beta (v - Sᵀk); S <- S + k eᵀ; o = Sᵀq.
    q / k heads (kv_heads of `dim`) shared by groups of value heads, each of q, k, v through a causal convolution of
    `conv` taps and silu, q and k scaled to unit length; read-out normed per head and gated by a low-rank sigmoid gate."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int = 4
    kind: str = "channel_delta"


@dataclass
class ParallelMixerSpec:
    """Two mixers side by side on the same input; each result is RMS-normed over the model width with its own weight and
    the mixer returns `scale` times their sum."""
    left: Any
    right: Any
    scale: float = 0.5
    kind: str = "parallel"


@dataclass
class PairEmbeddingSpec:
    """A second embedding table indexed by a hash of (previous token, token): row (prev * mul_prev + tok * mul_cur) mod
    buckets, and row `buckets` for a sequence's first token."""
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass
class DenseMlpSpec:
    """down(act(up h)), or with `gated` down(act(gate h) * (up h)).  act "xielu": z > 0: softplus(p) z^2 + z/2, else
    (1/2 + softplus(q)) (e^z - 1 - z) + z/2, with the layer's own (p, q) in the tensor `act`."""
    ff: int
    act: str = "relu2"
    gated: bool = False
    kind: str = "dense"


@dataclass
class MoeMlpSpec:
    """Mixture of experts: `experts` feed-forward layers of inner size `ff`, `top` per token.  groups > 1: the experts
    form equal groups of neighbours, a group scores the sum of its `group_top` largest choice scores and only the `keep` best
    groups can be chosen.  Weights = chosen scores over their sum, times `scale`.  shared_ff > 0: one more expert runs
    for every token, times a per-token sigmoid gate when shared_gate."""
    experts: int
    top: int
    ff: int
    act: str = "relu2"
    score: str = "sigmoid"
    groups: int = 1
    keep: int = 1
    group_top: int = 2
    scale: float = 1.0
    normalise: bool = True
    shared_ff: int = 0
    shared_gate: bool = True
    gated: bool = False             # experts with a gate projection: act "glu_clamped" is min(g, limit) sigmoid(1.702 ·) (clamp(u) + 1)
    limit: float = 0.0
    shared_limit: float = 0.0
    router_bias: bool = False       # `router.b` is added to the router logits
    identity: int = 0               # router outputs beyond `experts` that stand for identity experts (output = input, no tensors);
                                    # groups are formed over experts + identity
    choice_bias: bool = False       # `correction` [experts + identity] is added to the scores for the choice only (group scores, top)
    kind: str = "moe"


@dataclass
class HybridLayerSpec:
    mixer: Any
    mlp: Optional[DenseMlpSpec]


class HybridConfig:
    """What the configurations of the hybrid decoder family share: the JSON schema of the checkpoint's ``config.json``
    (``architecture``, ``vocab``, ``width``, ``norm.eps`` and ``layers`` — a list of ``{"type", "mixer": {...},
    "mlp": {...} | null}``), parsing of the layer list into specs, and the checkpoint I/O.  A design states

    * ``block``: "sandwich" — mixer and feed-forward one after the other, each between a norm before and a norm after,
      x += norm(sublayer(norm(x))); "parallel" — both read norms of the same x, x += residual_mult · (mixer + ff);
      "parallel_shared" — the same with ONE norm that both sublayers read;
    * ``tied_head``: the logits are taken against the embedding table (no ``head`` tensor); ``embed_norm``: a norm
      (``embed.norm``) right after the embedding;
    * ``norm_offset``: what is added to a stored norm weight (1 for weights stored around zero);
    * which mixer types and feed-forward kinds it has (`_parse_mixer`, `_parse_mlp`)."""

    model_type = "hybrid"
    architecture = "Hybrid"
    block = "sandwich"
    norm_offset = 0.0
    default_eps = 1e-6
    tied_head = False
    embed_norm = False
    learned_positions = False

    def __init__(self, vocab: int, width: int, layers: Any, norm: Optional[Dict[str, Any]] = None,
                 logit_scale: float = 1.0, logit_softcap: Optional[float] = None, residual_mult: float = 1.0,
                 embedding: Optional[Dict[str, Any]] = None, loop: Optional[Dict[str, Any]] = None,
                 token_side: Optional[Dict[str, Any]] = None, max_positions: Optional[int] = None, **extra: Any):
        self.vocab_size = int(vocab)
        self.hidden_size = int(width)
        self.rms_norm_eps = float((norm or {}).get("eps", self.default_eps))
        self.logit_scale = float(logit_scale)
        self.logit_softcap = float(logit_softcap) if logit_softcap else 0.0
        self.residual_mult = float(residual_mult)
        self.embedding_dict = copy.deepcopy(embedding) if embedding else None
        bg = (embedding or {}).get("bigram")
        self.pair_embedding = PairEmbeddingSpec(int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])) if bg else None
        # layers [start, stop) run `times` times in a row with the same weights (every pass has its own cache and state)
        self.loop = {k: int(loop[k]) for k in ("start", "stop", "times")} if loop else None
        # per-layer token input: a second embedding table holds `dim` numbers per layer and token
        self.token_side_dim = int(token_side["dim"]) if token_side else 0
        # learned position rows added to the token embedding (designs with `learned_positions`)
        self.max_positions = int(max_positions) if max_positions else 0
        self.layer_dicts = copy.deepcopy(list(layers))
        self.layers = [HybridLayerSpec(mixer=self._parse_mixer(i, d), mlp=self._parse_mlp(i, d.get("mlp")))
                       for i, d in enumerate(self.layer_dicts)]
        self.extra = {k: v for k, v in extra.items() if k != "architecture"}
        # generation defaults the front-end reads from every config
        self.pad_token_id, self.bos_token_id, self.eos_token_id = 0, -1, -1
        self.validate()

    # ------------------------------------------------------------------ what a design defines
    def _parse_mixer(self, i: int, d: Dict[str, Any]) -> Any:
        raise NotImplementedError

    def _parse_mlp(self, i: int, mlp: Optional[Dict[str, Any]]) -> Any:
        raise NotImplementedError

    def _validate_layer(self, i: int, l: "HybridLayerSpec") -> None:
        pass

    def _own_keys(self) -> Dict[str, Any]:
        return {}

    # ------------------------------------------------------------------ shared
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def layer_runs(self) -> List[int]:
        """The layer index of every layer run, in execution order (without a loop: every layer once)."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * t + list(range(b, n))

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.layers:
            raise ValueError("vocab, width and layers must be non-empty")
        if self.loop and not (0 <= self.loop["start"] <= self.loop["stop"] <= len(self.layers) and self.loop["times"] >= 1):
            raise ValueError(f"loop {self.loop} does not fit {len(self.layers)} layers")
        if self.token_side_dim < 0 or self.max_positions < 0 or (self.learned_positions and self.max_positions <= 0):
            raise ValueError("token_side.dim and max_positions must be positive where the design has them")
        for i, l in enumerate(self.layers):
            self._validate_layer(i, l)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.rms_norm_eps}, "layers": copy.deepcopy(self.layer_dicts)}
        if self.embedding_dict:
            d["embedding"] = copy.deepcopy(self.embedding_dict)
        if self.loop:
            d["loop"] = dict(self.loop)
        if self.token_side_dim:
            d["token_side"] = {"dim": self.token_side_dim}
        if self.max_positions:
            d["max_positions"] = self.max_positions
        d.update(self._own_keys())
        d.update(self.extra)
        return d

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "HybridConfig":
        return cls(**d)

    @classmethod
    def from_json_file(cls, path: str) -> "HybridConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    @classmethod
    def from_pretrained(cls, path: str) -> "HybridConfig":
        return cls.from_json_file(os.path.join(path, CONFIG_NAME) if os.path.isdir(path) else path)

    def save_pretrained(self, save_directory: str) -> None:
        os.makedirs(save_directory, exist_ok=True)
        with open(os.path.join(save_directory, CONFIG_NAME), "w") as f:
            json.dump(self.to_dict(), f, indent=1, sort_keys=True)

    def __repr__(self) -> str:
        return f"{type(self).__name__} {json.dumps(self.to_dict(), sort_keys=True)}"


class FoliraxConfig(HybridConfig):
    """Folirax: a decoder whose layers mix gated linear attention and softmax attention (rotary on part of each head,
    unit-norm q / k, per-head output gates, layers that share another layer's keys and values), every sublayer wrapped
    in a zero-centred RMS norm before and after, squared-ReLU feed-forward, scaled and soft-capped logits.

    Besides the shared keys its ``config.json`` has ``logit_scale`` and ``logit_softcap``.
    """

    model_type = "folirax"
    architecture = "Folirax"
    block = "sandwich"
    norm_offset = 1.0

    def _parse_mixer(self, i: int, d: Dict[str, Any]) -> Any:
        m = d["mixer"]
        kind = d["type"]
        if kind == "gla":
            return GlaMixerSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), tau=float(m["tau"]))
        if kind == "attention":
            return AttentionMixerSpec(
                heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
                scale=float(m["scale"]), rot=RotarySpec.parse(m.get("rot")),
                kv_from=None if m.get("kv_from") is None else int(m["kv_from"]))
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")

    def _parse_mlp(self, i: int, mlp: Optional[Dict[str, Any]]) -> Any:
        if mlp is None:
            return None
        if mlp.get("kind", "dense") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        return DenseMlpSpec(ff=int(mlp["ff"]), act=str(mlp.get("act", "relu2")))

    def _validate_layer(self, i: int, l: HybridLayerSpec) -> None:
        m = l.mixer
        if m.kind == "attention":
            if m.heads % m.kv_heads:
                raise ValueError(f"layer {i}: heads {m.heads} not a multiple of kv_heads {m.kv_heads}")
            if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                raise ValueError(f"layer {i}: rot.dims {m.rot.dims} must be even and at most dim {m.dim}")
            if m.kv_from is not None:
                if not 0 <= m.kv_from < i:
                    raise ValueError(f"layer {i}: kv_from {m.kv_from} must name an earlier layer")
                src = self.layers[m.kv_from].mixer
                if src.kind != "attention" or src.kv_from is not None:
                    raise ValueError(f"layer {i}: kv_from {m.kv_from} is not an attention layer with its own keys")
                if (src.kv_heads, src.dim, src.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ValueError(f"layer {i}: key / value sizes differ from layer {m.kv_from}")
        elif m.tau <= 0:
            raise ValueError(f"layer {i}: tau must be positive")

    def _own_keys(self) -> Dict[str, Any]:
        return {"logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap}


class NikonexConfig(HybridConfig):
    """Nikonex: a decoder of parallel blocks — mixer and feed-forward read two norms of the same residual stream and
    their sum, times ``residual_mult``, is added to it.  Mixers: attention through low-rank latents with a shared
    rotated key part, frequency-interpolated rotary embedding and a sliding window ("latent_attention"), and linear
    attention with a fixed decay per head ("retention").  Feed-forward: a mixture of squared-ReLU experts with sigmoid
    scores, group-limited choice and a gated shared expert.  Plain norm weights, plain logits."""

    model_type = "nikonex"
    architecture = "Nikonex"
    block = "parallel"
    norm_offset = 0.0

    def _parse_mixer(self, i: int, d: Dict[str, Any]) -> Any:
        m = d["mixer"]
        kind = d["type"]
        if kind == "latent_attention":
            return LatentAttentionMixerSpec(
                heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                rot=RotarySpec.parse(m.get("rot"), "interleaved"), window=int((m.get("mask") or {}).get("size") or 0))
        if kind == "retention":
            return RetentionMixerSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                      decay=[float(a) for a in m["decay"]], rot=RotarySpec.parse(m.get("rot"), "half"))
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")

    def _parse_mlp(self, i: int, mlp: Optional[Dict[str, Any]]) -> Any:
        if mlp is None:
            return None
        if mlp.get("kind", "moe") != "moe":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        r = mlp["router"]
        g = r.get("groups") or {}
        shared = mlp.get("shared") or {}
        return MoeMlpSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]), act="relu2",
                          score="sigmoid", groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))),
                          group_top=2, scale=float(r.get("scale", 1.0)), normalise=True,
                          shared_ff=int(shared.get("ff", 0)), shared_gate=True)

    def _validate_layer(self, i: int, l: HybridLayerSpec) -> None:
        m = l.mixer
        if m.kind == "latent_attention":
            if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.rot_dim):
                raise ValueError(f"layer {i}: rot.dims {m.rot.dims} must be even and at most rot_dim {m.rot_dim}")
            if m.rot_dim > 0 and m.rot is None:
                raise ValueError(f"layer {i}: rot_dim {m.rot_dim} without rot")
            if min(m.heads, m.dim + m.rot_dim, m.vdim, m.q_rank, m.kv_rank) <= 0 or m.window < 0:
                raise ValueError(f"layer {i}: sizes must be positive")
        else:
            if len(m.decay) != m.heads:
                raise ValueError(f"layer {i}: {len(m.decay)} decays for {m.heads} heads")
            if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                raise ValueError(f"layer {i}: rot.dims {m.rot.dims} must be even and at most dim {m.dim}")
        f = l.mlp
        if f is not None:
            if not 1 <= f.top <= f.experts:
                raise ValueError(f"layer {i}: top {f.top} of {f.experts} experts")
            if f.groups > 1 and (f.experts % f.groups or not 1 <= f.keep <= f.groups
                                 or f.keep * (f.experts // f.groups) < f.top):
                raise ValueError(f"layer {i}: {f.groups} groups (keep {f.keep}) cannot give {f.top} of {f.experts} experts")

    def _own_keys(self) -> Dict[str, Any]:
        return {"residual_mult": self.residual_mult}


class BazulornConfig(HybridConfig):
    """Bazulorn: a decoder of parallel blocks with ONE norm per block — ``x += mixer(norm1 x) + ff(norm1 x)`` — whose token
    embedding adds a row of a hashed (previous token, token) table and is normed, and whose logits are taken against the
    embedding table.  Mixers: "parallel" — softmax attention (q / k / v biases, no rotation, unit-RMS values, sliding window,
    a sink in the softmax denominator, weights mixed across heads) beside a selective state space layer, each result normed
    over the model width, half their sum — and "channel_delta", a gated delta rule with one decay per key channel.
    Feed-forward: a gated tanh-gelu layer or a mixture of clamped gated experts (biased router, softmax over the chosen
    logits) plus a shared expert.

    ``config.json``: ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram.{buckets, mul_prev, mul_cur}`` and ``layers[i]`` =
    ``{type, mixer, mlp}`` with, for "parallel", ``mixer.left.{heads, kv_heads, dim, vdim, scale, mask.size}`` and
    ``mixer.right.{heads, vdim, state, groups, conv, norm_groups}``; for "channel_delta", ``mixer.{heads, kv_heads, dim, vdim,
    conv}``; ``mlp`` null, ``{kind: dense, ff}`` or ``{kind: moe, router.{experts, top}, expert.{ff, limit}, shared.{ff, limit}}``."""

    model_type = "bazulorn"
    architecture = "Bazulorn"
    block = "parallel_shared"
    norm_offset = 0.0
    tied_head = True
    embed_norm = True

    def _parse_mixer(self, i: int, d: Dict[str, Any]) -> Any:
        m = d["mixer"]
        kind = d["type"]
        if kind == "parallel":
            a, r = m["left"], m["right"]
            left = AttentionMixerSpec(
                heads=int(a["heads"]), kv_heads=int(a.get("kv_heads", a["heads"])), dim=int(a["dim"]), vdim=int(a["vdim"]),
                scale=float(a["scale"]), rot=None, kv_from=None, qk_unit_norm=False, head_gate=False, bias=True,
                v_unit_norm=True, window=int((a.get("mask") or {}).get("size") or 0), sink=True, talking_heads=True)
            right = StateSpaceMixerSpec(heads=int(r["heads"]), vdim=int(r["vdim"]), state=int(r["state"]),
                                        groups=int(r.get("groups", 1)), conv=int(r["conv"]),
                                        norm_groups=int(r.get("norm_groups", 1)))
            return ParallelMixerSpec(left=left, right=right, scale=0.5)
        if kind == "channel_delta":
            return DeltaMixerSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                  vdim=int(m["vdim"]), conv=int(m["conv"]))
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")

    def _parse_mlp(self, i: int, mlp: Optional[Dict[str, Any]]) -> Any:
        if mlp is None:
            return None
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            return DenseMlpSpec(ff=int(mlp["ff"]), act="gelu_tanh", gated=True)
        if kind == "moe":
            r = mlp["router"]
            shared = mlp.get("shared") or {}
            return MoeMlpSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]), act="glu_clamped",
                              score="softmax", groups=1, keep=1, scale=1.0, normalise=True, shared_ff=int(shared.get("ff", 0)),
                              shared_gate=False, gated=True, limit=float(mlp["expert"]["limit"]),
                              shared_limit=float(shared.get("limit", mlp["expert"]["limit"])), router_bias=True)
        raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")

    def _validate_layer(self, i: int, l: HybridLayerSpec) -> None:
        m = l.mixer
        if m.kind == "parallel":
            a, r = m.left, m.right
            if min(a.heads, a.kv_heads, a.dim, a.vdim) <= 0 or a.heads % a.kv_heads or a.window < 0:
                raise ValueError(f"layer {i}: attention sizes heads {a.heads}, kv_heads {a.kv_heads}, window {a.window}")
            if min(r.heads, r.vdim, r.state, r.groups, r.norm_groups) <= 0 or r.heads % r.groups:
                raise ValueError(f"layer {i}: {r.heads} state space heads in {r.groups} groups")
            if (r.heads * r.vdim) % r.norm_groups or not 1 <= r.conv <= 8:
                raise ValueError(f"layer {i}: inner size {r.heads * r.vdim} in {r.norm_groups} norm groups, {r.conv} taps")
        else:
            if min(m.heads, m.kv_heads, m.dim, m.vdim) <= 0 or m.heads % m.kv_heads or not 1 <= m.conv <= 8:
                raise ValueError(f"layer {i}: delta rule sizes heads {m.heads}, kv_heads {m.kv_heads}, {m.conv} taps")
        f = l.mlp
        if f is not None and f.kind == "moe" and not 1 <= f.top <= f.experts:
            raise ValueError(f"layer {i}: top {f.top} of {f.experts} experts")

    def validate(self) -> None:
        super().validate()
        if self.pair_embedding is not None and self.pair_embedding.buckets <= 0:
            raise ValueError("embedding.bigram.buckets must be positive")


class DatozenConfig(HybridConfig):
    """Datozen: a decoder of parallel blocks with ONE norm per block — ``x += attention(norm1 x) + ff(norm1 x)`` — followed by a
    per-layer token input, ``y = proj(gelu(gate x) * Es[token, slice of the layer]); x += norm(y)``.  A stretch of layers can run
    several times over with the same weights (``loop``), each pass with keys and values of its own.  The token embedding adds a
    learned position row; the logits are taken against the embedding table.

    Mixer "attention": grouped heads; q and k normed per head with a weight before the rotation; rotary embedding in the
    half-split pairing with frequency interpolation; values rotated at their own position and the head's sum rotated back at the
    query's; keys of the query's block of ``mask.size`` positions only; a learned logit per head in the softmax denominator; a
    sigmoid gate per head.  Feed-forward: dense with the two-parameter "xielu" activation, or a mixture of silu-gated experts
    with softmax scores over experts and identity experts, a choice bias, groups limited by their best member, unnormalised
    weights and a shared expert.

    ``config.json``: ``vocab``, ``width``, ``norm.eps``, ``max_positions``, ``token_side.dim``, ``loop.{start, stop, times}`` and
    ``layers[i]`` = ``{type: "attention", mixer: {heads, kv_heads, dim, vdim, scale, mask.size, rot.{dims, base, scaling.{factor,
    original, fast, slow}}}, mlp}`` with ``mlp`` null, ``{kind: dense, ff}`` or ``{kind: moe, router.{experts, top, identity,
    groups.{count, keep}}, expert.ff, shared.ff}``."""

    model_type = "datozen"
    architecture = "Datozen"
    block = "parallel_shared"
    norm_offset = 0.0
    default_eps = 1e-5
    tied_head = True
    embed_norm = False
    learned_positions = True

    def _parse_mixer(self, i: int, d: Dict[str, Any]) -> Any:
        m = d["mixer"]
        kind = d["type"]
        if kind != "attention":
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        rot = RotarySpec.parse(m.get("rot"), "half")
        return AttentionMixerSpec(
            heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
            scale=float(m["scale"]), rot=rot, kv_from=None, qk_unit_norm=False, head_gate=True, qk_norm=True,
            chunk=int((m.get("mask") or {}).get("size") or 0), sink=True, sink_learned=True, v_rot=rot is not None)

    def _parse_mlp(self, i: int, mlp: Optional[Dict[str, Any]]) -> Any:
        if mlp is None:
            return None
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            return DenseMlpSpec(ff=int(mlp["ff"]), act="xielu", gated=False)
        if kind == "moe":
            r = mlp["router"]
            g = r.get("groups") or {}
            shared = mlp.get("shared") or {}
            return MoeMlpSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]), act="silu",
                              score="softmax", groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))),
                              group_top=1, scale=1.0, normalise=False, shared_ff=int(shared.get("ff", 0)), shared_gate=False,
                              gated=True, identity=int(r.get("identity", 0)), choice_bias=True)
        raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")

    def _validate_layer(self, i: int, l: HybridLayerSpec) -> None:
        m = l.mixer
        if min(m.heads, m.kv_heads, m.dim, m.vdim) <= 0 or m.heads % m.kv_heads or m.chunk < 0:
            raise ValueError(f"layer {i}: attention sizes heads {m.heads}, kv_heads {m.kv_heads}, block {m.chunk}")
        if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim or m.vdim % 2):
            raise ValueError(f"layer {i}: rot.dims {m.rot.dims} must be even and at most dim {m.dim}, vdim {m.vdim} even")
        f = l.mlp
        if f is not None and f.kind == "moe":
            n = f.experts + f.identity
            if not 1 <= f.top <= n:
                raise ValueError(f"layer {i}: top {f.top} of {n} experts")
            if f.groups > 1 and (n % f.groups or not 1 <= f.keep <= f.groups or f.keep * (n // f.groups) < f.top):
                raise ValueError(f"layer {i}: {f.groups} groups (keep {f.keep}) cannot give {f.top} of {n} experts")
