"""CPU-side checks of the Bazulorn integration: configuration schema, registry, tensor inventory, and properties of the
float64 oracle that need no device (causality, the window, the convolution's reach)."""
import json

import pytest
import torch

from jax_llama_b200.config import BazulornConfig, NikonexConfig
from jax_llama_b200.models import registry
from jax_llama_b200.models.hybrid_engine import tensor_shapes
from tests import bazulorn_oracle as O

MOE = {"kind": "moe", "expert": {"ff": 10, "limit": 1.5}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 14, "limit": 0.5}}
LAYERS = [
    {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 3}, "mlp": {"kind": "dense", "ff": 20}},
    {"type": "parallel",
     "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "mask": {"size": 7}},
               "right": {"heads": 3, "vdim": 4, "state": 5, "groups": 3, "conv": 2, "norm_groups": 2}},
     "mlp": MOE},
    {"type": "channel_delta", "mixer": {"heads": 2, "dim": 8, "vdim": 6, "conv": 4}, "mlp": None},
]


def cfg_dict(**over):
    d = {"architecture": "Bazulorn", "vocab": 50, "width": 24, "norm": {"eps": 1e-5},
         "embedding": {"bigram": {"buckets": 31, "mul_prev": 7, "mul_cur": 3}}, "layers": json.loads(json.dumps(LAYERS))}
    d.update(over)
    return d


def test_config_round_trip(tmp_path):
    c = BazulornConfig.from_dict(cfg_dict())
    assert c.vocab_size == 50 and c.hidden_size == 24 and c.num_hidden_layers == 3
    assert c.block == "parallel_shared" and c.tied_head and c.embed_norm and NikonexConfig.block == "parallel"
    assert (c.pair_embedding.buckets, c.pair_embedding.mul_prev, c.pair_embedding.mul_cur) == (31, 7, 3)
    d, p = c.layers[0].mixer, c.layers[1].mixer
    assert d.kind == "channel_delta" and (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (4, 2, 8, 6, 3)
    assert c.layers[2].mixer.kv_heads == 2 and c.layers[2].mlp is None
    a, s = p.left, p.right
    assert p.kind == "parallel" and p.scale == 0.5
    assert a.window == 7 and a.sink and a.talking_heads and a.bias and a.v_unit_norm and a.rot is None and not a.head_gate
    assert (s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups) == (3, 4, 5, 3, 2, 2)
    f = c.layers[1].mlp
    assert (f.experts, f.top, f.ff, f.limit, f.shared_ff, f.shared_limit) == (6, 2, 10, 1.5, 14, 0.5)
    assert f.gated and f.router_bias and f.score == "softmax" and not f.shared_gate
    g = c.layers[0].mlp
    assert g.gated and g.act == "gelu_tanh" and g.ff == 20
    c.save_pretrained(str(tmp_path))
    again = BazulornConfig.from_pretrained(str(tmp_path))
    assert again.to_dict() == c.to_dict()
    assert registry.resolve(str(tmp_path))[:2] == ("bazulorn", BazulornConfig)
    assert registry.kernel_subset("bazulorn") == "hybrid" and "float32" in registry.gpu_dtypes("bazulorn")


def test_config_defaults_and_validation():
    d = cfg_dict()
    del d["layers"][1]["mixer"]["left"]["mask"]
    del d["layers"][1]["mlp"]["shared"]
    c = BazulornConfig.from_dict(d)
    assert c.layers[1].mixer.left.window == 0 and c.layers[1].mlp.shared_ff == 0
    for bad in (lambda d: d["layers"][1]["mixer"]["left"].update(kv_heads=3),
                lambda d: d["layers"][1]["mixer"]["right"].update(groups=2),
                lambda d: d["layers"][1]["mixer"]["right"].update(norm_groups=5),
                lambda d: d["layers"][0]["mixer"].update(conv=9),
                lambda d: d["layers"][0]["mixer"].update(kv_heads=3),
                lambda d: d["layers"][1]["mlp"]["router"].update(top=7),
                lambda d: d["layers"][0].update(type="retention"),
                lambda d: d["embedding"]["bigram"].update(buckets=0)):
        e = cfg_dict()
        bad(e)
        with pytest.raises((ValueError, KeyError)):
            BazulornConfig.from_dict(e)


def test_tensor_inventory():
    c = BazulornConfig.from_dict(cfg_dict())
    present = {"l0.mix.a1": (3, 24), "l0.mix.g1": (9, 24)}
    shapes = tensor_shapes(c, decay_rank=5, present=present)
    assert "head" not in shapes and shapes["embed"] == (50, 24) and shapes["bigram"] == (32, 24) and shapes["embed.norm"] == (24,)
    assert shapes["l0.mix.a1"] == (3, 24) and shapes["l0.mix.a2"] == (32, 3) and shapes["l0.mix.dt_bias"] == (32,)
    assert shapes["l0.mix.g1"] == (9, 24) and shapes["l0.mix.g2"] == (24, 9) and shapes["l2.mix.a1"] == (5, 24)
    assert shapes["l0.mix.q"] == (16, 24) and shapes["l0.mix.q.conv"] == (16, 3) and shapes["l0.mix.v.conv"] == (24, 3)
    assert shapes["l0.mix.b"] == (4, 24) and shapes["l0.mix.norm"] == (6,) and shapes["l0.mix.o"] == (24, 24)
    assert shapes["l0.mlp.gate"] == (20, 24) and shapes["l0.mlp.down"] == (24, 20) and "l0.norm2" not in shapes
    assert shapes["l1.mix.left.q.b"] == (32,) and shapes["l1.mix.left.k"] == (16, 24) and shapes["l1.mix.left.talk"] == (4, 4)
    assert shapes["l1.mix.left.v.b"] == (12,) and shapes["l1.mix.left.out"] == (24,) and shapes["l1.mix.right.out"] == (24,)
    inner, gn = 12, 15
    assert shapes["l1.mix.right.in"] == (2 * inner + 2 * gn + 3, 24) and shapes["l1.mix.right.conv"] == (inner + 2 * gn, 2)
    assert shapes["l1.mix.right.conv.b"] == (inner + 2 * gn,) and shapes["l1.mix.right.norm"] == (inner,)
    assert shapes["l1.mix.right.A_log"] == shapes["l1.mix.right.D"] == shapes["l1.mix.right.dt_bias"] == (3,)
    assert shapes["l1.mlp.router.b"] == (6,) and shapes["l1.mlp.e5.gate"] == (10, 24) and shapes["l1.mlp.shared.gate"] == (14, 24)
    assert not any(k.startswith("l2.mlp") for k in shapes)


def _random(c, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = {}
    for name, shape in tensor_shapes(c, decay_rank=4).items():
        if len(shape) == 1:
            t[name] = (1.0 if "norm" in name or name.endswith(".out") else 0.0) + 0.3 * torch.randn(shape, generator=g)
        else:
            t[name] = torch.randn(shape, generator=g) / shape[1] ** 0.5
    return t


def test_oracle_is_causal_and_bounded_by_its_windows():
    """A token changes nothing before it; through a layer whose only path back is the windowed attention (state space
    output off, no hashed rows) a token outside the window changes nothing after it either."""
    c = BazulornConfig.from_dict(cfg_dict())
    t = _random(c)
    toks = [3, 9, 27, 4, 11, 45, 6, 6, 30, 2, 17, 8]
    base = O.forward(toks, t, c.to_dict())
    other = list(toks)
    other[7] = 40
    moved = O.forward(other, t, c.to_dict())
    assert (base[:7] - moved[:7]).abs().max() == 0 and (base[7:] - moved[7:]).abs().max() > 1e-3
    one = cfg_dict(layers=[json.loads(json.dumps(LAYERS[1]))])
    one["layers"][0]["mlp"] = None
    one["layers"][0]["mixer"]["left"]["mask"]["size"] = 3
    c1 = BazulornConfig.from_dict(one)
    t1 = _random(c1, 1)
    t1["bigram"].zero_()
    t1["l0.mix.right.o"].zero_()
    a = O.forward(toks, t1, c1.to_dict())
    other = list(toks)
    other[4] = 40
    b = O.forward(other, t1, c1.to_dict())
    assert (a[4:7] - b[4:7]).abs().max() > 1e-4 and (a[7:] - b[7:]).abs().max() == 0


def test_oracle_convolution_and_routing():
    x = torch.arange(12, dtype=torch.float64).view(6, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = O.causal_conv(x, w)
    assert y[0].tolist() == [0.0, 1.0] and y[2].tolist() == [100 * 4 + 10 * 2 + 0, 5.0] and torch.equal(y[:, 1], x[:, 1])
    t = {"r.router": torch.eye(4, dtype=torch.float64), "r.router.b": torch.tensor([0.0, 0.0, 0.0, 2.5], dtype=torch.float64)}
    idx, wt = O.route(torch.tensor([[3.0, 1.0, 2.0, 0.0]], dtype=torch.float64), t, "r.", 2)
    assert idx.tolist() == [[0, 3]] and abs(float(wt[0, 0]) - 1 / (1 + 2.718281828 ** -0.5)) < 1e-6
