"""CPU-side checks of the Datozen integration: configuration schema, layer runs, registry, tensor inventory, and
properties of the float64 oracle that need no device (causality, the blocks of the mask, relative positions, the router)."""
import json
import math

import pytest
import torch

from jax_llama_b200.config import BazulornConfig, DatozenConfig
from jax_llama_b200.models import registry
from jax_llama_b200.models.hybrid_engine import tensor_shapes
from jax_llama_b200.models.mixers import rotary_frequencies
from tests import datozen_oracle as O

ROT = {"dims": 4, "base": 50.0, "scaling": {"factor": 3.0, "original": 32, "fast": 6.0, "slow": 1.0}}
MOE = {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 6, "top": 2, "identity": 2, "groups": {"count": 4, "keep": 2}},
       "shared": {"ff": 14}}
LAYERS = [
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "mask": {"size": 5}, "rot": ROT},
     "mlp": {"kind": "dense", "ff": 20}},
    {"type": "attention", "mixer": {"heads": 3, "dim": 6, "vdim": 4, "scale": 0.5, "rot": {"dims": 6, "base": 9.0}}, "mlp": MOE},
    {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.2}, "mlp": None},
]


def cfg_dict(**over):
    d = {"architecture": "Datozen", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "max_positions": 40, "token_side": {"dim": 3},
         "loop": {"start": 1, "stop": 3, "times": 2}, "layers": json.loads(json.dumps(LAYERS))}
    d.update(over)
    return d


def test_config_round_trip(tmp_path):
    c = DatozenConfig.from_dict(cfg_dict())
    assert c.vocab_size == 50 and c.hidden_size == 24 and c.num_hidden_layers == 3
    assert c.block == "parallel_shared" and c.tied_head and not c.embed_norm and c.learned_positions
    assert not BazulornConfig.learned_positions
    assert c.layer_runs() == [0, 1, 2, 1, 2] and c.token_side_dim == 3 and c.max_positions == 40
    a, b, d = (l.mixer for l in c.layers)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.chunk, a.window) == (4, 2, 8, 6, 5, 0)
    assert a.qk_norm and a.head_gate and a.sink and a.sink_learned and a.v_rot and not a.qk_unit_norm and not a.bias
    assert a.rot.layout == "half" and a.rot.dims == 4 and a.rot.scaling.factor == 3.0 and b.rot.scaling is None
    assert b.kv_heads == 3 and b.chunk == 0 and d.rot is None and not d.v_rot and c.layers[2].mlp is None
    f = c.layers[1].mlp
    assert (f.experts, f.identity, f.top, f.ff, f.groups, f.keep, f.group_top, f.shared_ff) == (6, 2, 2, 10, 4, 2, 1, 14)
    assert f.gated and f.act == "silu" and f.score == "softmax" and f.choice_bias and not f.normalise and not f.shared_gate
    g = c.layers[0].mlp
    assert not g.gated and g.act == "xielu" and g.ff == 20
    c.save_pretrained(str(tmp_path))
    again = DatozenConfig.from_pretrained(str(tmp_path))
    assert again.to_dict() == c.to_dict()
    assert registry.resolve(str(tmp_path))[:2] == ("datozen", DatozenConfig)
    from jax_llama_b200.ops.build import SUBSETS
    sub = registry.kernel_subset("datozen")
    assert "float32" in registry.gpu_dtypes("datozen") and set(SUBSETS[sub]) < set(SUBSETS["hybrid"])
    assert "seq_token.cu" in SUBSETS[sub] and not {"gla_scan.cu", "delta_scan.cu", "decode_attn.cu"} & set(SUBSETS[sub])


def test_layer_runs_and_defaults():
    d = cfg_dict()
    del d["loop"], d["token_side"]
    del d["layers"][1]["mlp"]["shared"], d["layers"][1]["mlp"]["router"]["groups"], d["layers"][1]["mlp"]["router"]["identity"]
    c = DatozenConfig.from_dict(d)
    assert c.layer_runs() == [0, 1, 2] and c.token_side_dim == 0
    f = c.layers[1].mlp
    assert f.shared_ff == 0 and f.groups == 1 and f.identity == 0
    assert "loop" not in c.to_dict() and "token_side" not in c.to_dict()
    for loop, runs in (((0, 3, 2), [0, 1, 2, 0, 1, 2]), ((0, 1, 3), [0, 0, 0, 1, 2]), ((2, 3, 1), [0, 1, 2]), ((1, 1, 5), [0, 1, 2])):
        e = cfg_dict(loop={"start": loop[0], "stop": loop[1], "times": loop[2]})
        assert DatozenConfig.from_dict(e).layer_runs() == runs == O.layer_runs(e)


def test_validation():
    for bad in (lambda d: d["layers"][0]["mixer"].update(kv_heads=3),
                lambda d: d["layers"][0]["mixer"]["rot"].update(dims=10),
                lambda d: d["layers"][0]["mixer"]["rot"].update(dims=3),
                lambda d: d["layers"][1]["mixer"].update(vdim=5),
                lambda d: d["layers"][1]["mlp"]["router"].update(top=9),
                lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=3),
                lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(keep=5),
                lambda d: d["layers"][0].update(type="retention"),
                lambda d: d["loop"].update(stop=4),
                lambda d: d["loop"].update(times=0),
                lambda d: d.pop("max_positions")):
        e = cfg_dict()
        bad(e)
        with pytest.raises((ValueError, KeyError)):
            DatozenConfig.from_dict(e)


def test_tensor_inventory():
    c = DatozenConfig.from_dict(cfg_dict())
    shapes = tensor_shapes(c)
    assert "head" not in shapes and "embed.norm" not in shapes and shapes["embed"] == (50, 24) and shapes["pos"] == (40, 24)
    assert shapes["side.embed"] == (50, 9) and shapes["l2.side.gate"] == (3, 24) and shapes["l2.side.proj"] == (24, 3)
    assert shapes["l0.side.norm"] == (24,) and "l0.norm2" not in shapes
    assert shapes["l0.mix.q"] == (32, 24) and shapes["l0.mix.k"] == (16, 24) and shapes["l0.mix.v"] == (12, 24)
    assert shapes["l0.mix.q.norm"] == shapes["l0.mix.k.norm"] == (8,) and shapes["l0.mix.sink"] == (4,)
    assert shapes["l0.mix.g"] == (4, 24) and shapes["l0.mix.o"] == (24, 24)
    assert shapes["l0.mlp.up"] == (20, 24) and shapes["l0.mlp.act"] == (2,) and "l0.mlp.gate" not in shapes
    assert shapes["l1.mlp.router"] == (8, 24) and shapes["l1.mlp.correction"] == (8,) and "l1.mlp.e6.up" not in shapes
    assert shapes["l1.mlp.e5.gate"] == (10, 24) and shapes["l1.mlp.shared.down"] == (24, 14) and "l1.mlp.shared.sg" not in shapes
    assert not any(k.startswith("l2.mlp") for k in shapes)
    assert tensor_shapes(c, present={"pos": (64, 24)})["pos"] == (64, 24)


def _random(c, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = {}
    for name, shape in tensor_shapes(c).items():
        if len(shape) == 1:
            t[name] = (1.0 if "norm" in name else 0.0) + 0.3 * torch.randn(shape, generator=g)
        else:
            t[name] = torch.randn(shape, generator=g) / shape[1] ** 0.5
    return t


def test_oracle_is_causal_and_bounded_by_its_blocks():
    """A token changes nothing before it; through one layer of attention it changes nothing beyond its own block either."""
    c = DatozenConfig.from_dict(cfg_dict())
    t = _random(c)
    toks = [3, 9, 27, 4, 11, 45, 6, 6, 30, 2, 17, 8]
    base = O.forward(toks, t, c.to_dict())
    other = list(toks)
    other[7] = 40
    moved = O.forward(other, t, c.to_dict())
    assert (base[:7] - moved[:7]).abs().max() == 0 and (base[7:] - moved[7:]).abs().max() > 1e-3
    one = cfg_dict(layers=[json.loads(json.dumps(LAYERS[0]))])
    del one["loop"]
    c1 = DatozenConfig.from_dict(one)
    t1 = _random(c1, 1)
    a = O.forward(toks, t1, c1.to_dict())
    other = list(toks)
    other[6] = 40                                            # block 5 .. 9
    b = O.forward(other, t1, c1.to_dict())
    assert (a[6:10] - b[6:10]).abs().min() > 1e-6 and (a[10:] - b[10:]).abs().max() == 0 and (a[:6] - b[:6]).abs().max() == 0


def test_oracle_attention_depends_on_relative_positions_only():
    """Keys, queries and values all turn with their positions and the sum turns back: without blocks, shifting every position
    by the same amount leaves a layer's output as it is."""
    m = dict(LAYERS[0]["mixer"])
    del m["mask"]
    c = DatozenConfig.from_dict(cfg_dict(layers=[{"type": "attention", "mixer": m, "mlp": None}], loop=None))
    t = _random(c, 2)
    h = torch.randn(9, 24, dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    a = O.attention(h, t, "l0.mix.", m, 1e-5, first=0)
    b = O.attention(h, t, "l0.mix.", m, 1e-5, first=13)
    assert (a - b).abs().max() < 1e-9
    m5 = dict(m, mask={"size": 5})
    assert (O.attention(h, t, "l0.mix.", m5, 1e-5, first=0) - O.attention(h, t, "l0.mix.", m5, 1e-5, first=13)).abs().max() > 1e-4


def test_interpolated_frequencies_match_the_engine_tables():
    from jax_llama_b200.config import RotaryScaling
    for dims, base, sc in ((4, 50.0, ROT["scaling"]), (40, 30000.0, {"factor": 6.0, "original": 256, "fast": 16.0, "slow": 2.0}),
                           (16, 100.0, None), (6, 2.0, {"factor": 1.5, "original": 8, "fast": 2.0, "slow": 0.25})):
        f, mult = O.frequencies(dims, base, sc)
        g, gm = rotary_frequencies(dims, base, RotaryScaling(**sc) if sc else None)
        assert torch.allclose(f, g, rtol=1e-12, atol=0) and abs(mult - gm) < 1e-12
    f, mult = O.frequencies(8, 10000.0, {"factor": 4.0, "original": 64, "fast": 1e9, "slow": 1e-9})
    assert mult == pytest.approx(0.1 * math.log(4.0) + 1.0)


def test_oracle_router_and_activation():
    t = {"r.router": torch.eye(6, dtype=torch.float64) * 4.0,
         "r.correction": torch.tensor([0.0, 0.0, 0.9, 0.0, 0.0, -0.5], dtype=torch.float64)}
    mlp = {"router": {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 2}}}
    h = torch.tensor([[3.0, 1.0, 0.0, 0.5, 2.0, 2.5]], dtype=torch.float64) / 4.0
    idx, wt = O.route(h, t, "r.", mlp)
    s = torch.softmax(h[0] * 4.0, -1)
    # groups (0, 1), (2, 3), (4, 5): choice scores s + correction; the bias lifts expert 2 into the choice, the weights stay s
    assert sorted(idx[0].tolist()) == [0, 2] and torch.allclose(wt[0].sort().values, torch.stack([s[2], s[0]]).sort().values)
    z = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64)
    y = O.xielu(z, torch.tensor(0.0, dtype=torch.float64), torch.tensor(0.0, dtype=torch.float64))
    ln2 = math.log(2.0)
    assert y.tolist() == pytest.approx([(0.5 + ln2) * (math.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, ln2 * 9.0 + 1.5])
