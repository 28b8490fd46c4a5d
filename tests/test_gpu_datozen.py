"""Datozen on the hybrid engine against the plain float64 statement of the design (`datozen_oracle.py`).

Small configurations with random weights; every test builds its own.  The float32 engine is held to a tight bound, the
bfloat16 engine to the error that rounding its operands causes.
"""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from jax_llama_b200.config import DatozenConfig                                   # noqa: E402
from jax_llama_b200.generation import LLaMA                                       # noqa: E402
from jax_llama_b200.models.datozen import DatozenForCausalLM                      # noqa: E402
from jax_llama_b200.models.hybrid_engine import HybridEngine, random_tensors      # noqa: E402
from jax_llama_b200.ops import seq_kernels as SK                                  # noqa: E402
from jax_llama_b200.tokenizers import IdTokenizer                                 # noqa: E402

from tests import datozen_oracle as O                                             # noqa: E402

TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, cfg):
    """Rounding the operands of every layer run to bfloat16 adds up along the stack: the bound grows with the runs beyond four."""
    return TOL[dtype] * (max(1.0, len(cfg.layer_runs()) / 4.0) if dtype == torch.bfloat16 else 1.0)


SCALING = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, identity=2, groups=(4, 2), shared=16):
    r = {"experts": experts, "top": top}
    if identity:
        r["identity"] = identity
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def att(heads=4, kv_heads=2, dim=16, vdim=12, chunk=20, scale=0.3, rot=8, base=100.0, scaling=SCALING, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    return {"type": "attention", "mixer": m, "mlp": mlp}


def config(layers, vocab=96, width=72, eps=1e-5, side=6, loop=None, positions=512, dtype=None):
    """With dtype bfloat16 every expert of a layer is chosen (top = all router outputs, no group limit): rounding the router's
    input to bfloat16 moves its logits by parts in a thousand, which among random logits flips a close choice every few dozen
    tokens, and the oracle would then follow other experts.  The choice itself is checked in float32 and on the router alone."""
    layers = json.loads(json.dumps(layers))
    if dtype == torch.bfloat16:
        for l in layers:
            if l["mlp"] is not None and l["mlp"]["kind"] == "moe":
                r = l["mlp"]["router"]
                r["top"] = r["experts"] + r.get("identity", 0)
                r.pop("groups", None)
    d = {"architecture": "Datozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "max_positions": positions, "layers": layers}
    if side:
        d["token_side"] = {"dim": side}
    if loop:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return DatozenConfig.from_dict(d)


MIXED = [att(mlp=dense()), att(heads=3, kv_heads=3, dim=8, vdim=20, chunk=7, rot=8, scaling=None, mlp=moe()),
         att(heads=6, kv_heads=1, dim=12, vdim=8, chunk=0, rot=4, mlp=moe(experts=4, top=1, identity=0, groups=None, shared=0)),
         att(heads=2, kv_heads=2, dim=10, vdim=10, chunk=33, rot=10, base=7.0)]


def build(cfg, dtype, seed=0, graph=True, tweak=None):
    tensors = random_tensors(cfg, "cuda", seed)
    g = torch.Generator(device="cuda").manual_seed(seed + 1000)

    def rnd(name, mean, std):
        tensors[name] = (mean + std * torch.randn(tensors[name].shape, device="cuda", generator=g)).to(torch.bfloat16)

    for name in list(tensors):
        if name.endswith("q.norm") or name.endswith("k.norm") or name.endswith("side.norm"):
            rnd(name, 1.0, 0.3)
        if name.endswith("mix.sink"):                                    # sinks that take from nothing to most of the weight
            rnd(name, 0.0, 2.0)
        if name.endswith("mlp.act"):
            rnd(name, 0.0, 1.0)
        if name.endswith("mlp.correction"):
            rnd(name, 0.0, 0.05)
        if name == "pos":
            rnd(name, 0.0, 0.5)
        if name == "side.embed":
            rnd(name, 0.0, 1.0)
    if tweak is not None:
        tweak(tensors)
    eng = HybridEngine(cfg, tensors, dtype=dtype, device="cuda", use_cuda_graph=graph)
    return eng, {k: v.cpu() for k, v in tensors.items()}


def err(got, want):
    """Centred RMS difference over the vocabulary relative to the RMS of the wanted logits, worst row."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


def tokens(n, vocab, seed):
    return torch.randint(1, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def oracle_logits(cfg, cpu_tensors, toks, streams=None):
    return O.forward(toks, cpu_tensors, cfg.to_dict(), streams)


def feed(vals):
    return torch.tensor(vals, dtype=torch.int32).pin_memory()


def i32(vals):
    return torch.tensor(vals, dtype=torch.int32, device="cuda")


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_position_rows_with_padding_and_decoding(dtype):
    """Two rows, one left-padded by three; the prompt, then two single tokens: positions count from each row's first real
    token and go on across calls; padding rows are zero."""
    V, W, P = 50, 40, 32
    g = torch.Generator().manual_seed(1)
    t = {"embed": torch.randn(V, W, generator=g).to(torch.bfloat16), "pos": torch.randn(P, W, generator=g).to(torch.bfloat16)}
    seqs = [tokens(8, V, 2), tokens(5, V, 3)]
    d = {k: v.cuda().to(dtype) for k, v in t.items()}
    length, pad = i32([0]), i32([0, 3])
    ids = torch.zeros(2, 6, dtype=torch.int32)
    ids[0] = torch.tensor(seqs[0][:6])
    ids[1, 3:] = torch.tensor(seqs[1][:3])
    got = [SK.embed_pos(ids.cuda(), d["embed"], d["pos"], length, pad, 2, 6)]
    for j in range(2):
        length.fill_(6 + j)
        got.append(SK.embed_pos(i32([seqs[0][6 + j], seqs[1][3 + j]]), d["embed"], d["pos"], length, pad, 2, 1))
    want = [O.embed_tokens(s, t) for s in seqs]
    x = got[0].view(2, 6, W).double().cpu()
    assert (x[0] - want[0][:6]).abs().max() < 1e-5 and (x[1, 3:] - want[1][:3]).abs().max() < 1e-5
    assert x[1, :3].abs().max() == 0
    for j in range(2):
        y = got[1 + j].double().cpu()
        assert (y[0] - want[0][6 + j]).abs().max() < 1e-5 and (y[1] - want[1][3 + j]).abs().max() < 1e-5


@pytest.mark.parametrize("rows", [3, 200])
@pytest.mark.parametrize("pq", [(0.0, 0.0), (1.3, -0.7), (-2.0, 2.5)])
def test_two_parameter_activation(rows, pq):
    """The activation as the linear kernels apply it, on both sides of zero, near zero and far out (few rows: the
    weight-streaming kernel; many: the tiled one)."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(rows, 24, generator=g) * 3.0
    x[0, :6] = torch.tensor([0.0, 1e-4, -1e-4, 30.0, -30.0, -90.0])
    eye = torch.eye(24)
    p0 = float(O.softplus(torch.tensor(pq[0], dtype=O.F64)))
    p1 = 0.5 + float(O.softplus(torch.tensor(pq[1], dtype=O.F64)))
    got = SK.linear(x.cuda(), eye.cuda(), act=SK.ACT_XIELU, p0=p0, p1=p1)
    want = O.xielu(x.double(), torch.tensor(pq[0], dtype=O.F64), torch.tensor(pq[1], dtype=O.F64))
    assert ((got.double().cpu() - want).abs() / (1.0 + want.abs())).max() < 1e-5


@pytest.mark.parametrize("experts,identity,top,groups", [(6, 2, 2, (4, 2)), (5, 0, 1, None), (7, 1, 8, None), (40, 8, 3, (6, 2)),
                                                         (4, 4, 3, (2, 1)), (9, 3, 4, (3, 3))])
def test_router_with_choice_bias_groups_and_identity_experts(experts, identity, top, groups):
    """Chosen experts and weights against the oracle's router: the bias moves the choice and not the weights, negative choice
    scores stay above a masked group, identity experts are reported as -1 and their weights summed."""
    N, W, M = experts + identity, 32, 64
    g = torch.Generator().manual_seed(experts * 10 + top)
    t = {"router": torch.randn(N, W, generator=g), "correction": torch.randn(N, generator=g) * 0.2 - 0.3}
    h = torch.randn(M, W, generator=g)
    mlp = moe(experts=experts, top=top, identity=identity, groups=groups)
    idx_w, wt_w = O.route(h.double(), t, "", mlp)
    z = (h.double() @ t["router"].double().T).float().cuda()
    ident = torch.empty(M, dtype=torch.float32, device="cuda")
    gc, gk = groups if groups else (1, 1)
    idx, wt = SK.moe_route(z, N, top, gc, gk, 1, SK.SCORE_SOFTMAX, False, 1.0, choice_bias=t["correction"].cuda(), n_real=experts,
                           ident_w=ident)
    idx, wt = idx.cpu(), wt.double().cpu()
    for m in range(M):
        want = {int(e): float(w) for e, w in zip(idx_w[m], wt_w[m])}
        real = {e: w for e, w in want.items() if e < experts}
        got = {int(e): float(w) for e, w in zip(idx[m], wt[m]) if e >= 0}
        assert set(got) == set(real), m
        assert all(abs(got[e] - real[e]) < 1e-6 for e in real)
        assert int((idx[m] < 0).sum()) == len(want) - len(real)
        assert abs(float(ident[m]) - sum(w for e, w in want.items() if e >= experts)) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5, 8, 9, 70])
def test_token_input_for_few_and_for_many_rows(dtype, rows):
    """The per-layer token input on the stream alone: up to eight rows run the gate kernel that holds the small projection, more
    run two products around a gate kernel; both against the oracle, with the norm of the next block formed on the way."""
    from jax_llama_b200.models.hybrid_engine import TokenSide
    V, W, n, layer, L = 30, 56, 6, 2, 4
    g = torch.Generator().manual_seed(rows)
    t = {"side.embed": torch.randn(V, L * n, generator=g).to(torch.bfloat16), "l2.side.gate": (torch.randn(n, W, generator=g) / 7).to(torch.bfloat16),
         "l2.side.proj": torch.randn(W, n, generator=g).to(torch.bfloat16), "l2.side.norm": (1 + 0.3 * torch.randn(W, generator=g)).to(torch.bfloat16)}
    w_next = (1 + 0.3 * torch.randn(W, generator=g)).to(torch.bfloat16)
    x = torch.randn(rows, W, generator=g) * 2
    toks = tokens(rows, V, 5)
    want_y = O.token_side(x.double(), toks, t, "l2.", layer, n, 1e-5)
    want_x = x.double() + want_y
    want_h = O.rms_norm(want_x, w_next.double(), 1e-5)
    side = TokenSide(t["side.embed"].cuda().to(dtype), layer * n,
                     {k: t["l2.side." + k].cuda().to(dtype) for k in ("gate", "proj", "norm")})
    xd = x.cuda().clone()
    h = side.run(xd, i32(toks), w_next.cuda().to(dtype), 1e-5)
    tol = 1e-4 if dtype == torch.float32 else 4e-2
    assert (xd.double().cpu() - want_x).abs().max() < tol * 4
    assert (h.double().cpu() - want_h).abs().max() < tol * 4


SINGLE = {
    "attention": [att()],
    "attention_plain_rotation": [att(scaling=None, rot=16, chunk=0)],
    "attention_unrotated": [att(rot=0)],
    "attention_one_value_head": [att(heads=4, kv_heads=1, dim=8, vdim=32, chunk=5)],
    "attention_every_head_its_own": [att(heads=3, kv_heads=3, dim=12, vdim=6, chunk=64, rot=12)],
    "attention_and_dense": [att(mlp=dense())],
    "attention_and_experts": [att(mlp=moe())],
    "experts_without_extras": [att(mlp=moe(experts=5, top=2, identity=0, groups=None, shared=0))],
    "one_group_kept": [att(mlp=moe(experts=9, top=2, identity=3, groups=(4, 1), shared=8))],
    "seventeen_query_heads_per_value_head": [att(heads=34, kv_heads=2, dim=8, vdim=8, chunk=50, rot=4)],
    "value_rows_of_320_channels": [att(heads=2, kv_heads=1, dim=16, vdim=320, chunk=40, rot=16)],
    "keys_of_264_channels": [att(heads=2, kv_heads=2, dim=264, vdim=8, chunk=0, rot=100, scale=0.06)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_single_mechanism_models(dtype, name):
    cfg = config(SINGLE[name], side=0 if "unrotated" in name else 6, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=3)
    toks = tokens(75, cfg.vocab_size, 9)
    want = oracle_logits(cfg, cpu, toks)
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got, want) < tol(dtype, cfg)
    stream = eng.begin_stream(torch.tensor([toks[:70]], device="cuda"), None, max_length=80, eos_token_id=-1)
    rows = []
    for t in toks[70:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[70:]) < tol(dtype, cfg)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("loop", [None, (1, 3, 2), (0, 4, 3), (2, 3, 1), (3, 4, 4)])
def test_residual_stream_after_every_layer_run(dtype, loop):
    """The stream after every layer run of a looped stack: a repeated layer keeps its weights and its slice of the token
    table, and every pass has keys and values of its own."""
    cfg = config(MIXED, loop=loop, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=4)
    toks = tokens(50, cfg.vocab_size, 11)
    want_streams = []
    want = oracle_logits(cfg, cpu, toks, want_streams)
    eng.capture_streams = []
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    streams, eng.capture_streams = eng.capture_streams, None
    assert len(streams) == len(want_streams) == len(cfg.layer_runs())
    for r, (a, b) in enumerate(zip(streams, want_streams)):
        assert (a.double().cpu() - b).abs().max() < (2e-3 if dtype == torch.float32 else 0.6), r
    assert err(got, want) < tol(dtype, cfg)


def test_other_constants():
    """Another eps, base, scale, interpolation and width; a table of exactly as many positions as the prompt has tokens."""
    layers = [att(heads=2, kv_heads=1, dim=24, vdim=16, chunk=11, scale=0.07, rot=20, base=31.0,
                  scaling={"factor": 2.5, "original": 16, "fast": 3.0, "slow": 0.5}, mlp=dense(ff=17)),
              att(heads=5, kv_heads=5, dim=6, vdim=4, chunk=3, rot=2, base=2.0, scaling=None, mlp=moe(experts=3, top=3, identity=1, groups=(2, 2), ff=9, shared=5))]
    cfg = config(layers, vocab=41, width=50, eps=3e-3, side=1, loop=(0, 1, 2), positions=60)
    eng, cpu = build(cfg, torch.float32, seed=2)
    toks = tokens(60, cfg.vocab_size, 1)
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got, oracle_logits(cfg, cpu, toks)) < TOL[torch.float32]
    with pytest.raises(ValueError):
        eng.generate(torch.tensor([toks], device="cuda"), None, max_length=62)


# ------------------------------------------------------------------------------------------ decoding, portions, batches
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("prompt", [1, 2, 31, 33])
def test_decode_matches_prefill_and_oracle(dtype, prompt):
    cfg = config(MIXED, loop=(1, 3, 2), dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=7)
    toks = tokens(prompt + 45, cfg.vocab_size, 13)
    want = oracle_logits(cfg, cpu, toks)
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole, want) < tol(dtype, cfg)
    stream = eng.begin_stream(torch.tensor([toks[:prompt]], device="cuda"), None, max_length=len(toks) + 2, eos_token_id=-1)
    rows = [stream.logits()[0].clone()]
    for t in toks[prompt:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[prompt - 1:]) < tol(dtype, cfg)
    assert err(torch.stack(rows), whole[prompt - 1:]) < tol(dtype, cfg)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """Three hundred tokens decoded one by one after a two-token prompt, across many block borders."""
    cfg = config([att(chunk=37, mlp=moe()), att(chunk=64, heads=2, kv_heads=1, mlp=dense())], loop=(0, 2, 2), dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=21)
    toks = tokens(302, cfg.vocab_size, 5)
    want = oracle_logits(cfg, cpu, toks)
    stream = eng.begin_stream(torch.tensor([toks[:2]], device="cuda"), None, max_length=310, eos_token_id=-1)
    rows = [stream.logits()[0].clone()]
    for t in toks[2:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[1:]) < tol(dtype, cfg)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 30], [33, 2, 9], [5, 64, 3], [1, 2, 200]])
def test_prompt_in_portions(dtype, cuts):
    """The same prompt fed to one cache in portions of several sizes, down to two tokens (and one): blocks of positions count
    from the start of the sequence, not of the portion."""
    cfg = config(MIXED, loop=(0, 2, 2), dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=14)
    toks = tokens(sum(cuts), cfg.vocab_size, 31)
    want = oracle_logits(cfg, cpu, toks)
    cache = eng.new_cache(1, len(toks) + 2)
    cache.set_index(0)
    got, at = [], 0
    for n in cuts:
        got.append(eng.forward(torch.tensor([toks[at:at + n]], device="cuda"), cache=cache).logits[0])
        at += n
    assert err(torch.cat(got), want) < tol(dtype, cfg)


def run_unequal_batch(cfg, dtype, lens, extra, seed):
    """Left-padded batch of prompts of the given lengths, then `extra` tokens decoded together; every row is compared with
    the oracle run of that request alone."""
    eng, cpu = build(cfg, dtype, seed=seed)
    seqs = [tokens(n + extra, cfg.vocab_size, 20 + n + 100 * b) for b, n in enumerate(lens)]
    S, B = max(lens), len(lens)
    ids = torch.zeros((B, S), dtype=torch.long)
    mask = torch.zeros((B, S), dtype=torch.int32)
    rows = []
    for b, (n, s) in enumerate(zip(lens, seqs)):
        ids[b, S - n:] = torch.tensor(s[:n])
        mask[b, S - n:] = 1
        rows += [b * S + S - n + j for j in range(n)]
    stream = eng.begin_stream(ids.cuda(), mask.cuda(), max_length=S + extra + 1, eos_token_id=-1, logit_rows=torch.tensor(rows))
    got_prompt = stream.prompt_logits().clone()
    steps = []
    for j in range(extra):
        stream.step(feed([s[n + j] for n, s in zip(lens, seqs)]))
        steps.append(stream.logits().clone())
    stream.close()
    at = 0
    for b, (n, s) in enumerate(zip(lens, seqs)):
        want = oracle_logits(cfg, cpu, s)
        assert err(got_prompt[at:at + n], want[:n]) < tol(dtype, cfg), b
        assert err(torch.stack([x[b] for x in steps]), want[n:]) < tol(dtype, cfg), b
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_equals_each_alone(dtype):
    """Prompts of 1, 7 and 40 tokens in one batch: padding must touch neither the positions, the blocks of the mask, the
    rotation of keys and values, the token inputs, nor the choice of experts of the real tokens."""
    run_unequal_batch(config(MIXED, loop=(1, 3, 2), dtype=dtype), dtype, [1, 7, 40], 36, seed=6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_odd_sizes_and_a_batch_of_twenty(dtype):
    """Sizes that fit no vector width or tile in a batch of twenty unequal requests: more rows than the pairwise expert
    path, the one-launch token input and the weight-streaming kernel take."""
    layers = [att(heads=3, kv_heads=3, dim=10, vdim=14, chunk=9, rot=6, mlp=moe(experts=9, top=2, ff=10, identity=1, groups=(5, 3), shared=6)),
              att(heads=3, kv_heads=1, dim=12, vdim=10, chunk=0, rot=12, mlp=moe(experts=3, top=1, ff=5, identity=0, groups=None, shared=0)),
              att(heads=1, kv_heads=1, dim=6, vdim=2, chunk=4, rot=2, mlp=dense(ff=11))]
    cfg = config(layers, vocab=77, width=90, side=5, dtype=dtype)
    run_unequal_batch(cfg, dtype, [3, 17, 1, 9, 30, 2, 12, 25, 8, 21, 4, 5, 6, 7, 11, 13, 14, 15, 16, 29], 12, seed=17)


def test_realistic_head_sizes():
    """128- and 64-wide heads, eight query heads per key/value head, experts on the tensor-core path."""
    layers = [att(heads=8, kv_heads=1, dim=128, vdim=128, chunk=96, rot=64, mlp=moe(experts=6, top=2, ff=64, identity=2, groups=None, shared=64)),
              att(heads=4, kv_heads=2, dim=64, vdim=128, chunk=0, rot=64, mlp=dense(ff=256))]
    run_unequal_batch(config(layers, width=256, vocab=128, side=16, dtype=torch.bfloat16), torch.bfloat16, [5, 150, 131], 40, seed=13)


def test_state_and_cache_are_clean_when_used_again():
    """The same decode state serves request after request: a second, shorter request must see nothing of the first (old
    keys invisible, old left-pad counts gone, positions from zero again)."""
    cfg = config(MIXED, loop=(1, 3, 2))
    eng, cpu = build(cfg, torch.float32, seed=8)
    a, b = tokens(50, cfg.vocab_size, 1), tokens(9, cfg.vocab_size, 2)
    pad_ids = torch.zeros((2, 50), dtype=torch.long)
    pad_ids[0] = torch.tensor(a)
    pad_ids[1, 41:] = torch.tensor(b)
    mask = (torch.arange(50)[None, :] >= torch.tensor([0, 41])[:, None]).int()
    out1 = eng.generate(pad_ids.cuda(), mask.cuda(), max_length=60, eos_token_id=-1)
    st = eng._decode_state(2, 60)
    ids2 = torch.tensor([b, b[::-1]])
    out2 = eng.generate(ids2.cuda(), None, max_length=60, eos_token_id=-1)          # same (B, max_length): same state, same cache
    assert eng._decode_state(2, 60) is st
    fresh, _ = build(cfg, torch.float32, seed=8)
    out3 = fresh.generate(ids2.cuda(), None, max_length=60, eos_token_id=-1)
    assert torch.equal(out2, out3)
    assert out1.shape == (2, 60)
    eng.release_state(st)
    assert (2, 60) not in eng._decode_states
    out4 = eng.generate(ids2.cuda(), None, max_length=60, eos_token_id=-1)
    assert torch.equal(out4, out3)


# ------------------------------------------------------------------------------------------ made-to-show inputs
A_TOK, B_TOK = 61, 60
DIM, ROT, WIDTH = 64, 32, 48


def _planted_attention(chunk, dtype, seed=5, sink=0.0, dim=DIM, vdim=12, rot=ROT):
    """One layer of attention alone.  Tokens A and B embed as unit vectors and the position rows are zero, so the layer sees
    sqrt(width) times one column of each projection for them.  A's key, in every key/value head, and B's query, in the first
    query head of that group, are the same vector on the unrotated channels: after the head norms their score is
    scale * dim = 24 at any distance, five deviations of a random key's score above zero."""
    layer = att(heads=4, kv_heads=2, dim=dim, vdim=vdim, chunk=chunk, scale=24.0 / dim, rot=rot)
    cfg = config([layer], vocab=64, width=WIDTH, side=4)

    def tweak(t):
        t["pos"].zero_()
        t["l0.norm1"].fill_(1.0)
        for tok, ch in ((B_TOK, 0), (A_TOK, 1)):
            t["embed"][tok] = 0
            t["embed"][tok, ch] = 1.0
        p = "l0.mix."
        t[p + "q.norm"].fill_(1.0)
        t[p + "k.norm"].fill_(1.0)
        t[p + "sink"].fill_(sink)
        u = torch.zeros(dim, device="cuda")
        u[rot:] = torch.randn(dim - rot, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
        for c in range(2):
            t[p + "k"][dim * c:dim * (c + 1), 1] = u.to(t[p + "k"].dtype)
            t[p + "q"][dim * 2 * c:dim * (2 * c + 1), 0] = u.to(t[p + "q"].dtype)
    eng, cpu = build(cfg, dtype, seed=seed, tweak=tweak)
    return cfg, eng, cpu


def _check_last(cfg, eng, cpu, toks, dtype, at, matters):
    """The last token's logits in a whole prompt and decoded alone, against the oracle; `matters`: whether replacing the
    planted token (at `at`) must move them."""
    want = oracle_logits(cfg, cpu, toks)
    without = list(toks)
    without[at] = 59
    moved = err(oracle_logits(cfg, cpu, without)[-1:], want[-1:])
    assert (moved > 4 * TOL[dtype]) if matters else (moved < 1e-9), moved
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole[-1:], want[-1:]) < TOL[dtype]
    stream = eng.begin_stream(torch.tensor([toks[:-1]], device="cuda"), None, max_length=len(toks) + 3, eos_token_id=-1)
    stream.step(feed([toks[-1]]))
    assert err(stream.logits()[:1], want[-1:]) < TOL[dtype]
    stream.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 1, 31, 32, 33, 63, 64, 290])
def test_one_far_key_decides(dtype, far):
    """Attention without blocks: the planted key stands once at position `far` among 300 random ones and B is the last
    token.  A kernel that drops or misplaces it (edges of the 32-key tiles, the first slots, hundreds back) moves the
    logits far beyond the tolerance."""
    cfg, eng, cpu = _planted_attention(0, dtype)
    toks = [2 + (i % 50) for i in range(300)]
    toks[far] = A_TOK
    toks.append(B_TOK)
    _check_last(cfg, eng, cpu, toks, dtype, far, True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [2, 24, 32, 33, 70])
@pytest.mark.parametrize("where", ["first_of_block", "last_of_previous", "next", "far_outside", "query_opens_a_block"])
def test_block_edge_decides(dtype, chunk, where):
    """The planted key stands on the first position of the query's block, on the last of the block before, right before
    the query, or far behind; or the query itself opens a block and sees nothing but itself.  Attention is all that reaches
    back in this model, so a key outside the block must not matter at all."""
    n = 200 if where != "query_opens_a_block" else (200 // chunk) * chunk        # the query's position
    start = n // chunk * chunk
    at = {"first_of_block": start, "last_of_previous": start - 1, "next": n - 1, "far_outside": start - 64,
          "query_opens_a_block": n - 1}[where]
    if at == n:                                                                  # a block of one position: there is no key before the query in it
        at = n - 1
    cfg, eng, cpu = _planted_attention(chunk, dtype)
    toks = [2 + (i % 50) for i in range(n)]
    toks[at] = A_TOK
    toks.append(B_TOK)
    _check_last(cfg, eng, cpu, toks, dtype, at, start <= at < n)


@pytest.mark.parametrize("chunk", [0, 24, 33, 64, 70, 128, 200])
@pytest.mark.parametrize("where", ["first_of_block", "last_of_previous", "next", "far_outside", "query_opens_a_block"])
def test_block_edge_decides_on_the_tensor_core_path(chunk, where):
    """The same planted key with 128-wide keys and values in bfloat16, where prompts run the tcgen05 kernel: blocks that end
    inside a key tile or a query tile, three query tiles, the sink and the gate in the kernel's epilogue."""
    n = 300 if where != "query_opens_a_block" or not chunk else (300 // chunk) * chunk
    size = chunk or 10 ** 6
    start = n // size * size
    at = {"first_of_block": start, "last_of_previous": max(start - 1, 0), "next": n - 1, "far_outside": max(start - 64, 0),
          "query_opens_a_block": n - 1}[where]
    at = min(at, n - 1)
    cfg, eng, cpu = _planted_attention(chunk, torch.bfloat16, sink=22.0, dim=128, vdim=128, rot=64)
    assert eng.layers[0].mixer._flash_masked_shape()
    toks = [2 + (i % 50) for i in range(n)]
    toks[at] = A_TOK
    toks.append(B_TOK)
    _check_last(cfg, eng, cpu, toks, torch.bfloat16, at, start <= at < n)
    want = oracle_logits(cfg, cpu, toks)
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole, want) < TOL[torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoded_queries_leave_the_planted_key_behind(dtype):
    """The planted key is in the prompt; B is then decoded again and again: A is seen until the query's position enters
    the next block."""
    chunk = 12
    cfg, eng, cpu = _planted_attention(chunk, dtype)
    toks = [2 + (i % 50) for i in range(40)] + [A_TOK] + [B_TOK] * 20            # A at 40: block 36 .. 47
    want = oracle_logits(cfg, cpu, toks)
    other = list(toks)
    other[40] = 59
    moved = [err(a[None], b[None]) for a, b in zip(oracle_logits(cfg, cpu, other), want)]
    assert all(m > 4 * TOL[dtype] for m in moved[41:48]) and all(m < 1e-9 for m in moved[48:])
    stream = eng.begin_stream(torch.tensor([toks[:41]], device="cuda"), None, max_length=70, eos_token_id=-1)
    rows = []
    for t in toks[41:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[41:]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sink", [-30.0, 20.0, 27.0, 60.0])
def test_the_sink_takes_the_weight_of_the_planted_key(dtype, sink):
    """A sink logit far below the planted score changes nothing, one near it shares the weight, one far above takes all of
    it: the heads' outputs scale accordingly (the logit is a number of its own, not scaled, and counts once)."""
    cfg, eng, cpu = _planted_attention(0, dtype, sink=sink)
    toks = [2 + (i % 50) for i in range(90)]
    toks[17] = A_TOK
    toks.append(B_TOK)
    want = oracle_logits(cfg, cpu, toks)
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole, want) < TOL[dtype]
    stream = eng.begin_stream(torch.tensor([toks[:-1]], device="cuda"), None, max_length=len(toks) + 3, eos_token_id=-1)
    stream.step(feed([toks[-1]]))
    assert err(stream.logits()[:1], want[-1:]) < TOL[dtype]
    stream.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_values_turn_with_the_distance(dtype):
    """The planted value reaches the query turned by their distance: the same key two positions further back gives other
    logits (the oracle says how much), and the engine follows in prompts and in decoding."""
    cfg, eng, cpu = _planted_attention(0, dtype)
    base = [2 + (i % 50) for i in range(80)]
    outs = []
    for at in (70, 68):
        toks = list(base)
        toks[at] = A_TOK
        toks.append(B_TOK)
        want = oracle_logits(cfg, cpu, toks)
        outs.append(want[-1])
        _check_last(cfg, eng, cpu, toks, dtype, at, True)
    assert err(outs[0][None], outs[1][None]) > 4 * TOL[dtype]


# ------------------------------------------------------------------------------------------ the framework's entry points
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_front_end(dtype, tmp_path):
    """save_pretrained → registry → `LLaMA.generate_from_str` (left-padded batch, scheduler, on-device arg-max): every
    generated token is the oracle's arg-max given its prefix, up to near-ties."""
    from jax_llama_b200.models import registry

    cfg = config(MIXED, vocab=80, loop=(1, 3, 2), dtype=dtype)
    model = DatozenForCausalLM(cfg, dtype=dtype, seed=12, _do_init=True)
    model.save_pretrained(str(tmp_path))
    assert registry.resolve(str(tmp_path))[0] == "datozen"
    loaded = registry.load_pretrained(str(tmp_path), dtype=dtype, device="cuda")
    assert isinstance(loaded, DatozenForCausalLM) and loaded.config.to_dict() == cfg.to_dict()
    llm = LLaMA(loaded.params, loaded, IdTokenizer(cfg.vocab_size))
    prompts = ["7 8 9 10 11 12", "40", "3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3"]
    texts = llm.generate_from_str(prompts, max_gen_len=24, temperature=0.0)
    cpu = {k: v.cpu() for k, v in loaded.params.items()}
    for p, t in zip(prompts, texts):
        ids = [int(x) for x in t.split()]
        n0 = len(p.split()) + 1
        assert ids[:n0] == [1] + [int(x) for x in p.split()]
        assert len(ids) > n0
        want = oracle_logits(cfg, cpu, ids)
        for j in range(n0, len(ids)):
            row = want[j - 1]
            assert row[ids[j]] >= row.max() - (1e-3 if dtype == torch.float32 else 0.15), (p, j)
    sampled = llm.generate_from_str(prompts[:1], max_gen_len=8, temperature=0.9, top_p=0.9)
    assert len(sampled[0].split()) >= 7


def test_command_line_generates_from_a_checkpoint_directory(tmp_path):
    """examples/example.py --model_dir: registry, loader, engine, scheduler and sampler behind the command line."""
    cfg = config(MIXED, vocab=80, loop=(1, 3, 2))
    DatozenForCausalLM(cfg, seed=3, _do_init=True).save_pretrained(str(tmp_path))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "example.py"), "--model_dir", str(tmp_path), "--prompt",
                        "7 8 9", "--prompt", "40", "--max_gen_len", "6", "--temperature", "0"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip() and not l.startswith("=")]
    assert lines[0].split()[:4] == ["1", "7", "8", "9"] and lines[1].split()[:2] == ["1", "40"]
    assert all(0 <= int(t) < 80 for l in lines[:2] for t in l.split())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_batches_that_come_and_go(dtype, tmp_path):
    """bin/trace_run on a saved checkpoint: a request alone, a batch of three unequal requests decoded together while its
    shorter ones end, a second batch that opens while the first is still live, a prompt as long as the position table;
    every wanted row against the oracle of that request alone."""
    import numpy as np

    cfg = config(MIXED, vocab=80, loop=(1, 3, 2), positions=48, dtype=getattr(torch, dtype))
    model = DatozenForCausalLM(cfg, seed=5, _do_init=True)
    model.save_pretrained(str(tmp_path / "m"))
    cpu = {k: v.cpu() for k, v in model.params.items()}
    seq = {"a": tokens(30, 80, 1), "b": tokens(12, 80, 2), "c": tokens(47, 80, 3), "d": tokens(9, 80, 4), "e": tokens(26, 80, 5),
           "f": tokens(48, 80, 6)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": seq["a"][:25], "want": [0, 24]}], "end": []}]
    for j in range(25, 30):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [seq["a"][j]], "want": [0] if j % 2 else []}],
                      "end": ["a"] if j == 29 else []})
    steps.append({"step": len(steps), "entries": [{"id": "b", "tokens": seq["b"][:9], "want": [8]},
                                                   {"id": "c", "tokens": seq["c"][:41], "want": list(range(0, 41, 5))},
                                                   {"id": "d", "tokens": seq["d"][:6], "want": []}], "end": []})
    for j in range(3):
        live = [("b", 9 + j, 12), ("c", 41 + j, 47), ("d", 6 + j, 9)]
        ent = [{"id": r, "tokens": [seq[r][at]], "want": [0]} for r, at, n in live]
        steps.append({"step": len(steps), "entries": ent, "end": [r for r, at, n in live if at == n - 1]})
    steps.append({"step": len(steps), "entries": [{"id": "e", "tokens": seq["e"][:20], "want": [19]},
                                                   {"id": "a2", "tokens": seq["a"][:3], "want": [2]}], "end": ["a2"]})
    for j in range(6):
        ent = [{"id": "e", "tokens": [seq["e"][20 + j]], "want": [0]}]
        if j < 3:
            ent.insert(0, {"id": "c", "tokens": [seq["c"][44 + j]], "want": [0]})
        steps.append({"step": len(steps), "entries": ent, "end": (["c"] if j == 2 else []) + (["e"] if j == 5 else [])})
    steps.append({"step": len(steps), "entries": [{"id": "f", "tokens": seq["f"], "want": [0, 47]}], "end": ["f"]})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out",
                        str(out), "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    seq["a2"] = seq["a"]
    full = {k: oracle_logits(cfg, cpu, v) for k, v in seq.items()}
    at = {k: 0 for k in seq}
    bound = tol(getattr(torch, dtype), cfg)
    for s in steps:
        want = []
        for e in s["entries"]:
            want += [full[e["id"]][at[e["id"]] + w] for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        path = out / f"{s['step']}.f32"
        if not want:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(want), 80).copy())
        assert err(got, torch.stack(want)) < bound, s["step"]
