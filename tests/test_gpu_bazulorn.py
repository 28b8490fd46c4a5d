"""Bazulorn on the hybrid engine against the plain float64 statement of the design (`bazulorn_oracle.py`).

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

from jax_llama_b200.config import BazulornConfig                                  # noqa: E402
from jax_llama_b200.generation import LLaMA                                       # noqa: E402
from jax_llama_b200.models.bazulorn import BazulornForCausalLM                    # noqa: E402
from jax_llama_b200.models.hybrid_engine import HybridEngine, random_tensors      # noqa: E402
from jax_llama_b200.ops import seq_kernels as SK                                  # noqa: E402
from jax_llama_b200.tokenizers import IdTokenizer                                 # noqa: E402

from tests import bazulorn_oracle as O                                            # noqa: E402

TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, limit=1.5, shared=16, shared_limit=0.75):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared, "limit": shared_limit}
    return m


def par(heads=4, kv_heads=2, dim=16, vdim=12, window=20, scale=0.3, s_heads=4, s_vdim=8, state=16, groups=2, conv=4,
        norm_groups=2, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        left["mask"] = {"size": window}
    right = {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=16, vdim=12, conv=4, mlp=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def config(layers, vocab=96, width=72, eps=1e-5, buckets=61, mul_prev=37, mul_cur=11, dtype=None):
    """With dtype bfloat16 every expert of a layer is chosen (top = experts): rounding the router's input to bfloat16
    moves its logits by parts in a thousand, which among random logits flips a close choice every few dozen tokens, and
    the oracle would then follow other experts.  The choice itself is checked in float32 and on the router alone."""
    layers = json.loads(json.dumps(layers))
    if dtype == torch.bfloat16:
        for l in layers:
            if l["mlp"] is not None and l["mlp"]["kind"] == "moe":
                l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
    return BazulornConfig.from_dict({"architecture": "Bazulorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
                                     "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
                                     "layers": layers})


MIXED = [delta(mlp=dense()), par(mlp=moe()), delta(heads=3, kv_heads=3, dim=8, vdim=20, conv=3, mlp=moe(experts=4, top=1, shared=0)),
         par(heads=3, kv_heads=3, dim=8, vdim=24, window=0, s_heads=3, s_vdim=12, state=8, groups=1, conv=2, norm_groups=1)]


def build(cfg, dtype, seed=0, graph=True, tweak=None, rank=5):
    tensors = random_tensors(cfg, "cuda", seed, decay_rank=rank)
    g = torch.Generator(device="cuda").manual_seed(seed + 1000)
    for name in list(tensors):
        if name.endswith(".out") or name.endswith("mix.norm"):            # branch norms and head norms around one
            tensors[name] = (1.0 + 0.2 * torch.randn(tensors[name].shape, device="cuda", generator=g)).to(torch.bfloat16)
        if name.endswith("A_log"):                                       # decays from fast to slow
            tensors[name] = (torch.rand(tensors[name].shape, device="cuda", generator=g) * 4.0 - 3.0).to(torch.bfloat16)
        if name.endswith(".b") or name.endswith("dt_bias") or name.endswith(".D"):
            tensors[name] = (0.5 * torch.randn(tensors[name].shape, device="cuda", generator=g)).to(torch.bfloat16)
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
def test_pair_embedding_with_padding_and_carried_token(dtype):
    """Two rows, one left-padded by three; the prompt, then two single tokens: the hashed row follows the previous token
    across calls, a sequence's first token takes the table's last row, padding rows are zero."""
    V, W, n, mp, mc = 50, 40, 13, 1000003, 77
    g = torch.Generator().manual_seed(1)
    t = {"embed": torch.randn(V, W, generator=g).to(torch.bfloat16), "bigram": torch.randn(n + 1, W, generator=g).to(torch.bfloat16),
         "embed.norm": (1 + 0.1 * torch.randn(W, generator=g)).to(torch.bfloat16)}
    cfg = {"embedding": {"bigram": {"buckets": n, "mul_prev": mp, "mul_cur": mc}}, "norm": {"eps": 1e-5}}
    seqs = [tokens(8, V, 2), tokens(5, V, 3)]
    d = {k: v.cuda().to(dtype) for k, v in t.items()}
    prev, length, pad = i32([7, 7]), i32([0]), i32([0, 3])
    ids = torch.zeros(2, 6, dtype=torch.int32)
    ids[0] = torch.tensor(seqs[0][:6])
    ids[1, 3:] = torch.tensor(seqs[1][:3])
    got = [SK.embed_pair_norm(ids.cuda(), d["embed"], d["bigram"], d["embed.norm"], prev, length, pad, 2, 6, n, mp, mc, 1e-5)]
    for j in range(2):
        length.fill_(6 + j)
        got.append(SK.embed_pair_norm(i32([seqs[0][6 + j], seqs[1][3 + j]]), d["embed"], d["bigram"], d["embed.norm"], prev,
                                      length, pad, 2, 1, n, mp, mc, 1e-5))
    want = [O.embed_tokens(s, t, cfg) for s in seqs]
    x = got[0].view(2, 6, W).double().cpu()
    assert (x[0] - want[0][:6]).abs().max() < 1e-5 and (x[1, 3:] - want[1][:3]).abs().max() < 1e-5
    assert x[1, :3].abs().max() == 0
    for j in range(2):
        y = got[1 + j].double().cpu()
        assert (y[0] - want[0][6 + j]).abs().max() < 1e-5 and (y[1] - want[1][3 + j]).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("cuts", [[150], [1, 1, 1, 1, 1, 1, 1, 1, 1], [2, 5, 1, 70, 3], [65, 64, 2]])
def test_causal_convolution_with_state(dtype, taps, cuts):
    """The convolution over a sequence fed in portions (its last taps − 1 inputs carried as state) equals the one over
    the whole; a second row is left-padded in the first portion.  Portions shorter than the filter, of one token, and
    longer than a CTA's time chunk."""
    C, B, extra = 37, 2, 4
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g).to(torch.bfloat16)
    bias = torch.randn(C, generator=g).to(torch.bfloat16)
    T = sum(cuts)
    pad = min(cuts[0] - 1, 5)
    x = torch.randn(B, T, C + extra, generator=g)
    want = [O.silu(O.causal_conv(x[0, :, extra:].double(), w.double(), bias.double())),
            O.silu(O.causal_conv(x[1, pad:, extra:].double(), w.double(), bias.double()))]
    state = torch.zeros(B, max(taps - 1, 1), C, device="cuda")
    length, padl = i32([0]), i32([0, pad])
    got, at = [], 0
    for n in cuts:
        y = x[:, at:at + n].reshape(B * n, C + extra).cuda().contiguous()
        length.fill_(at)
        got.append(SK.causal_conv(y, extra, w.cuda().to(dtype), bias.cuda().to(dtype), state, length, padl, B, n).view(B, n, C))
        at += n
    got = torch.cat(got, 1).double().cpu()
    assert (got[0] - want[0]).abs().max() < 1e-5
    assert (got[1, pad:] - want[1]).abs().max() < 1e-5 and (pad == 0 or got[1, :pad].abs().max() == 0)


def test_small_kernels_around_the_mixers():
    """norm_mean2, gated_groupnorm, both gated activations and the mix of per-head weighted sums against float64."""
    g = torch.Generator().manual_seed(3)
    M, W = 5, 70
    a, b = torch.randn(M, W, generator=g), torch.randn(M, W, generator=g) * 3
    wa, wb = torch.randn(W, generator=g), torch.randn(W, generator=g)
    got = SK.norm_mean2(a.cuda(), wa.cuda(), b.cuda(), wb.cuda(), 0.5, 1e-3)
    want = 0.5 * (O.rms_norm(a.double(), wa.double(), 1e-3) + O.rms_norm(b.double(), wb.double(), 1e-3))
    assert (got.double().cpu() - want).abs().max() < 1e-5
    H, P, groups = 6, 10, 3
    o, x, z = (torch.randn(M, H * P, generator=g) for _ in range(3))
    skip, w = torch.randn(H, generator=g), torch.randn(H * P, generator=g)
    got = SK.gated_groupnorm(o.cuda(), x.cuda(), skip.cuda(), P, z.cuda(), w.cuda(), groups, 1e-2)
    v = (o.double() + skip.double().repeat_interleave(P) * x.double()) * O.silu(z.double())
    want = O.rms_norm(v.view(M, groups, -1), None, 1e-2).reshape(M, -1) * w.double()
    assert (got.double().cpu() - want).abs().max() < 1e-5
    F = 9
    y = torch.randn(M, 2 * F + 3, generator=g) * 2
    got = SK.glu_act(y.cuda(), 0, F + 3, F, torch.float32, kind=SK.GLU_CLAMPED, limit=0.8, alpha=1.702)
    ga, u = y[:, :F].double().clamp(max=0.8), y[:, F + 3:].double().clamp(-0.8, 0.8)
    assert (got.double().cpu() - ga * torch.sigmoid(1.702 * ga) * (u + 1)).abs().max() < 1e-6
    got = SK.glu_act(y.cuda(), 0, F + 3, F, torch.float32, kind=SK.GLU_PRODUCT, act=SK.ACT_GELU_TANH)
    assert (got.double().cpu() - O.gelu_tanh(y[:, :F].double()) * y[:, F + 3:].double()).abs().max() < 1e-6
    Hh, G, Dv = 6, 3, 5
    part = torch.randn(M, Hh, G, Dv, generator=g)
    mix = torch.randn(Hh, Hh, generator=g)
    out = torch.zeros(M, Hh * Dv, device="cuda")
    for c0, gc in ((0, 2), (2, 1)):                                       # value heads two at a time, then the last
        SK.talk_mix(part[:, :, c0:c0 + gc].contiguous().cuda(), mix.cuda(), out, Hh, G, gc, c0, Dv)
    want = torch.stack([torch.einsum("g,mgd->md", mix[h].double(), part[:, :, h // 2].double()) for h in range(Hh)], 1)
    assert (out.double().cpu().view(M, Hh, Dv) - want).abs().max() < 1e-5


@pytest.mark.parametrize("experts,top", [(6, 2), (5, 1), (7, 7), (40, 3)])
def test_router_with_bias(experts, top):
    g = torch.Generator().manual_seed(experts)
    M, W = 33, 24
    h = torch.randn(M, W, generator=g)
    t = {"r.router": torch.randn(experts, W, generator=g), "r.router.b": torch.randn(experts, generator=g)}
    z = (h @ t["r.router"].T).cuda().contiguous()
    idx, wt = SK.moe_route(z, experts, top, 1, 1, 2, SK.SCORE_SOFTMAX, True, 1.0, bias=t["r.router.b"].cuda())
    widx, wwt = O.route(h.double(), t, "r.", top)
    order = idx.cpu().long().argsort(-1)
    worder = widx.argsort(-1)
    assert torch.equal(idx.cpu().long().gather(1, order), widx.gather(1, worder))
    assert (wt.cpu().double().gather(1, order) - wwt.gather(1, worder)).abs().max() < 1e-5


SINGLE = {
    "delta_alone": [delta()],
    "delta_one_qk_head_wide_keys": [delta(heads=3, kv_heads=1, dim=80, vdim=10, conv=2)],
    "delta_key_of_33": [delta(heads=2, kv_heads=2, dim=33, vdim=7, conv=1)],
    "delta_keys_above_256": [delta(heads=1, kv_heads=1, dim=264, vdim=6, conv=2)],
    "attention_and_state_space": [par()],
    "one_kv_head_window_one": [par(heads=4, kv_heads=1, dim=8, vdim=16, window=1, s_heads=2, groups=2, norm_groups=4)],
    "no_window_one_group": [par(heads=2, kv_heads=2, dim=24, vdim=8, window=0, s_heads=6, s_vdim=4, state=40, groups=1, conv=3,
                                norm_groups=1)],
    "wide_value_rows": [par(heads=6, kv_heads=6, dim=8, vdim=96, window=9, s_heads=1, s_vdim=8, state=8, groups=1, norm_groups=1)],
    "dense_ff": [delta(mlp=dense(ff=50))],
    "experts_top_one_no_shared": [delta(mlp=moe(experts=5, top=1, ff=10, shared=0))],
    "experts_all_chosen": [par(mlp=moe(experts=3, top=3, ff=8, limit=0.2, shared=40, shared_limit=5.0))],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_single_mechanism_models(dtype, name):
    """One layer of each kind with sizes that the usual configurations make equal or one (one key/value head, a window
    of one, no window, value rows above the attention kernel's width, keys above 32 channels, one tap)."""
    cfg = config(SINGLE[name], dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=3)
    toks = tokens(45, cfg.vocab_size, 9)
    assert err(eng.forward(torch.tensor([toks], device="cuda")).logits[0], oracle_logits(cfg, cpu, toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_stream_after_every_layer(dtype):
    cfg = config(MIXED, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=2)
    toks = tokens(40, cfg.vocab_size, 7)
    eng.capture_streams = []
    eng.forward(torch.tensor([toks], device="cuda"))
    want = []
    oracle_logits(cfg, cpu, toks, want)
    assert len(eng.capture_streams) == len(want) == len(MIXED)
    for i, (g, w) in enumerate(zip(eng.capture_streams, want)):
        assert g.dtype == torch.float32
        assert (g.double().cpu() - w).abs().max() < (1e-4 if dtype == torch.float32 else 5e-2) * w.abs().max(), i


def test_other_constants():
    """eps, score scale, limits, hash multipliers and table size far from the usual values."""
    layers = [par(window=3, scale=2.5, conv=5, mlp=moe(limit=0.05, shared_limit=9.0)), delta(conv=8, mlp=dense(ff=8))]
    cfg = config(layers, eps=0.3, buckets=3, mul_prev=2 ** 31 - 1, mul_cur=99991, vocab=77, width=90)
    eng, cpu = build(cfg, torch.float32, seed=11)
    toks = tokens(50, cfg.vocab_size, 4)
    assert err(eng.forward(torch.tensor([toks], device="cuda")).logits[0], oracle_logits(cfg, cpu, toks)) < TOL[torch.float32]


# ------------------------------------------------------------------------------------------ prefill vs decoding
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("prompt", [1, 2, 31, 33])
def test_decode_matches_prefill_and_oracle(dtype, prompt):
    """The prompt in one step, then 70 tokens one by one through the graph-replayed step: the window passes over decoded
    tokens, the convolutions' state, the 32-key blocks of the attention kernels and the first tokens of a sequence
    (where the sink holds most of the weight) are all crossed."""
    cfg = config(MIXED, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=4)
    toks = tokens(prompt + 70, cfg.vocab_size, prompt)
    want = oracle_logits(cfg, cpu, toks)
    stream = eng.begin_stream(torch.tensor([toks[:prompt]], device="cuda"), None, max_length=len(toks) + 1, eos_token_id=-1,
                              logit_rows=torch.arange(prompt))
    assert err(stream.prompt_logits(), want[:prompt]) < TOL[dtype]
    rows = []
    for t in toks[prompt:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    assert err(torch.stack(rows), want[prompt:]) < TOL[dtype]
    stream.close()
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole, want) < TOL[dtype]
    if dtype == torch.float32:
        assert err(torch.stack(rows), whole[prompt:]) < 5e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """Three hundred tokens decoded one by one after a two-token prompt."""
    cfg = config([delta(mlp=moe()), par(window=40, mlp=moe(shared=0))], dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=21)
    toks = tokens(302, cfg.vocab_size, 5)
    want = oracle_logits(cfg, cpu, toks)
    stream = eng.begin_stream(torch.tensor([toks[:2]], device="cuda"), None, max_length=310, eos_token_id=-1)
    rows = [stream.logits()[0].clone()]
    for t in toks[2:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[1:]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 30], [33, 2, 9], [5, 64, 3], [1, 2, 200]])
def test_prompt_in_portions(dtype, cuts):
    """The same prompt fed to one cache in portions of several sizes, down to two tokens (and one)."""
    cfg = config(MIXED, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=14)
    toks = tokens(sum(cuts), cfg.vocab_size, 31)
    want = oracle_logits(cfg, cpu, toks)
    cache = eng.new_cache(1, len(toks) + 2)
    cache.set_index(0)
    got, at = [], 0
    for n in cuts:
        got.append(eng.forward(torch.tensor([toks[at:at + n]], device="cuda"), cache=cache).logits[0])
        at += n
    assert err(torch.cat(got), want) < TOL[dtype]


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
        assert err(got_prompt[at:at + n], want[:n]) < TOL[dtype], b
        assert err(torch.stack([x[b] for x in steps]), want[n:]) < TOL[dtype], b
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_equals_each_alone(dtype):
    """Prompts of 1, 7 and 40 tokens in one batch: padding must touch neither the recurrent states, the convolutions'
    inputs, the hashed embedding row, the visible keys and the window, nor the choice of experts of the real tokens."""
    run_unequal_batch(config(MIXED, dtype=dtype), dtype, [1, 7, 40], 36, seed=6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_odd_sizes_and_a_batch_of_twenty(dtype):
    """Sizes that fit no vector width or tile in a batch of twenty unequal requests: more rows than the pairwise expert
    path and the weight-streaming kernel take, so decoding runs the sorted experts and the GEMMs."""
    layers = [par(heads=3, kv_heads=3, dim=10, vdim=14, window=9, s_heads=3, s_vdim=6, state=10, groups=3, conv=3, norm_groups=3,
                  mlp=moe(experts=9, top=2, ff=10, shared=6)),
              delta(heads=3, kv_heads=1, dim=12, vdim=10, conv=2, mlp=moe(experts=3, top=1, ff=5, shared=0))]
    cfg = config(layers, vocab=77, width=90, dtype=dtype)
    run_unequal_batch(cfg, dtype, [3, 17, 1, 9, 30, 2, 12, 25, 8, 21, 4, 5, 6, 7, 11, 13, 14, 15, 16, 29], 12, seed=17)


@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_rule_in_a_grid_that_fills_the_gpu(dtype):
    """Twenty rows of 64 x 64 heads: the scan then keeps 32 key channels per thread instead of 8 (prompt and decoding)."""
    cfg = config([delta(heads=4, kv_heads=2, dim=64, vdim=64, mlp=dense(ff=24))], dtype=dtype)
    run_unequal_batch(cfg, dtype, [3, 17, 1, 9, 30, 2, 12, 25, 8, 21, 4, 5, 6, 7, 11, 13, 14, 15, 16, 29], 10, seed=19)


def test_realistic_head_sizes():
    """64-wide attention heads, state space heads of 64 x 64 with a state of 128, delta-rule heads of 128 x 64."""
    layers = [par(heads=4, kv_heads=2, dim=64, vdim=64, window=48, s_heads=4, s_vdim=64, state=128, groups=1, mlp=moe(ff=64)),
              delta(heads=4, kv_heads=2, dim=128, vdim=64, mlp=dense(ff=256))]
    run_unequal_batch(config(layers, width=256, vocab=128, dtype=torch.bfloat16), torch.bfloat16, [5, 150, 131], 40, seed=13)


def test_state_and_cache_are_clean_when_used_again():
    """The same decode state serves request after request: a second, shorter request must see nothing of the first
    (recurrent and convolution states zeroed, old keys invisible, old left-pad counts and previous tokens gone)."""
    cfg = config(MIXED)
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


def _bare_input(t, width):
    """No hashed rows, unit norms before the mixer, and unit-vector embeddings for tokens A (channel 1) and B (channel 0):
    the mixer of layer 0 then sees sqrt(width) times one column of each projection for them."""
    t["bigram"].zero_()
    t["embed.norm"].fill_(1.0)
    t["l0.norm1"].fill_(1.0)
    for tok, ch in ((B_TOK, 0), (A_TOK, 1)):
        t["embed"][tok] = 0
        t["embed"][tok, ch] = 1.0


def _planted_attention(window, dtype, seed=5):
    """Token A's key, in every key/value head, is a multiple of token B's query in the first query head of that group:
    when B asks, A's single key takes nearly all of those heads' weight among hundreds of random keys."""
    layer = par(heads=4, kv_heads=2, dim=16, vdim=12, window=window, scale=1.0)
    cfg = config([layer], vocab=64, width=48)

    def tweak(t):
        _bare_input(t, 48)
        _state_space_off(t)
        p = "l0.mix.left."
        for n in ("q.b", "k.b"):
            t[p + n].zero_()
        q_col = t[p + "q"][:, 0].float().view(4, 16)                    # B's query per head, up to sqrt(width)
        for c in range(2):
            qc = q_col[2 * c]
            t[p + "k"][16 * c:16 * (c + 1), 1] = (qc / (qc @ qc) * (20.0 / 48.0)).to(t[p + "k"].dtype)     # score(B -> A) = 20
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


def _state_space_off(t):
    """The right-hand mixer's state would also carry the planted token: switch its output off so that only the attention
    can tell whether the token is there."""
    t["l0.mix.right.o"].zero_()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 1, 31, 32, 33, 63, 64, 290])
def test_one_far_key_decides(dtype, far):
    """Attention without a window: the planted key stands once at position `far` among 300 random ones and B is the last
    token.  A kernel that drops or misplaces it (edges of the 32-key blocks, the first slots, hundreds back) moves the
    logits far beyond the tolerance."""
    cfg, eng, cpu = _planted_attention(0, dtype)
    toks = [2 + (i % 50) for i in range(300)]
    toks[far] = A_TOK
    toks.append(B_TOK)
    _check_last(cfg, eng, cpu, toks, dtype, far, True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [2, 24, 32, 33, 70])
@pytest.mark.parametrize("back", ["inside", "outside", "next", "far_outside"])
def test_window_edge_decides(dtype, window, back):
    """The planted key stands on the last position the window still shows, on the first it hides, right before the
    query, or far behind the window.  The state space half is switched off and the convolution-free attention is then
    all that reaches back, so a key outside the window must not matter at all."""
    d = {"inside": window - 1, "outside": window, "next": 1, "far_outside": window + 64}[back]
    layer = par(heads=4, kv_heads=2, dim=16, vdim=12, window=window, scale=1.0)
    cfg = config([layer], vocab=64, width=48)

    def tweak(t):
        _bare_input(t, 48)
        _state_space_off(t)
        p = "l0.mix.left."
        for n in ("q.b", "k.b"):
            t[p + n].zero_()
        q_col = t[p + "q"][:, 0].float().view(4, 16)
        for c in range(2):
            qc = q_col[2 * c]
            t[p + "k"][16 * c:16 * (c + 1), 1] = (qc / (qc @ qc) * (20.0 / 48.0)).to(t[p + "k"].dtype)
    eng, cpu = build(cfg, dtype, seed=5, tweak=tweak)
    n = 200
    toks = [2 + (i % 50) for i in range(n)]
    toks[n - d] = A_TOK
    toks.append(B_TOK)
    _check_last(cfg, eng, cpu, toks, dtype, n - d, d < window)


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_slides_over_decoded_tokens(dtype):
    """The planted key is in the prompt; B is then decoded again and again: A is seen until it leaves the window."""
    window = 12
    cfg, eng, cpu = _planted_attention(window, dtype)
    toks = [2 + (i % 50) for i in range(40)] + [A_TOK] + [B_TOK] * 20
    want = oracle_logits(cfg, cpu, toks)
    assert err(want[41 + window - 2:41 + window - 1], want[41 + window - 1:41 + window]) > 10 * TOL[dtype]   # A leaves here
    stream = eng.begin_stream(torch.tensor([toks[:41]], device="cuda"), None, max_length=70, eos_token_id=-1)
    rows = []
    for t in toks[41:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[41:]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_the_weight_of_unwelcome_keys(dtype):
    """All scores far below zero (the keys' bias points against the queries' bias): nearly all weight goes to the sink and
    the attention's output nearly vanishes; a softmax without the sink would return an average of the values instead."""
    cfg = config([par(heads=2, kv_heads=2, dim=8, vdim=8, window=0, scale=1.0)], vocab=64, width=48)

    def tweak(t):
        p = "l0.mix.left."
        t[p + "q"].mul_(0.05)
        t[p + "k"].mul_(0.05)
        t[p + "q.b"].fill_(1.5)
        t[p + "k.b"].fill_(-1.5)                                         # every score is about -18
    eng, cpu = build(cfg, dtype, seed=9, tweak=tweak)
    toks = tokens(40, 64, 3)
    want = oracle_logits(cfg, cpu, toks)
    no_sink = {k: v.clone() for k, v in cpu.items()}
    no_sink["l0.mix.left.k.b"].fill_(1.5)                                # welcome keys: the values come through
    assert err(oracle_logits(cfg, no_sink, toks), want) > 4 * TOL[dtype]
    assert err(eng.forward(torch.tensor([toks], device="cuda")).logits[0], want) < TOL[dtype]


def _slow_memory(kind):
    """One layer whose recurrence forgets slowly; the filler token writes nothing into the state."""
    if kind == "delta":
        return [delta(heads=2, kv_heads=2, dim=16, vdim=16, conv=1)]
    return [par(heads=2, kv_heads=2, dim=8, vdim=8, window=1, s_heads=2, s_vdim=16, state=16, groups=1, conv=1, norm_groups=1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["delta", "state_space"])
@pytest.mark.parametrize("gap", [2, 7, 15, 16, 17, 216])
def test_recurrent_state_keeps_a_far_token(dtype, kind, gap):
    """Slow decays and a filler token whose key (delta rule) or input (state space layer) is cut to zero, so the state
    holds only what two planted tokens wrote, `gap` steps and one step back.  Read-outs are normed, so one token alone
    would hide a wrong decay; the mix of the two shows decay^(gap−1): a state that is lost, reset or decayed wrongly at an
    edge of the scan's token chunks moves the logits.  In a prompt and decoded token by token."""
    filler, first, second = 5, 40, 41
    cfg = config(_slow_memory(kind), vocab=64, width=48)

    def tweak(t):
        t["bigram"].zero_()
        t["embed.norm"].fill_(1.0)
        t["l0.norm1"].fill_(1.0)
        t["embed"][filler] = 0
        t["embed"][filler, 3] = 1.0
        if kind == "delta":
            t["l0.mix.A_log"].fill_(-7.0)
            t["l0.mix.v"][:, 3] = 0                                      # silu(0) = 0: the filler corrects towards nothing ...
            t["l0.mix.b"][:, 3] = -30.0                                  # ... with beta = 0
        else:
            t["l0.mix.right.A_log"].fill_(-7.0)
            t["l0.mix.right.in"][32:64, 3] = 0                           # the filler's x: nothing is written
            t["l0.mix.right.conv.b"].zero_()
            t["l0.mix.left.o"].zero_()
    eng, cpu = build(cfg, dtype, seed=7, tweak=tweak)
    n = 230
    toks = [filler] * n
    toks[n - 1 - gap], toks[n - 2] = first, second
    want = oracle_logits(cfg, cpu, toks)
    other = list(toks)
    other[n - 1 - gap] = first + 2
    assert err(oracle_logits(cfg, cpu, other)[-1:], want[-1:]) > 3 * TOL[dtype]
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got[n - 1 - gap:], want[n - 1 - gap:]) < TOL[dtype]
    cut = 10
    stream = eng.begin_stream(torch.tensor([toks[:cut]], device="cuda"), None, max_length=n + 2, eos_token_id=-1)
    rows = []
    for t in toks[cut:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows)[n - 1 - gap - cut:], want[n - 1 - gap:]) < TOL[dtype]


# ------------------------------------------------------------------------------------------ the framework's entry points
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_front_end(dtype, tmp_path):
    """save_pretrained → registry → `LLaMA.generate_from_str` (left-padded batch, scheduler, on-device arg-max): every
    generated token is the oracle's arg-max given its prefix, up to near-ties."""
    from jax_llama_b200.models import registry

    cfg = config(MIXED, vocab=80, dtype=dtype)
    model = BazulornForCausalLM(cfg, dtype=dtype, seed=12, _do_init=True)
    model.save_pretrained(str(tmp_path))
    assert registry.resolve(str(tmp_path))[0] == "bazulorn"
    loaded = registry.load_pretrained(str(tmp_path), dtype=dtype, device="cuda")
    assert isinstance(loaded, BazulornForCausalLM) and loaded.config.to_dict() == cfg.to_dict()
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
    cfg = config(MIXED, vocab=80)
    BazulornForCausalLM(cfg, seed=3, _do_init=True).save_pretrained(str(tmp_path))
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
    shorter ones end, a second batch that opens while the first is still live; every wanted row against the oracle of
    that request alone."""
    import numpy as np

    cfg = config(MIXED, vocab=80, dtype=getattr(torch, dtype))
    model = BazulornForCausalLM(cfg, seed=5, _do_init=True)
    model.save_pretrained(str(tmp_path / "m"))
    cpu = {k: v.cpu() for k, v in model.params.items()}
    seq = {"a": tokens(30, 80, 1), "b": tokens(12, 80, 2), "c": tokens(47, 80, 3), "d": tokens(9, 80, 4), "e": tokens(26, 80, 5)}
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
    tol = TOL[getattr(torch, dtype)]
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
        assert err(got, torch.stack(want)) < tol, s["step"]
