"""Plain float64 statement of the Datozen decoder, one function per mechanism, for one sequence at a time.

Nothing here imports the package: the functions take the checkpoint's tensors (name -> tensor) and the configuration as
the dictionary ``config.json`` holds, and recompute every token from the whole prefix (no cache carried over).

Notation: T tokens at positions 0 .. T-1, W model width.  Linear weights are [out, in].

  embedding     x_t = E[tok_t] + P[t]
  layer run     h = norm1(x);  x <- x + attention(h) + ff(h);  then the token side input
                y = Wp (gelu(Wg x) * Es[tok_t, slice of the layer]);  x <- x + y / rms(y) * w_side
  schedule      layers [0, start), then layers [start, stop) `times` times over, then [stop, L); a repeated layer shares its
                weights and its slice of Es between passes, never its keys and values
  attention     grouped heads; q, k normed per head (weight shared by the heads), then rotated on the leading rot.dims
                channels (pairs i, i + dims/2; interpolated frequencies); values rotated at their own position over all
                their channels with plain frequencies, the head's sum rotated back at the query's position; keys of the
                query's block of mask.size positions only; a learned logit per head joins the softmax denominator; a
                sigmoid gate per head from the layer input
  feed-forward  dense with the two-parameter quadratic / exponential activation, or a mixture of silu-gated experts with
                softmax scores, a choice bias, group limits by the best member, identity experts and a shared expert
  output        model norm with ``final.norm``, logits against the embedding table
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def embed_tokens(tokens, t, first=0):
    T = len(tokens)
    return t["embed"].to(F64)[tokens] + t["pos"].to(F64)[first:first + T]


def frequencies(dims, base, scaling=None):
    """(per-pair frequency [dims/2], factor on cos and sin)."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, pos, freq, mult=1.0, sign=1.0):
    """x [T, heads, n] with pairs (i, i + len(freq)) on its leading 2·len(freq) channels, turned by sign · pos · freq."""
    n2 = freq.shape[0]
    ang = sign * pos.to(F64)[:, None] * freq[None, :]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    u, v = x[..., :n2], x[..., n2:2 * n2]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * n2:]], -1)


def attention(h, t, p, m, eps, first=0):
    """h [T, W] at positions first .. first + T - 1 (the whole sequence when first == 0)."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    g = lambda n: t[p + n].to(F64)
    pos = torch.arange(first, first + T)
    q = rms_norm((h @ g("q").T).view(T, H, D), g("q.norm"), eps)
    k = rms_norm((h @ g("k").T).view(T, G, D), g("k.norm"), eps)
    v = (h @ g("v").T).view(T, G, Dv)
    rot = m.get("rot")
    if rot:
        f, mult = frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q, k = rotate_half(q, pos, f, mult), rotate_half(k, pos, f, mult)
        fv, _ = frequencies(Dv, float(rot["base"]), None)
        v = rotate_half(v, pos, fv)
    i, j = pos[:, None], pos[None, :]
    seen = j <= i
    size = int((m.get("mask") or {}).get("size") or 0)
    if size > 0:
        seen = seen & (i // size == j // size)
    gate = torch.sigmoid(h @ g("g").T)                                  # [T, H]
    sink = g("sink")
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hh in range(H):
        c = hh // (H // G)
        s = (q[:, hh] @ k[:, c].T) * float(m["scale"])
        s = s.masked_fill(~seen, -math.inf)
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink[hh])
        e = torch.exp(s - mx)
        w = e / (e.sum(-1, keepdim=True) + torch.exp(sink[hh] - mx))
        out[:, hh] = w @ v[:, c]
    if rot:
        out = rotate_half(out, pos, fv, sign=-1.0)
    out = out * gate[:, :, None]
    return out.reshape(T, H * Dv) @ g("o").T


def dense_ff(h, t, p):
    a = t[p + "act"].to(F64)
    return xielu(h @ t[p + "up"].to(F64).T, a[0], a[1]) @ t[p + "down"].to(F64).T


def gated_expert(h, t, p):
    return (silu(h @ t[p + "gate"].to(F64).T) * (h @ t[p + "up"].to(F64).T)) @ t[p + "down"].to(F64).T


def route(h, t, p, mlp):
    """(chosen indices [T, top], their weights [T, top]) over experts + identity experts."""
    r = mlp["router"]
    E, n_id, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    N = E + n_id
    s = torch.softmax(h @ t[p + "router"].to(F64).T, -1)                # [T, N]
    choice = s + t[p + "correction"].to(F64) if p + "correction" in t else s.clone()
    grp = r.get("groups")
    if grp and int(grp["count"]) > 1:
        n, keep = int(grp["count"]), int(grp["keep"])
        best = choice.view(-1, n, N // n).max(-1).values                # [T, n]
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, -1).indices, True)
        choice = choice.masked_fill(~kept[:, :, None].expand(-1, n, N // n).reshape(-1, N), -math.inf)
    idx = choice.topk(top, -1).indices
    return idx, s.gather(1, idx)


def moe_ff(h, t, p, mlp):
    E = int(mlp["router"]["experts"])
    idx, wt = route(h, t, p, mlp)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=F64)
    for tok in range(h.shape[0]):
        for e, w in zip(idx[tok].tolist(), wt[tok]):
            y = gated_expert(h[tok:tok + 1], t, f"{p}e{e}.")[0] if e < E else h[tok]
            out[tok] += w * y
    if mlp.get("shared"):
        out = out + gated_expert(h, t, p + "shared.")
    return out


def token_side(x, tokens, t, p, layer, dim, eps):
    e = t["side.embed"].to(F64)[tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ t[p + "side.gate"].to(F64).T) * e) @ t[p + "side.proj"].to(F64).T
    return rms_norm(y, t[p + "side.norm"].to(F64), eps)


def layer_runs(cfg):
    """Layer index of every run, in order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(tokens, t, cfg, streams=None):
    """Logits [T, vocab] of a whole sequence; `streams` (a list) receives the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = embed_tokens(tokens, t)
    side = cfg.get("token_side")
    for i in layer_runs(cfg):
        l, p = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, t[p + "norm1"].to(F64), eps)
        y = attention(h, t, p + "mix.", l["mixer"], eps)
        mlp = l.get("mlp")
        if mlp:
            y = y + (dense_ff(h, t, p + "mlp.") if mlp.get("kind", "dense") == "dense" else moe_ff(h, t, p + "mlp.", mlp))
        x = x + y
        if side:
            x = x + token_side(x, tokens, t, p, i, int(side["dim"]), eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, t["final.norm"].to(F64), eps) @ t["embed"].to(F64).T
