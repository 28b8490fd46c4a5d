"""Plain float64 statement of the Bazulorn decoder, one function per mechanism, for one sequence at a time.

Nothing here imports the package: the functions take the checkpoint's tensors (name -> tensor) and the configuration as
the dictionary ``config.json`` holds, and recompute every token from the whole prefix (no cache, no state carried over).

Notation: T tokens, W model width.  Linear weights are [out, in].

  embedding        x_t = E[tok_t] + Bg[r_t],  r_t = (tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets, r_0 = buckets;
                   then the model norm with weight ``embed.norm``
  layer            h = norm1(x);  x <- x + mixer(h) + ff(h)
  "parallel"       mixer = (norm(left(h)) * w_left + norm(right(h)) * w_right) / 2 over the model width
     left          softmax attention with q/k/v biases, values scaled to unit RMS per head, a window, one more unit in the
                   denominator (a sink that carries no value), the heads' weights mixed by a [H, H] matrix afterwards
     right         selective state space layer: S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t per head
  "channel_delta"  gated delta rule with one decay per key channel
  feed-forward     gated dense layer (tanh gelu) or a mixture of clamped gated experts plus one shared expert
  output           model norm with ``final.norm``, logits against the embedding table
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


def embed_tokens(tokens, t, cfg):
    """tokens: list of ints -> [T, W] after the embedding norm."""
    bg = cfg["embedding"]["bigram"]
    n = int(bg["buckets"])
    rows = [n] + [(tokens[i - 1] * int(bg["mul_prev"]) + tokens[i] * int(bg["mul_cur"])) % n for i in range(1, len(tokens))]
    x = t["embed"].to(F64)[tokens] + t["bigram"].to(F64)[rows]
    return rms_norm(x, t["embed.norm"].to(F64), cfg["norm"]["eps"])


def causal_conv(x, w, bias=None):
    """x [T, C], w [C, taps] (last column multiplies the current token), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j:j + T] * w[:, j]
    return y if bias is None else y + bias


def sink_attention(h, t, p, m, eps):
    """The left half of a "parallel" mixer.  p: tensor prefix, m: its sizes."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    window = int((m.get("mask") or {}).get("size") or 0)
    g = lambda n: t[p + n].to(F64)
    q = (h @ g("q").T + g("q.b")).view(T, H, D)
    k = (h @ g("k").T + g("k.b")).view(T, G, D)
    v = rms_norm((h @ g("v").T + g("v.b")).view(T, G, Dv), None, eps)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if window <= 0 else ((j <= i) & (i - j < window))
    wts = torch.zeros(H, T, T, dtype=F64)
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh // (H // G)].T) * float(m["scale"])
        s = s.masked_fill(~seen, -math.inf)
        mx = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - mx)
        wts[hh] = e / (torch.exp(-mx) + e.sum(-1, keepdim=True))
    mixed = torch.einsum("hg,gij->hij", g("talk"), wts)
    out = torch.stack([mixed[hh] @ v[:, hh // (H // G)] for hh in range(H)], 1)          # [T, H, Dv]
    return out.reshape(T, H * Dv) @ g("o").T


def state_space(h, t, p, m, eps):
    """The right half of a "parallel" mixer."""
    T = h.shape[0]
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * P
    g = lambda n: t[p + n].to(F64)
    y = h @ g("in").T
    z, xbc, dt = y[:, :inner], y[:, inner:2 * inner + 2 * G * N], y[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, g("conv"), g("conv.b")))
    x = xbc[:, :inner].view(T, H, P)
    Bm = xbc[:, inner:inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + g("dt_bias"))                                                      # [T, H]
    decay = torch.exp(-torch.exp(g("A_log")) * dt)
    out = torch.zeros(T, H, P, dtype=F64)
    for hh in range(H):
        grp = hh // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for s in range(T):
            S = decay[s, hh] * S + dt[s, hh] * torch.outer(Bm[s, grp], x[s, hh])
            out[s, hh] = S.T @ Cm[s, grp] + g("D")[hh] * x[s, hh]
    o = out.reshape(T, inner) * silu(z)
    ng = int(m["norm_groups"])
    o = rms_norm(o.view(T, ng, inner // ng), None, eps).reshape(T, inner) * g("norm")
    return o @ g("o").T


def parallel_mixer(h, t, p, m, eps):
    left = rms_norm(sink_attention(h, t, p + "left.", m["left"], eps), t[p + "left.out"].to(F64), eps)
    right = rms_norm(state_space(h, t, p + "right.", m["right"], eps), t[p + "right.out"].to(F64), eps)
    return 0.5 * (left + right)


def channel_delta(h, t, p, m, eps):
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    g = lambda n: t[p + n].to(F64)
    q = silu(causal_conv(h @ g("q").T, g("q.conv"))).view(T, G, D)
    k = silu(causal_conv(h @ g("k").T, g("k.conv"))).view(T, G, D)
    v = silu(causal_conv(h @ g("v").T, g("v.conv"))).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ g("b").T)                                                    # [T, H]
    a = (h @ g("a1").T) @ g("a2").T + g("dt_bias")
    decay = torch.exp(-torch.exp(g("A_log"))[None, :, None] * softplus(a).view(T, H, D))  # [T, H, D]
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hh in range(H):
        kv = hh // (H // G)
        S = torch.zeros(D, Dv, dtype=F64)
        for s in range(T):
            S = decay[s, hh][:, None] * S
            u = beta[s, hh] * (v[s, hh] - S.T @ k[s, kv])
            S = S + torch.outer(k[s, kv], u)
            out[s, hh] = S.T @ q[s, kv]
    gate = torch.sigmoid((h @ g("g1").T) @ g("g2").T).view(T, H, Dv)
    o = rms_norm(out, g("norm"), eps) * gate
    return o.reshape(T, H * Dv) @ g("o").T


def dense_ff(h, t, p):
    g = lambda n: t[p + n].to(F64)
    return (gelu_tanh(h @ g("gate").T) * (h @ g("up").T)) @ g("down").T


def expert(h, t, p, limit):
    g = lambda n: t[p + n].to(F64)
    a = torch.clamp(h @ g("gate").T, max=limit)
    u = torch.clamp(h @ g("up").T, min=-limit, max=limit)
    return (a * torch.sigmoid(1.702 * a) * (u + 1.0)) @ g("down").T


def route(h, t, p, top):
    """-> (experts [T, top], weights [T, top]): the largest logits, softmax over the chosen ones."""
    z = h @ t[p + "router"].to(F64).T + t[p + "router.b"].to(F64)
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def moe_ff(h, t, p, mlp):
    top = int(mlp["router"]["top"])
    idx, wt = route(h, t, p, top)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=F64)
    for s in range(h.shape[0]):
        for c in range(top):
            out[s] += wt[s, c] * expert(h[s:s + 1], t, f"{p}e{int(idx[s, c])}.", float(mlp["expert"]["limit"]))[0]
    if mlp.get("shared"):
        out = out + expert(h, t, p + "shared.", float(mlp["shared"]["limit"]))
    return out


def forward(tokens, t, cfg, streams=None):
    """tokens: list of ints -> logits [T, vocab]; `streams` (a list) receives the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed_tokens(tokens, t, cfg)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, t[p + "norm1"].to(F64), eps)
        if layer["type"] == "parallel":
            y = parallel_mixer(h, t, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(h, t, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(h, t, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, t, p + "mlp.", mlp))
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, t["final.norm"].to(F64), eps)
    return x @ t["embed"].to(F64).T
