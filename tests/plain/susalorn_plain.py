"""Plain, slow Susalorn decoder: whole sequences, no cache, one function per mechanism.

Written from the design's equations with elementary torch operations on the CPU, in 64-bit on
the stored (bfloat16-rounded) weights.  It shares no code with ``enginekernel_b200``: it takes a
``config.json`` dictionary and a dictionary of tensors by checkpoint name.

Notation: T tokens at positions p = 0..T-1, width W, n residual streams; latent attention with H
heads of d unrotated + r rotated query/key dimensions, value size e, latent size c; delta mixer
with H value heads of size e, G key heads of size d, K convolution taps.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def lin(x, w):
    """W x for every row of x; W is stored [out, in]."""
    return x @ w.to(F).T


def embedding(table, ids):
    return table[torch.as_tensor(ids, dtype=torch.long)].to(F)


def stream_norm(x, weight, eps):
    return rms(x, eps) * weight.to(F)


# ---------------------------------------------------------------- several residual streams
def streams_read(xs, w_in):
    """u = sum over streams s of in[s] * x_s; xs is [T, n, W]."""
    return torch.einsum("s,tsw->tw", w_in.to(F), xs)


def streams_write(xs, y, w_mix, w_out):
    """x_t <- sum_s mix[s, t] x_s + out[t] * y for all t at once."""
    return torch.einsum("st,asw->atw", w_mix.to(F), xs) + w_out.to(F)[None, :, None] * y[:, None, :]


# ---------------------------------------------------------------- rotation with stretched frequencies
def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims) for i < dims/2; with scaling the blend of f_i and f_i / factor along a
    ramp between the dimensions that turn `fast` and `slow` times within `original` positions.
    Returns (frequencies, factor on cos and sin)."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, mult):
    """x [..T.., dims] with T on axis 0: pair (i, i + dims/2) turned by position * f_i."""
    half = freqs.numel()
    ang = torch.as_tensor(positions, dtype=F)[:, None] * freqs[None, :]
    cos, sin = torch.cos(ang) * mult, torch.sin(ang) * mult
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]], -1)


# ---------------------------------------------------------------- latent attention
def sink_softmax(scores, mask, sink):
    """exp(s_j) / (exp(sink) + sum over visible j' of exp(s_j'))."""
    m = torch.maximum(torch.where(mask, scores, torch.full_like(scores, -1e300)).amax(-1, keepdim=True),
                      torch.as_tensor(float(sink), dtype=F))
    e = torch.where(mask, torch.exp(scores - m), torch.zeros_like(scores))
    return e / (torch.exp(float(sink) - m) + e.sum(-1, keepdim=True))


def latent_attention(h, w, p, m, eps, positions=None):
    """The whole latent-attention mixer on normalised input h [T, W]."""
    t = h.shape[0]
    n_heads, d, r, e, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = list(range(t)) if positions is None else positions
    rot = m["rot"]
    freqs, mult = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    cq = rms(lin(h, w[p + "dq"]), eps) * w[p + "dq.norm"].to(F)
    q = lin(cq, w[p + "uq"]).view(t, n_heads, d + r)
    q_flat, q_rot = q[..., :d], rotate(q[..., d:], pos, freqs, mult)
    dkv = lin(h, w[p + "dkv"])
    lat = rms(dkv[:, :c], eps) * w[p + "dkv.norm"].to(F)
    k_rot = rotate(dkv[:, c:], pos, freqs, mult)                   # one for all heads
    k_flat = lin(lat, w[p + "uk"]).view(t, n_heads, d)
    v = lin(lat, w[p + "uv"]).view(t, n_heads, e)
    pp = torch.as_tensor(pos)
    mask = pp[None, :] <= pp[:, None]
    out = torch.zeros(t, n_heads, e, dtype=F)
    for a in range(n_heads):
        s = (q_flat[:, a] @ k_flat[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = sink_softmax(s, mask, w[p + "sink"].to(F)[a]) @ v[:, a]
    return lin(out.reshape(t, -1), w[p + "o"])


# ---------------------------------------------------------------- delta rule with a decay per key channel
def short_convolution(x, taps):
    """y[t, c] = sum_j taps[c, K-1-j] * x[t-j, c], zeros before the start; then silu."""
    t, k = x.shape[0], taps.shape[1]
    pad = torch.cat([torch.zeros(k - 1, x.shape[1], dtype=F), x], 0)
    y = torch.zeros_like(x)
    for j in range(k):
        y = y + pad[k - 1 - j:k - 1 - j + t] * taps.to(F)[:, k - 1 - j]
    return y * torch.sigmoid(y)


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_scan(q, k, v, beta, g):
    """Per head: S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k, g [T, H, d]; v [T, H, e]; beta [T, H]."""
    t, n_heads, d = q.shape
    e = v.shape[-1]
    s = torch.zeros(n_heads, d, e, dtype=F)
    out = torch.zeros(t, n_heads, e, dtype=F)
    for i in range(t):
        s = s * g[i][:, :, None]
        u = beta[i][:, None] * (v[i] - torch.einsum("hde,hd->he", s, k[i]))
        s = s + k[i][:, :, None] * u[:, None, :]
        out[i] = torch.einsum("hde,hd->he", s, q[i])
    return out


def channel_delta(h, w, p, m, eps):
    t = h.shape[0]
    n_heads, n_kv, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = n_heads // n_kv
    q = short_convolution(lin(h, w[p + "q"]), w[p + "q.conv"]).view(t, n_kv, d)
    k = short_convolution(lin(h, w[p + "k"]), w[p + "k.conv"]).view(t, n_kv, d)
    v = short_convolution(lin(h, w[p + "v"]), w[p + "v.conv"]).view(t, n_heads, e)
    q = (unit(q) * d ** -0.5).repeat_interleave(rep, 1)
    k = unit(k).repeat_interleave(rep, 1)
    beta = torch.sigmoid(lin(h, w[p + "b"]))
    a = lin(lin(h, w[p + "a1"]), w[p + "a2"]) + w[p + "dt_bias"].to(F)
    rate = torch.exp(w[p + "A_log"].to(F))[None, :, None]
    g = torch.exp(-rate * torch.nn.functional.softplus(a).view(t, n_heads, d))
    o = delta_scan(q, k, v, beta, g)
    gate = torch.sigmoid(lin(lin(h, w[p + "g1"]), w[p + "g2"])).view(t, n_heads, e)
    o = rms(o, eps) * w[p + "norm"].to(F) * gate
    return lin(o.reshape(t, -1), w[p + "o"])


# ---------------------------------------------------------------- feed-forwards
def dense_mlp(h, w, p):
    g = lin(h, w[p + "gate"])
    return lin(g * torch.sigmoid(g) * lin(h, w[p + "up"]), w[p + "down"])


def route(h, w_router, r):
    """Chosen experts [T, top] and their weights: softmax scores, only experts of the `keep` groups
    with the largest best score, the `top` largest of those, scores over their sum times scale."""
    s = torch.softmax(lin(h, w_router), -1)
    n = s.shape[-1]
    groups = r.get("groups")
    allowed = s
    if groups:
        per = n // groups["count"]
        best = s.view(-1, groups["count"], per).amax(-1)
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(groups["keep"], -1).indices, True)
        allowed = torch.where(kept.repeat_interleave(per, 1), s, torch.full_like(s, -1.0))
    idx = allowed.topk(r["top"], -1).indices
    val = s.gather(1, idx)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def expert(h, w, p):
    return lin(torch.relu(lin(h, w[p + "up"])) ** 2, w[p + "down"])


def moe(h, w, p, mlp):
    idx, wt = route(h, w[p + "router"], mlp["router"])
    out = torch.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        y = expert(h, w, f"{p}e{e}.")
        out = out + y * (wt * (idx == e)).sum(-1, keepdim=True)
    return out


def feed_forward(h, w, p, mlp):
    return dense_mlp(h, w, p) if mlp["kind"] == "dense" else moe(h, w, p, mlp)


# ---------------------------------------------------------------- the model
def layer_runs(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = list(range(loop["start"]))
    for _ in range(loop["times"]):
        order += list(range(loop["start"], loop["stop"]))
    return order + list(range(loop["stop"], n))


def forward(cfg, w, ids, return_layers=False):
    """Logits [T, vocab] (and the stream after every layer run) of one sequence from position 0."""
    eps = cfg["norm"]["eps"]
    n = cfg.get("streams")
    x = embedding(w["embed"], ids)
    xs = x[:, None, :].repeat(1, n, 1) if n else None
    after = []
    for i in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        mix = latent_attention if layer["type"] == "latent_attention" else channel_delta
        subs = [("hc1.", "norm1", lambda h: mix(h, w, p + "mix.", layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append(("hc2.", "norm2", lambda h: feed_forward(h, w, p + "mlp.", layer["mlp"])))
        for hc, norm, fn in subs:
            if n:
                u = streams_read(xs, w[p + hc + "in"])
                y = fn(stream_norm(u, w[p + norm], eps))
                xs = streams_write(xs, y, w[p + hc + "mix"], w[p + hc + "out"])
            else:
                x = x + fn(stream_norm(x, w[p + norm], eps))
        after.append(xs.sum(1) if n else x)
    x = xs.sum(1) if n else x
    logits = lin(stream_norm(x, w["final.norm"], eps), w["embed"])
    return (logits, torch.stack(after)) if return_layers else logits


def logits(cfg, w, ids):
    return forward(cfg, w, ids)


def greedy(cfg, w, ids, n_new):
    """The n_new tokens that arg-max decoding appends to ids (the whole sequence is run again each time)."""
    ids, out = list(ids), []
    for _ in range(n_new):
        nxt = int(forward(cfg, w, ids)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
