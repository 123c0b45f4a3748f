"""Plain, slow Lopazen decoder: whole sequences, no cache, one function per mechanism.

Written from the design's equations with elementary torch operations on the CPU, in 64-bit on
the stored (bfloat16-rounded) weights.  It shares no code with ``enginekernel_b200``: it takes a
``config.json`` dictionary and a dictionary of tensors by checkpoint name.

Notation: T tokens at positions p = 0..T-1, width W, H query heads and G key heads of size d.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def embedding(table, ids, scale):
    """Row ``id`` of the table times the model's embedding scale."""
    return table[torch.as_tensor(ids, dtype=torch.long)].to(F) * scale


def stream_norm(x, weight, eps):
    """The norm in front of a mixer, a feed-forward or the output: rms(x) * w."""
    return rms(x, eps) * weight.to(F)


def projections(h, wq, bq, wk, bk, n_heads, n_kv, d):
    """q = Wq h + bq as [T, H, d]; k = Wk h + bk as [T, G, d]; the values are k as it stands."""
    q = (h @ wq.to(F).T + bq.to(F)).view(-1, n_heads, d)
    k = (h @ wk.to(F).T + bk.to(F)).view(-1, n_kv, d)
    return q, k, k.clone()


def head_norm(x, weight, eps):
    """RMS norm of every head over its d values, one weight vector for all heads."""
    return rms(x, eps) * weight.to(F)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    p = torch.as_tensor(positions, dtype=torch.long)
    return 1.0 + coef * torch.log(torch.div(p + 1, every, rounding_mode="floor").to(F) + 1.0)


def sink_softmax(scores, mask):
    """exp(s_j) / (1 + sum over visible j' of exp(s_j')): an extra unit term in the denominator."""
    e = torch.where(mask, torch.exp(scores), torch.zeros_like(scores))
    return e / (1.0 + e.sum(-1, keepdim=True))


def attention(q, k, v, scale, positions=None):
    """Causal grouped attention: query head h reads key head h // (H / G); position i sees j <= i."""
    t, n_heads, d = q.shape
    n_kv = k.shape[1]
    pos = torch.arange(t) if positions is None else torch.as_tensor(positions)
    mask = pos[None, :] <= pos[:, None]
    out = torch.zeros(t, n_heads, v.shape[-1], dtype=F)
    for h in range(n_heads):
        g = h // (n_heads // n_kv)
        w = sink_softmax((q[:, h] @ k[:, g].T) * scale, mask)
        out[:, h] = w @ v[:, g]
    return out.reshape(t, -1)


def mixer(h, w, prefix, m, eps):
    """The whole attention mixer of one layer on normalised input ``h`` [T, W]."""
    n_heads, n_kv, d = m["heads"], m["kv_heads"], m["dim"]
    q, k, v = projections(h, w[prefix + "q"], w[prefix + "q.b"], w[prefix + "k"], w[prefix + "k.b"],
                          n_heads, n_kv, d)
    q = head_norm(q, w[prefix + "q.norm"], eps)
    k = head_norm(k, w[prefix + "k.norm"], eps)
    temp = m.get("q_temp")
    if temp is not None:
        q = q * query_temperature(range(h.shape[0]), temp["coef"], temp["every"])[:, None, None]
    return attention(q, k, v, m["scale"]) @ w[prefix + "o"].to(F).T


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def feed_forward(h, w, prefix):
    """down(gelu_tanh(gate h) * (up h))."""
    return (gelu_tanh(h @ w[prefix + "gate"].to(F).T) * (h @ w[prefix + "up"].to(F).T)) @ w[prefix + "down"].to(F).T


def layer_runs(cfg):
    """(layer, whether the embedding output is added before it) in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, False) for i in range(loop["start"])]
    for p in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, p > 0 and i == loop["start"]))
    return runs + [(i, False) for i in range(loop["stop"], n)]


def hidden_states(cfg, w, ids, collect=None):
    eps = cfg["norm"]["eps"]
    x = embedding(w["embed"], ids, cfg["embedding"]["scale"])
    first = x.clone()
    for i, again in layer_runs(cfg):
        if again:
            x = x + first
        layer, p = cfg["layers"][i], f"l{i}."
        x = x + mixer(stream_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        if layer["mlp"] is not None:
            x = x + feed_forward(stream_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        if collect is not None:
            collect.append(x.clone())
    return x


def logits(cfg, w, ids):
    """[T, vocab]: the output norm, then the embedding table itself (without its scale)."""
    x = hidden_states(cfg, w, ids)
    return (stream_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].to(F).T).to(torch.float32)


def greedy(cfg, w, ids, n_new):
    """``n_new`` tokens by arg-max, each from a full pass over the sequence so far."""
    ids, out = list(ids), []
    for _ in range(n_new):
        nxt = int(torch.argmax(logits(cfg, w, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out
