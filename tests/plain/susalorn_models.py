"""Small Susalorn configurations for tests and a writer of model folders of the tests' own.

The shapes differ from one another in everything the configuration can say: one, two, three or no
residual streams; latent attention whose value size differs from its key size and whose two latents
differ; cached rows of 48, 40, 96 and 192 values; rotations of 4 to 32 values with and without
stretched frequencies; delta mixers with one to all key heads per value head, key sizes 16 to 128,
convolutions of 2 to 5 taps and low-rank pairs of unlike inner sizes; dense and routed feed-forwards,
routers with and without groups, keeping one or several; layers without a feed-forward; a loop at the
start, in the middle, at the end or none; a width that is no multiple of 8.  Weights are drawn wide
enough for attention and routing to be far from uniform.
"""

from __future__ import annotations

import json
import math
import os

import torch


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scaling=None, base=10000.0, scale=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention",
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot,
                      "rot_dim": rot_dim, "scale": scale if scale is not None else 1.5 / math.sqrt(dim + rot_dim),
                      "vdim": vdim}}


def delta(heads, kv_heads, dim, vdim, conv, ranks):
    return {"type": "channel_delta", "ranks": ranks,
            "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, ff, top, groups=None, scale=1.0):
    router = {"experts": experts, "scale": scale, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"expert": {"ff": ff}, "kind": "moe", "router": router}


def config(width, vocab, layers, streams=None, loop=None, eps=1e-5):
    """``layers``: (mixer entry, mlp entry or None) pairs."""
    cfg = {"architecture": "Susalorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [dict(m, mlp=f) for m, f in layers]}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def file_config(cfg):
    """What goes into config.json: the inner sizes of the low-rank pairs are tensor shapes, not keys."""
    out = json.loads(json.dumps(cfg))
    for layer in out["layers"]:
        layer.pop("ranks", None)
    return out


# three streams; attention first; a loop over the last two layers; a layer without feed-forward
MIXED = config(96, 211, [
    (latent(3, 24, 8, 40, 48, 40, scaling=(4.0, 64, 8.0, 1.0)), moe(8, 48, 2, groups=(4, 2), scale=1.7)),
    (delta(4, 2, 16, 24, 3, (8, 12)), dense(80)),
    (latent(2, 16, 16, 16, 24, 32, scaling=(16.0, 32, 4.0, 0.5), base=100.0), None)],
    streams=3, loop=(1, 3, 2))
# one plain residual stream; a router without groups; no loop
PLAIN = config(128, 157, [
    (delta(2, 2, 64, 32, 2, (16, 4)), moe(6, 40, 3)),
    (latent(5, 32, 16, 32, 64, 80), dense(144))], eps=1e-6)
# a single residual stream that still has its coefficients; a width no product kernel takes; all
# value heads on one key head; a loop from the first layer
ODD = config(100, 89, [
    (delta(3, 1, 40, 20, 5, (5, 7)), moe(4, 36, 2, groups=(2, 1), scale=3.0)),
    (latent(2, 20, 4, 12, 28, 36, scaling=(2.0, 16, 2.0, 1.0)), dense(52)),
    (delta(2, 2, 24, 40, 1, (3, 3)), None)],
    streams=1, loop=(0, 2, 2), eps=1e-4)
# two streams; key size 128; a cached row of 192 values; many experts, several groups kept; a loop
# at the end that runs once
WIDE = config(256, 301, [
    (delta(4, 2, 128, 64, 4, (24, 16)), moe(16, 32, 6, groups=(4, 3), scale=2.5)),
    (latent(8, 64, 32, 48, 96, 160, scaling=(8.0, 128, 16.0, 2.0)), moe(12, 64, 1))],
    streams=2, loop=(1, 2, 1))

SHAPES = {"mixed": MIXED, "plain": PLAIN, "odd": ODD, "wide": WIDE}


def tensor_shapes(cfg):
    w, v, n = cfg["width"], cfg["vocab"], cfg.get("streams")
    shapes = {"embed": (v, w), "final.norm": (w,)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        shapes[p + "norm1"] = (w,)
        subs = ["hc1."]
        if layer["type"] == "latent_attention":
            h, d, r, e, a, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            shapes.update({p + "mix.dq": (a, w), p + "mix.dq.norm": (a,), p + "mix.uq": (h * (d + r), a),
                           p + "mix.dkv": (c + r, w), p + "mix.dkv.norm": (c,), p + "mix.uk": (h * d, c),
                           p + "mix.uv": (h * e, c), p + "mix.sink": (h,), p + "mix.o": (w, h * e)})
        else:
            h, g, d, e, k = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = layer["ranks"]
            shapes.update({p + "mix.q": (g * d, w), p + "mix.q.conv": (g * d, k), p + "mix.k": (g * d, w),
                           p + "mix.k.conv": (g * d, k), p + "mix.v": (h * e, w), p + "mix.v.conv": (h * e, k),
                           p + "mix.b": (h, w), p + "mix.A_log": (h,), p + "mix.norm": (e,),
                           p + "mix.a1": (ra, w), p + "mix.a2": (h * d, ra), p + "mix.dt_bias": (h * d,),
                           p + "mix.g1": (rg, w), p + "mix.g2": (h * e, rg), p + "mix.o": (w, h * e)})
        mlp = layer["mlp"]
        if mlp is not None:
            subs.append("hc2.")
            shapes[p + "norm2"] = (w,)
            if mlp["kind"] == "dense":
                shapes.update({p + "mlp.gate": (mlp["ff"], w), p + "mlp.up": (mlp["ff"], w), p + "mlp.down": (w, mlp["ff"])})
            else:
                shapes[p + "mlp.router"] = (mlp["router"]["experts"], w)
                for e in range(mlp["router"]["experts"]):
                    shapes[f"{p}mlp.e{e}.up"] = (mlp["expert"]["ff"], w)
                    shapes[f"{p}mlp.e{e}.down"] = (w, mlp["expert"]["ff"])
        if n is not None:
            for hc in subs:
                shapes.update({p + hc + "in": (n,), p + hc + "out": (n,), p + hc + "mix": (n, n)})
    return shapes


def make_tensors(cfg, seed, dtype=torch.bfloat16, sharp=1.0):
    """Matrices N(0, 1/in); gains 1 + 0.2 N; stream coefficients near (1/n, 1, identity); decay rates
    spread over two decades; ``sharp`` multiplies the query up-projection and the router (and, below 1, its
    square the experts' output)."""
    g = torch.Generator().manual_seed(seed)
    n = cfg.get("streams") or 1
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.2 * t
        elif name.endswith(".in"):
            t = 1.0 / n + 0.3 * t
        elif name.endswith(".out"):
            t = 1.0 + 0.3 * t
        elif ".hc" in name and last == "mix":
            t = torch.eye(n) + 0.15 * t
        elif last == "conv":
            t = 0.6 * t
        elif last == "A_log":
            t = 1.5 * t - 1.0
        elif last in ("dt_bias", "sink"):
            pass
        elif name == "embed":
            pass
        else:
            t = t / math.sqrt(shape[1])
            if last in ("uq", "router"):
                t = t * 1.5 * sharp
            if ".mlp.e" in name and last == "down" and sharp < 1.0:
                t = t * sharp * sharp            # mild weights: a token sent to another expert moves little
            if last in ("a2", "g2", "b"):
                t = t * 1.5
        out[name] = t.to(dtype)
    return out


def write_folder(folder, cfg, tensors):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(file_config(cfg), f)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def random_prompts(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]
