"""Small Lopazen configurations for tests and a writer of model folders of the tests' own.

The shapes differ from one another in every size and option: heads per group (1, 2, 4, all on
one key head), head sizes that take different attention kernels (40: the general one; 32: the
mma.sync ones; 64 and 128: the TMA / tcgen05 ones), a loop at the start, in the middle or none,
a loop that runs once, layers without a feed-forward, query temperatures that step every 1, 5,
16 or 100 positions, embedding scales of 1 and more.  Weights are drawn wide enough for the
attention to be far from uniform (scores of a few units), so that a wrong key, a missing sink
or a temperature one position off moves the logits by much more than rounding does.
"""

from __future__ import annotations

import json
import math
import os

import torch


def attention_layer(heads, kv_heads, dim, ff, coef=0.5, every=16, scale=None):
    return {"type": "attention",
            "mixer": {"dim": dim, "vdim": dim, "heads": heads, "kv_heads": kv_heads,
                      "q_temp": {"coef": coef, "every": every},
                      "scale": scale if scale is not None else 2.0 / math.sqrt(dim)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(width, vocab, layers, loop=None, scale=1.0, eps=1e-5):
    cfg = {"architecture": "Lopazen", "vocab": vocab, "width": width, "embedding": {"scale": scale},
           "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# group of 2, head size 32, a loop in the middle that runs three times, one layer without feed-forward
LOOPED = config(96, 211, [attention_layer(6, 3, 32, 160, 0.7, 16), attention_layer(6, 3, 32, None, 0.3, 5),
                          attention_layer(6, 3, 32, 112, 0.5, 1), attention_layer(6, 3, 32, 64, 0.9, 100)],
                loop=(1, 3, 3), scale=3.5)
# every query head its own key head, head size 64, no loop, layers of different head counts
FLAT = config(128, 157, [attention_layer(2, 2, 64, 96, 0.4, 7), attention_layer(4, 4, 64, 200, 0.0, 1)],
              scale=1.0, eps=1e-6)
# all query heads on one key head, head size 40 (no 16-byte rows of 16-bit values), a loop from
# layer 0 that runs twice, and a last layer without feed-forward
ODD = config(72, 89, [attention_layer(3, 1, 40, 48, 0.6, 3), attention_layer(3, 1, 40, None, 0.2, 64)],
             loop=(0, 1, 2), scale=8.0, eps=1e-5)
# head size 128, four query heads a key head, a loop over everything that runs once
WIDE = config(160, 301, [attention_layer(8, 2, 128, 256, 0.5, 32), attention_layer(4, 1, 128, 96, 1.0, 2)],
              loop=(0, 2, 1), scale=12.0, eps=1e-5)

# sizes that no fast path takes: a width and feed-forward sizes that are no multiples of 8, head
# sizes 20 and 36 in different layers (so also cache groups of different shapes), 3 x 20 = 60 and
# 2 x 36 = 72 values into the output projection, a loop that ends with the last layer
RAGGED = config(100, 77, [attention_layer(3, 3, 20, 52, 0.5, 4), attention_layer(2, 1, 36, 30, 0.8, 9),
                          attention_layer(6, 2, 20, None, 0.1, 2)],
                loop=(1, 3, 2), scale=2.0, eps=1e-4)

SHAPES = {"looped": LOOPED, "flat": FLAT, "odd": ODD, "wide": WIDE, "ragged": RAGGED}


def tensor_shapes(cfg):
    w, v = cfg["width"], cfg["vocab"]
    shapes = {"embed": (v, w), "final.norm": (w,)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        shapes.update({p + "norm1": (w,), p + "mix.q": (m["heads"] * m["dim"], w),
                       p + "mix.q.b": (m["heads"] * m["dim"],), p + "mix.k": (m["kv_heads"] * m["dim"], w),
                       p + "mix.k.b": (m["kv_heads"] * m["dim"],), p + "mix.q.norm": (m["dim"],),
                       p + "mix.k.norm": (m["dim"],), p + "mix.o": (w, m["heads"] * m["vdim"])})
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "norm2": (w,), p + "mlp.gate": (ff, w), p + "mlp.up": (ff, w),
                           p + "mlp.down": (w, ff)})
    return shapes


def make_tensors(cfg, seed, dtype=torch.bfloat16):
    """Matrices N(0, 1/in), the embedding N(0, 1) / scale-ish, gains 1 + 0.2 N, biases 0.5 N."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.2 * t
        elif name.endswith(".b"):
            t = 0.5 * t
        elif name == "embed":
            t = t / max(1.0, cfg["embedding"]["scale"]) ** 0.5
        else:
            t = t / math.sqrt(shape[1])
        out[name] = t.to(dtype)
    return out


def write_folder(folder, cfg, tensors):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def random_prompts(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]
