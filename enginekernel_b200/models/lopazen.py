"""Lopazen decoder: configuration -> model description.

Per token: x = embed[id] * embedding.scale.  Each layer is pre-norm, x += mixer(rms(x) * w1) and,
if it has a feed-forward, x += down(gelu_tanh(gate h) * (up h)) with h = rms(x) * w2.  The
mixer is grouped-query attention without rotation: q and k projections with biases, a per-head
RMS norm of q and k with one weight vector for all heads, the query multiplied by
1 + coef * ln(floor((p + 1) / every) + 1) at position p, the values being the keys as
projected (before their norm; there is no value projection), scores (q . k) * scale over all
earlier positions and the token itself, and a softmax whose denominator holds one more term of 1
(a sink of score 0 without a value).  A stretch of layers may run several times with the same
weights: every pass has cache entries of its own, and before each pass but the first the
embedding output is added to x.  Output: RMS norm, then logits against the embedding table
(unscaled).  Positions count from 0; there is no limit on them but the cache's.

Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{q,q.b,k,k.b,q.norm,k.norm,o}``, ``l<i>.mlp.{gate,up,down}``.  This module only names
parts and sizes; the parts know nothing of Lopazen.
"""

from __future__ import annotations

from ..config.lopazen import LopazenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec
from ..registry import register_architecture

MAX_POSITIONS = 1 << 30      # the design sets no limit; positions are 32-bit on the device


def build_lopazen(cfg: LopazenConfig) -> ModelSpec:
    layers, ignorable = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = PartSpec(
            "attention",
            {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
             "head_dim": m.dim, "scale": m.scale, "qk_norm_eps": cfg.norm_eps, "window": None,
             "position": None, "bias": ("q", "k"), "values": "keys",
             "query_temperature": (m.q_temp_coef, m.q_temp_every) if m.q_temp_coef != 0.0 else None,
             "sink": 0.0},
            {"q": p + "mix.q", "k": p + "mix.k", "o": p + "mix.o", "q_bias": p + "mix.q.b",
             "k_bias": p + "mix.k.b", "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm"})
        norms = {"pre_mixer": PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps},
                                       {"gain": p + "norm1"})}
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff,
                                         "activation": "gelu_tanh"},
                           {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"})
            norms["pre_feed_forward"] = PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps},
                                                 {"gain": p + "norm2"})
        else:
            ignorable.append(p + "norm2")       # a file may keep the unused weight
        layers.append(LayerSpec(PartSpec("pre_norm"), mixer, ffn, norms))

    schedule = [RunSpec(layer, entry, add_embedding=again)
                for entry, (layer, again) in enumerate(cfg.runs())]
    embedding = TensorSpec("embed", (cfg.vocab, cfg.width), "embedding")
    spec = ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=embedding, layers=layers, schedule=schedule,
        final_norm=PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps}, {"gain": "final.norm"}),
        lm_head=TensorSpec("lm_head", (cfg.vocab, cfg.width), "linear", optional_alias=embedding.name),
        embedding_multiplier=cfg.embedding_scale, ignorable=tuple(ignorable))
    spec.check()
    return spec


register_architecture(LopazenConfig.architecture, LopazenConfig, build_lopazen)
