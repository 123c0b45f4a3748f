"""Susalorn decoder: configuration -> model description.

x = embed[id].  Layers are pre-norm, x += mixer(rms(x) w1) and, with a feed-forward, x += ff(rms(x) w2);
with ``streams`` in the configuration the one x is n copies that each sublayer reads as a mixture and
writes into all at once (``parts/hyper.py``), and the output reads their sum.  Mixers: attention through
a low-rank latent with a rotated key part shared by the heads, stretched rotation frequencies and a
learned sink score per head (``parts/latent_attention.py``), or a gated delta rule with a decay per key
channel behind short convolutions (``parts/delta.py``).  Feed-forwards: SwiGLU, or routed experts with
squared-relu experts and a router limited to the best groups (``parts/moe.py``).  A stretch of layers may
run several times with the same weights, every pass with cache entries of its own and nothing else in
between.  Output: RMS norm, then logits against the embedding table.

Tensor names: ``embed``, ``final.norm``, per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc{1,2}.{in,out,mix}``,
``l<i>.mix.*`` and ``l<i>.mlp.*`` as the parts' docstrings list them.  This module only names parts and
sizes; the parts know nothing of Susalorn.
"""

from __future__ import annotations

from ..config.susalorn import ChannelDeltaConfig, DenseMlpConfig, LatentAttentionConfig, SusalornConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec
from ..registry import register_architecture

MAX_POSITIONS = 1 << 30      # the design sets no limit; positions are 32-bit on the device


def _mixer(cfg: SusalornConfig, m, p: str) -> PartSpec:
    if isinstance(m, LatentAttentionConfig):
        position = None
        if m.rot_dim > 0:
            params = {"rotary_dim": m.rot_dims, "theta": m.rot_base}
            if m.rot_scaling is not None:
                s = m.rot_scaling
                params.update(factor=s.factor, original=s.original, fast=s.fast, slow=s.slow)
            position = PartSpec("rope_stretched", params)
        return PartSpec(
            "latent_attention",
            {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
             "v_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps,
             "position": position, "sink": True},
            {"dq": p + "dq", "dq_norm": p + "dq.norm", "uq": p + "uq", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm",
             "uk": p + "uk", "uv": p + "uv", "o": p + "o", "sink": p + "sink"})
    assert isinstance(m, ChannelDeltaConfig)
    return PartSpec(
        "channel_delta",
        {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
         "v_dim": m.vdim, "conv": m.conv, "eps": cfg.norm_eps, "rank": m.rank},
        {"q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
         "v_conv": p + "v.conv", "b": p + "b", "A_log": p + "A_log", "dt_bias": p + "dt_bias", "a1": p + "a1",
         "a2": p + "a2", "g1": p + "g1", "g2": p + "g2", "norm": p + "norm", "o": p + "o"})


def _feed_forward(cfg: SusalornConfig, mlp, p: str) -> PartSpec:
    if isinstance(mlp, DenseMlpConfig):
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "activation": "silu"},
                        {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    weights = {"router": p + "router"}
    for e in range(mlp.experts):
        weights[f"up_{e}"] = f"{p}e{e}.up"
        weights[f"down_{e}"] = f"{p}e{e}.down"
    return PartSpec("routed_experts",
                    {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "experts": mlp.experts, "top": mlp.top,
                     "groups": mlp.groups, "keep": mlp.keep, "scale": mlp.scale, "activation": "relu2"}, weights)


def build_susalorn(cfg: SusalornConfig) -> ModelSpec:
    layers, ignorable = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm = lambda name: PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps}, {"gain": p + name})
        norms = {"pre_mixer": norm("norm1")}
        hc = {"in1": p + "hc1.in", "out1": p + "hc1.out", "mix1": p + "hc1.mix"}
        ffn = None
        if layer.mlp is not None:
            ffn = _feed_forward(cfg, layer.mlp, p + "mlp.")
            norms["pre_feed_forward"] = norm("norm2")
            hc.update(in2=p + "hc2.in", out2=p + "hc2.out", mix2=p + "hc2.mix")
        else:                                   # a file may keep the unused sublayer's weights
            ignorable += [p + "norm2", p + "hc2.in", p + "hc2.out", p + "hc2.mix"]
        if cfg.streams is not None:
            block = PartSpec("hyper_connections", {"streams": cfg.streams, "hidden_size": cfg.width}, hc)
        else:
            block = PartSpec("pre_norm")
        layers.append(LayerSpec(block, _mixer(cfg, layer.mixer, p + "mix."), ffn, norms))

    schedule = [RunSpec(layer, entry) for entry, layer in enumerate(cfg.runs())]
    embedding = TensorSpec("embed", (cfg.vocab, cfg.width), "embedding")
    spec = ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=embedding, layers=layers, schedule=schedule,
        final_norm=PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps}, {"gain": "final.norm"}),
        lm_head=TensorSpec("lm_head", (cfg.vocab, cfg.width), "linear", optional_alias=embedding.name),
        ignorable=tuple(ignorable))
    spec.check()
    return spec


register_architecture(SusalornConfig.architecture, SusalornConfig, build_susalorn)
