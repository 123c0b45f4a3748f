"""Pre-norm layer over several residual streams (hyper-connections).

A token carries n copies x_0 .. x_{n-1} of the stream, all equal to the embedding output at the
start.  A sublayer f (the mixer, then the feed-forward) with its norm reads one mixture of them
and writes into all of them at once from the old values:

    u = sum_s in[s] x_s;    y = f(norm(u));    x_t <- sum_s mix[s, t] x_s + out[t] y.

After the last layer the model's stream is the sum of the copies.  Parameters: ``streams`` (n),
``hidden_size``.  Tensors: ``in1`` [n], ``out1`` [n], ``mix1`` [n, n] (indexed [from, to]) for the
mixer and ``in2``, ``out2``, ``mix2`` for the feed-forward (absent in a layer without one).
Norms: ``pre_mixer``, ``pre_feed_forward``.  The copies live in 32-bit, [T, n, hidden]; the write of
one sublayer, the read of the next and - for a norm that is gain * u * rsqrt(mean(u^2) + eps) over the
row (``Norm.deferrable``) - that norm are one kernel; any other norm is called on the mixture.
"""

from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..ops import kernels
from ..registry import register_part
from .base import Block
from .spec import TensorSpec


@dataclasses.dataclass
class StreamWrite:
    """A sublayer's output that has not been written into the streams yet."""
    y: torch.Tensor
    mix: torch.Tensor
    out: torch.Tensor


@register_part("block", "hyper_connections")
class HyperConnectionBlock(Block):
    @classmethod
    def norm_names(cls, spec):
        return ["pre_mixer"]

    @classmethod
    def tensors(cls, spec):
        n, w = int(spec.params["streams"]), spec.weights
        out = []
        for q in ("1", "2"):
            if "in" + q in w:
                out += [TensorSpec(w["in" + q], (n,), "gain"), TensorSpec(w["out" + q], (n,), "gain"),
                        TensorSpec(w["mix" + q], (n, n), "linear")]
        return out

    def __init__(self, spec, dtype, device, mixer, feed_forward, norms):
        super().__init__(spec, dtype, device, mixer, feed_forward, norms)
        self.n = int(self.param("streams"))
        self.hidden = int(self.param("hidden_size"))
        if not 1 <= self.n <= kernels.MAX_RESIDUAL_STREAMS:
            raise ValueError(f"hyper_connections: 1 to {kernels.MAX_RESIDUAL_STREAMS} streams, not {self.n}")
        if feed_forward is not None and ("pre_feed_forward" not in norms or "in2" not in spec.weights):
            raise ValueError("hyper_connections: a feed-forward needs the norm 'pre_feed_forward' and in2/out2/mix2")
        self.coef = {}

    def load(self, tensors):
        for role, name in self.spec.weights.items():
            self.coef[role] = tensors[name].to(torch.float32).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * 4 for t in self.coef.values())

    # -- what the blocks carry ---------------------------------------------------------
    def open_stream(self, stream, ctx):
        streams = ctx.workspace.get("residual_streams", (ctx.n_tokens, self.n, self.hidden), torch.float32)
        kernels.hc_broadcast(streams, stream, ctx.n_tokens)
        return streams

    def collapse(self, streams, pending, ctx):
        x = ctx.workspace.get("stream", (ctx.n_tokens, self.hidden), torch.float32)
        self._step(streams, pending, None, x, ctx)
        return x, None

    def _step(self, streams, pending: Optional[StreamWrite], read_in, u, ctx, norm=None):
        kw = dict(read_in=read_in, u=u, norm=norm)
        if pending is not None:
            kw.update(y=pending.y, write_mix=pending.mix, write_out=pending.out)
        kernels.hc_step(streams, ctx.n_tokens, **kw)

    def _read_normed(self, streams, pending, read_in, norm_part, ctx):
        """The write of ``pending``, the read with ``read_in`` and ``norm_part`` of what was read."""
        spec = norm_part.deferrable()
        if spec is not None:
            gain, eps = spec
            normed = ctx.workspace.get("normed", (ctx.n_tokens, self.hidden), self.dtype)
            self._step(streams, pending, read_in, None, ctx, norm=(gain, float(eps), normed))
            return normed
        u = ctx.workspace.get("stream_read", (ctx.n_tokens, self.hidden), torch.float32)
        self._step(streams, pending, read_in, u, ctx)
        return norm_part.forward(u, ctx)

    def forward(self, streams, pending, ctx, entry, writes_cache=True):
        c = self.coef
        a = self._read_normed(streams, pending, c["in1"], self.norms["pre_mixer"], ctx)
        y = self.mixer.forward(a, ctx, entry, writes_cache)
        pending = StreamWrite(y, c["mix1"], c["out1"])
        if self.feed_forward is None:
            return pending
        a = self._read_normed(streams, pending, c["in2"], self.norms["pre_feed_forward"], ctx)
        y = self.feed_forward.forward(a, ctx)
        return StreamWrite(y, c["mix2"], c["out2"])
