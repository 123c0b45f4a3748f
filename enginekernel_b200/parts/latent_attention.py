"""Attention through a low-rank latent: queries, keys and values are up-projections of small
vectors, and only the key/value latent is cached.

Per token, with h the normalised input, H heads, per head d unrotated and r rotated query/key
dimensions, value size e, query latent size a and key/value latent size c:

    c_q = gain_dq * rms(W_dq h)                 q_h = W_uq,h c_q = [q_h,flat (d) ; q_h,rot (r)]
    [l ; k_rot] = W_dkv h                       lat = gain_dkv * rms(l)   (c values; k_rot is not normed)
    k_h = [W_uk,h lat ; rot(k_rot)]             v_h = W_uv,h lat
    score_h(i, j) = scale * (q_h,flat(i) . k_h,flat(j) + rot(q_h,rot(i)) . rot(k_rot(j))),  j <= i
    p = softmax over j with one more term exp(sink_h) in the denominator (no value)
    out = W_o [sum_j p_h(i, j) v_h(j)]_h

The cache holds one row [lat ; rot(k_rot)] per token (``CacheSpec.planes == 1``, one head), padded
with zeros to the row length D that the attention kernels take, and attention runs in the absorbed
form: the query of head h becomes [W_uk,h^T q_h,flat ; rot(q_h,rot)] (D values), all H heads read
the same cached rows as keys AND as values, and W_uv,h is applied to the first c values of each
head's result.  That is grouped-query attention with one key head, so the framework's attention
kernels run it (with a sink score per head): the mma.sync kernels for rows of up to 256 values, the
general kernel beyond (up to 1,024).

Parameters: ``hidden_size``, ``num_heads``, ``head_dim`` (d), ``rot_dim`` (r), ``v_dim`` (e),
``q_rank`` (a), ``kv_rank`` (c), ``scale``, ``eps``, ``position`` (a rotary PartSpec over ``rot_dim``
values, or None), ``sink`` (True: a learned score per head).  Tensors: ``dq`` [a, hidden],
``dq_norm`` [a], ``uq`` [H (d + r), a], ``dkv`` [c + r, hidden], ``dkv_norm`` [c], ``uk`` [H d, c],
``uv`` [H e, c], ``o`` [hidden, H e], ``sink`` [H].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..registry import lookup_part, register_part
from .base import Mixer
from .spec import CacheSpec, TensorSpec


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        hid, nh, d, r, e = p["hidden_size"], p["num_heads"], p["head_dim"], p["rot_dim"], p["v_dim"]
        a, c = p["q_rank"], p["kv_rank"]
        out = [TensorSpec(w["dq"], (a, hid)), TensorSpec(w["dq_norm"], (a,), "gain"),
               TensorSpec(w["uq"], (nh * (d + r), a)), TensorSpec(w["dkv"], (c + r, hid)),
               TensorSpec(w["dkv_norm"], (c,), "gain"), TensorSpec(w["uk"], (nh * d, c)),
               TensorSpec(w["uv"], (nh * e, c)), TensorSpec(w["o"], (hid, nh * e))]
        if p.get("sink"):
            out.append(TensorSpec(w["sink"], (nh,)))
        return out

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.num_heads, self.head_dim = g("hidden_size"), g("num_heads"), g("head_dim")
        self.rot_dim, self.v_dim, self.q_rank, self.kv_rank = g("rot_dim"), g("v_dim"), g("q_rank"), g("kv_rank")
        self.scale, self.eps = float(self.param("scale")), float(self.param("eps"))
        self.has_sink = bool(spec.params.get("sink"))
        pos = spec.params.get("position")
        self.position = lookup_part("position", pos.kind)(pos, dtype, device) if pos else None
        if self.position is not None and self.position.rotary_dim > self.rot_dim:
            raise ValueError("latent_attention: the rotation covers more than rot_dim values")
        # the cached row: latent and rotated key part, padded to what every attention kernel takes
        self.row = -(-(self.kv_rank + self.rot_dim) // 32) * 32
        if self.row > kernels.GENERIC_MAX_HEAD_DIM:
            raise kernels.KernelError(f"latent_attention: a cached row of {self.row} values (kv_rank + rot_dim) exceeds "
                                      f"the attention kernels' limit of {kernels.GENERIC_MAX_HEAD_DIM}")
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = None
        self.gain_q = self.gain_kv = self.sinks = None

    def cache_spec(self):
        return CacheSpec("kv", heads=1, head_dim=self.row, planes=1)

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def load(self, tensors):
        w = self.spec.weights
        nh, d, e, c = self.num_heads, self.head_dim, self.v_dim, self.kv_rank
        down = [tensors[w["dq"]], tensors[w["dkv"]]]          # (zero rows up to a multiple of 64, for the library's product)
        n = down[0].shape[0] + down[1].shape[0]
        down.append(torch.zeros((-n % 64, self.hidden), dtype=down[0].dtype, device=down[0].device))
        self.w_down = torch.cat(down, 0).to(self.dtype).contiguous()
        self.w_uq = tensors[w["uq"]].to(self.dtype).contiguous()
        # [heads, in, out] for the per-head products: the absorbed query reads W_uk transposed,
        # which is how it is stored ([H d, c] = [heads, d, c]); W_uv [H e, c] is turned once
        self.w_uk = tensors[w["uk"]].to(self.dtype).view(nh, d, c).contiguous()
        self.w_uv = tensors[w["uv"]].to(self.dtype).view(nh, e, c).transpose(1, 2).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()
        self.gain_q = tensors[w["dq_norm"]].to(torch.float32).contiguous()
        self.gain_kv = tensors[w["dkv_norm"]].to(torch.float32).contiguous()
        if self.has_sink:
            self.sinks = tensors[w["sink"]].to(torch.float32).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * t.element_size() for t in (self.w_down, self.w_uq, self.w_uk, self.w_uv, self.w_o))

    def forward(self, x, ctx, entry, writes_cache=True):
        t, nh, ws = ctx.n_tokens, self.num_heads, ctx.workspace
        a, c, r, d, e, row = self.q_rank, self.kv_rank, self.rot_dim, self.head_dim, self.v_dim, self.row
        pos = self.position
        rot_dims = pos.rotary_dim if pos is not None else 0
        cos, sin = (pos.cos, pos.sin) if pos is not None else (None, None)
        # both down-projections in one product, kept in 32-bit for the norms and the rotation
        down = linear(x, self.w_down, ctx, "latent_down", n_rows=t, out_dtype=torch.float32, wide_f32="library")
        cq = ws.get("latent_cq", (t, a), self.dtype)
        kernels.latent_prepare(cq, down, t, self.gain_q, self.gain_kv, self.eps, cos, sin, rot_dims,
                               ctx.positions, ctx.token_slot, entry.k_pages, entry.block_table, a, c, r,
                               write_cache=writes_cache)
        q = linear(cq, self.w_uq, ctx, "latent_q", n_rows=t)
        q_abs = ws.get("latent_q_abs", (t, nh, row), self.dtype)
        kernels.head_linear(q_abs, q[:t].view(t, nh, d + r), self.w_uk, t, nh, d, c,
                            rot=(r, rot_dims, cos, sin, ctx.positions))
        o_lat = ws.get("latent_attn", (t, nh * row), self.dtype)
        self._attend(o_lat, q_abs.view(t, nh * row), ctx, entry)
        o = ws.get("attn_out", (t, nh, e), self.dtype)
        kernels.head_linear(o, o_lat.view(t, nh, row), self.w_uv, t, nh, c, e)
        return linear(o.view(t, nh * e), self.w_o, ctx, "attn_proj", n_rows=t)

    def _attend(self, out, q, ctx, entry):
        """One key head of ``row`` values, read as keys and as values; H query heads."""
        t, nh, row = ctx.n_tokens, self.num_heads, self.row
        pages, table = entry.k_pages, entry.block_table
        common = dict(sinks=self.sinks)
        if not ctx.is_decode and kernels.attention_prefill_supported(self.dtype, row, nh, 1):
            kernels.attention_prefill_bf16(out, q, t, ctx.positions, ctx.token_slot, ctx.cu_seqlens, ctx.n_seqs,
                                           pages, pages, table, nh, 1, row, self.scale, None, **common)
            return
        fast = ctx.is_decode and kernels.attention_decode_supported(self.dtype, row)
        if fast:
            blocks = t * -(-nh // 16)
            resident = 3 * kernels.sm_count(self.device)
            splits = max(1, min(resident // max(blocks, 1), -(-ctx.max_context // 128)))
            per_split = 0
        else:
            splits = 1
            if t * nh < 2 * kernels.sm_count(self.device) and ctx.max_context > 512:
                splits = max(1, min(-(-ctx.max_context // 256), -(-4 * kernels.sm_count(self.device) // (t * nh)), 64))
            per_split = -(-(-(-ctx.max_context // splits)) // 128) * 128 if splits > 1 else 0
            splits = -(-ctx.max_context // per_split) if splits > 1 else 1
        acc = ml = None
        if splits > 1:
            acc = ctx.workspace.get("attn_part_acc", (t, nh, splits, row), torch.float32)
            ml = ctx.workspace.get("attn_part_ml", (t, nh, splits, 2), torch.float32)
        fn = kernels.attention_decode_bf16 if fast else kernels.attention_generic
        fn(out, q, t, ctx.positions, ctx.token_slot, pages, pages, table, nh, 1, row, self.scale, None,
           splits, per_split, acc, ml, **common)
