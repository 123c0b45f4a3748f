"""The Susalorn decoder in the engine against the plain implementation, mechanism by mechanism and
then whole models under every way of cutting the work.

Part one drives the new kernels alone: the residual streams' read and write, the latent's norms,
rotation and cache row, the per-head products, the delta rule's convolution with its carried inputs,
its scan from a carried state, its output norm and gate, the router and the experts' products.  Part
two runs one-layer models of each mixer with weights made sharp, so that one far token decides, and
part three four small models of unlike shapes (tests/plain/susalorn_models.py) through ``Engine``:
whole prompts, prompts in portions down to two tokens, token-by-token decoding, unequal batches,
slots, pages and states used again, long decoding, and greedy generation through the scheduler.
"""

import json
import math

import pytest
import torch

from tests import helpers
from tests.plain import susalorn_models as models
from tests.plain import susalorn_plain as plain
from tests.test_kernels_gpu import DEV, DTYPES, TOL, K, rel, rnd

pytestmark = pytest.mark.gpu
F32 = torch.float32


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ===================================================================== mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,width,tokens", [(1, 40, 3), (2, 100, 17), (3, 96, 5), (4, 256, 33), (8, 72, 2)])
def test_residual_streams_read_and_write(dtype, n, width, tokens):
    k = K()
    x = rnd(tokens, width, seed=1)
    xs = torch.empty(tokens, n, width, device=DEV)
    k.hc_broadcast(xs, x, tokens)
    assert torch.equal(xs, x[:, None, :].expand(-1, n, -1))
    xs = rnd(tokens, n, width, seed=2)
    w_in, w_out, mix = rnd(n, seed=3), rnd(n, seed=4), rnd(n, n, seed=5)
    y = rnd(tokens, width, dtype=dtype, seed=6)
    u = torch.empty(tokens, width, device=DEV)
    k.hc_step(xs.clone(), tokens, read_in=w_in, u=u)                                # read alone
    assert rel(u, plain.streams_read(xs.double().cpu(), w_in.cpu())) <= 1e-6
    got = xs.clone()
    k.hc_step(got, tokens, y=y, write_mix=mix, write_out=w_out, read_in=w_in, u=u)  # write, then read
    want = plain.streams_write(xs.double().cpu(), y.double().cpu(), mix.cpu(), w_out.cpu())
    assert rel(got, want) <= 1e-6                      # the streams stay 32-bit whatever y's type
    assert rel(u, plain.streams_read(want, w_in.cpu())) <= 1e-6
    got2 = xs.clone()
    k.hc_step(got2, tokens, y=y, write_mix=mix, write_out=w_out, u=u)               # write, then the plain sum
    assert rel(u, want.sum(1)) <= 1e-6
    gain, normed = 1 + 0.2 * rnd(width, seed=7), torch.full((tokens, width), 7.0, dtype=dtype, device=DEV)
    for with_u in (True, False):                                                    # ... and the norm of what was read
        got3, u3 = xs.clone(), torch.full((tokens, width), 7.0, device=DEV)
        k.hc_step(got3, tokens, y=y, write_mix=mix, write_out=w_out, read_in=w_in, u=u3 if with_u else None,
                  norm=(gain, 1e-5, normed))
        assert rel(got3, want) <= 1e-6
        assert rel(normed, plain.stream_norm(plain.streams_read(want, w_in.cpu()), gain.cpu(), 1e-5)) <= TOL[dtype]
        assert (rel(u3, plain.streams_read(want, w_in.cpu())) <= 1e-6) if with_u else bool((u3 == 7.0).all())
    k.hc_step(xs.clone(), tokens, read_in=w_in, norm=(gain, 1e-5, normed))          # read and norm alone
    assert rel(normed, plain.stream_norm(plain.streams_read(xs.double().cpu(), w_in.cpu()), gain.cpu(), 1e-5)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("a,c,r,rot,row", [(48, 40, 8, 8, 64), (24, 32, 16, 16, 64), (20, 36, 4, 4, 64), (96, 160, 32, 32, 192),
                                           (16, 24, 12, 8, 64)])
def test_latent_norms_rotation_and_cache_row(dtype, a, c, r, rot, row):
    """Tokens of three sequences at positions on both sides of page borders; one row is not written."""
    k = K()
    pos = [0, 1, 63, 64, 65, 127, 128, 200, -1]
    slot = [0, 0, 1, 1, 1, 2, 2, 2, 0]
    t = len(pos)
    proj = rnd(t, a + c + r + 3, seed=1, scale=2.0)
    gq, gkv = 1 + 0.3 * rnd(a, seed=2), 1 + 0.3 * rnd(c, seed=3)
    f, mult = plain.rotary_frequencies(rot, 100.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0})
    ang = torch.arange(256, dtype=torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * mult).float().to(DEV), (torch.sin(ang) * mult).float().to(DEV)
    pages = torch.full((13, 1, 64, row), 7.0, dtype=dtype, device=DEV)
    table = i32([[5, 1, 9, 0], [2, 12, 3, 0], [4, 6, 8, 11]])
    cq = torch.empty(t, a, dtype=dtype, device=DEV)
    eps = 1e-5
    k.latent_prepare(cq, proj, t, gq, gkv, eps, cos, sin, rot, i32(pos), i32(slot), pages, table, a, c, r)
    pj = proj.double().cpu()
    assert rel(cq, plain.rms(pj[:, :a], eps) * gq.double().cpu()) <= TOL[dtype]
    for i, (p, s) in enumerate(zip(pos, slot)):
        if p < 0:
            continue
        got = pages[int(table[s, p // 64]), 0, p % 64].double().cpu()
        lat = plain.rms(pj[i:i + 1, a:a + c], eps)[0] * gkv.double().cpu()
        kr = plain.rotate(pj[i:i + 1, a + c:a + c + r], [p], f, mult)[0]
        assert rel(got[:c + r], torch.cat([lat, kr])) <= TOL[dtype], i
        assert got[c + r:].abs().sum().item() == 0
    assert (pages == 7.0).sum().item() == pages.numel() - (t - 1) * row      # nothing else was touched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,n_in,n_out,r,rot,tokens", [(3, 24, 40, 8, 8, 11), (8, 64, 160, 32, 32, 70), (2, 20, 36, 4, 4, 1),
                                                           (5, 130, 300, 0, 0, 9)])
def test_products_per_head(dtype, heads, n_in, n_out, r, rot, tokens):
    k = K()
    x = rnd(tokens, heads, n_in + r, dtype=dtype, seed=1)
    w = rnd(heads, n_in, n_out, dtype=dtype, seed=2, scale=n_in ** -0.5)
    want = torch.einsum("thi,hio->tho", x[..., :n_in].double().cpu(), w.double().cpu())
    out = torch.full((tokens, heads, n_out), 7.0, dtype=dtype, device=DEV)
    k.head_linear(out, x, w, tokens, heads, n_in, n_out)
    assert rel(out, want) <= TOL[dtype]
    if r:
        stride = -(-(n_out + r) // 32) * 32
        pos = [(7 * i) % 250 for i in range(tokens)]
        f, mult = plain.rotary_frequencies(rot, 10000.0, None)
        ang = torch.arange(256, dtype=torch.float64)[:, None] * f[None, :]
        cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
        out = torch.full((tokens, heads, stride), 7.0, dtype=dtype, device=DEV)
        k.head_linear(out, x, w, tokens, heads, n_in, n_out, rot=(r, rot, cos, sin, i32(pos)))
        assert rel(out[..., :n_out], want) <= TOL[dtype]
        assert rel(out[..., n_out:n_out + r], plain.rotate(x[..., n_in:].double().cpu(), pos, f, mult)) <= TOL[dtype]
        assert out[..., n_out + r:].abs().sum().item() == 0


def _delta_inputs(t, heads, kv_heads, dim, vdim, seed):
    g = torch.Generator().manual_seed(seed)
    q = plain.unit(torch.randn(t, kv_heads, dim, generator=g, dtype=torch.float64)) * dim ** -0.5
    k_ = plain.unit(torch.randn(t, kv_heads, dim, generator=g, dtype=torch.float64))
    v = torch.randn(t, heads, vdim, generator=g, dtype=torch.float64)
    beta = torch.rand(t, heads, generator=g, dtype=torch.float64)
    decay = torch.rand(t, heads, dim, generator=g, dtype=torch.float64) ** 0.2       # mostly near 1
    return q, k_, v, beta, decay


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 24), (2, 2, 64, 32), (3, 1, 40, 20), (2, 1, 128, 64),
                                                     (1, 1, 200, 70)])
def test_delta_scan_alone_and_from_a_carried_state(heads, kv_heads, dim, vdim):
    """Three sequences of unequal lengths in one launch; then the same tokens in two launches (the
    second starts from the state the first left) and one token at a time, in slots that were used before."""
    k = K()
    lens = [37, 1, 90]
    rows = k.delta_state_rows(dim)
    per_slot = heads * vdim * rows + 8
    rep = heads // kv_heads
    data = [_delta_inputs(n, heads, kv_heads, dim, vdim, 10 + i) for i, n in enumerate(lens)]
    want = [plain.delta_scan(q.repeat_interleave(rep, 1), kk.repeat_interleave(rep, 1), v, b, g) for q, kk, v, b, g in data]

    def run(cuts, slots):
        state = torch.zeros(6, per_slot, device=DEV)
        state[:, -8:] = 3.0                                   # what lies behind S in a slot is not the scan's
        out = [torch.zeros(n, heads * vdim) for n in lens]
        for step in cuts:                                     # step: per sequence (start, stop)
            live = [(i, a, b) for i, (a, b) in enumerate(step) if b > a]
            cat = lambda j: torch.cat([data[i][j][a:b].reshape(b - a, -1) for i, a, b in live]).float().to(DEV)
            n = sum(b - a for _, a, b in live)
            cu = [0]
            for _, a, b in live:
                cu.append(cu[-1] + b - a)
            pos = [p for _, a, b in live for p in range(a, b)]
            slot = [slots[i] for i, a, b in live for _ in range(a, b)]
            o = torch.full((n, heads * vdim), 7.0, device=DEV)
            k.delta_scan(o, cat(0), cat(1), cat(2), cat(3), cat(4), state, i32(cu), i32(pos), i32(slot), len(live),
                         heads, kv_heads, dim, vdim)
            for j, (i, a, b) in enumerate(live):
                out[i][a:b] = o[cu[j]:cu[j + 1]].cpu()
        assert (state[:, -8:] == 3.0).all()
        return out

    with pytest.raises(k.KernelError):                        # S is moved 16 bytes at a time
        k.delta_scan(torch.empty(1, heads * vdim, device=DEV), *[torch.zeros(1, 8, device=DEV)] * 5,
                     torch.zeros(2, per_slot + 1, device=DEV), i32([0, 1]), i32([0]), i32([0]), 1, heads, kv_heads, dim, vdim)
    whole = run([[(0, n) for n in lens]], [4, 0, 2])
    for o, w in zip(whole, want):
        assert rel(o, w.reshape(o.shape)) <= 2e-5
    two = run([[(0, 20), (0, 1), (0, 2)], [(20, 37), (1, 1), (2, 90)]], [1, 5, 3])
    single = run([[(i, min(i + 1, n)) for n in lens] for i in range(max(lens))], [0, 1, 2])
    for a, b, w in zip(two, single, want):
        assert rel(a, w.reshape(a.shape)) <= 2e-5 and rel(b, w.reshape(b.shape)) <= 2e-5


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps,ra,rg", [(4, 2, 16, 24, 3, 8, 12), (2, 2, 64, 32, 2, 16, 4),
                                                                 (3, 1, 40, 20, 5, 5, 7), (2, 2, 24, 40, 1, 3, 3)])
def test_delta_convolution_norms_decays_and_carried_inputs(heads, kv_heads, dim, vdim, taps, ra, rg):
    """A sequence of 11 tokens whole, and cut 1 + 2 + 8 behind another sequence: the convolution reads
    the inputs that the state carried over, also when a portion is shorter than the taps."""
    k = K()
    cq, cv = kv_heads * dim, heads * vdim
    nch = 2 * cq + cv
    width = nch + heads + ra + rg
    t = 11
    proj = rnd(t, width + 2, seed=1)
    conv = rnd(nch, taps, seed=2, scale=0.6)
    a2, g2 = rnd(heads * dim, ra, seed=3), rnd(cv, rg, seed=4)
    dt_bias, a_log, norm_w = rnd(heads * dim, seed=5), rnd(heads, seed=6), 1 + 0.2 * rnd(vdim, seed=7)
    pj = proj.double().cpu()
    sc = lambda x, w: plain.short_convolution(x, w.cpu())
    want_q = plain.unit(sc(pj[:, :cq], conv[:cq]).view(t, kv_heads, dim)) * dim ** -0.5
    want_k = plain.unit(sc(pj[:, cq:2 * cq], conv[cq:2 * cq]).view(t, kv_heads, dim))
    want_v = sc(pj[:, 2 * cq:nch], conv[2 * cq:])
    want_b = torch.sigmoid(pj[:, nch:nch + heads])
    a = pj[:, nch + heads:nch + heads + ra] @ a2.double().cpu().T + dt_bias.double().cpu()
    want_g = torch.exp(-torch.exp(a_log.double().cpu()).repeat_interleave(dim) * torch.nn.functional.softplus(a))
    s_values = heads * vdim * k.delta_state_rows(dim)
    shape = (heads, kv_heads, dim, vdim, taps, ra, rg)

    def run(cuts):
        state = torch.zeros(3, s_values + nch * (taps - 1), device=DEV)
        state[:, :s_values] = 5.0
        got = [torch.zeros(t, n) for n in (cq, cq, cv, heads)]
        other = rnd(4, width + 2, seed=9)
        for a_, b_ in cuts:
            n = b_ - a_
            rows = torch.cat([other[:2], proj[a_:b_]])          # another sequence's two tokens in front
            pos, slot, cu = [0, 1] + list(range(a_, b_)), [0, 0] + [2] * n, [0, 2, 2 + n]
            outs = [torch.full((n + 2, m), 7.0, device=DEV) for m in (cq, cq, cv, heads)]
            k.delta_prepare(*outs, rows, n + 2, conv, state, s_values, i32(pos), i32(slot), shape)
            k.delta_conv_tail(state, s_values, rows, i32(cu), i32(pos), i32(slot), 2, nch, taps)
            state[0, s_values:] = 0                              # the other sequence always starts anew
            for g_, o in zip(got, outs):
                g_[a_:b_] = o[2:].cpu()
        assert (state[:, :s_values] == 5.0).all()
        return got

    for cuts in ([(0, t)], [(0, 1), (1, 3), (3, t)], [(i, i + 1) for i in range(t)]):
        q_, k_, v_, b_ = run(cuts)
        assert rel(q_, want_q.reshape(t, -1)) <= 2e-5 and rel(k_, want_k.reshape(t, -1)) <= 2e-5, cuts
        assert rel(v_, want_v) <= 2e-5 and rel(b_, want_b) <= 2e-5, cuts

    decay = torch.full((t, heads * dim), 7.0, device=DEV)       # the second halves of the low-rank pairs
    k.delta_low_rank(decay, proj, t, nch + heads, a2.t().contiguous(), bias=dt_bias, a_log=a_log, dim=dim)
    assert rel(decay, want_g) <= 2e-5
    gate = torch.full((t, cv), 7.0, device=DEV)
    k.delta_low_rank(gate, proj, t, nch + heads + ra, g2.t().contiguous())
    want_gate = torch.sigmoid(pj[:, width - rg:width] @ g2.double().cpu().T)
    assert rel(gate, want_gate) <= 2e-5

    for dtype in DTYPES:                                         # the output norm and its gate
        o = rnd(t, cv, seed=11, scale=3.0)
        y = torch.empty(t, cv, dtype=dtype, device=DEV)
        pos = list(range(t - 1)) + [-1]
        k.delta_out_norm(y, o, gate, norm_w, 1e-5, i32(pos), t, shape)
        want = plain.rms(o.double().cpu().view(t, heads, vdim), 1e-5) * norm_w.double().cpu() * want_gate.view(t, heads, vdim)
        assert rel(y[:-1], want.reshape(t, -1)[:-1]) <= TOL[dtype]
        assert y[-1].abs().max().item() == 0


@pytest.mark.parametrize("experts,top,groups", [(8, 2, (4, 2)), (6, 3, None), (4, 2, (2, 1)), (16, 6, (4, 3)), (12, 1, None),
                                                (64, 8, (8, 4)), (40, 33, (2, 2))])
def test_router_against_the_plain_one(experts, top, groups):
    k = K()
    t = 97
    logits = rnd(t, experts, seed=experts, scale=2.0)
    chosen = torch.empty(t, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(t, top, device=DEV)
    n_groups, keep = groups or (1, 1)
    k.moe_route(chosen, weight, logits, t, n_groups, keep, top, 2.5)
    r = {"experts": experts, "top": top, "scale": 2.5}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    idx, wt = plain.route(logits.double().cpu(), torch.eye(experts), r)
    assert torch.equal(chosen.cpu().long(), idx)                 # in the order of their scores
    assert rel(weight, wt) <= 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,experts,top,groups,tokens", [(96, 48, 8, 2, (4, 2), 50), (100, 36, 4, 2, (2, 1), 7),
                                                                (256, 32, 16, 6, (4, 3), 300), (128, 40, 6, 3, None, 1)])
def test_routed_experts_part(dtype, width, ff, experts, top, groups, tokens):
    """The part as a whole (router, plan, both products, the sum in the order chosen) against the plain one;
    the router is made sharp so that 16-bit inputs choose as 64-bit ones do."""
    from enginekernel_b200.parts.moe import RoutedExperts
    from enginekernel_b200.parts.spec import PartSpec
    mlp = models.moe(experts, ff, top, groups, scale=1.3)
    names = {"router": "router"}
    w = {"router": rnd(experts, width, dtype=torch.bfloat16, seed=1, scale=4 * width ** -0.5)}
    for e in range(experts):
        names[f"up_{e}"], names[f"down_{e}"] = f"e{e}.up", f"e{e}.down"
        w[f"e{e}.up"] = rnd(ff, width, dtype=torch.bfloat16, seed=10 + e, scale=width ** -0.5)
        w[f"e{e}.down"] = rnd(width, ff, dtype=torch.bfloat16, seed=100 + e, scale=ff ** -0.5)
    n_groups, keep = groups or (1, 1)
    part = RoutedExperts(PartSpec("routed_experts", {"hidden_size": width, "intermediate_size": ff, "experts": experts,
                                                     "top": top, "groups": n_groups, "keep": keep, "scale": 1.3,
                                                     "activation": "relu2"}, names), dtype, DEV)
    part.load(w)
    x = rnd(tokens, width, dtype=dtype, seed=5)
    ctx = helpers.make_context(dtype, DEV, list(range(tokens)), [0] * tokens, [0, tokens])
    got = part.forward(x, ctx)
    want = plain.moe(x.double().cpu(), {k_: v.cpu() for k_, v in w.items()}, "", mlp)
    rows = ((got.double().cpu() - want).abs().amax(-1) / want.abs().max()) <= TOL[dtype] * 2
    assert rows.float().mean().item() >= (1.0 if dtype == F32 else 0.97)
    assert part.bytes_read_per_step(1) < part.bytes_read_per_step(10 ** 6)


# ===================================================================== one mixer, sharp weights
def _one_layer(mixer_entry, width, vocab, streams):
    return models.config(width, vocab, [(mixer_entry, None)], streams=streams)


ONE_LAYER = {
    "latent": _one_layer(models.latent(3, 24, 8, 40, 48, 40, scaling=(4.0, 64, 8.0, 1.0), scale=0.9), 96, 600, 2),
    "latent_wide": _one_layer(models.latent(6, 64, 32, 48, 96, 160, scaling=(8.0, 256, 32.0, 1.0), scale=0.5), 128, 600, None),
    # a cached row of 304 values: beyond what the mma.sync attention kernels take, so the general kernel runs it
    "latent_long_row": _one_layer(models.latent(2, 16, 16, 24, 32, 288, scale=0.7), 64, 600, None),
    "delta": _one_layer(models.delta(4, 2, 16, 24, 3, (8, 12)), 96, 83, 3),
    "delta_wide": _one_layer(models.delta(2, 1, 128, 64, 4, (24, 16)), 128, 83, None),
}


@pytest.fixture(scope="module")
def one_layer_engines(tmp_path_factory):
    from enginekernel_b200 import Engine
    made = {}

    def get(tag, dtype):
        if (tag, dtype) not in made:
            cfg = ONE_LAYER[tag]
            w = models.make_tensors(cfg, 5, sharp=1.0)
            folder = models.write_folder(str(tmp_path_factory.mktemp("one_" + tag)), cfg, w)
            made[(tag, dtype)] = (Engine(folder, dtype, max_tokens=2048, max_batch=4), cfg, w)
        return made[(tag, dtype)]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", list(ONE_LAYER))
def test_one_mixer_whole_then_token_by_token(one_layer_engines, tag, dtype):
    eng, cfg, w = one_layer_engines(tag, dtype)
    ids = models.random_prompts(cfg, [330], seed=2)[0]
    want = plain.logits(cfg, w, ids)
    assert helpers.rel_err(helpers.whole(eng, ids), want) <= helpers.TOL[dtype]
    got = helpers.tail_one_by_one(eng, ids, 140)              # across three page borders
    assert helpers.rel_err(got, want) <= helpers.TOL[dtype]


def _best_key_token(cfg, w, last_token, last_pos, key_pos):
    """The vocabulary token whose key at ``key_pos`` scores highest against the query of ``last_token`` at
    ``last_pos`` in some head of layer 0 (from the plain pieces), and that score minus the query's own."""
    m, eps, p = cfg["layers"][0]["mixer"], cfg["norm"]["eps"], "l0.mix."
    d, r, c, nh = m["dim"], m["rot_dim"], m["kv_rank"], m["heads"]
    x = plain.embedding(w["embed"], list(range(cfg["vocab"])))
    if "streams" in cfg:
        x = x * w["l0.hc1.in"].double().sum()
    h = plain.stream_norm(x, w["l0.norm1"], eps)
    f, mult = plain.rotary_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = plain.lin(plain.rms(plain.lin(h[last_token:last_token + 1], w[p + "dq"]), eps) * w[p + "dq.norm"].double(),
                  w[p + "uq"]).view(1, nh, d + r)
    q_rot = plain.rotate(q[..., d:], [last_pos], f, mult)[0]
    dkv = plain.lin(h, w[p + "dkv"])
    lat = plain.rms(dkv[:, :c], eps) * w[p + "dkv.norm"].double()
    k_flat = plain.lin(lat, w[p + "uk"]).view(-1, nh, d)

    def scores(pos):
        k_rot = plain.rotate(dkv[:, c:], [pos] * cfg["vocab"], f, mult)
        return (torch.einsum("hd,vhd->vh", q[0, :, :d], k_flat) + (k_rot @ q_rot.T)).mul(m["scale"])
    far = scores(key_pos)
    far[:cfg["vocab"] // 2] = -1e9                        # the prompts are drawn from the lower half
    best = int(far.amax(-1).argmax())
    return best, float(far[best].max() - scores(last_pos)[last_token].max())


@pytest.mark.parametrize("tag", ["latent", "latent_wide"])
@pytest.mark.parametrize("key_pos", [0, 1, 63, 64, 255, 256, 317])
def test_one_far_key_among_hundreds_decides(one_layer_engines, tag, key_pos):
    """The token whose key fits the last query best is put at ``key_pos`` - the first places, both sides
    of page borders, just before the end - among 320 others: the last logits follow it, in a prompt
    and when the last tokens are decoded alone."""
    eng, cfg, w = one_layer_engines(tag, "float32")
    a = [t % (cfg["vocab"] // 2) for t in models.random_prompts(cfg, [320], seed=3)[0]]
    b = list(a)
    b[key_pos], margin = _best_key_token(cfg, w, a[-1], 319, key_pos)      # a token that is nowhere else
    wa, wb = plain.logits(cfg, w, a)[-1], plain.logits(cfg, w, b)[-1]
    assert (wa - wb).abs().max() > 1e-2 * wa.abs().max(), margin        # the key is seen
    for run in (helpers.whole, lambda e, ids: helpers.tail_one_by_one(e, ids, 3)):
        gb = run(eng, b)[-1]
        assert helpers.rel_err(gb, wb) <= helpers.TOL["float32"]
        assert helpers.rel_err(run(eng, a)[-1] - gb, wa - wb) <= 1e-3


@pytest.mark.parametrize("tag", ["delta", "delta_wide"])
@pytest.mark.parametrize("changed", [0, 63, 64, 300, 318])
def test_one_changed_token_moves_the_last_logits(one_layer_engines, tag, changed):
    """The same prompt with one token changed: what the state carries of it moves the logits at the end in
    the engine as in the plain model, in a prompt and when the last tokens are decoded alone."""
    eng, cfg, w = one_layer_engines(tag, "float32")
    a = models.random_prompts(cfg, [320], seed=3)[0]
    b = list(a)
    b[changed] = (a[changed] + 1) % cfg["vocab"]
    wa, wb = plain.logits(cfg, w, a)[-1], plain.logits(cfg, w, b)[-1]
    if changed >= 300:
        assert (wa - wb).abs().max() > 1e-4 * wa.abs().max()
    for run in (helpers.whole, lambda e, ids: helpers.tail_one_by_one(e, ids, 3)):
        ga, gb = run(eng, a)[-1], run(eng, b)[-1]
        assert (ga - gb - (wa - wb).float()).abs().max().item() <= 2e-2 * float((wa - wb).abs().max()) + 2e-5 * float(wa.abs().max())


def test_the_sink_takes_weight_from_every_key(one_layer_engines, tmp_path):
    """Raising one head's sink score by 6 must change the logits as it does in the plain model."""
    from enginekernel_b200 import Engine
    _, cfg, w = one_layer_engines("latent", "float32")
    w2 = dict(w)
    s = w["l0.mix.sink"].float().clone()
    s[1] += 6.0
    w2["l0.mix.sink"] = s.to(torch.bfloat16)
    eng = Engine(models.write_folder(str(tmp_path / "m"), cfg, w2), "float32", max_tokens=512, max_batch=2)
    ids = models.random_prompts(cfg, [100], seed=4)[0]
    want, base = plain.logits(cfg, w2, ids), plain.logits(cfg, w, ids)
    assert (want - base).abs().max() > 1e-3 * base.abs().max()
    assert helpers.rel_err(helpers.whole(eng, ids), want) <= helpers.TOL["float32"]
    assert helpers.rel_err(helpers.tail_one_by_one(eng, ids, 70), want) <= helpers.TOL["float32"]


# ===================================================================== whole models
SEEDS = {"mixed": 11, "plain": 12, "odd": 13, "wide": 14}
TAGS = list(models.SHAPES)
# 32-bit runs take sharp weights and every row must fit.  In bfloat16 a router score that rounds the other
# way sends a token to another expert; that moves its logits by much more than rounding does, and through the
# delta rule's state and the cached latents also, less and less, the rows behind it (the plain model would
# do the same, were it rounded).  So those runs take milder weights, the typical row must fit,
# and 85 rows in a hundred (or all but two) must lie within five times the limit; the strict 16-bit
# comparisons are the one-mixer models above, which have no router.
SHARP = {"float32": 1.0, "bfloat16": 0.4}
ALLOWED = {"float32": 1.0, "bfloat16": 0.85}


@pytest.fixture(scope="module")
def weights():
    return {(tag, dtype): models.make_tensors(cfg, SEEDS[tag], sharp=SHARP[dtype])
            for tag, cfg in models.SHAPES.items() for dtype in SHARP}


@pytest.fixture(scope="module")
def engines(tmp_path_factory, weights):
    from enginekernel_b200 import Engine
    made = {}

    def get(tag, dtype):
        if (tag, dtype) not in made:
            folder = models.write_folder(str(tmp_path_factory.mktemp("susalorn_" + tag)), models.SHAPES[tag],
                                         weights[(tag, dtype)])
            made[(tag, dtype)] = Engine(folder, dtype, max_tokens=4096, max_batch=8)
        return made[(tag, dtype)]
    return get


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().amax(-1) / want.abs().max()
    limit = helpers.TOL[dtype] * (5 if dtype == "bfloat16" else 1)
    inside = (err <= limit).sum().item()
    assert inside >= ALLOWED[dtype] * err.numel() or err.numel() - inside <= (2 if dtype == "bfloat16" else 0), \
        f"{what} {dtype}: {inside} of {err.numel()} rows within {limit}, worst {err.max():.3e}"
    if dtype == "bfloat16":
        assert err.median().item() <= helpers.TOL[dtype], f"{what}: median {err.median():.3e}"


def want_logits(weights, tag, ids, dtype):
    return plain.logits(models.SHAPES[tag], weights[(tag, dtype)], ids)


def in_portions(engine, tokens, sizes):
    slot = engine.open_sequence()
    try:
        rows, at = [], 0
        for n in list(sizes) + [len(tokens)]:
            part = tokens[at:at + n]
            if not part:
                break
            rows.append(engine.step([(slot, part, list(range(len(part))))]).cpu())
            at += len(part)
        return torch.cat(rows, 0)
    finally:
        engine.close_sequence(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_whole_prompts(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    for j, n in enumerate((1, 2, 7, 33, 64, 65, 130, 200, 530)):       # (from 512 tokens on the convolution has a kernel of its own)
        ids = models.random_prompts(models.SHAPES[tag], [n], seed=40 + j)[0]
        close(helpers.whole(eng, ids), want_logits(weights, tag, ids, dtype), dtype, f"{tag} length {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_prompt_then_token_by_token(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [150], seed=77)[0]
    got = helpers.tail_one_by_one(eng, ids, 40)
    close(got, want_logits(weights, tag, ids, dtype), dtype, tag)
    if dtype == "float32":
        assert helpers.rel_err(got, helpers.whole(eng, ids)) <= 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_prompts_in_portions(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [210], seed=78)[0]
    want = want_logits(weights, tag, ids, dtype)
    for sizes in ((2, 2, 2, 3, 17), (64, 64, 2), (63, 2, 65), (1, 127, 2), (129,)):
        close(in_portions(eng, ids, sizes), want, dtype, f"{tag} portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_unequal_batches_and_reuse(engines, weights, tag, dtype):
    """Requests of unequal lengths start together and end at different steps; three such batches in a row
    through the same few slots, pages and states, then everything is free again."""
    eng = engines(tag, dtype)
    shapes = [((5, 9, 13), (3, 9, 1)), ((1, 70, 31, 16), (1, 64, 20, 16)), ((66, 2, 140), (65, 1, 100))]
    for j, (lens, heads) in enumerate(shapes):
        seqs = models.random_prompts(models.SHAPES[tag], lens, seed=200 + j)
        got = helpers.batch_then_steps(eng, seqs, heads)
        for ids, g in zip(seqs, got):
            close(g, want_logits(weights, tag, ids, dtype), dtype, f"{tag} batch {j} length {len(ids)}")
    assert eng.cache.book.open_slots() == []
    assert eng.cache.free_tokens() == eng.cache.num_pages * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_one_by_one(engines, weights, dtype):
    eng = engines("odd", dtype)
    ids = models.random_prompts(models.SHAPES["odd"], [7], seed=5)[0]
    close(helpers.tail_one_by_one(eng, ids, tail=6), want_logits(weights, "odd", ids, dtype), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["mixed", "plain"])
def test_long_decoding(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [420], seed=9)[0]
    close(helpers.tail_one_by_one(eng, ids, tail=410), want_logits(weights, tag, ids, dtype), dtype, tag)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(tmp_path, dtype):
    """``Engine.generate_all``: five requests of unequal lengths through two slots, so the scheduler forms
    several batches and the captured decode step runs on slots and states used before."""
    from enginekernel_b200 import Engine
    cfg = models.SHAPES["mixed"]
    w = models.make_tensors(cfg, 21)
    w["embed"] = (w["embed"].float() * 0.3).to(torch.bfloat16)
    folder = models.write_folder(str(tmp_path / "m"), cfg, w)
    eng = Engine(folder, dtype, max_tokens=2048, max_batch=2)
    prompts = models.random_prompts(cfg, [3, 70, 17, 64, 1], seed=8)
    got = eng.generate_all(prompts, 12)
    distinct = set()
    for ids, out in zip(prompts, got):
        assert len(out) == 12
        want = plain.greedy(cfg, w, ids, 12)
        distinct.update(want)
        if dtype == "float32":
            assert out == want
        else:
            assert out[:1] == want[:1]
    assert len(distinct) > 3
    assert eng.cache.book.open_slots() == []


def test_sizes_only_the_file_knows_and_unused_tensors(tmp_path):
    """The low-rank pairs' inner sizes come from the file; a layer without feed-forward may still carry its
    second norm and stream coefficients; a file whose pair disagrees or that lacks a tensor is refused."""
    from enginekernel_b200 import Engine
    from enginekernel_b200.weights.checkpoint import WeightsError
    cfg = models.SHAPES["odd"]
    w = models.make_tensors(cfg, 2)
    w["l2.norm2"] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    w["l2.hc2.in"] = torch.ones(1, dtype=torch.bfloat16)
    eng = Engine(models.write_folder(str(tmp_path / "a"), cfg, w), "float32", max_tokens=256, max_batch=2)
    ids = models.random_prompts(cfg, [20], seed=1)[0]
    assert helpers.rel_err(helpers.whole(eng, ids), plain.logits(cfg, w, ids)) <= helpers.TOL["float32"]
    bad = dict(w)
    bad["l0.mix.a2"] = torch.zeros(3 * 40, 6, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="inner sizes"):
        Engine(models.write_folder(str(tmp_path / "b"), cfg, bad), "float32", max_tokens=256, max_batch=2)
    del w["l1.mix.sink"]
    with pytest.raises(WeightsError, match="l1.mix.sink"):
        Engine(models.write_folder(str(tmp_path / "c"), cfg, w), "float32", max_tokens=256, max_batch=2)


def test_command_line_and_trace_replay(tmp_path):
    """``random-model`` writes a Susalorn folder from a configuration file (the low-rank pairs take the
    configuration's ``rank``), ``generate`` prints the plain model's greedy tokens for it, and
    ``bin/trace_run`` replays steps over the same folder."""
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors import safe_open
    from tests.test_cli_gpu import ROOT, run_cli
    cfg = models.SHAPES["odd"]
    raw = models.file_config(cfg)
    for layer in raw["layers"]:
        if layer["type"] == "channel_delta":
            layer["mixer"]["rank"] = 6
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(raw))
    folder = tmp_path / "model"
    run_cli("random-model", "--config", str(config_file), "--seed", "5", "--out", str(folder))
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        w = {name: f.get_tensor(name) for name in f.keys()}
    assert set(w) == set(models.tensor_shapes(cfg))
    assert w["l0.mix.a1"].shape[0] == 6 and w["l2.mix.g2"].shape[1] == 6
    prompts = models.random_prompts(cfg, (3, 40), seed=4)
    ids = ";".join(",".join(str(t) for t in p) for p in prompts)
    out = run_cli("generate", "--model", str(folder), "--dtype", "float32", "--prompt-ids", ids, "--out-len", "5")
    rows = [json.loads(line) for line in out.strip().splitlines()]
    assert [r["tokens"] for r in rows] == [plain.greedy(cfg, w, p, 5) for p in prompts]

    steps = [{"step": 0, "entries": [{"id": "a", "tokens": prompts[1][:30], "want": [0, 29]},
                                     {"id": "b", "tokens": prompts[0][:1], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": prompts[1][30:31], "want": [0]},
                                     {"id": "b", "tokens": prompts[0][1:2], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": prompts[1][31:32], "want": [0]}], "end": ["a"]}]
    out_dir = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(folder), "--dtype",
                        "float32", "--out", str(out_dir), "--max-tokens", "128"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    a, b = plain.logits(cfg, w, prompts[1][:32]), plain.logits(cfg, w, prompts[0][:2])
    want = {0: torch.stack([a[0], a[29]]), 1: torch.stack([a[30], b[1]]), 2: a[31:32]}
    for n, rows_wanted in want.items():
        got = torch.from_numpy(np.fromfile(str(out_dir / f"{n}.f32"), dtype="<f4").reshape(rows_wanted.shape))
        assert helpers.rel_err(got, rows_wanted) <= helpers.TOL["float32"], n
