"""The Lopazen decoder in the engine against the plain implementation, mechanism by mechanism
and then whole models under every way of cutting the work.

Part one drives single kernels with inputs made so that a fault shows: one far key whose score
stands out, scores so low that only the sink is left, positions on both sides of every step of
the query temperature.  Part two runs four small models of unlike shapes (tests/plain/
lopazen_models.py) through ``Engine``: whole prompts, prompts in portions, token-by-token
decoding, unequal batches, slots and pages used again, long decoding, and greedy generation
through the scheduler.
"""

import math

import pytest
import torch

from tests import helpers
from tests.plain import lopazen_models as models
from tests.plain import lopazen_plain as plain
from tests.test_kernels_gpu import DEV, DTYPES, TOL, K, Pages, rel, rnd

pytestmark = pytest.mark.gpu


# ===================================================================== mechanisms alone
def sink_attention(q, keys, values, pos, scale, sink, window=None):
    """q [NH, D] at position ``pos`` over keys/values [len, NKV, D]: softmax with exp(sink) added to
    the denominator, in 64-bit."""
    nh, nkv = q.shape[0], keys.shape[1]
    lo = 0 if not window else max(0, pos - window + 1)
    kk = keys[lo:pos + 1].double().repeat_interleave(nh // nkv, 1)
    vv = values[lo:pos + 1].double().repeat_interleave(nh // nkv, 1)
    s = torch.einsum("hd,jhd->hj", q.double(), kk) * scale
    e = torch.exp(s)
    p = e / (math.exp(sink) + e.sum(-1, keepdim=True))
    return torch.einsum("hj,jhd->hd", p, vv).reshape(-1)


def _filled_pages(lens, nkv, d, dtype, seed):
    pages = Pages(len(lens), max(lens), nkv, d, dtype, seed=seed)
    kv = []
    for s, n in enumerate(lens):
        keys, vals = rnd(n, nkv, d, dtype=dtype, seed=10 + s), rnd(n, nkv, d, dtype=dtype, seed=20 + s)
        pages.fill(s, keys, vals)
        kv.append((keys.cpu(), vals.cpu()))
    return pages, kv


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (6, 3, 48), (3, 1, 40), (8, 2, 128), (5, 5, 24)])
def test_sink_in_the_general_kernel(dtype, nq, nkv, d):
    """Single tokens at many positions, with and without key splits and windows.  Row 3 has one
    far key that dominates; row 5 has scores so low that the sink takes nearly all the weight and
    the output must be close to zero - without the sink it would be an average of values."""
    k = K()
    lens = [1, 64, 65, 517, 130]
    pages, kv = _filled_pages(lens, nkv, d, dtype, seed=3)
    toks = [(0, 0), (1, 63), (2, 64), (3, 516), (3, 0), (3, 255), (4, 129), (4, 64), (2, -1)]
    t = len(toks)
    q = rnd(t, nq * d + 3 * d, dtype=dtype, seed=30)
    q[3, :d] = (kv[3][0][3, 0].float() * 4).to(dtype)
    q[5] = q[5] * 0
    q[5, :nq * d] = -(kv[3][0][:256, 0].float().mean(0) * 40).repeat(nq).to(dtype)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    for sink in (0.0, 1.5, -2.0):
        for window, splits, per in ((None, 1, 0), (None, 5, 128), (100, 1, 0), (64, 3, 192)):
            out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
            acc = torch.empty(t * nq * splits * d, device=DEV)
            ml = torch.empty(t * nq * splits * 2, device=DEV)
            k.attention_generic(out, q, t, positions, slots, pages.k, pages.v, pages.table, nq, nkv, d,
                                scale, window, splits, per, acc, ml, sink=sink)
            for i, (s, p) in enumerate(toks):
                if p < 0:
                    assert out[i].abs().max().item() == 0
                    continue
                want = sink_attention(q[i, :nq * d].view(nq, d).cpu(), kv[s][0], kv[s][1], p, scale, sink, window)
                # against the size of the values, not of this row: rows that the sink empties are near zero
                err = (out[i].double().cpu() - want).abs().max().item() / kv[s][1].double().abs().max().item()
                assert err <= TOL[dtype], (sink, window, splits, i, err)


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 32), (6, 3, 64), (32, 8, 128), (5, 5, 96), (20, 1, 64)])
def test_sink_in_the_decode_kernels(nq, nkv, d):
    """The two bfloat16 decode kernels (streaming through registers; fed by TMA with the splits of
    a token in one cluster): the sink is counted once however the keys are split."""
    k = K()
    dtype = torch.bfloat16
    lens = [1, 64, 65, 517, 130, 16, 17, 1100]
    pages, kv = _filled_pages(lens, nkv, d, dtype, seed=5)
    toks = [(0, 0), (1, 63), (2, 64), (3, 516), (4, 129), (5, 15), (6, 16), (7, 1099), (3, 300), (2, -1)]
    t = len(toks)
    q = rnd(t, nq * d + 2 * nkv * d, dtype=dtype, seed=31)
    q[3, :d] = (kv[3][0][3, 0].float() * 4).to(dtype)              # a far key dominates
    q[7, :nq * d] = -(kv[7][0][:, 0].float().mean(0) * 40).repeat(nq).to(dtype)   # the sink dominates
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)

    def compare(out, sink, window, what):
        for i, (s, p) in enumerate(toks):
            if p < 0:
                continue
            want = sink_attention(q[i, :nq * d].view(nq, d).cpu(), kv[s][0], kv[s][1], p, scale, sink, window)
            err = (out[i].double().cpu() - want).abs().max().item() / kv[s][1].double().abs().max().item()
            assert err <= TOL[dtype], (what, sink, window, i, err)

    for sink in (0.0, 2.0):
        for window, splits in ((None, 1), (None, 4), (100, 2), (None, 9)):
            out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
            acc = torch.empty(t * nq * splits * d, device=DEV)
            ml = torch.empty(t * nq * splits * 2, device=DEV)
            k.attention_decode_bf16(out, q, t, positions, slots, pages.k, pages.v, pages.table, nq, nkv, d,
                                    scale, window, splits, 0, acc, ml, sink=sink)
            compare(out, sink, window, ("registers", splits))
        if k.attention_decode_tma_supported(dtype, d, nq, nkv):
            for window, splits in ((None, 1), (None, 4), (100, 2), (None, 8)):
                out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
                k.attention_decode_tma(out, q, t, positions, slots, pages.k, pages.v, pages.table, nq, nkv,
                                       d, scale, window, splits, sink=sink)
                k.check_tc_status(DEV)
                compare(out, sink, window, ("tma", splits))


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (6, 2, 48), (32, 8, 128), (5, 5, 80), (3, 1, 64), (8, 2, 128)])
def test_sink_in_the_prompt_kernels(nq, nkv, d):
    """The mma.sync and the tcgen05 prompt kernels: several sequences, some continuing a cached prefix."""
    k = K()
    dtype = torch.bfloat16
    seqs = [(1, 0), (64, 0), (65, 0), (517, 0), (130, 100), (200, 199), (300, 37)]
    pages, kv = _filled_pages([n for n, _ in seqs], nkv, d, dtype, seed=7)
    rows, positions, slots, cu = [], [], [], [0]
    for s, (n, start) in enumerate(seqs):
        for p in range(start, n):
            rows.append((s, p))
            positions.append(p)
            slots.append(s)
        cu.append(len(rows))
    t = len(rows)
    q = rnd(t, nq * d + nkv * d, dtype=dtype, seed=30)             # rows as wide as q and k together
    far = rows.index((3, 516))
    q[far, :d] = (kv[3][0][3, 0].float() * 4).to(dtype)
    low = rows.index((3, 400))
    q[low, :nq * d] = -(kv[3][0][:401, 0].float().mean(0) * 40).repeat(nq).to(dtype)
    positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    variants = [k.attention_prefill_bf16]
    if k.attention_prefill_tc_supported(dtype, d, nq, nkv):
        variants.append(k.attention_prefill_tc)
    for fn in variants:
        for sink, window in ((0.0, None), (1.0, 100), (0.0, 64)):
            out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
            fn(out, q, t, positions, slots, cu_t, len(seqs), pages.k, pages.v, pages.table, nq, nkv, d,
               scale, window, sink=sink)
            if fn is k.attention_prefill_tc:
                k.check_tc_status(DEV)
            outc, qc = out.cpu(), q.cpu()
            picks = sorted(set(list(range(0, t, 11)) + [far, low, t - 1, cu[4], cu[5], cu[6], cu[1] - 1, cu[2]]))
            for i in picks:
                s, p = rows[i]
                want = sink_attention(qc[i, :nq * d].view(nq, d), kv[s][0], kv[s][1], p, scale, sink, window)
                err = (outc[i].double() - want).abs().max().item() / kv[s][1].double().abs().max().item()
                assert err <= TOL[dtype], (fn.__name__, sink, window, i, err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,every", [(4, 2, 48, 5), (6, 3, 40, 1), (8, 1, 128, 64), (2, 2, 24, 3),
                                            (3, 3, 64, 128)])
def test_bias_head_norm_temperature_and_values_from_keys(dtype, nq, nkv, d, every):
    """What happens between the q/k projection and the cache: bias, per-head norm, the query
    temperature at positions on both sides of its steps, keys stored normalised and values stored
    as the keys were projected."""
    k = K()
    coef, eps = 0.7, 1e-5
    pos_list = [0, every - 1, every, every + 1, 2 * every - 1, 2 * every, 63, 64, 65, 127, 128, 129, 255, 256, 700]
    pos_list = sorted(set(p for p in pos_list if p >= 0))
    t = len(pos_list)
    pages = Pages(2, 800, nkv, d, dtype, seed=1)
    raw = rnd(t, (nq + nkv) * d, dtype=dtype, seed=2)
    qb, kb = rnd(nq * d, seed=3, scale=0.5), rnd(nkv * d, seed=4, scale=0.5)
    qg, kg = 1 + 0.2 * rnd(d, seed=5), 1 + 0.2 * rnd(d, seed=6)
    positions = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    slots = torch.tensor([i % 2 for i in range(t)], dtype=torch.int32, device=DEV)
    qkv = raw.clone()
    empty = torch.zeros((1, 0), dtype=torch.float32, device=DEV)
    k.qk_prepare_kv(qkv, t, qg, kg, empty, empty, 0, positions, slots, pages.k, pages.v, pages.table, nq, nkv,
                    d, eps, q_bias=qb, k_bias=kb, q_temperature=(coef, every), values_from_keys=True)
    q0 = raw[:, :nq * d].double().cpu() + qb.double().cpu()
    k0 = raw[:, nq * d:].double().cpu() + kb.double().cpu()
    qn = plain.head_norm(q0.view(t, nq, d), qg.cpu(), eps) * \
        plain.query_temperature(pos_list, coef, every)[:, None, None]
    kn = plain.head_norm(k0.view(t, nkv, d), kg.cpu(), eps)
    assert rel(qkv[:, :nq * d], qn.reshape(t, -1)) <= TOL[dtype]
    for i, p in enumerate(pos_list):
        page = int(pages.table[i % 2, p // 64])
        assert rel(pages.k[page, :, p % 64], kn[i]) <= TOL[dtype], p
        assert rel(pages.v[page, :, p % 64], k0[i].view(nkv, d)) <= TOL[dtype], p
    # the temperature is not a constant: its first step lies where the design puts it
    first = plain.query_temperature([every - 2 if every > 1 else 0, every - 1], coef, every)
    assert (every == 1 and first[0] > 1) or (first[0] == 1.0 and first[1] > 1.0)


def _prepared(raw, qb, kb, qg, kg, pos_list, nq, nkv, d, coef, every, eps):
    """What the cache and the query rows must hold, from the plain functions: (q, k normalised, v)."""
    t = raw.shape[0]
    q0 = raw[:, :nq * d].double().cpu() + qb.double().cpu()
    k0 = raw[:, nq * d:].double().cpu() + kb.double().cpu()
    qn = plain.head_norm(q0.view(t, nq, d), qg.cpu(), eps) * \
        plain.query_temperature(pos_list, coef, every)[:, None, None]
    return qn.reshape(t, -1), plain.head_norm(k0.view(t, nkv, d), kg.cpu(), eps), k0.view(t, nkv, d)


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 64), (8, 2, 128), (3, 1, 256), (40, 8, 128)])
def test_prepare_of_many_tokens(nq, nkv, d):
    """The form that takes a whole token a block (16-bit rows, 128 tokens and more, no rotation)."""
    k = K()
    dtype, coef, every, eps = torch.bfloat16, 0.4, 7, 1e-6
    t = 333
    pos_list = list(dict.fromkeys((i * 5) % 700 for i in range(t)))   # 140 positions, each once
    t = len(pos_list)
    assert t >= 128
    pages = Pages(1, 800, nkv, d, dtype, seed=1)
    raw = rnd(t, (nq + nkv) * d, dtype=dtype, seed=2)
    qb, kb = rnd(nq * d, seed=3, scale=0.5), rnd(nkv * d, seed=4, scale=0.5)
    qg, kg = 1 + 0.2 * rnd(d, seed=5), 1 + 0.2 * rnd(d, seed=6)
    positions = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    slots = torch.zeros(t, dtype=torch.int32, device=DEV)
    qkv = raw.clone()
    empty = torch.zeros((1, 0), dtype=torch.float32, device=DEV)
    k.qk_prepare_kv(qkv, t, qg, kg, empty, empty, 0, positions, slots, pages.k, pages.v, pages.table, nq, nkv,
                    d, eps, q_bias=qb, k_bias=kb, q_temperature=(coef, every), values_from_keys=True)
    qn, kn, k0 = _prepared(raw, qb, kb, qg, kg, pos_list, nq, nkv, d, coef, every, eps)
    assert rel(qkv[:, :nq * d], qn) <= TOL[dtype]
    kd, vd = pages.dense(0, 700)
    idx = torch.tensor(pos_list)
    assert rel(kd.cpu()[idx], kn) <= TOL[dtype]
    assert rel(vd.cpu()[idx], k0) <= TOL[dtype]


@pytest.mark.parametrize("m,nq,nkv,hidden", [(1, 4, 2, 320), (8, 8, 2, 1024), (33, 3, 1, 136), (64, 8, 8, 512)])
def test_projection_with_the_prepare_in_its_epilogue(m, nq, nkv, hidden):
    """The q/k product of few rows (heads of 128) that adds the biases, normalises the heads, applies
    the query temperature and stores keys and values itself."""
    k = K()
    dtype, d, coef, every, eps = torch.bfloat16, 128, 0.6, 3, 1e-5
    pos_list = [(7 * i + 2) % 400 for i in range(m)]
    pages = Pages(m, 400, nkv, d, dtype, seed=1)
    x = rnd(m, hidden, dtype=dtype, seed=2)
    w = rnd((nq + nkv) * d, hidden, dtype=dtype, seed=3, scale=hidden ** -0.5)
    qb, kb = rnd(nq * d, seed=4, scale=0.5), rnd(nkv * d, seed=5, scale=0.5)
    qg, kg = 1 + 0.2 * rnd(d, seed=6), 1 + 0.2 * rnd(d, seed=7)
    positions = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    slots = torch.arange(m, dtype=torch.int32, device=DEV)
    qkv = torch.zeros(m, (nq + nkv) * d, dtype=dtype, device=DEV)
    for k_split in (1, 2, None):
        pages.k.zero_()
        pages.v.zero_()
        k.gemm_tc_qkv_prepare(qkv, x, w, m, qg, kg, eps, None, None, positions, slots, pages.k, pages.v,
                              pages.table, nq, nkv, k_split=k_split, q_bias=qb, k_bias=kb,
                              q_temperature=(coef, every), values_from_keys=True)
        k.check_tc_status(DEV)
        raw = x.double() @ w.double().t()
        qn, kn, k0 = _prepared(raw, qb, kb, qg, kg, pos_list, nq, nkv, d, coef, every, eps)
        assert rel(qkv[:, :nq * d], qn) <= 4e-3, k_split
        for i, p in enumerate(pos_list):
            page = int(pages.table[i, p // 64])
            assert rel(pages.k[page, :, p % 64], kn[i]) <= 4e-3
            assert rel(pages.v[page, :, p % 64], k0[i]) <= 4e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_gate_and_embedding_added_again(dtype):
    k = K()
    rows, inter = 37, 200
    gu = rnd(rows, 2 * inter, dtype=dtype, seed=1, scale=3.0)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    k.act_mul(out, gu, "gelu_tanh")
    g, u = gu[:, :inter].double().cpu(), gu[:, inter:].double().cpu()
    assert rel(out, plain.gelu_tanh(g) * u) <= TOL[dtype]
    table = rnd(50, 72, dtype=dtype, seed=2)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    stream = torch.zeros(4, 72, device=DEV)
    k.embed(stream, table, ids, 4, scale=2.5)
    first = stream.clone()
    stream += 1.0
    k.embed(stream, table, ids, 4, scale=2.5, accumulate=True)
    assert rel(stream, 2 * first.double().cpu() + 1.0) <= 1e-6
    assert rel(first, plain.embedding(table.cpu(), ids.cpu().tolist(), 2.5)) <= 1e-6


@pytest.mark.parametrize("m,n,k_", [(1, 256, 128), (17, 1000, 200), (64, 2560, 1024), (65, 1040, 72),
                                    (300, 528, 200), (1000, 2048, 512)])
def test_gelu_gate_in_the_products(m, n, k_):
    """The gate/up product with the tanh form of GELU in its epilogue: the swapped tcgen05 form for
    few rows (K split over a cluster, through scratch, or not), the kernel on pairs of SMs for many."""
    k = K()
    x = rnd(m, k_, dtype=torch.bfloat16, seed=1, scale=2.0)
    w = rnd(n, k_, dtype=torch.bfloat16, seed=2, scale=0.05)
    prod = x.double() @ w.double().t()
    inter = n // 2
    want = (plain.gelu_tanh(prod[:, :inter]) * prod[:, inter:]).cpu()
    act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    if m <= 64:
        for k_split, cluster in ((1, True), (3, True), (3, False), (None, True)):
            act.fill_(9.0)
            k.gemm_tc_bf16(act, x, w, k.EPI_GEGLU, swap=True, k_split=k_split, cluster=cluster)
            k.check_tc_status(DEV)
            assert rel(act, want) <= 4e-3, (k_split, cluster)
    else:
        k.gemm_pair_bf16(act, x, w, k.PAIR_EPI_GEGLU)
        k.check_tc_status(DEV)
        assert rel(act, want) <= 4e-3
        k.gemm_tc_bf16(act, x, w, k.EPI_GEGLU, swap=False)
        k.check_tc_status(DEV)
        assert rel(act, want) <= 4e-3
    # and it is not the SiLU gate
    silu = (prod[:, :inter] / (1 + torch.exp(-prod[:, :inter])) * prod[:, inter:]).cpu()
    assert rel(act, silu) > 2e-2


# ===================================================================== whole models
SEEDS = {"looped": 11, "flat": 12, "odd": 13, "wide": 14, "ragged": 15}


@pytest.fixture(scope="module")
def weights():
    return {tag: models.make_tensors(cfg, SEEDS[tag]) for tag, cfg in models.SHAPES.items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory, weights):
    return {tag: models.write_folder(str(tmp_path_factory.mktemp("lopazen_" + tag)), cfg, weights[tag])
            for tag, cfg in models.SHAPES.items()}


@pytest.fixture(scope="module")
def engines(folders):
    from enginekernel_b200 import Engine
    cache = {}

    def get(tag, dtype):
        if (tag, dtype) not in cache:
            cache[(tag, dtype)] = Engine(folders[tag], dtype, max_tokens=4096, max_batch=8)
        return cache[(tag, dtype)]
    return get


def want_logits(weights, tag, ids):
    return plain.logits(models.SHAPES[tag], weights[tag], ids)


def in_portions(engine, tokens, sizes):
    """One request alone, its tokens in portions of the given sizes (the last one takes the rest)."""
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


TAGS = list(models.SHAPES)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_whole_prompts(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    for j, n in enumerate((1, 2, 7, 33, 64, 65, 130, 200)):
        ids = models.random_prompts(models.SHAPES[tag], [n], seed=40 + j)[0]
        err = helpers.rel_err(helpers.whole(eng, ids), want_logits(weights, tag, ids))
        assert err <= helpers.TOL[dtype], f"{tag} {dtype} length {n}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_prompt_then_token_by_token(engines, weights, tag, dtype):
    """The last 40 of 150 tokens one per step: across a page border and several temperature steps."""
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [150], seed=77)[0]
    want = want_logits(weights, tag, ids)
    got = helpers.tail_one_by_one(eng, ids, 40)
    err = helpers.rel_err(got, want)
    assert err <= helpers.TOL[dtype], f"{tag} {dtype}: {err:.3e}"
    if dtype == "float32":
        assert helpers.rel_err(got, helpers.whole(eng, ids)) <= 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_prompts_in_portions(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [210], seed=78)[0]
    want = want_logits(weights, tag, ids)
    for sizes in ((2, 2, 2, 3, 17), (64, 64, 2), (63, 2, 65), (1, 127, 2), (129,)):
        err = helpers.rel_err(in_portions(eng, ids, sizes), want)
        assert err <= helpers.TOL[dtype], f"{tag} {dtype} portions {sizes}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_unequal_batches_and_reuse(engines, weights, tag, dtype):
    """Requests of unequal lengths start together and end at different steps; three such batches
    in a row through the same few slots and pages, then everything is free again."""
    eng = engines(tag, dtype)
    shapes = [((5, 9, 13), (3, 9, 1)), ((1, 70, 31, 16), (1, 64, 20, 16)), ((66, 2, 140), (65, 1, 100))]
    for j, (lens, heads) in enumerate(shapes):
        seqs = models.random_prompts(models.SHAPES[tag], lens, seed=200 + j)
        got = helpers.batch_then_steps(eng, seqs, heads)
        for ids, g in zip(seqs, got):
            err = helpers.rel_err(g, want_logits(weights, tag, ids))
            assert err <= helpers.TOL[dtype], f"{tag} {dtype} batch {j} length {len(ids)}: {err:.3e}"
    assert eng.cache.book.open_slots() == []
    assert eng.cache.free_tokens() == eng.cache.num_pages * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_one_by_one(engines, weights, dtype):
    eng = engines("odd", dtype)
    ids = models.random_prompts(models.SHAPES["odd"], [6], seed=5)[0]
    got = helpers.tail_one_by_one(eng, ids, tail=5)
    assert helpers.rel_err(got, want_logits(weights, "odd", ids)) <= helpers.TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["looped", "flat"])
def test_long_decoding(engines, weights, tag, dtype):
    """Hundreds of single-token steps across many page borders and temperature steps."""
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [600], seed=9)[0]
    got = helpers.tail_one_by_one(eng, ids, tail=590)
    err = helpers.rel_err(got, want_logits(weights, tag, ids))
    assert err <= helpers.TOL[dtype], f"{err:.3e}"


def test_a_far_token_decides(engines, weights):
    """The same prompt with one early token changed: the logits at the end must move, in the
    engine as in the plain model (the design has no window, so nothing is ever out of sight)."""
    tag = "flat"
    eng = engines(tag, "float32")
    a = models.random_prompts(models.SHAPES[tag], [300], seed=3)[0]
    b = list(a)
    b[1] = (a[1] + 1) % models.SHAPES[tag]["vocab"]
    ga, gb = helpers.tail_one_by_one(eng, a, 3)[-1], helpers.tail_one_by_one(eng, b, 3)[-1]
    wa, wb = want_logits(weights, tag, a)[-1], want_logits(weights, tag, b)[-1]
    assert (wa - wb).abs().max() > 1e-3 * wa.abs().max()
    assert helpers.rel_err(ga - gb, wa - wb) <= 2e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(tmp_path, dtype):
    """``Engine.generate_all``: five requests of unequal lengths through two slots, so the
    scheduler forms several batches and the captured decode step runs on slots used before."""
    from enginekernel_b200 import Engine
    cfg = models.SHAPES["looped"]
    w = models.make_tensors(cfg, 21)
    w["embed"] = (w["embed"].float() * 0.15).to(torch.bfloat16)      # else the tied head repeats the last token
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
        else:                                  # a near tie may flip a token in 16 bits: the start must agree
            assert out[:2] == want[:2]
    assert len(distinct) > 3
    assert eng.cache.book.open_slots() == []


def test_a_stored_but_unused_norm_and_wrong_shapes(tmp_path):
    """A layer without feed-forward may still carry its second norm in the file; a file with a
    missing bias is refused with the tensor's name."""
    from enginekernel_b200 import Engine
    from enginekernel_b200.weights.checkpoint import WeightsError
    cfg = models.SHAPES["odd"]
    w = models.make_tensors(cfg, 2)
    w["l1.norm2"] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    eng = Engine(models.write_folder(str(tmp_path / "a"), cfg, w), "float32", max_tokens=256, max_batch=2)
    ids = models.random_prompts(cfg, [20], seed=1)[0]
    assert helpers.rel_err(helpers.whole(eng, ids), plain.logits(cfg, w, ids)) <= helpers.TOL["float32"]
    del w["l0.mix.k.b"]
    with pytest.raises(WeightsError, match="l0.mix.k.b"):
        Engine(models.write_folder(str(tmp_path / "b"), cfg, w), "float32", max_tokens=256, max_batch=2)


def test_command_line_and_trace_replay(tmp_path):
    """``random-model`` writes a Lopazen folder from a configuration file, ``generate`` prints the
    plain model's greedy tokens for it, and ``bin/trace_run`` replays steps over the same folder."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors import safe_open
    from tests.test_cli_gpu import ROOT, run_cli
    cfg = models.SHAPES["odd"]
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    run_cli("random-model", "--config", str(config_file), "--seed", "5", "--out", str(folder))
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        w = {name: f.get_tensor(name) for name in f.keys()}
    assert set(w) == set(models.tensor_shapes(cfg))
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
