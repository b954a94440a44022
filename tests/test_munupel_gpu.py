"""Munupel on the GPU against the plain implementation (tests/plain_munupel.py): every mechanism's kernels
alone (the layer norm that completes the stream, biases and rescaled rotation at the cache write, the masks,
the score cap, the sink and the gates of the attention kernels, on CUDA cores and on tensor cores), then
whole models through trace replay in every way of cutting, and greedy generation through the entry point."""
import math

import numpy as np
import pytest
import torch

import plain_munupel as pm
import replay_util as ru
from munupel_util import MU_A, MU_B, MU_C, sharpen, write_model

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
F64 = torch.float64


def rel(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def err_word():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H", [(1, 40), (19, 72), (300, 1024), (5, 4100)])
def test_layer_norm_completes_the_stream_and_normalises_it(dtype, T, H):
    """The stream plus two sublayer results plus a bias on every row, written back, and its layer norm
    (mean off, variance with eps inside the root, weight and bias); then the norm of chosen rows."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(T + H)
    x = torch.randn(T, H, generator=g) * 3 + 1.5
    a, b = torch.randn(T, H, generator=g).to(DT[dtype]), torch.randn(T, H, generator=g).to(DT[dtype])
    rb, w, c = torch.randn(H, generator=g), torch.randn(H, generator=g), torch.randn(H, generator=g)
    eps = 1e-5
    xd, out = x.cuda(), torch.empty(T, H, dtype=DT[dtype], device="cuda")
    ops.layernorm(xd, w.cuda(), c.cuda(), eps, out, deltas=(a.cuda(), b.cuda()), row_bias=rb.cuda(), writeback=True)
    v = x.double() + a.double() + b.double() + rb.double()
    want = pm.layer_norm({"n": w.double(), "n.b": c.double()}, "n", v, eps)
    assert rel(xd, v) <= 1e-6
    assert rel(out, want) <= (3e-6 if dtype == "float32" else 1e-2)
    rows = [T - 1, 0, T // 2]
    some = torch.empty(3, H, dtype=DT[dtype], device="cuda")
    ops.layernorm(xd, w.cuda(), c.cuda(), eps, some, rows=i32(rows))
    assert rel(some, want[rows]) <= (3e-6 if dtype == "float32" else 1e-2)
    # the plain adds: one term, two terms and a bias; a bias on the rows of a projection's result
    y = x.cuda()
    ops.add_rows(y, (a.cuda(),))
    ops.add_rows(y, (a.cuda(), b.cuda()), rb.cuda())
    assert rel(y, x.double() + 2 * a.double() + b.double() + rb.double()) <= 1e-6
    z = a.cuda().clone()
    ops.add_row_bias(z, rb.cuda())
    assert rel(z, a.double() + rb.double()) <= (1e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,dk,dv,rot", [(6, 2, 24, 40, {"dims": 12, "base": 10000.0}),
                                             (4, 4, 16, 16, {"dims": 16, "base": 300.0, "scaling": {
                                                 "factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}}),
                                             (2, 1, 64, 32, {"dims": 2, "base": 3.0}),
                                             (8, 2, 64, 64, {"dims": 32, "base": 1000000.0, "scaling": {
                                                 "factor": 8.0, "original": 2048, "fast": 16.0, "slow": 2.0}}),
                                             (4, 1, 128, 64, {"dims": 128, "base": 10000.0}),
                                             (2, 2, 32, 48, {"dims": 16, "base": 10000.0}),
                                             (3, 1, 20, 28, {"dims": 20, "base": 250000.0, "scaling": {
                                                 "factor": 3.0, "original": 256, "fast": 24.0, "slow": 1.5}})])
def test_biases_and_rescaled_rotation_at_the_cache_write(dtype, nq, nkv, dk, dv, rot):
    """One kernel adds the biases of q, k and v, rotates the first dims of every query and key head by the
    token's position (slowed frequencies, cosine and sine times the rule's factor) and writes keys and values
    to the token's place in shuffled pages; the columns behind the value heads (a gate's) stay."""
    from rllm_b200.kernels import ops
    from rllm_b200.parts.registry import build_part
    from rllm_b200.parts.spec import PartSpec
    g = torch.Generator().manual_seed(dk)
    page, positions, tseq = 8, [0, 1, 9, 130, 4000, 7], [0, 0, 0, 1, 2, 1]
    T, extra = len(positions), 5
    width = nq * dk + nkv * (dk + dv)
    rows = torch.randn(T, width + extra, generator=g).to(DT[dtype])
    bias = torch.randn(width, generator=g)
    sc = rot.get("scaling")
    part = build_part("position_encoding", PartSpec.of(
        "rotary", head_dim=dk, rotary_dim=rot["dims"], theta=rot["base"],
        scaling=None if sc is None else dict(sc, kind="yarn")))
    inv_freq, rd = part.fused_rotary(torch.device("cuda"))
    f, mag = pm.rotation_frequencies(rot)
    assert rd == rot["dims"] and rel(inv_freq, torch.tensor(f, dtype=F64)) <= 1e-12
    assert abs(float(getattr(part, "magnitude", 1.0)) - mag) <= 1e-12
    table = torch.tensor([[3, 1, -1], [0, 20, 17], [5, 2, 4]], dtype=torch.int32)
    table = torch.cat([table, torch.full((3, 510), 6, dtype=torch.int32)], dim=1)     # far positions: page 6
    kc = torch.zeros(24, nkv, page, dk, dtype=DT[dtype], device="cuda")
    vc = torch.zeros(24, nkv, page, dv, dtype=DT[dtype], device="cuda")
    qkv, err = rows.cuda(), err_word()
    ops.head_norm_kv_write(qkv, i32(positions), i32(tseq), None, None, 0.0, table.cuda(), kc, vc, nq, nkv, dk, dv, err,
                           bias=bias.cuda(), inv_freq=inv_freq, rotary_dim=rd, magnitude=mag)
    assert int(err.item()) == 0
    full = rows[:, :width].double() + bias.double()
    pos = torch.tensor(positions)
    q = pm.rotate(full[:, :nq * dk].reshape(T, nq, dk), rot, pos)
    k = pm.rotate(full[:, nq * dk: (nq + nkv) * dk].reshape(T, nkv, dk), rot, pos)
    v = full[:, (nq + nkv) * dk:].reshape(T, nkv, dv)
    tol = 3e-6 if dtype == "float32" else 1e-2
    assert rel(qkv[:, :nq * dk], q.reshape(T, -1)) <= tol
    assert torch.equal(qkv[:, width:].cpu(), rows[:, width:])
    for t, (p, s) in enumerate(zip(positions, tseq)):
        pg = int(table[s, p // page])
        assert rel(kc[pg, :, p % page], k[t]) <= tol and rel(vc[pg, :, p % page], v[t]) <= tol


# ---------------------------------------------------------------------------
# the attention kernels with masks, cap, sink and gates
# ---------------------------------------------------------------------------
def visible(kind, i, j, size, keep):
    if kind == "chunk":
        return pm.sees_chunk(i, j, size)
    if kind == "window" and size:
        return pm.sees_window_keep(i, j, size, keep)
    return j <= i                                        # (a window of 0: every earlier key)


def plain_attend(q, k, v, i, h, kvh, kind, size, keep, scale, cap, sink):
    """Row i, head h in float64: scaled (capped) scores over the visible keys, softmax whose denominator
    may hold exp(sink) as well."""
    js = [j for j in range(i + 1) if visible(kind, i, j, size, keep)]
    s = (k[js, kvh] @ q[i, h]) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
    e = torch.exp(s - top)
    den = e.sum() + (0.0 if sink is None else torch.exp(sink[h] - top))
    return (e / den) @ v[js, kvh]


def attention_case(dtype, path, nq, nkv, dk, dv, page, lens, news, scale, kind="window", size=0, keep=0, cap=0.0,
                   sinks=False, gate=None, boost=None, seed=0):
    """Sequences on shuffled pages; the last ``news[s]`` tokens of sequence s are this step's queries (every
    key, theirs included, is in the pages already).  ``path`` "simt": the CUDA-core kernel; "mma": the
    tensor-core kernels, the decode kernel for the sequences with one query (they come first) and the prompt
    kernel for the rest; "tcgen05": the same with the tcgen05 prompt kernel.  Returns (got, want) [T, nq, dv]."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    per = [-(-n // page) for n in lens]
    perm = torch.randperm(sum(per) + 3, generator=g)
    table = torch.full((S, max(per)), -1, dtype=torch.int32)
    kc = torch.zeros(sum(per) + 3, nkv, page, dk, dtype=DT[dtype])
    vc = torch.zeros(sum(per) + 3, nkv, page, dv, dtype=DT[dtype])
    sink = torch.randn(nq, generator=torch.Generator().manual_seed(seed + 1000)) * 2 + 1 if sinks else None
    gw = 0 if gate is None else (nq if gate == "head" else nq * dv)
    rows, positions, tseq, want = [], [], [], []
    at = 0
    for s, (n, new) in enumerate(zip(lens, news)):
        table[s, :per[s]] = perm[at:at + per[s]].to(torch.int32)
        at += per[s]
        q = torch.randn(n, nq, dk, generator=g)
        k = torch.randn(n, nkv, dk, generator=g)
        v = torch.randn(n, nkv, dv, generator=g).to(DT[dtype])
        gt = torch.randn(n, gw, generator=g).to(DT[dtype]) * 2
        if boost is not None:
            boost(s, q, k)
        q, k = q.to(DT[dtype]), k.to(DT[dtype])
        for j in range(n):
            kc[table[s, j // page], :, j % page] = k[j]
            vc[table[s, j // page], :, j % page] = v[j]
        for i in range(n - new, n):
            rows.append(torch.cat([q[i].reshape(-1), gt[i], torch.zeros((-(nq * dk + gw)) % 8, dtype=DT[dtype])]))
            positions.append(i)
            tseq.append(s)
            o = torch.stack([plain_attend(q.double(), k.double(), v.double(), i, h, h // (nq // nkv), kind, size, keep,
                                          scale, cap, None if sink is None else sink.double()) for h in range(nq)])
            if gate == "head":
                o = o * torch.sigmoid(gt[i].double())[:, None]
            elif gate == "element":
                o = o * torch.sigmoid(gt[i].double()).view(nq, dv)
            want.append(o)
    qg = torch.stack(rows).cuda()
    T = len(rows)
    kcd, vcd, err = kc.cuda(), vc.cuda(), err_word()
    out = torch.empty(T, nq * dv, dtype=DT[dtype], device="cuda")
    gview = qg[:, nq * dk: nq * dk + gw] if gate else None              # (rows padded to a multiple of 8 elements)
    window = size if kind == "window" else 0
    opts = dict(keep_first=keep if kind == "window" else 0, chunk=size if kind == "chunk" else 0, softcap=cap,
                sinks=None if sink is None else sink.cuda(), gate=gview, gate_per_head=gate == "head")
    if path == "simt":
        ops.attention_simt_kv(qg, qg.shape[1], out, kcd, vcd, table.cuda(), i32(positions), i32(tseq), nq, nkv, window,
                              scale, err, **opts)
    else:
        assert dk == dv and dtype == "bfloat16"
        nd = sum(1 for n in news if n == 1)
        assert all(n == 1 for n in news[:nd]) and all(n > 1 for n in news[nd:])
        q_start = i32([0] + list(np.cumsum(news)))
        if nd:
            ops.attention_decode_bf16(qg, qg.shape[1], out, kcd, vcd, table.cuda(), i32(lens), nd, max(lens[:nd]), nq,
                                      nkv, dk, window, scale, err, **opts)
        if S > nd:
            prompt = ops.attention_prefill_tcgen05 if path == "tcgen05" else ops.attention_prefill_bf16
            prompt(qg, qg.shape[1], out, kcd, vcd, table.cuda(), q_start, i32(lens), nd, S, T - nd,
                                       nq, nkv, dk, window, scale, err, **opts)
    assert int(err.item()) == 0
    return out.view(T, nq, dv), torch.stack(want)


CASES = [  # nq, nkv, dk, dv, page, kind, size, keep, cap, sinks, gate
    (6, 2, 24, 40, 16, "window", 11, 3, 0.0, True, "head"),
    (4, 4, 16, 16, 4, "chunk", 13, 0, 5.0, False, "element"),
    (2, 1, 40, 24, 8, "window", 37, 20, 0.0, True, None),
    (3, 1, 20, 28, 16, "chunk", 50, 0, 0.0, False, "head"),
    (8, 2, 64, 64, 16, "window", 64, 1, 2.0, True, "element"),
    (8, 1, 32, 32, 16, "chunk", 32, 0, 2.0, True, "head"),
    (2, 2, 128, 128, 16, "window", 1, 2, 0.0, False, None),
    (4, 1, 16, 16, 8, "chunk", 1, 0, 0.0, False, None),
    (4, 2, 64, 64, 16, "window", 200, 130, 0.0, True, "head"),
    (16, 1, 128, 128, 16, "chunk", 128, 0, 30.0, False, "element"),
]


def takes(path, dk, dv, page):
    if path == "mma":
        return dk == dv and dk in (16, 32, 64, 128)
    if path == "tcgen05":
        return dk == dv and dk in (64, 128) and page in (16, 32, 64)
    return True


@pytest.mark.parametrize("dtype,path", [("float32", "simt"), ("bfloat16", "simt"), ("bfloat16", "mma"),
                                        ("bfloat16", "tcgen05")])
@pytest.mark.parametrize("case", CASES)
def test_masks_cap_sink_and_gates_in_the_attention_kernels(dtype, path, case):
    """Two decoded tokens, a prompt portion behind a cached prefix and a whole short prompt in one step,
    keys on shuffled pages, against the formula in float64: a window beside kept first keys, chunks, a
    tanh cap on the scores, a sink in the denominator, a gate per head or per element."""
    nq, nkv, dk, dv, page, kind, size, keep, cap, sinks, gate = case
    if not takes(path, dk, dv, page):
        pytest.skip("the tensor-core kernels take keys and values of one size: 16, 32, 64 or 128 (tcgen05: 64, 128)")
    got, want = attention_case(dtype, path, nq, nkv, dk, dv, page, [141, 300, 83, 19], [1, 1, 50, 19], dk ** -0.5 * 3,
                               kind=kind, size=size, keep=keep, cap=cap, sinks=sinks, gate=gate, seed=nq + dk)
    assert rel(got, want) <= (3e-6 if dtype == "float32" else 2e-2)


def _one_loud_key(key_pos, n, new, path, **kw):
    """All queries and the key at ``key_pos`` point along one axis, no other key has anything there: whoever
    sees that key returns (nearly) its value."""
    def boost(s, q, k):
        q.mul_(0.05)
        q[:, :, 0] = 6.0
        k[:, :, 0] = 0.0
        k[key_pos].mul_(0.05)
        k[key_pos, :, 0] = 6.0
    dtype = "float32" if path == "simt" else "bfloat16"
    d = 64 if path == "tcgen05" else 16
    return attention_case(dtype, path, 2, 1, d, d, kw.pop("page", 16), [n], [new], 4.0, boost=boost, **kw)


@pytest.mark.parametrize("path", ["simt", "mma", "tcgen05"])
@pytest.mark.parametrize("new", [1, 30, 200])
@pytest.mark.parametrize("size,keep,page", [(5, 2, 16), (16, 1, 16), (17, 20, 4), (100, 7, 16), (64, 64, 16), (130, 3, 8)])
def test_keys_at_the_edges_of_the_window_and_of_the_kept_first(path, new, size, keep, page):
    """The last query must see the oldest key of its window and not the one before it; it must see the last
    of the kept first keys and not the next one (which is far outside the window); as a decoded token and in
    a prompt portion, edges on and off page borders."""
    if not takes(path, 64, 64, page):
        pytest.skip("the tcgen05 kernel takes pages of 16, 32 or 64 keys")
    n = 3 * size + keep + 270
    last = n - 1
    tol = 3e-6 if path == "simt" else 2e-2
    kw = dict(kind="window", size=size, keep=keep, page=page, seed=size)
    pairs = [(last - size + 1, last - size), (keep - 1, keep)]
    for seen, hidden in pairs:
        g1, w1 = _one_loud_key(seen, n, new, path, **kw)
        g0, w0 = _one_loud_key(hidden, n, new, path, **kw)
        assert rel(g1, w1) <= tol and rel(g0, w0) <= tol
        assert float((w1[-1] - w0[-1]).abs().max()) > 0.2
        assert float((g1[-1].double().cpu() - w0[-1]).abs().max()) > 0.2


@pytest.mark.parametrize("path", ["simt", "mma", "tcgen05"])
@pytest.mark.parametrize("new", [1, 30, 200])
@pytest.mark.parametrize("size,page", [(5, 16), (16, 16), (13, 4), (112, 16), (128, 16), (200, 8)])
def test_keys_at_the_edges_of_a_chunk(path, new, size, page):
    """A query at the start, in the middle and at the end of its chunk sees the chunk's first key and not
    the last key of the chunk before; chunks are counted from the sequence's first position."""
    if not takes(path, 64, 64, page):
        pytest.skip("the tcgen05 kernel takes pages of 16, 32 or 64 keys")
    tol = 3e-6 if path == "simt" else 2e-2
    for n in (3 * size + 1, 3 * size + size // 2 + 1, 4 * size):
        if new > 1 and n <= new:
            continue
        first = (n - 1) // size * size
        kw = dict(kind="chunk", size=size, page=page, seed=size)
        g1, w1 = _one_loud_key(first, n, new, path, **kw)
        g0, w0 = _one_loud_key(first - 1, n, new, path, **kw)
        assert rel(g1, w1) <= tol and rel(g0, w0) <= tol
        if first < n - 1:                                # (a query that is its chunk's first key sees itself only)
            assert float((w1[-1] - w0[-1]).abs().max()) > 0.2
            assert float((g1[-1].double().cpu() - w0[-1]).abs().max()) > 0.2


@pytest.mark.parametrize("path", ["simt", "mma", "tcgen05"])
def test_the_sink_takes_its_share_and_the_cap_holds_the_scores(path):
    """A sink as large as the largest score halves the result against no sink; a cap far below the scores
    makes the weights nearly equal."""
    dtype = "float32" if path == "simt" else "bfloat16"
    tol = 3e-6 if path == "simt" else 2e-2
    d = 64 if path == "tcgen05" else 32
    args = (dtype, path, 4, 2, d, d, 16, [1, 77], [1, 40], d ** -0.5)
    g1, w1 = attention_case(*args, sinks=True, seed=5)
    g0, w0 = attention_case(*args, sinks=False, seed=5)
    assert rel(g1, w1) <= tol and rel(g0, w0) <= tol
    assert float((w1 - w0).abs().max()) > 0.1
    # the first token of a sequence sees itself and the sink only
    assert float(w1[0].abs().max()) < float(w0[0].abs().max())
    gc, wc = attention_case(*args, cap=0.01, seed=5)
    assert rel(gc, wc) <= tol and float((wc - w0).abs().max()) > 0.1


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def mu_dirs(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("mu_a")), MU_A, 31, sharpen),
            "B": write_model(str(tmp_path_factory.mktemp("mu_b")), MU_B, 32, sharpen),
            "C": write_model(str(tmp_path_factory.mktemp("mu_c")), MU_C, 33, sharpen)}


CFG = {"A": MU_A, "B": MU_B, "C": MU_C}


def plain_rows(folder, dtype, reqs):
    cfg, w = pm.read_model_dir(folder, round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    return {r: pm.forward(cfg, w, toks).numpy() for r, toks in reqs.items()}


def compare(got, want, reqs, dtype, what):
    for r, toks in reqs.items():
        have = np.stack([got[(r, p)] for p in range(len(toks))])
        err = np.abs(have - want[r]).max(axis=1) / np.abs(want[r]).max()
        assert np.isfinite(have).all()
        assert err.max() <= TOL[dtype], (what, r, int(err.argmax()), float(err.max()))


def make_requests(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name", ["A", "B"])
def test_layers_match_the_plain_residual_after_every_run(mu_dirs, name):
    """The stream after every entry of the layer list (an entry that uses another's tensors counts as a run
    of its own) in float32."""
    from rllm_b200.engine.loading import load_model
    from rllm_b200.engine.replay import TraceSession
    cfg, w = pm.read_model_dir(mu_dirs[name])
    toks = make_requests(CFG[name]["vocab"], [75], seed=2)["r0"]
    want = []
    pm.forward(cfg, w, toks, want)
    _, model = load_model(mu_dirs[name], dtype="float32")
    sess = TraceSession(model, 128, 16, 2)
    trace, orig = [], sess.runner.build_context

    def with_trace(entries):
        ctx, a, b = orig(entries)
        ctx.extras["residual_trace"] = trace
        return ctx, a, b

    sess.runner.build_context = with_trace
    sess.step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    assert len(trace) == len(want) == len(CFG[name]["layers"])
    for i, (g, x) in enumerate(zip(trace, want)):
        assert rel(g, x) <= 1e-5, i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("A", 16), ("A", 4), ("B", 16), ("B", 8), ("C", 16)])
def test_every_way_of_cutting_gives_the_plain_logits(mu_dirs, name, page, dtype):
    """Whole prompts, token by token from the first token on, portions down to two tokens, and mixed
    batches of up to four live requests whose pages are given back and used again (the pool holds exactly
    the peak); every position's logits are compared.  The prompts pass every window, every chunk border and
    the kept first tokens; windowed and chunked groups give pages back while a request is still running."""
    V = CFG[name]["vocab"]
    reqs = make_requests(V, [61, 1, 2, 17, 150, 33, 5], seed=7)
    want = plain_rows(mu_dirs[name], dtype, reqs)
    for what, tb in (("whole", ru.trace_whole(reqs)), ("one by one", ru.trace_tail_decode(reqs, tail=1000)),
                     ("tail decoded", ru.trace_tail_decode(reqs, tail=45)),
                     ("portions", ru.trace_portions(reqs, seed=1)), ("portions b", ru.trace_portions(reqs, seed=4)),
                     ("mixed", ru.trace_mixed(reqs, seed=2, live=4, tail=6)),
                     ("mixed b", ru.trace_mixed(reqs, seed=3, live=3, tail=30))):
        got = ru.run_trace(mu_dirs[name], dtype, tb, V, page_size=page, max_live=4)
        compare(got, want, reqs, dtype, f"{name}/{dtype}/page {page}/{what}")


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("bfloat16", "B")])
def test_long_decoding_past_every_window_chunk_and_many_pages(mu_dirs, dtype, name):
    """A prompt of 3 tokens, then 260 tokens one by one (pages of 8: windows and chunks give pages back on
    the way, the kept first tokens' pages stay), beside a second request that starts later."""
    V = CFG[name]["vocab"]
    reqs = make_requests(V, [263, 120], seed=9)
    want = plain_rows(mu_dirs[name], dtype, reqs)
    tb = ru.TraceBuilder()
    a, b = reqs["r0"], reqs["r1"]
    tb.step([("r0", a[:3])])
    for i in range(3, 263):
        entries = [("r0", a[i:i + 1])]
        j = i - 60
        if j == 0:
            entries.append(("r1", b[:25]))
        elif 0 < j < 96:
            entries.append(("r1", b[24 + j:25 + j]))
        tb.step(entries, end=(["r0"] if i == 262 else []) + (["r1"] if j == 95 else []))
    got = ru.run_trace(mu_dirs[name], dtype, tb, V, page_size=8)
    compare(got, want, reqs, dtype, "long decoding")


def test_a_far_kept_token_decides_a_decoded_token(mu_dirs, tmp_path):
    """A window of 5 that keeps the first 9 tokens, sinks that take no share, peaked attention: a query far
    behind the window still reads the kept tokens at their true positions, from pages of 4 that stay while
    the pages between are given back.  Decoding goes on for many windows; the plain model without kept
    tokens differs by far more than rounding."""
    def edit(w):
        sharpen(w)
        for n, t in w.items():
            if n.endswith("mix.sink"):
                t.fill_(-20.0)
    folder = write_model(str(tmp_path / "kept"), MU_C, 35, edit)
    V = MU_C["vocab"]
    reqs = make_requests(V, [90], seed=3)
    want = plain_rows(folder, "float32", reqs)
    got = ru.run_trace(folder, "float32", ru.trace_tail_decode(reqs, tail=80), V, page_size=4)
    compare(got, want, reqs, "float32", "kept token")
    # without the kept tokens the plain model differs by far more than rounding at positions behind the window
    cfg, w = pm.read_model_dir(folder)
    for L in cfg["layers"]:
        if L["type"] == "attention_2":
            L["mixer"]["mask"]["keep_first"] = 0
    other = pm.forward(cfg, w, reqs["r0"]).numpy()
    assert np.abs(other[40:] - want["r0"][40:]).max() > 10 * TOL["float32"] * np.abs(want["r0"]).max()


def test_the_runner_as_a_program_and_pools_no_larger_than_asked(mu_dirs):
    """bin/trace_run as a child process with a pool of exactly the peak of live tokens and its four slots."""
    V = MU_B["vocab"]
    reqs = make_requests(V, [40, 70, 9, 64, 3, 20], seed=13)
    want = plain_rows(mu_dirs["B"], "float32", reqs)
    tb = ru.trace_mixed(reqs, seed=5, live=4, tail=4)
    got = ru.run_trace(mu_dirs["B"], "float32", tb, V, page_size=16, subprocess_mode=True, max_live=None)
    compare(got, want, reqs, "float32", "child process")


def plain_greedy(cfg, w, prompt, n_new):
    seq, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(pm.forward(cfg, w, seq)[-1]))
        out.append(t)
        seq.append(t)
    return out


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("float32", "C"), ("bfloat16", "B")])
def test_greedy_generation_through_the_entry_point(mu_dirs, dtype, name):
    """Nine requests through LLM.generate with the scheduler cutting prompts into portions of at most 16
    tokens beside decoding requests, CUDA graphs for the decode steps, more requests than sequences at a
    time.  float32: the plain implementation's tokens.  bfloat16: its choice at (nearly) all places where
    that is clear."""
    from rllm_b200 import LLM, SamplingParams
    V = CFG[name]["vocab"]
    rng = np.random.default_rng(17)
    prompts = [[int(t) for t in rng.integers(0, V, size=int(n))] for n in (5, 41, 1, 23, 60, 2, 9, 30, 14)]
    n_new = 12
    llm = LLM(mu_dirs[name], dtype="fp32" if dtype == "float32" else "bf16", block_size=8, num_gpu_blocks=96,
              max_num_seqs=4, max_num_batched_tokens=24, long_prefill_token_threshold=16, enable_prefix_caching=False)
    assert llm.engine.runner.capture_graphs
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    cfg, w = pm.read_model_dir(mu_dirs[name], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    clear = wrong = 0
    for p, o in zip(prompts, outs):
        got = o.outputs[0].token_ids
        assert len(got) == n_new
        if dtype == "float32":
            assert got == plain_greedy(cfg, w, p, n_new)
            continue
        seq = list(p)
        for t in got:
            row = pm.forward(cfg, w, seq)[-1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 6e-2 * float(row.abs().max()):
                clear += 1
                wrong += t != int(torch.argmax(row))
            seq.append(t)
    assert dtype == "float32" or (clear >= 20 and wrong <= 0.05 * clear), (clear, wrong)
    assert any(g.graph is not None for g in llm.engine.runner.graphs.values())
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0


@pytest.mark.parametrize("nq,nkv,d,rd,bias,kind", [(8, 2, 64, 32, True, "chunk"), (4, 4, 16, 16, True, "chunk"),
                                                    (16, 1, 128, 64, False, "window"), (6, 2, 32, 0, True, "window")])
def test_decode_with_bias_rotation_and_cache_write_in_the_attention_kernel(nq, nkv, d, rd, bias, kind):
    """The decode attention that adds the biases, rotates (cosine and sine times the rule's factor) and writes
    the token's key and value itself leaves the same bits in the cache as the kernel that prepares prompt
    portions, and returns what the attention over those pages returns."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(d + nq)
    page, lens = 16, [1, 37, 300, 129]
    S, mag = len(lens), 1.2079
    per = [-(-n // page) for n in lens]
    table = torch.full((S, max(per)), -1, dtype=torch.int32)
    perm = torch.randperm(sum(per), generator=g)
    at = 0
    for s in range(S):
        table[s, :per[s]] = perm[at:at + per[s]].to(torch.int32)
        at += per[s]
    kc = torch.randn(sum(per), nkv, page, d, generator=g).bfloat16().cuda()
    vc = torch.randn(sum(per), nkv, page, d, generator=g).bfloat16().cuda()
    gw = nq * d if kind == "chunk" else nq
    width = (nq + 2 * nkv) * d + gw
    width += (-width) % 8
    rows = torch.randn(S, width, generator=g).bfloat16().cuda()
    b = (torch.randn((nq + 2 * nkv) * d, generator=g) * 2).cuda() if bias else None
    inv_freq = (10000.0 ** (-torch.arange(rd // 2, dtype=F64) * 2 / max(rd, 1))).cuda() if rd else None
    sink = None if kind == "chunk" else torch.randn(nq, generator=g).cuda()
    opts = dict(keep_first=0 if kind == "chunk" else 3, chunk=64 if kind == "chunk" else 0,
                softcap=7.0 if kind == "chunk" else 0.0, sinks=sink, gate_per_head=kind != "chunk")
    window = 0 if kind == "chunk" else 50
    positions, tseq, err = i32([n - 1 for n in lens]), i32(list(range(S))), err_word()
    # a: prepared by the glue kernel, then attention from the pages
    qa, ka, va = rows.clone(), kc.clone(), vc.clone()
    ops.head_norm_kv_write(qa, positions, tseq, None, None, 0.0, table.cuda(), ka, va, nq, nkv, d, d, err, bias=b,
                           inv_freq=inv_freq, rotary_dim=rd, magnitude=mag)
    oa = torch.empty(S, nq * d, dtype=torch.bfloat16, device="cuda")
    ops.attention_decode_bf16(qa, width, oa, ka, va, table.cuda(), i32(lens), S, max(lens), nq, nkv, d, window, 0.2, err,
                              gate=qa[:, (nq + 2 * nkv) * d: (nq + 2 * nkv) * d + gw], **opts)
    # b: all of it in the attention kernel
    qb, kb, vb = rows.clone(), kc.clone(), vc.clone()
    ob = torch.empty_like(oa)
    ops.attention_decode_bf16(qb, width, ob, kb, vb, table.cuda(), i32(lens), S, max(lens), nq, nkv, d, window, 0.2, err,
                              inv_freq=inv_freq, rotary_dim=rd, write_kv=True, bias=b, magnitude=mag,
                              gate=qb[:, (nq + 2 * nkv) * d: (nq + 2 * nkv) * d + gw], **opts)
    assert int(err.item()) == 0
    assert torch.equal(ka, kb) and torch.equal(va, vb)
    assert not torch.equal(ka, kc) and not torch.equal(va, vc)
    assert float((oa.float() - ob.float()).abs().max()) <= 2e-2 * float(oa.float().abs().max())


def test_the_command_line_with_prefix_sharing_and_forked_samples(mu_dirs, capsys):
    """`rllm generate` on a Munupel folder in float32: greedy tokens of the plain model for two prompts of which
    the second repeats the first's 40 tokens (its pages are found again: the kept first pages and those the
    first query sees) and goes on; then two sampled continuations of one prompt, which fork from its pages."""
    import json
    from rllm_b200.cli import main
    V = MU_A["vocab"]
    rng = np.random.default_rng(23)
    first = [int(t) for t in rng.integers(0, V, size=40)]
    second = first + [int(t) for t in rng.integers(0, V, size=9)]
    ids = lambda p: ",".join(str(t) for t in p)
    common = ["--dtype", "fp32", "--num-gpu-blocks", "64", "--block-size", "8", "--max-num-seqs", "2", "--ignore-eos",
              "--json"]
    code = main(["generate", mu_dirs["A"], "--prompt-ids", ids(first), "-p", ids(first), "-p", ids(second),
                 "--max-tokens", "6", "--temperature", "0", "--enable-prefix-caching", "true"] + common)
    assert code == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().split("\n")]
    cfg, w = pm.read_model_dir(mu_dirs["A"])
    assert [l["token_ids"] for l in lines] == [plain_greedy(cfg, w, first, 6), plain_greedy(cfg, w, first, 6),
                                               plain_greedy(cfg, w, second, 6)]
    code = main(["generate", mu_dirs["A"], "--prompt-ids", ids(second), "--max-tokens", "5", "--temperature", "0.8",
                 "-n", "2", "--seed", "3"] + common)
    assert code == 0
    line = json.loads(capsys.readouterr().out.strip())
    assert [o["index"] for o in line["outputs"]] == [0, 1] and all(len(o["token_ids"]) == 5 for o in line["outputs"])
    assert all(0 <= t < V for o in line["outputs"] for t in o["token_ids"])
