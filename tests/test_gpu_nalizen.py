"""The Nalizen design in the layer-list family (post-norm blocks with layer norms that carry a bias, a token shift in front of every
mixer, a scaled and tied embedding, the per-layer token input; grouped-query attention with half-split rotation, wavelength-band
frequency scaling, per-head query / key norm after the rotation, sliding window, output gate and shared key / value caches; the
HGRN2 recurrence; gated dense feed-forwards and routed ones with a softmax over the chosen logits and squared-ReLU experts)
against the plain float64 statement in oracle/nalizen_oracle.py.  Every test mints its own small random checkpoint."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - b).max() / max(np.abs(b).max(), 1e-30))


def close_bf16(a, b):
    """bfloat16 matrices against the float64 oracle, row by row (rounding is about 1e-2 of the scale for most rows)."""
    e = np.abs(np.asarray(a, np.float64) - b).max(-1) / max(np.abs(b).max(), 1e-30)
    return float(np.median(e)) < 2e-2 and float(np.quantile(e, 0.95)) < 5e-2 and float(e.max()) < 0.25


@pytest.fixture(scope="module")
def no():
    import nalizen_oracle
    return nalizen_oracle


@pytest.fixture(scope="module")
def mk(tmp_path_factory, no):
    """mk(cfg, seed, quant, chunk, context, edit) -> (dsk.Model, weights): mints the checkpoint, loads it through Model.from_dir."""
    import dsk
    root = tmp_path_factory.mktemp("nal")
    made, n = [], [0]

    def get(cfg, seed=0, quant="fp32", chunk=8, context=512, edit=None):
        W = no.random_weights(cfg, seed)
        if edit:
            edit(W)
            W = {k: no.bf16_to_f64(no.to_bf16(v)).reshape(v.shape) for k, v in W.items()}
        n[0] += 1
        d = no.write(str(root / f"m{n[0]}"), cfg, W)
        m = dsk.Model.from_dir(d, quant=quant, chunk=chunk, context=context)
        made.append(m)
        m.dir = d
        return m, W

    yield get
    for m in made:
        m.close()


def tokens_for(cfg, n, seed=0):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], n).astype(np.int32)


def check_all_schedules(m, no, cfg, W, toks, tol=F32_TOL):
    exp, exp_layers = no.run(cfg, W, toks)
    n = len(toks)
    got, got_layers = m.forward_chunk(toks, 0, range(n), layers=True)
    assert got_layers.shape == exp_layers.shape
    assert rel(got_layers, exp_layers) < tol
    assert rel(got, exp) < tol
    k = n // 2
    rows = [m.forward_chunk(toks[:k], 0, range(k))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(k, n)]
    assert rel(np.concatenate(rows), exp) < tol
    return exp


# ---- each mechanism alone -------------------------------------------------------------------------------------------------
BARE = dict(heads=3, kv_heads=3, dim=8, vdim=8, size=None, dims=0)
BANDS = {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 40}     # with base 30 over 10 pairs: kept, blended and slowed pairs


@pytest.mark.parametrize("kind", ["bare", "rotation", "partial_rotation", "scaled_rotation", "window", "grouped", "one_key_head", "value_size",
                                  "shared_cache", "shared_cache_wider_window", "recurrence", "recurrence_sizes", "dense_ff", "routed_ff", "routed_top1",
                                  "routed_all", "no_token_input", "no_embedding_key", "no_shift", "layer_without_ff"])
def test_mechanism_alone(mk, no, kind):
    """From plain causal attention without rotation, window or feed-forward, one mechanism at a time (the oracle and the model
    read the same config.json keys, so a key left out switches the same thing off in both)."""
    a, layers, kw, edit = dict(BARE), None, {}, None
    if kind == "rotation":
        a.update(dims=8, base=100.0)
    elif kind == "partial_rotation":
        a.update(dim=10, dims=4, base=7.0)
    elif kind == "scaled_rotation":
        a.update(dim=20, dims=20, base=30.0, scaling=BANDS)
    elif kind == "window":
        a.update(size=5)
    elif kind == "grouped":
        a.update(heads=6, kv_heads=2)
    elif kind == "one_key_head":
        a.update(heads=4, kv_heads=1)
    elif kind == "value_size":
        a.update(vdim=5)
    elif kind == "shared_cache":
        layers = [no.att(**dict(a, size=6, dims=8)), no.rec(), no.att(**dict(a, size=6, dims=8, scale=0.5, kv_from=0)), no.att(**dict(a, size=3, dims=8, kv_from=0))]
    elif kind == "shared_cache_wider_window":
        layers = [no.att(**dict(a, size=3)), no.att(**dict(a, size=9, kv_from=0)), no.att(**dict(a, size=None, kv_from=0))]
    elif kind == "recurrence":
        layers = [no.rec()]
    elif kind == "recurrence_sizes":
        layers = [no.rec(heads=1, dim=3, vdim=9), no.rec(heads=5, dim=36, vdim=2), no.rec(heads=2, dim=16, vdim=40)]
    elif kind == "dense_ff":
        a.update(ff=24)
    elif kind == "routed_ff":
        a.update(ff=(6, 2, 10))
    elif kind == "routed_top1":
        a.update(ff=(4, 1, 7))
    elif kind == "routed_all":
        a.update(ff=(3, 3, 5))
    elif kind == "no_token_input":
        kw = dict(side=0)
    elif kind == "no_shift":
        def edit(W):
            W["l0.shift"][:] = 0.0
    elif kind == "layer_without_ff":
        layers = [no.rec(ff=None), no.att(**dict(a, ff=12)), no.rec(ff=(4, 2, 6)), no.att(**dict(a, ff=None))]
    cfg = no.model_config(layers or [no.att(**a)], **kw)
    if kind == "no_embedding_key":
        del cfg["embedding"]
    m, W = mk(cfg, seed=3, chunk=16, edit=edit)
    check_all_schedules(m, no, cfg, W, tokens_for(cfg, 26, 1))


def test_mechanisms_matter(no):
    """The parts are not no-ops in the oracle: the same weights with one of them removed give other logits."""
    full = no.model_config([no.att(heads=4, kv_heads=2, dim=20, dims=20, base=30.0, scaling=BANDS, size=5, ff=12), no.rec(ff=(5, 2, 8)),
                            no.att(heads=4, kv_heads=2, dim=20, dims=20, base=30.0, scaling=BANDS, size=9, kv_from=0)])
    W = no.random_weights(full, 2)
    toks = tokens_for(full, 20, 2)
    base = no.run(full, W, toks)[0]

    def without(f):
        cfg = json.loads(json.dumps(full))
        f(cfg)
        return no.run(cfg, W, toks)[0]
    assert rel(without(lambda c: c["layers"][0]["mixer"]["rot"].pop("scaling")), base) > 1e-3
    assert rel(without(lambda c: c["layers"][0]["mixer"].pop("rot")), base) > 1e-3
    assert rel(without(lambda c: c["layers"][0]["mixer"].pop("mask")), base) > 1e-3
    assert rel(without(lambda c: c["layers"][2]["mixer"]["mask"].update(size=8)), base) > 1e-4
    assert rel(without(lambda c: c["embedding"].update(scale=1.0)), base) > 1e-3
    assert rel(without(lambda c: c.pop("token_side")), base) > 1e-3
    for name, value in (("l0.shift", 0.0), ("l1.shift", 0.0), ("l0.norm1.b", 0.0), ("final.norm.b", 0.0), ("l1.mix.lower", 0.0), ("l1.mix.f.b", 0.0),
                        ("l1.mlp.router.b", 0.0), ("l0.mix.g", 0.0)):
        W2 = dict(W, **{name: np.full_like(W[name], value)})
        assert rel(no.run(full, W2, toks)[0], base) > 1e-4, name
    f = no.rot_frequencies({"dims": 20, "base": 30.0, "scaling": BANDS})
    plain = no.rot_frequencies({"dims": 20, "base": 30.0})
    ratios = [a / b for a, b in zip(f, plain)]
    assert ratios[0] == 1.0 and abs(ratios[-1] - 0.2) < 1e-12 and any(0.21 < r < 0.99 for r in ratios)      # all three bands occur


def test_router_picks_and_weights(no):
    idx, w = no.route(np.array([0.5, 2.0, 2.0, -1.0, 1.0]), 3)
    assert idx == [1, 2, 4] and abs(w.sum() - 1.0) < 1e-12 and abs(w[0] - w[1]) < 1e-15 and abs(w[2] / w[0] - np.exp(-1.0)) < 1e-12


# ---- schedules: whole prompt, token by token, portions ------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full(mk, no):
    cfg = no.small_config()
    m, W = mk(cfg, seed=11, chunk=8)
    toks = tokens_for(cfg, 70, 4)
    exp, exp_layers = no.run(cfg, W, toks)
    return cfg, m, W, toks, exp, exp_layers


def test_whole_prompt(full):
    cfg, m, W, toks, exp, exp_layers = full
    got, got_layers = m.forward_chunk(toks, 0, range(len(toks)), layers=True)   # 70 tokens = 9 internal steps of 8
    assert rel(got_layers, exp_layers) < F32_TOL
    assert rel(got, exp) < F32_TOL


def test_token_by_token_equals_prefill(full):
    cfg, m, W, toks, exp, _ = full
    rows = [m.forward(int(t), i)[0].copy() for i, t in enumerate(toks)]
    assert rel(np.array(rows), exp) < F32_TOL


@pytest.mark.parametrize("chunk", [8, 64])      # steps below 32 tokens: the decode-sized kernels; 32 and more: the matrix-product path
@pytest.mark.parametrize("sizes", [[2] * 35, [3, 2, 5, 2, 7, 1, 8, 9, 2, 16, 2, 13], [33, 2, 35], [1, 69], [32, 38]])
def test_portions(mk, no, full, chunk, sizes):
    cfg, _, W, toks, exp, _ = full
    m, _ = mk(cfg, seed=11, chunk=chunk)
    assert sum(sizes) == len(toks)
    p, rows = 0, []
    for c in sizes:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c)))
        p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_first_tokens_and_single_token_sequence(full, no):
    cfg, m, W, toks, exp, _ = full
    for n in (1, 2, 3, 4):
        assert rel(m.forward_chunk(toks[:n], 0, range(n)), exp[:n]) < F32_TOL
    one = no.run(cfg, W, [7])[0]
    assert rel(m.forward_chunk([7], 0, [0]), one) < F32_TOL
    assert rel(m.forward(7, 0)[0], one[0]) < F32_TOL


# ---- states: interleaved sequences, states given back and used again ---------------------------------------------------
def test_interleaved_sequences_and_state_reuse(full, no):
    cfg, m, W, toks, exp, _ = full
    other = tokens_for(cfg, 41, 9)
    exp_o = no.run(cfg, W, other)[0]
    sa, sb = m.new_state(), m.new_state()
    ra, rb, pa, pb = [], [], 0, 0
    for ca, cb in [(5, 2), (1, 9), (17, 3), (2, 11), (45, 16)]:
        ra.append(m.forward_chunk(toks[pa:pa + ca], pa, range(ca), state=sa)); pa += ca
        rb.append(m.forward_chunk(other[pb:pb + cb], pb, range(cb), state=sb)); pb += cb
    assert rel(np.concatenate(ra), exp) < F32_TOL
    assert rel(np.concatenate(rb), exp_o) < F32_TOL
    # give both back and run each request in the other's state: nothing of the previous owner may show (shifted inputs,
    # recurrent states, ring rows)
    m.reset(state=sa); m.reset(state=sb)
    assert rel(m.forward_chunk(other, 0, range(len(other)), state=sa), exp_o) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(len(toks)), state=sb), exp) < F32_TOL
    # position 0 starts a new sequence by itself; a shorter request after a longer one in the same state
    assert rel(m.forward_chunk(other[:9], 0, range(9), state=sb), exp_o[:9]) < F32_TOL
    rows = [m.forward_chunk(other[i:i + 1], i, [0], state=sa) for i in range(12)]       # and token by token over a used state
    assert rel(np.concatenate(rows), exp_o[:12]) < F32_TOL


# ---- sliding window: edges ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("chunk", [8, 64])
@pytest.mark.parametrize("size,reader", [(1, None), (2, None), (5, None), (16, None), (3, 9), (2, 30)])
def test_window_edge_sensitivity(mk, no, size, reader, chunk):
    """Attention layers without feed-forwards.  One layer: the logits at position i depend on the keys of positions
    i - size + 1 .. i, and a key depends on its own token and on the one before (token shift): token i - size is the earliest that
    counts.  With a second layer that reads the first one's keys and values through a wider window of `reader` positions, its
    oldest visible key is that of position i - reader + 1, so token i - reader is the earliest.  Changing the token before the
    earliest changes nothing, bit for bit; changing the earliest must.  In prompts and in decoding."""
    a = dict(heads=4, kv_heads=2, dim=8, vdim=8, dims=8, base=50.0)
    layers = [no.att(**dict(a, size=size))] + ([no.att(**dict(a, size=reader, kv_from=0))] if reader else [])
    cfg = no.model_config(layers)
    m, W = mk(cfg, seed=21, chunk=chunk)
    n, reach = 50, reader or size

    def logits_at(toks, i, decode):
        if decode:
            m.forward_chunk(toks[:max(1, i - 6)], 0, [])
            for p in range(max(1, i - 6), i):
                m.forward_chunk(toks[p:p + 1], p, [])
            return m.forward_chunk(toks[i:i + 1], i, [0])[0]
        return m.forward_chunk(toks[:i + 1], 0, [i])[0]

    base = tokens_for(cfg, n, 5)
    for i in (n - 1, n - 8):
        first_in = i - reach
        for decode in (False, True):
            ref = logits_at(base, i, decode)
            outside = base.copy()
            outside[first_in - 1] = (outside[first_in - 1] + 1) % cfg["vocab"]
            assert np.array_equal(logits_at(outside, i, decode), ref)
            inside = base.copy()
            inside[first_in] = (inside[first_in] + 1) % cfg["vocab"]
            assert np.abs(logits_at(inside, i, decode) - ref).max() > 1e-5


@pytest.mark.parametrize("chunk", [8, 64])
def test_window_edges_and_far_keys_vs_oracle(mk, no, chunk):
    """Sharp attention (score scale 6: unit-RMS queries and keys of 8 to 12 entries give scores of up to +-70) over windows of 23
    and 150 positions, a reader of the wide window's cache with a window of 61, and a recurrent layer between, so dominant keys
    fall on every offset to step, ring and window borders, far back and next to the edge.  Prompt in uneven portions, then
    decoding while the windows move over the decoded tokens."""
    cfg = no.model_config([no.att(heads=3, dim=8, size=23, scale=6.0, dims=4, base=20.0), no.rec(heads=2, dim=6, vdim=5, ff=(4, 2, 6)),
                           no.att(heads=4, kv_heads=2, dim=12, vdim=6, size=150, scale=6.0, dims=12, base=1000.0, scaling={"factor": 3.0, "low": 1.0, "high": 5.0, "original": 64}, ff=20),
                           no.att(heads=4, kv_heads=2, dim=12, vdim=6, size=61, scale=6.0, dims=12, base=1000.0, scaling={"factor": 3.0, "low": 1.0, "high": 5.0, "original": 64}, kv_from=2)])
    m, W = mk(cfg, seed=23, chunk=chunk)
    n = 330
    toks = tokens_for(cfg, n, 6)
    exp = no.run(cfg, W, toks)[0]
    p, rows = 0, []
    for c in [7, 16, 2, 31, 9, 64, 23, 40]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    while p < n:
        rows.append(m.forward_chunk(toks[p:p + 1], p, [0])); p += 1
    assert rel(np.concatenate(rows), exp) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL


FAR, ASKS = 39, 38      # the token whose key is to be found, and the token whose query looks for it


def far_key_model(no, mk, chunk, size, shared):
    """The query matrix is the key matrix behind a map that sends the embedding of token ASKS to that of token FAR (no token
    shift, no rotation, so a key is a function of its token alone): the unit-RMS query of ASKS equals the unit-RMS key of FAR
    (score 32 per head) and meets every other key, its own included, at about 0 +- 6.  `shared`: the asking layer is a second
    one that reads the first one's keys and values (whose own window is short)."""
    a = dict(heads=2, kv_heads=2, dim=32, vdim=8, scale=1.0, dims=0)
    layers = [no.att(**dict(a, size=4)), no.att(**dict(a, size=size, kv_from=0))] if shared else [no.att(**dict(a, size=size))]
    cfg = no.model_config(layers, vocab=40, side=0)

    def edit(W):
        ea, eb = W["embed"][FAR], W["embed"][ASKS]
        last = f"l{len(layers) - 1}."
        W[last + "mix.q"][:] = W["l0.mix.k"] @ (np.eye(len(ea)) + np.outer(ea - eb, eb) / (eb @ eb))
        for i in range(len(layers)):
            W[f"l{i}.shift"][:] = 0.0
        if shared:                       # the first layer adds nothing to the stream: the second one's queries see the embeddings
            W["l0.norm1"][:] = 0.0
            W["l0.norm1.b"][:] = 0.0
    return (cfg,) + mk(cfg, seed=33, chunk=chunk, edit=edit)


@pytest.mark.parametrize("shared", [False, True])
def test_far_key_dominates(mk, no, shared):
    """A single key far back, among hundreds, takes nearly all of the softmax: its token occurs once, 288 positions back at the
    far end of a window of 300.  Losing it (a wrong first row, a ring row reused too early, a ring sized for the owner's window
    instead of the reader's) moves the logits by O(1), as the oracle shows when the token is taken out."""
    toks = np.random.RandomState(1).randint(0, 38, 299).astype(np.int32)
    toks[10], toks[-1] = FAR, ASKS
    cfg, m, W = far_key_model(no, mk, 16, 300, shared)
    rows = no.run(cfg, W, toks)[0]
    lost = toks.copy()
    lost[10] = 0
    assert rel(no.run(cfg, W, lost)[0][298:], rows[298:]) > 0.05          # the far key carries the result in the oracle
    got = [m.forward_chunk(toks[:250], 0, [249])] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(250, 299)]
    assert rel(np.concatenate(got), rows[249:]) < F32_TOL      # decoded, the step size far below the window's size
    assert rel(m.forward_chunk(toks, 0, [298]), rows[298:]) < F32_TOL
    _, m2, _ = far_key_model(no, mk, 128, 300, shared)         # in a prompt, through the matrix-product path
    assert rel(m2.forward_chunk(toks, 0, [298]), rows[298:]) < F32_TOL


def test_recurrence_remembers_far_tokens(mk, no):
    """Forget gates close to 1 (lower bounds of 0.996 and more): the state still holds the first tokens after 300 steps, so a
    state that was lost, reset or rounded along the way shows.  Whole prompt, portions, and decoding from a carried state."""
    cfg = no.model_config([no.rec(heads=2, dim=6, vdim=10, ff=None), no.rec(heads=3, dim=4, vdim=4, ff=8)], side=0)

    def edit(W):
        for i in (0, 1):
            W[f"l{i}.mix.lower"][:] = 0.996 + 0.003 * np.random.RandomState(i).rand(*W[f"l{i}.mix.lower"].shape)
    m, W = mk(cfg, seed=37, chunk=32, edit=edit)
    n = 320
    toks = tokens_for(cfg, n, 2)
    exp = no.run(cfg, W, toks)[0]
    other = toks.copy()
    other[3] = (other[3] + 1) % cfg["vocab"]
    assert rel(no.run(cfg, W, other)[0][-1:], exp[-1:]) > 1e-3            # token 3 still matters at the end, in the oracle
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL
    p, rows = 0, []
    for c in [70, 2, 33, 100, 5]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    while p < n:
        rows.append(m.forward_chunk(toks[p:p + 1], p, [0])); p += 1
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_long_decoding_wraps_the_ring(mk, no):
    """Steps of 2 tokens, windows of 5 and 3 and a reader with a window of 4: the rings have 6 and 4 rows, so 160 decoded tokens
    go round them many times, while the recurrent layer's state is carried all the way."""
    cfg = no.model_config([no.att(heads=2, size=5, ff=12), no.rec(ff=(3, 1, 5)), no.att(heads=4, kv_heads=1, dim=6, vdim=16, size=3, dims=2),
                           no.att(heads=2, size=4, kv_from=0, ff=None)])
    m, W = mk(cfg, seed=29, chunk=2)
    toks = tokens_for(cfg, 160, 8)
    exp = no.run(cfg, W, toks)[0]
    rows = [m.forward_chunk(toks[:3], 0, range(3))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(3, 160)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(160)), exp) < F32_TOL


def test_context_limit_is_enforced(mk, no):
    import dsk
    cfg = no.model_config([no.att(size=None)])
    m, W = mk(cfg, seed=1, chunk=8, context=20)       # causal attention: the cache holds 20 positions and no more
    m.forward_chunk(tokens_for(cfg, 20), 0, [19])
    with pytest.raises(dsk.DskError):
        m.forward_chunk([1], 20, [0])


def test_bad_configs_are_refused(no):
    import dsk
    for layers in ([no.att(heads=4, kv_heads=3)],                                   # query heads must split evenly over the key heads
                   [no.att(), no.att(kv_from=1)],                                   # a layer cannot read its own cache
                   [no.rec(), no.att(kv_from=0)],                                   # nor that of a layer that is no attention layer
                   [no.att(), no.att(kv_from=0), no.att(kv_from=1)],                # nor that of a layer that has none of its own
                   [no.att(dim=8), no.att(dim=6, kv_from=0)],                       # key sizes must agree
                   [no.att(dim=8, dims=10)],                                        # more rotated entries than a head has
                   [no.att(ff=(3, 4, 5))]):                                         # more experts chosen than there are
        hc, sp = dsk.nalizen_from_config(no.model_config(layers), quant="fp32", max_seq_len=32)
        with pytest.raises(dsk.DskError):
            dsk.Model(hc, layers=sp)
    cfg = no.model_config([no.att()])
    cfg["layers"][0]["type"] = "unheard_of"
    with pytest.raises(dsk.DskError):
        dsk.nalizen_from_config(cfg)
    cfg = no.model_config([no.att(ff=4)])
    cfg["layers"][0]["mlp"]["kind"] = "unheard_of"
    with pytest.raises(dsk.DskError):
        dsk.nalizen_from_config(cfg)


# ---- other sizes --------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["ones", "odd", "wide", "recurrence_first", "attention_only", "recurrence_only"])
def test_other_sizes(mk, no, case):
    kw = {}
    if case == "ones":      # every count that can be 1 is 1
        layers = [no.att(heads=1, kv_heads=1, dim=2, vdim=1, size=1, dims=2, ff=1), no.rec(heads=1, dim=1, vdim=1, ff=(1, 1, 1)),
                  no.att(heads=1, kv_heads=1, dim=2, vdim=1, size=1, dims=2, kv_from=0)]
        kw = dict(width=3, vocab=3, side=1)
    elif case == "odd":     # nothing is a multiple of 4; three query heads per key head; rotation of one pair only
        layers = [no.att(heads=9, kv_heads=3, dim=7, vdim=5, size=11, dims=2, base=3.0, ff=5), no.rec(heads=3, dim=7, vdim=11, ff=(7, 3, 9)),
                  no.att(heads=9, kv_heads=3, dim=7, vdim=5, size=17, dims=2, base=3.0, kv_from=0, ff=(5, 1, 3)), no.att(heads=5, kv_heads=5, dim=6, vdim=3, size=7, dims=6)]
        kw = dict(width=42, vocab=97, side=7)
    elif case == "wide":    # larger sizes: 16 heads of 64 over 4 key heads, a window wider than the prompt, recurrent heads of 128 x 64
        layers = [no.rec(heads=4, dim=128, vdim=64, ff=(8, 2, 96)),
                  no.att(heads=16, kv_heads=4, dim=64, vdim=32, size=128, scale=0.11, dims=48, base=50000.0, scaling={"factor": 16.0, "low": 0.5, "high": 6.0, "original": 256}, ff=320),
                  no.rec(heads=2, dim=200, vdim=96, ff=None),
                  no.att(heads=16, kv_heads=4, dim=64, vdim=32, size=16, scale=0.11, dims=48, base=50000.0, scaling={"factor": 16.0, "low": 0.5, "high": 6.0, "original": 256}, kv_from=1, ff=(16, 4, 64))]
        kw = dict(width=192, vocab=300, side=24)
    elif case == "recurrence_first":
        layers = [no.rec(ff=12), no.att(ff=None), no.rec(heads=2, dim=6, vdim=2, ff=None), no.att(heads=6, kv_heads=3, vdim=8, size=9, ff=10)]
    elif case == "attention_only":
        layers = [no.att(ff=8), no.att(heads=2, kv_heads=1, vdim=12, size=4), no.att(heads=4, kv_heads=4, vdim=3, size=30, ff=8), no.att(heads=2, kv_heads=1, vdim=12, size=30, kv_from=1)]
    else:
        layers = [no.rec(ff=8), no.rec(heads=4, dim=2, vdim=3, ff=(3, 2, 4))]
    cfg = no.model_config(layers, **kw)
    m, W = mk(cfg, seed=31, chunk=16)
    toks = tokens_for(cfg, 45, 3)
    exp = check_all_schedules(m, no, cfg, W, toks)
    if case == "ones":      # a norm over one to three values turns rounding into sign flips: no bfloat16 comparison here
        return
    mb, _ = mk(cfg, seed=31, chunk=64, quant="bf16")            # the bfloat16 kernels on the same sizes, matrix-product attention
    assert close_bf16(mb.forward_chunk(toks, 0, range(45)), exp)
    rows = [mb.forward_chunk(toks[:20], 0, range(20))] + [mb.forward_chunk(toks[i:i + 1], i, [0]) for i in range(20, 45)]
    assert close_bf16(np.concatenate(rows), exp)


def test_large_steps_and_many_wanted_rows(mk, no):
    """A step above 256 tokens with every row wanted: two blocks of queries in the matrix-product attention, the second seeing
    keys of the first; the LM head runs over the wanted rows in several groups; the token shift and the recurrence run over
    several blocks of tokens."""
    cfg = no.model_config([no.att(heads=4, kv_heads=2, size=200, ff=24), no.rec(ff=(4, 2, 8)), no.att(heads=4, kv_heads=2, size=50, kv_from=0)])
    toks = tokens_for(cfg, 330, 7)
    for quant in ("fp32", "bf16"):
        m, W = mk(cfg, seed=41, chunk=512, quant=quant)
        exp = no.run(cfg, W, toks)[0]
        ok = (lambda a, b: rel(a, b) < F32_TOL) if quant == "fp32" else close_bf16
        assert ok(m.forward_chunk(toks, 0, range(330)), exp)
        assert ok(m.forward_chunk(toks[:300], 0, [0, 150, 299]), exp[[0, 150, 299]])
        assert ok(m.forward_chunk(toks[300:], 300, range(30)), exp[300:])      # a portion that continues a long step


def test_bf16_matrices(mk, no):
    cfg = no.small_config()
    m, W = mk(cfg, seed=11, quant="bf16", chunk=8)
    toks = tokens_for(cfg, 50, 4)
    exp = no.run(cfg, W, toks)[0]
    assert close_bf16(m.forward_chunk(toks, 0, range(50)), exp)
    rows = [m.forward_chunk(toks[:30], 0, range(30))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(30, 50)]
    assert close_bf16(np.concatenate(rows), exp)


# ---- generation through the framework's own entry points -------------------------------------------------------------------------
def oracle_greedy(no, cfg, W, prompt, steps):
    seq = no.Sequence(cfg, W)
    for t in prompt:
        lg = seq.feed(int(t))
    out, margins = [], []
    for _ in range(steps):
        top = np.sort(lg)[-2:]
        margins.append(top[1] - top[0])
        out.append(int(np.argmax(lg)))
        lg = seq.feed(out[-1])
    return out, min(margins)


def test_greedy_generation(full, no):
    cfg, m, W, toks, exp, _ = full
    prompt, steps = toks[:12], 24
    want, margin = oracle_greedy(no, cfg, W, prompt, steps)
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    dev, _ = m.decode_greedy(len(prompt), steps)                # device loop: a captured step, arg-max fed back without the host
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    host = []
    for i in range(steps):                                      # the samplers' loop: dsk_sample -> dsk_forward
        host.append(m.sample(temperature=0.0))
        m.forward(host[-1], len(prompt) + i)
    assert list(dev) == host
    if margin > 1e-3:                                           # no near-tie along the way: the oracle must agree token for token
        assert host == want


def test_cli_completion(full, repo):
    cfg, m, W, toks, exp, _ = full
    exe = os.path.join(repo, "deepseek.cpp_b200", "main")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-C", os.path.join(repo, "deepseek.cpp_b200"), "main"], stdout=subprocess.DEVNULL)
    prompt, steps = [int(t) for t in toks[:9]], 10
    r = subprocess.run([exe, m.dir, "-I", ",".join(map(str, prompt)), "-q", "fp32", "-n", str(steps), "-t", "0", "-T", "128"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    ids = [int(x) for x in r.stdout.split("generated ids:")[1].split()]
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    dev, _ = m.decode_greedy(len(prompt), steps)
    assert ids == prompt + list(dev)


def test_trace_runner(full, repo, tmp_path):
    """bin/trace_run end to end: two requests in turn, portions, decoded tokens, a state given back and used again."""
    cfg, m, W, toks, exp, _ = full
    out = tmp_path / "out"
    out.mkdir()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [int(t) for t in toks[:33]], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [int(t) for t in toks[33:35]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [int(toks[35])], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": [int(t) for t in toks[:8]], "want": [7, 3]}], "end": ["b"]}]
    r = subprocess.run([sys.executable, os.path.join(repo, "bin", "trace_run"), "--model", m.dir, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    V = cfg["vocab"]
    g0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    g2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    g3 = np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, V)
    assert not (out / "1.f32").exists()
    assert rel(g0, exp[[0, 32]]) < F32_TOL and rel(g2, exp[[35]]) < F32_TOL and rel(g3, exp[[7, 3]]) < F32_TOL


# ---- random designs -----------------------------------------------------------------------------------------------------------------
def random_design(seed):
    import nalizen_oracle as no
    rng = np.random.RandomState(seed)
    n = int(rng.randint(2, 7))
    layers, owners = [], []

    def ff():
        r = rng.rand()
        if r < 0.25:
            return None
        if r < 0.5:
            return int(rng.randint(1, 40))
        E = int(rng.randint(1, 9))
        return (E, int(rng.randint(1, E + 1)), int(rng.randint(1, 20)))
    for i in range(n):
        if rng.rand() < 0.55:
            size = None if rng.rand() < 0.15 else int(rng.choice([1, 3, 8, 20, 33, 70]))
            scale = float(rng.uniform(0.1, 2.0))
            if owners and rng.rand() < 0.4:
                j = int(rng.choice(owners))
                mx = layers[j]["mixer"]
                rep = int(rng.choice([1, 2, 4]))
                layers.append(no.att(heads=mx["kv_heads"] * rep, kv_heads=mx["kv_heads"], dim=mx["dim"], vdim=mx["vdim"], size=size, scale=scale,
                                     dims=(mx.get("rot") or {}).get("dims", 0), base=(mx.get("rot") or {}).get("base", 1.0),
                                     scaling=(mx.get("rot") or {}).get("scaling"), kv_from=j, ff=ff()))
                continue
            G, rep, D = int(rng.choice([1, 2, 3])), int(rng.choice([1, 2, 4])), int(rng.choice([2, 4, 6, 10, 16]))
            dims = int(rng.choice([d for d in (0, 2, 4, 6, 10, 16) if d <= D]))
            sc = None
            if dims and rng.rand() < 0.6:
                low = float(rng.choice([0.5, 1.0, 2.0]))
                sc = {"factor": float(rng.choice([2.0, 8.0, 32.0])), "low": low, "high": low + float(rng.choice([1.0, 3.0, 7.0])), "original": int(rng.choice([8, 32, 200]))}
            owners.append(i)
            layers.append(no.att(heads=G * rep, kv_heads=G, dim=D, vdim=int(rng.choice([2, 5, 8])), size=size, scale=scale, dims=dims,
                                 base=float(rng.choice([5.0, 100.0, 10000.0, 500000.0])), scaling=sc, ff=ff()))
        else:
            layers.append(no.rec(heads=int(rng.choice([1, 2, 3, 5])), dim=int(rng.choice([1, 4, 6, 10, 33])), vdim=int(rng.choice([1, 3, 8, 20])), ff=ff()))
    return no.model_config(layers, width=int(rng.choice([8, 20, 36, 50])), vocab=int(rng.randint(5, 90)), eps=float(rng.choice([1e-6, 1e-5, 1e-3])),
                           emb_scale=float(rng.choice([0.25, 1.0, 2.5])), side=int(rng.choice([0, 1, 3, 8])))


@pytest.mark.parametrize("seed", range(10))
def test_random_designs(mk, no, seed):
    """Layer count and order, every size, windows, cache sharing, rotation and its scaling, routers and the constants drawn at
    random; whole prompt, prompt + decoded tail, uneven portions (steps on both attention paths)."""
    cfg = random_design(100 + seed)
    m, W = mk(cfg, seed=seed, chunk=40)
    n = 90
    toks = tokens_for(cfg, n, seed)
    exp = no.run(cfg, W, toks)[0]
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL
    rows = [m.forward_chunk(toks[:60], 0, range(60))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(60, n)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    p, rows = 0, []
    for c in [3, 34, 2, 2, 17, 5, 27]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL
