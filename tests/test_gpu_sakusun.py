"""The Sakusun design in the layer-list family (post-norm blocks with input convolutions, gated sublayer results, single-number
RMS norms and layer scale; scaled embedding plus bigram table; grouped-query attention with value matrix, biases, score cap,
distance-bucket bias, window with kept first positions, sink and value mixing; latent attention with a query latent, a rotated
shared key part and an output gate; gated GELU feed-forward) against the plain float64 statement in oracle/sakusun_oracle.py.
Every test mints its own small random checkpoint."""
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
def so():
    import sakusun_oracle
    return sakusun_oracle


@pytest.fixture(scope="module")
def mk(tmp_path_factory, so):
    """mk(cfg, seed, quant, chunk, context, edit) -> (dsk.Model, weights): mints the checkpoint, loads it through Model.from_dir."""
    import dsk
    root = tmp_path_factory.mktemp("sak")
    made, n = [], [0]

    def get(cfg, seed=0, quant="fp32", chunk=8, context=512, edit=None):
        W = so.random_weights(cfg, seed)
        if edit:
            edit(W)
            W = {k: so.bf16_to_f64(so.to_bf16(v)).reshape(v.shape) for k, v in W.items()}
        n[0] += 1
        d = so.write(str(root / f"m{n[0]}"), cfg, W)
        m = dsk.Model.from_dir(d, quant=quant, chunk=chunk, context=context)
        made.append(m)
        m.dir = d
        return m, W

    yield get
    for m in made:
        m.close()


def tokens_for(cfg, n, seed=0):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], n).astype(np.int32)


def peaky(W):
    for k in W:
        if k.endswith("mix.q.norm") or k.endswith("mix.dq.norm"):
            W[k] *= 6.0          # scores x 6: a few keys take nearly all the weight, so a wrong edge or a lost key moves the output by O(1)


def check_all_schedules(m, so, cfg, W, toks, tol=F32_TOL, layers=True):
    exp, exp_layers = so.run(cfg, W, toks)
    n = len(toks)
    if layers:
        got, got_layers = m.forward_chunk(toks, 0, range(n), layers=True)
        assert got_layers.shape == exp_layers.shape
        assert rel(got_layers, exp_layers) < tol
    else:
        got = m.forward_chunk(toks, 0, range(n))
    assert rel(got, exp) < tol
    k = n // 2
    rows = [m.forward_chunk(toks[:k], 0, range(k))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(k, n)]
    assert rel(np.concatenate(rows), exp) < tol
    return exp


# ---- each mechanism alone -------------------------------------------------------------------------------------------------
BARE = dict(heads=3, kv_heads=3, dim=8, vdim=8, size=None, softcap=None, bias_max=None, v_mix=False)


@pytest.mark.parametrize("kind", ["bare", "cap", "distance_bias", "distance_bias_odd", "window", "kept_first", "kept_beyond_window", "grouped", "one_key_head",
                                  "value_size", "value_mixing", "ff", "taps1", "taps2", "taps5", "no_bigram_collisions", "latent", "latent_partial_rotation",
                                  "latent_no_plain_rotation", "latent_ff"])
def test_mechanism_alone(mk, so, kind):
    """From plain causal attention without cap, bias, window or mixing, one mechanism at a time (the oracle and the model read the
    same config.json keys, so a key left out switches the same thing off in both)."""
    a, taps, layers, kw = dict(BARE), 3, None, {}
    if kind == "cap":
        a.update(softcap=0.7)                       # well inside the scores' range, so the tanh bends them
    elif kind == "distance_bias":
        a.update(bias_max=12, rel_rows=8)           # 4 exact buckets, 4 logarithmic ones, distances beyond 12 in the last
    elif kind == "distance_bias_odd":
        a.update(bias_max=30, rel_rows=7)
    elif kind == "window":
        a.update(size=5, keep_first=0)
    elif kind == "kept_first":
        a.update(size=5, keep_first=3)
    elif kind == "kept_beyond_window":
        a.update(size=2, keep_first=9)              # more kept positions than the window is wide
    elif kind == "grouped":
        a.update(heads=6, kv_heads=2)
    elif kind == "one_key_head":
        a.update(heads=4, kv_heads=1)
    elif kind == "value_size":
        a.update(vdim=5)
    elif kind == "value_mixing":
        layers = [so.att(**dict(BARE, v_mix=False)), so.att(**dict(BARE, v_mix=True)), so.lat(), so.att(**dict(BARE, v_mix=True, heads=6, kv_heads=3, vdim=8)),
                  so.att(**dict(BARE, v_mix=False)), so.att(**dict(BARE, v_mix=True, heads=2, kv_heads=1, vdim=24))]
    elif kind == "ff":
        a.update(ff=24)
    elif kind.startswith("taps"):
        taps = int(kind[4:])
        a.update(ff=12)
    elif kind == "no_bigram_collisions":
        kw = dict(buckets=4000, mul_prev=61, mul_cur=1)
    elif kind == "latent":
        layers = [so.lat()]
    elif kind == "latent_partial_rotation":
        layers = [so.lat(rot_dim=8, dims=4, base=7.0)]
    elif kind == "latent_no_plain_rotation":
        layers = [so.lat(rot_dim=6, dims=0)]
    elif kind == "latent_ff":
        layers = [so.lat(ff=20), so.lat(heads=2, dim=4, rot_dim=10, vdim=6, kv_rank=9, q_rank=30, ff=None)]
    cfg = so.model_config(layers or [so.att(**a)], taps=taps, **kw)
    m, W = mk(cfg, seed=3, chunk=16)
    check_all_schedules(m, so, cfg, W, tokens_for(cfg, 26, 1))


def test_mechanisms_matter(so):
    """The switches are not no-ops in the oracle: the same weights with one mechanism removed give other logits."""
    full = so.model_config([so.att(size=5, keep_first=2, softcap=0.7, bias_max=12, rel_rows=8, ff=12), so.att(size=4, keep_first=0, ff=None)])
    W = so.random_weights(full, 2)
    toks = tokens_for(full, 20, 2)
    base = so.run(full, W, toks)[0]

    def without(f):
        cfg = json.loads(json.dumps(full))
        f(cfg)
        return so.run(cfg, W, toks)[0]
    assert rel(without(lambda c: c["layers"][0]["mixer"].pop("softcap")), base) > 1e-3
    assert rel(without(lambda c: c["layers"][0]["mixer"].pop("bias_max")), base) > 1e-3
    assert rel(without(lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=0)), base) > 1e-3
    assert rel(without(lambda c: c["layers"][1]["mixer"].update(v_mix=False)), base) > 1e-3
    assert rel(without(lambda c: c["embedding"].update(scale=1.0)), base) > 1e-3
    W2 = dict(W, **{"l0.mix.sink": W["l0.mix.sink"] - 30.0})
    assert rel(so.run(full, W2, toks)[0], base) > 1e-3
    W3 = dict(W, **{"bigram": np.zeros_like(W["bigram"])})
    assert rel(so.run(full, W3, toks)[0], base) > 1e-3
    assert [so.rel_bucket(n, 8, 12) for n in (0, 3, 4, 5, 6, 8, 11, 12, 500)] == [0, 3, 4, 4, 5, 6, 7, 7, 7]


# ---- schedules: whole prompt, token by token, portions ------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full(mk, so):
    cfg = so.small_config()
    m, W = mk(cfg, seed=11, chunk=8)
    toks = tokens_for(cfg, 70, 4)
    exp, exp_layers = so.run(cfg, W, toks)
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
def test_portions(mk, so, full, chunk, sizes):
    cfg, _, W, toks, exp, _ = full
    m, _ = mk(cfg, seed=11, chunk=chunk)
    assert sum(sizes) == len(toks)
    p, rows = 0, []
    for c in sizes:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c)))
        p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_first_tokens_and_single_token_sequence(full, so):
    cfg, m, W, toks, exp, _ = full
    for n in (1, 2, 3, 4):
        assert rel(m.forward_chunk(toks[:n], 0, range(n)), exp[:n]) < F32_TOL
    one = so.run(cfg, W, [7])[0]
    assert rel(m.forward_chunk([7], 0, [0]), one) < F32_TOL
    assert rel(m.forward(7, 0)[0], one[0]) < F32_TOL


# ---- states: interleaved sequences, states given back and used again ---------------------------------------------------
def test_interleaved_sequences_and_state_reuse(full, so):
    cfg, m, W, toks, exp, _ = full
    other = tokens_for(cfg, 41, 9)
    exp_o = so.run(cfg, W, other)[0]
    sa, sb = m.new_state(), m.new_state()
    ra, rb, pa, pb = [], [], 0, 0
    for ca, cb in [(5, 2), (1, 9), (17, 3), (2, 11), (45, 16)]:
        ra.append(m.forward_chunk(toks[pa:pa + ca], pa, range(ca), state=sa)); pa += ca
        rb.append(m.forward_chunk(other[pb:pb + cb], pb, range(cb), state=sb)); pb += cb
    assert rel(np.concatenate(ra), exp) < F32_TOL
    assert rel(np.concatenate(rb), exp_o) < F32_TOL
    # give both back and run each request in the other's state: nothing of the previous owner may show (previous token,
    # convolution inputs, kept first rows, ring rows)
    m.reset(state=sa); m.reset(state=sb)
    assert rel(m.forward_chunk(other, 0, range(len(other)), state=sa), exp_o) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(len(toks)), state=sb), exp) < F32_TOL
    # position 0 starts a new sequence by itself; a shorter request after a longer one in the same state
    assert rel(m.forward_chunk(other[:9], 0, range(9), state=sb), exp_o[:9]) < F32_TOL
    rows = [m.forward_chunk(other[i:i + 1], i, [0], state=sa) for i in range(12)]       # and token by token over a used state
    assert rel(np.concatenate(rows), exp_o[:12]) < F32_TOL


# ---- window with kept first positions: edges -------------------------------------------------------------------------------------
@pytest.mark.parametrize("chunk", [8, 64])
@pytest.mark.parametrize("size,keep", [(1, 0), (2, 1), (5, 3), (16, 2)])
def test_window_edge_sensitivity(mk, so, size, keep, chunk):
    """One attention layer without a feed-forward: the logits at position i depend on the keys of positions i - size + 1 .. i and
    of the kept first positions; a key depends on its own token, on the taps - 1 tokens before (input convolution) and on one
    more (bigram row).  Changing the last token that reaches no visible key changes nothing, bit for bit; changing the first one
    that does must; likewise the last kept position against the one after it.  In prompts and in decoding."""
    taps = 3
    cfg = so.model_config([so.att(heads=4, kv_heads=2, size=size, keep_first=keep, bias_max=None, ff=None)], taps=taps, buckets=4000, mul_prev=61, mul_cur=1)
    m, W = mk(cfg, seed=21, chunk=chunk)
    n = 44

    def logits_at(toks, i, decode):
        if decode:
            m.forward_chunk(toks[:max(1, i - 6)], 0, [])
            for p in range(max(1, i - 6), i):
                m.forward_chunk(toks[p:p + 1], p, [])
            return m.forward_chunk(toks[i:i + 1], i, [0])[0]
        return m.forward_chunk(toks[:i + 1], 0, [i])[0]

    base = tokens_for(cfg, n, 5)
    for i in (n - 1, n - 8):
        first_in = i - size + 1 - (taps - 1) - 1          # the earliest token that reaches the oldest key of the window
        for decode in (False, True):
            ref = logits_at(base, i, decode)
            outside = base.copy()
            outside[first_in - 1] = (outside[first_in - 1] + 1) % cfg["vocab"]
            assert np.array_equal(logits_at(outside, i, decode), ref)
            inside = base.copy()
            inside[first_in] = (inside[first_in] + 1) % cfg["vocab"]
            assert np.abs(logits_at(inside, i, decode) - ref).max() > 1e-4
            if keep:
                kept = base.copy()
                kept[keep - 1] = (kept[keep - 1] + 1) % cfg["vocab"]
                assert np.abs(logits_at(kept, i, decode) - ref).max() > 1e-4
                after = base.copy()
                after[keep] = (after[keep] + 1) % cfg["vocab"]           # reaches the keys of positions keep .. keep + taps: none is visible
                assert np.array_equal(logits_at(after, i, decode), ref)


@pytest.mark.parametrize("chunk", [8, 64])
def test_window_edges_and_far_keys_vs_oracle(mk, so, chunk):
    """Peaky attention (scores x 6) over windows of 23 and 150 positions with kept first positions and a causal latent layer, so
    dominant keys fall on every offset to step, ring and window borders, far back and next to the edge.  Prompt in uneven
    portions, then decoding while both windows move over the decoded tokens."""
    cfg = so.model_config([so.att(heads=3, size=23, keep_first=4, bias_max=40, rel_rows=12), so.lat(heads=2, kv_rank=10, q_rank=7),
                           so.att(heads=4, kv_heads=2, dim=6, vdim=12, size=150, keep_first=1, scale=0.4, bias_max=100, rel_rows=20, ff=20)])
    m, W = mk(cfg, seed=23, chunk=chunk, edit=peaky)
    n = 330
    toks = tokens_for(cfg, n, 6)
    exp = so.run(cfg, W, toks)[0]
    p, rows = 0, []
    for c in [7, 16, 2, 31, 9, 64, 23, 40]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    while p < n:
        rows.append(m.forward_chunk(toks[p:p + 1], p, [0])); p += 1
    assert rel(np.concatenate(rows), exp) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL


FAR, ASKS = 39, 38      # the token whose key is to be found, and the token whose query looks for it


def far_key_model(so, mk, chunk, size, keep):
    """The query matrix is the key matrix behind a map that sends the embedding of token ASKS to that of token FAR (no biases,
    unit norm weights, no cap, no bias table, sinks far below; input convolution and bigram rows zeroed, so a key is a function
    of its token alone): the query of ASKS equals the key of FAR (32 per head after the norm) and meets every other key,
    its own included, at about 0 +- 6."""
    cfg = so.model_config([so.att(heads=2, dim=32, vdim=8, size=size, keep_first=keep, scale=1.0, softcap=None, bias_max=None, v_mix=False)], vocab=40,
                          buckets=50)

    def edit(W):
        ea, eb = W["embed"][FAR], W["embed"][ASKS]
        W["l0.mix.q"][:] = W["l0.mix.k"] @ (np.eye(len(ea)) + np.outer(ea - eb, eb) / (eb @ eb))
        for k in ("l0.mix.q.b", "l0.mix.k.b", "l0.canon1", "bigram"):
            W[k][:] = 0.0
        W["l0.mix.k.norm"][:] = 1.0
        W["l0.mix.q.norm"][:] = 1.0
        W["l0.mix.sink"][:] = -20.0
    return (cfg,) + mk(cfg, seed=33, chunk=chunk, edit=edit)


@pytest.mark.parametrize("case", ["window", "kept"])
def test_far_key_dominates(mk, so, case):
    """A single key far back, among hundreds, takes nearly all of the softmax: its token occurs once, either 288 positions back at
    the far end of a window of 300, or at a kept first position far outside a window of 50.  Losing it (a wrong first row, a
    ring row reused too early, kept rows overwritten) moves the logits by O(1), as the oracle shows when the token is taken out."""
    size, keep, at = (300, 0, 10) if case == "window" else (50, 3, 2)
    toks = np.random.RandomState(1).randint(0, 38, 299).astype(np.int32)
    toks[at], toks[-1] = FAR, ASKS
    cfg, m, W = far_key_model(so, mk, 16, size, keep)
    rows = so.run(cfg, W, toks)[0]
    lost = toks.copy()
    lost[at] = 0
    assert rel(so.run(cfg, W, lost)[0][298:], rows[298:]) > 0.05          # the far key carries the result in the oracle
    got = [m.forward_chunk(toks[:250], 0, [249])] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(250, 299)]
    assert rel(np.concatenate(got), rows[249:]) < F32_TOL      # decoded, the step size far below the window's size
    assert rel(m.forward_chunk(toks, 0, [298]), rows[298:]) < F32_TOL
    _, m2, _ = far_key_model(so, mk, 128, size, keep)          # in a prompt, through the matrix-product path
    assert rel(m2.forward_chunk(toks, 0, [298]), rows[298:]) < F32_TOL


def test_long_decoding_wraps_the_ring(mk, so):
    """Steps of 2 tokens, windows of 5 and 3 with kept first positions: the rings have 6 and 4 rows behind the kept ones, so 160
    decoded tokens go round them many times, while the latent layer's cache grows."""
    cfg = so.model_config([so.att(heads=2, size=5, keep_first=2, ff=12), so.lat(heads=2, ff=None), so.att(heads=4, kv_heads=1, dim=6, vdim=16, size=3, keep_first=4)])
    m, W = mk(cfg, seed=29, chunk=2)
    toks = tokens_for(cfg, 160, 8)
    exp = so.run(cfg, W, toks)[0]
    rows = [m.forward_chunk(toks[:3], 0, range(3))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(3, 160)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(160)), exp) < F32_TOL


def test_context_limit_is_enforced(mk, so):
    import dsk
    cfg = so.model_config([so.lat()])
    m, W = mk(cfg, seed=1, chunk=8, context=20)       # causal attention: the cache holds 20 positions and no more
    m.forward_chunk(tokens_for(cfg, 20), 0, [19])
    with pytest.raises(dsk.DskError):
        m.forward_chunk([1], 20, [0])


def test_bad_configs_are_refused(so):
    import dsk
    cfg = so.public_config(so.model_config([so.att(heads=4, kv_heads=3)]))  # query heads must split evenly over the key heads
    hc, sp = dsk.sakusun_from_config(cfg, quant="fp32", max_seq_len=32)
    with pytest.raises(dsk.DskError):
        dsk.Model(hc, layers=sp)
    cfg = so.public_config(so.model_config([so.att(vdim=8), so.att(vdim=6)]))   # mixed values must have one size
    hc, sp = dsk.sakusun_from_config(cfg, quant="fp32", max_seq_len=32)
    with pytest.raises(dsk.DskError):
        dsk.Model(hc, layers=sp)
    cfg = so.public_config(so.model_config([so.lat(rot_dim=4, dims=6)]))        # more rotated entries than the rotated part has
    hc, sp = dsk.sakusun_from_config(cfg, quant="fp32", max_seq_len=32)
    with pytest.raises(dsk.DskError):
        dsk.Model(hc, layers=sp)
    cfg = so.public_config(so.model_config([so.att()]))
    cfg["layers"][0]["type"] = "unheard_of"
    with pytest.raises(dsk.DskError):
        dsk.sakusun_from_config(cfg)


# ---- other sizes --------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["ones", "odd", "wide", "latent_first", "attention_only", "latent_only"])
def test_other_sizes(mk, so, case):
    kw = {}
    if case == "ones":      # every count that can be 1 is 1
        layers = [so.att(heads=1, kv_heads=1, dim=1, vdim=1, size=1, keep_first=1, bias_max=3, rel_rows=2, ff=1),
                  so.lat(heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=1, q_rank=1, ff=1)]
        kw = dict(width=3, vocab=3, taps=1, buckets=1, mul_prev=1, mul_cur=1)
    elif case == "odd":     # nothing is a multiple of 4; three query heads per key head; rotation of one pair only
        layers = [so.att(heads=9, kv_heads=3, dim=7, vdim=5, size=11, keep_first=5, bias_max=17, rel_rows=9, ff=5), so.lat(heads=5, dim=3, rot_dim=6, dims=2, vdim=7, kv_rank=11, q_rank=13),
                  so.att(heads=5, kv_heads=5, dim=3, vdim=3, size=7, keep_first=0, bias_max=200, rel_rows=31, ff=None)]
        kw = dict(width=42, vocab=97, taps=2, buckets=101, mul_prev=97, mul_cur=89)
    elif case == "wide":    # larger sizes: 16 heads of 64 over 4 key heads, a window wider than the prompt, a latent of 192 + 64
        layers = [so.lat(heads=8, dim=64, rot_dim=64, vdim=64, kv_rank=192, q_rank=160, scale=0.09, base=10000.0, ff=320),
                  so.att(heads=16, kv_heads=4, dim=64, vdim=32, size=128, keep_first=8, scale=0.125, softcap=30.0, bias_max=128, rel_rows=32, ff=320),
                  so.att(heads=8, kv_heads=8, dim=32, vdim=16, size=16, keep_first=4, scale=0.2, bias_max=64, rel_rows=16, ff=96)]
        kw = dict(width=192, vocab=300, taps=4, buckets=509, mul_prev=1000003, mul_cur=7919)
    elif case == "latent_first":
        layers = [so.lat(ff=12), so.att(ff=None), so.lat(heads=2, dim=6, rot_dim=2, ff=None), so.att(heads=6, kv_heads=3, vdim=8, size=9, ff=10)]
    elif case == "attention_only":
        layers = [so.att(v_mix=False, ff=8), so.att(heads=2, kv_heads=1, vdim=12, size=4, keep_first=0), so.att(heads=4, kv_heads=4, vdim=3, size=30, keep_first=30, ff=8)]
    else:
        layers = [so.lat(ff=8), so.lat(heads=4, dim=2, rot_dim=12, dims=8, vdim=3, kv_rank=5, q_rank=4, base=3.0, ff=None)]
    cfg = so.model_config(layers, **kw)
    m, W = mk(cfg, seed=31, chunk=16)
    toks = tokens_for(cfg, 45, 3)
    exp = check_all_schedules(m, so, cfg, W, toks)
    if case == "ones":      # a norm over one to three values turns rounding into sign flips: no bfloat16 comparison here
        return
    mb, _ = mk(cfg, seed=31, chunk=64, quant="bf16")            # the bfloat16 kernels on the same sizes, matrix-product attention
    assert close_bf16(mb.forward_chunk(toks, 0, range(45)), exp)
    rows = [mb.forward_chunk(toks[:20], 0, range(20))] + [mb.forward_chunk(toks[i:i + 1], i, [0]) for i in range(20, 45)]
    assert close_bf16(np.concatenate(rows), exp)


def test_large_steps_and_many_wanted_rows(mk, so):
    """A step above 256 tokens with every row wanted: two blocks of queries in the matrix-product attention, the second seeing
    keys of the first (and the kept first positions beyond its window); the LM head runs over the wanted rows in several
    groups; the input convolution runs over several blocks of tokens."""
    cfg = so.model_config([so.att(heads=4, kv_heads=2, size=200, keep_first=3, bias_max=300, rel_rows=24, ff=24), so.lat(heads=2), so.att(heads=4, kv_heads=4, vdim=4, size=50, keep_first=5)], taps=4)
    toks = tokens_for(cfg, 330, 7)
    for quant in ("fp32", "bf16"):
        m, W = mk(cfg, seed=41, chunk=512, quant=quant)
        exp = so.run(cfg, W, toks)[0]
        ok = (lambda a, b: rel(a, b) < F32_TOL) if quant == "fp32" else close_bf16
        assert ok(m.forward_chunk(toks, 0, range(330)), exp)
        assert ok(m.forward_chunk(toks[:300], 0, [0, 150, 299]), exp[[0, 150, 299]])
        assert ok(m.forward_chunk(toks[300:], 300, range(30)), exp[300:])      # a portion that continues a long step


def test_bf16_matrices(mk, so):
    cfg = so.small_config()
    m, W = mk(cfg, seed=11, quant="bf16", chunk=8)
    toks = tokens_for(cfg, 50, 4)
    exp = so.run(cfg, W, toks)[0]
    assert close_bf16(m.forward_chunk(toks, 0, range(50)), exp)
    rows = [m.forward_chunk(toks[:30], 0, range(30))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(30, 50)]
    assert close_bf16(np.concatenate(rows), exp)


# ---- generation through the framework's own entry points -------------------------------------------------------------------------
def oracle_greedy(so, cfg, W, prompt, steps):
    seq = so.Sequence(cfg, W)
    for t in prompt:
        lg = seq.feed(int(t))
    out, margins = [], []
    for _ in range(steps):
        top = np.sort(lg)[-2:]
        margins.append(top[1] - top[0])
        out.append(int(np.argmax(lg)))
        lg = seq.feed(out[-1])
    return out, min(margins)


def test_greedy_generation(full, so):
    cfg, m, W, toks, exp, _ = full
    prompt, steps = toks[:12], 24
    want, margin = oracle_greedy(so, cfg, W, prompt, steps)
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
    import sakusun_oracle as so
    rng = np.random.RandomState(seed)
    n = int(rng.randint(1, 6))
    gv = int(rng.choice([4, 6, 12]))          # value entries per token of the layers that mix values
    layers = []
    for _ in range(n):
        ff = int(rng.randint(1, 40)) if rng.rand() < 0.7 else None
        if rng.rand() < 0.5:
            G = int(rng.choice([1, 2, 3]))
            rep = int(rng.choice([1, 2, 4]))
            mix = bool(rng.rand() < 0.6)
            vd = gv // G if mix and gv % G == 0 else int(rng.choice([2, 5, 8]))
            mix = mix and gv % G == 0
            rows = int(rng.choice([2, 5, 8, 16]))
            layers.append(so.att(heads=G * rep, kv_heads=G, dim=int(rng.choice([2, 4, 6, 10, 16])), vdim=vd,
                                 size=None if rng.rand() < 0.15 else int(rng.choice([1, 3, 8, 20, 33, 70])), keep_first=int(rng.choice([0, 1, 4, 40])),
                                 scale=float(rng.uniform(0.1, 0.6)), softcap=None if rng.rand() < 0.3 else float(rng.choice([0.5, 5.0, 50.0])),
                                 bias_max=None if rng.rand() < 0.3 else rows // 2 + int(rng.choice([1, 7, 60])), rel_rows=rows, v_mix=mix, ff=ff))
        else:
            rd = int(rng.choice([2, 4, 6, 10]))
            layers.append(so.lat(heads=int(rng.choice([1, 2, 3, 5])), dim=int(rng.choice([1, 4, 6, 10])), rot_dim=rd, dims=int(rng.choice([d for d in (0, 2, 4, 6, 10) if d <= rd])),
                                 vdim=int(rng.choice([2, 5, 8])), kv_rank=int(rng.choice([3, 8, 17])), q_rank=int(rng.choice([2, 9, 20])),
                                 scale=float(rng.uniform(0.1, 0.6)), base=float(rng.choice([10.0, 1000.0, 50000.0])), ff=ff))
    return so.model_config(layers, width=int(rng.choice([8, 20, 36, 50])), vocab=int(rng.randint(5, 90)), taps=int(rng.choice([1, 2, 3, 4, 6])),
                           eps=float(rng.choice([1e-6, 1e-5, 1e-3])), emb_scale=float(rng.choice([0.25, 1.0, 3.0])), buckets=int(rng.choice([1, 7, 64, 1013])),
                           mul_prev=int(rng.randint(1, 100)), mul_cur=int(rng.randint(1, 100)))


@pytest.mark.parametrize("seed", range(10))
def test_random_designs(mk, so, seed):
    """Layer count and order, every size, windows, kept positions, caps, bias tables, mixing, rotation, taps and the embedding's
    constants drawn at random; whole prompt, prompt + decoded tail, uneven portions (steps on both attention paths)."""
    cfg = random_design(100 + seed)
    m, W = mk(cfg, seed=seed, chunk=40)
    n = 90
    toks = tokens_for(cfg, n, seed)
    exp = so.run(cfg, W, toks)[0]
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL
    rows = [m.forward_chunk(toks[:60], 0, range(60))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(60, n)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    p, rows = 0, []
    for c in [3, 34, 2, 2, 17, 5, 27]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL
