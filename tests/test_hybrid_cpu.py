"""CPU-side checks of the layer-list model family: config.json -> C-ABI description, the checkpoint reader, and the float64
oracle's own invariants (what a sequence carries is enough to continue it; a window hides what lies outside it)."""
import ctypes

import numpy as np
import pytest


@pytest.fixture(scope="module")
def ho():
    import hybrid_oracle
    return hybrid_oracle


def test_config_to_layer_specs(ho):
    import dsk
    cfg = ho.small_config()
    hc, specs = dsk.ARCHITECTURES[cfg["architecture"]](cfg, quant="fp32", max_seq_len=99, chunk=8)
    assert (hc.dim, hc.vocab_size, hc.n_layers, hc.max_seq_len, hc.chunk, hc.norm_groups, hc.side_dim) == (48, 61, 5, 99, 8, 3, 6)
    assert hc.quant == dsk.QUANT_IDS["fp32"] and abs(hc.residual_mult - 0.7) < 1e-7 and abs(hc.logit_scale - 1.5) < 1e-7
    a, s, b = specs[0], specs[1], specs[2]
    assert (a.mixer, a.att_heads, a.att_dim, a.att_vdim, a.att_kv_rank, a.att_window, a.att_kv_from) == (dsk.MIX_LATENT_SWA, 3, 12, 20, 40, 7, -1)
    assert (a.ff_kind, a.ff_experts, a.ff_top, a.ff_hidden) == (dsk.FF_MOE, 5, 2, 24) and abs(a.ff_limit - 1.5) < 1e-7
    assert (s.mixer, s.ssm_heads, s.ssm_vdim, s.ssm_state, s.ssm_groups, s.ssm_conv, s.ssm_norm_groups, s.ff_kind) == (dsk.MIX_SSD, 6, 10, 12, 3, 3, 2, dsk.FF_NONE)
    assert b.att_kv_from == 0 and specs[3].mixer == dsk.MIX_SSD        # a second type name of the same mechanism
    del cfg["token_side"]
    assert dsk.hybrid_from_config(cfg)[0].side_dim == 0
    cfg["layers"][0]["type"] = "unheard_of"
    with pytest.raises(dsk.DskError):
        dsk.hybrid_from_config(cfg)


def test_spec_structs_match_the_header(repo):
    """The ctypes mirrors must have the C structs' sizes (field order is checked by the GPU tests' results)."""
    import os
    import subprocess
    import tempfile

    import dsk
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "t.c")
        open(src, "w").write('#include "dsk.h"\n#include <stdio.h>\nint main(void){printf("%zu %zu\\n", sizeof(dsk_layer_spec), sizeof(dsk_hybrid_config));return 0;}')
        exe = os.path.join(td, "t")
        subprocess.check_call(["gcc", "-std=c99", "-I", os.path.join(repo, "include"), src, "-o", exe])
        a, b = map(int, subprocess.check_output([exe]).split())
    assert (a, b) == (ctypes.sizeof(dsk.LayerSpec), ctypes.sizeof(dsk.HybridConfig))


def test_checkpoint_roundtrip(ho, tmp_path):
    import dseek
    cfg = ho.small_config()
    W = ho.random_weights(cfg, 2)
    d = ho.write_checkpoint(str(tmp_path / "m"), cfg, W)
    cfg2, ts = dseek.read_config_dir(d)
    assert cfg2 == cfg and set(ts) == set(W)
    for k, t in ts.items():
        assert t.dtype == "BF16" and tuple(t.shape) == W[k].shape
        assert np.array_equal(ho.bf16_to_f64(np.asarray(t.data)).reshape(W[k].shape), W[k])


def test_oracle_window_and_carry(ho):
    """Oracle invariants: (1) with one attention layer a token outside the window cannot change the logits, one inside does;
    (2) the state-space carry continues a sequence: feeding a prefix to two Sequence objects and the same suffix gives equal logits."""
    win = 4
    cfg = {"architecture": "Desarax", "vocab": 23, "width": 16, "norm": {"eps": 1e-5, "groups": 1}, "residual_mult": 1.0, "logit_scale": 1.0,
           "layers": [{"type": "latent_attention", "mlp": None, "mixer": {"heads": 2, "dim": 4, "vdim": 4, "kv_rank": 6, "mask": {"size": win}, "scale": 1.0}}]}
    W = ho.random_weights(cfg, 4)
    toks = np.arange(12) % 23
    base = ho.run(cfg, W, toks)[0][-1]
    out, ins = toks.copy(), toks.copy()
    out[11 - win] += 1
    ins[11 - win + 1] += 1
    assert np.array_equal(ho.run(cfg, W, out)[0][-1], base)
    assert np.abs(ho.run(cfg, W, ins)[0][-1] - base).max() > 1e-6
    cfg2 = ho.small_config()
    W2 = ho.random_weights(cfg2, 5)
    full = ho.run(cfg2, W2, np.arange(20) % 61)[0]
    seq = ho.Sequence(cfg2, W2)
    rows = [seq.feed(int(t)) for t in np.arange(20) % 61]
    assert np.allclose(np.array(rows), full, rtol=0, atol=1e-12)


# ---- the Rutulix design ---------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def ro():
    import rutulix_oracle
    return rutulix_oracle


def test_rutulix_config_to_layer_specs(ro):
    import dsk
    cfg = ro.small_config()
    hc, specs = dsk.ARCHITECTURES[cfg["architecture"]](cfg, quant="bf16", max_seq_len=77, chunk=16)
    assert (hc.dim, hc.vocab_size, hc.n_layers, hc.max_seq_len, hc.chunk, hc.side_dim) == (44, 61, 4, 77, 16, 0)
    assert (hc.block, hc.norm_kind, hc.tie_head) == (dsk.BLOCK_SANDWICH, dsk.NORM_LAYER, 0)
    assert (hc.loop_start, hc.loop_stop, hc.loop_times) == (1, 3, 3) and hc.quant == dsk.QUANT_IDS["bf16"]
    a, b, c = specs[0], specs[1], specs[2]
    assert (a.mixer, a.att_heads, a.att_kv_heads, a.att_dim, a.att_vdim, a.att_mask, a.att_window, a.att_talk) == (dsk.MIX_GQA, 6, 2, 10, 10, dsk.MASK_CHUNK, 7, 1)
    assert (a.rot_dims, a.rot_original) == (6, 64) and abs(a.rot_base - 500.0) < 1e-3 and (a.rot_factor, a.rot_fast, a.rot_slow) == (4.0, 8.0, 1.0)
    assert (a.ff_kind, a.ff_hidden, a.ff_act) == (dsk.FF_DENSE, 28, dsk.ACT_XIELU) and abs(a.att_scale - 0.3) < 1e-7
    assert b.ff_kind == dsk.FF_NONE and b.rot_factor == 0.0 and b.rot_dims == 12       # no scaling: plain frequencies
    assert c.att_kv_heads == 1 and abs(c.rot_slow - 0.5) < 1e-7
    del cfg["loop"]
    assert dsk.rutulix_from_config(cfg)[0].loop_times == 0
    cfg["layers"][1]["type"] = "latent_attention"
    with pytest.raises(dsk.DskError):
        dsk.rutulix_from_config(cfg)


def test_rutulix_oracle_invariants(ro):
    """(1) the chunk mask: with one attention layer a token of the chunk before cannot change the logits, a token of the own chunk
    does; (2) the loop's run order; (3) a sequence fed in two parts equals the whole; (4) rotation keeps a pair's length up to
    the magnitude factor and depends on the position difference only."""
    cfg = ro.model_config([ro.att(heads=2, dim=4, size=4, dims=2, ff=8)], width=16, vocab=23)
    W = ro.random_weights(cfg, 4)
    toks = np.arange(12) % 23
    base = ro.run(cfg, W, toks)[0][-1]                   # position 11 sees 8 .. 11
    out, ins = toks.copy(), toks.copy()
    out[7] += 1
    ins[8] += 1
    assert np.array_equal(ro.run(cfg, W, out)[0][-1], base)
    assert np.abs(ro.run(cfg, W, ins)[0][-1] - base).max() > 1e-6
    cfg2 = ro.small_config()
    assert ro.layer_runs(cfg2) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    W2 = ro.random_weights(cfg2, 5)
    whole = ro.run(cfg2, W2, np.arange(20) % 61)[0]
    seq = ro.Sequence(cfg2, W2)
    rows = [seq.feed(int(t)) for t in np.arange(20) % 61]
    assert np.allclose(np.array(rows), whole, rtol=0, atol=1e-12)
    rot = {"dims": 4, "base": 50.0, "scaling": {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 0.5}}
    _, mag = ro.rotation_table(rot)
    v = np.random.RandomState(0).randn(2 * 6)
    r5, r9 = ro.rotate_heads(v, 2, 6, rot, 5), ro.rotate_heads(v, 2, 6, rot, 9)
    assert np.allclose(np.hypot(r5[:, 0], r5[:, 1]), mag * np.hypot(v.reshape(2, 6)[:, 0], v.reshape(2, 6)[:, 1]))
    assert np.array_equal(r5[:, 4:], v.reshape(2, 6)[:, 4:])                          # beyond dims: unchanged
    w = np.random.RandomState(1).randn(2 * 6)
    d1 = (ro.rotate_heads(v, 2, 6, rot, 5) * ro.rotate_heads(w, 2, 6, rot, 2)).sum()
    d2 = (ro.rotate_heads(v, 2, 6, rot, 9) * ro.rotate_heads(w, 2, 6, rot, 6)).sum()
    assert abs(d1 - d2) < 1e-9


# ---- the Sakusun design ---------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def so():
    import sakusun_oracle
    return sakusun_oracle


def test_sakusun_config_to_layer_specs(so):
    import dsk
    cfg = so.public_config(so.small_config())
    hc, specs = dsk.ARCHITECTURES[cfg["architecture"]](cfg, quant="bf16", max_seq_len=77, chunk=16)
    assert (hc.dim, hc.vocab_size, hc.n_layers, hc.max_seq_len, hc.chunk, hc.side_dim, hc.loop_times) == (44, 61, 5, 77, 16, 0, 0)
    assert (hc.block, hc.norm_kind, hc.norm_scalar, hc.tie_head, hc.canon_taps, hc.res_gate, hc.layer_scale) == (dsk.BLOCK_POST, dsk.NORM_RMS, 1, 0, 4, 1, 1)
    assert (hc.bigram_buckets, hc.bigram_mul_prev, hc.bigram_mul_cur) == (37, 5, 3) and abs(hc.embed_scale - 0.75) < 1e-7
    a, b, c, d, e = specs
    assert (a.mixer, a.att_heads, a.att_kv_heads, a.att_dim, a.att_vdim, a.att_mask, a.att_window, a.att_keep_first) == (dsk.MIX_GQA, 6, 2, 10, 6, dsk.MASK_WINDOW, 7, 3)
    assert (a.att_value_proj, a.att_bias, a.att_sink, a.att_vmix, a.att_talk, a.att_rel_max, a.rot_dims) == (1, 1, 1, 1, 0, 20, 0) and abs(a.att_softcap - 15.0) < 1e-6
    assert (a.ff_kind, a.ff_hidden, a.ff_act) == (dsk.FF_DENSE, 28, dsk.ACT_GEGLU)
    assert (b.mixer, b.att_heads, b.att_dim, b.att_rot_dim, b.att_vdim, b.att_kv_rank, b.att_q_rank, b.att_out_gate, b.rot_dims) == (dsk.MIX_MLA, 3, 12, 6, 10, 14, 9, 1, 6)
    assert b.att_window == 1 << 30 and b.ff_kind == dsk.FF_NONE and abs(b.rot_base - 500.0) < 1e-3
    assert c.att_kv_heads == 1 and c.att_keep_first == 0 and e.att_vmix == 0 and d.att_rot_dim == 8
    m = cfg["layers"][0]["mixer"]
    del m["softcap"], m["bias_max"], m["mask"], m["kv_heads"]
    a = dsk.sakusun_from_config(cfg)[1][0]
    assert (a.att_softcap, a.att_rel_max, a.att_window, a.att_keep_first, a.att_kv_heads) == (0.0, 0, 1 << 30, 0, 6)
    cfg["layers"][1]["type"] = "mamba2"
    with pytest.raises(dsk.DskError):
        dsk.sakusun_from_config(cfg)


def test_sakusun_oracle_invariants(so):
    """(1) window with kept first positions; (2) distance buckets: one per distance below half, logarithmic steps above, the last
    one from the limit on; (3) a sequence fed token by token equals the whole; (4) the input convolution's carry; (5) rotation
    depends on the position difference only and leaves the entries beyond `dims` alone."""
    mask = {"size": 4, "keep_first": 2}
    assert [j for j in range(12) if so.sees(mask, 9, j)] == [0, 1, 6, 7, 8, 9]
    assert [j for j in range(12) if so.sees(None, 3, j)] == [0, 1, 2, 3]
    bk = [so.rel_bucket(n, 16, 100) for n in range(0, 400)]
    assert bk[:8] == list(range(8)) and bk[8] == 8 and bk[99] == 15 and bk[100] == 15 and bk[399] == 15 and all(x <= y for x, y in zip(bk, bk[1:]))
    cfg = so.small_config()
    W = so.random_weights(cfg, 5)
    toks = np.arange(20) % 61
    whole = so.run(cfg, W, toks)[0]
    seq = so.Sequence(cfg, W)
    assert np.allclose(np.array([seq.feed(int(t)) for t in toks]), whole, rtol=0, atol=1e-12)
    w = np.random.RandomState(0).randn(5, 3)
    xs = [np.random.RandomState(i).randn(5) for i in range(4)]
    u = so.input_conv(w, [xs[1], xs[2]], xs[3])
    assert np.allclose(u, xs[3] + w[:, 0] * xs[1] + w[:, 1] * xs[2] + w[:, 2] * xs[3])
    rot = {"dims": 4, "base": 50.0}
    v, k = np.random.RandomState(1).randn(6), np.random.RandomState(2).randn(6)
    assert abs(so.rotate(v, rot, 5) @ so.rotate(k, rot, 2) - so.rotate(v, rot, 9) @ so.rotate(k, rot, 6)) < 1e-9
    assert np.array_equal(so.rotate(v, rot, 7)[4:], v[4:])


@pytest.fixture(scope="module")
def no():
    import nalizen_oracle
    return nalizen_oracle


def test_nalizen_config_to_layer_specs(no):
    import dsk
    cfg = no.small_config()
    hc, specs = dsk.ARCHITECTURES[cfg["architecture"]](cfg, quant="bf16", max_seq_len=77, chunk=16)
    assert (hc.dim, hc.vocab_size, hc.n_layers, hc.max_seq_len, hc.chunk, hc.side_dim, hc.loop_times) == (44, 61, 5, 77, 16, 5, 0)
    assert (hc.block, hc.norm_kind, hc.norm_bias, hc.norm_scalar, hc.tie_head, hc.token_shift, hc.canon_taps, hc.res_gate, hc.layer_scale) == \
        (dsk.BLOCK_POST, dsk.NORM_LAYER, 1, 0, 1, 1, 0, 0, 0)
    assert abs(hc.embed_scale - 1.5) < 1e-7 and hc.bigram_buckets == 0
    a, b, c, d, e = specs
    assert (a.mixer, a.att_heads, a.att_kv_heads, a.att_dim, a.att_vdim, a.att_mask, a.att_window, a.att_kv_from) == (dsk.MIX_GQA, 6, 2, 10, 6, dsk.MASK_WINDOW, 7, -1)
    assert (a.att_value_proj, a.att_bias, a.att_sink, a.att_talk, a.att_out_gate, a.att_qk_norm, a.rot_layout, a.rot_scale, a.rot_dims, a.rot_original) == \
        (1, 0, 0, 0, 1, dsk.QKNORM_HEAD, dsk.ROT_HALF, dsk.ROTSCALE_BANDS, 6, 40)
    assert (a.rot_factor, a.rot_fast, a.rot_slow) == (4.0, 3.0, 1.0) and abs(a.rot_base - 50.0) < 1e-4 and abs(a.att_scale - 0.6) < 1e-6
    assert (a.ff_kind, a.ff_hidden, a.ff_act) == (dsk.FF_DENSE, 28, dsk.ACT_GEGLU)
    assert (b.mixer, b.lin_heads, b.lin_dim, b.lin_vdim) == (dsk.MIX_HGRN2, 3, 5, 7)
    assert (b.ff_kind, b.ff_router, b.ff_expert, b.ff_experts, b.ff_top, b.ff_hidden) == (dsk.FF_MOE, dsk.ROUTER_TOP_SOFTMAX, dsk.EXPERT_RELU2, 5, 2, 12)
    assert (c.att_kv_from, c.att_window, c.ff_experts, c.ff_top) == (0, 4, 7, 3) and d.ff_kind == dsk.FF_NONE
    assert (e.rot_factor, e.rot_dims, e.att_kv_heads, e.att_kv_from) == (0.0, 12, 1, -1)
    m = cfg["layers"][4]["mixer"]
    del m["rot"], m["mask"], m["kv_heads"]
    del cfg["token_side"], cfg["embedding"]
    hc, specs = dsk.nalizen_from_config(cfg)
    assert (specs[4].rot_dims, specs[4].att_window, specs[4].att_kv_heads, hc.side_dim, hc.embed_scale) == (0, 1 << 30, 2, 0, 1.0)
    cfg["layers"][1]["type"] = "mamba2"
    with pytest.raises(dsk.DskError):
        dsk.nalizen_from_config(cfg)


def test_nalizen_oracle_invariants(no):
    """(1) a sequence fed token by token equals the whole; (2) the rotation depends on the position difference only, pairs the two
    halves of the rotated part and leaves the entries beyond `dims` alone; (3) the frequency bands; (4) the recurrence with a forget
    gate of 1 keeps its state and with 0 holds the last value; (5) the token shift; (6) the layer norm."""
    cfg = no.small_config()
    W = no.random_weights(cfg, 5)
    toks = np.arange(20) % 61
    whole = no.run(cfg, W, toks)[0]
    seq = no.Sequence(cfg, W)
    assert np.allclose(np.array([seq.feed(int(t)) for t in toks]), whole, rtol=0, atol=1e-12)
    rot = {"dims": 4, "base": 50.0}
    v, k = np.random.RandomState(1).randn(6), np.random.RandomState(2).randn(6)
    assert abs(no.rotate_half(v, rot, 5) @ no.rotate_half(k, rot, 2) - no.rotate_half(v, rot, 9) @ no.rotate_half(k, rot, 6)) < 1e-9
    assert np.array_equal(no.rotate_half(v, rot, 7)[4:], v[4:])
    one = no.rotate_half(np.array([1.0, 0.0, 0.0, 0.0, 9.0]), {"dims": 4, "base": 1.0}, 1)       # entry 0 turns into entry 2, not 1
    assert np.allclose(one, [np.cos(1.0), 0.0, np.sin(1.0), 0.0, 9.0])
    sc = {"factor": 10.0, "low": 1.0, "high": 2.0, "original": 100}
    f = no.rot_frequencies({"dims": 8, "base": 1000.0, "scaling": sc})
    p = no.rot_frequencies({"dims": 8, "base": 1000.0})
    assert f[0] == p[0] and abs(f[3] - p[3] / 10.0) < 1e-15                                       # wavelengths 6.3 and 1117 against the bounds 50 and 100
    mid = 2.0 * np.pi / 75.0
    s = (100.0 / 75.0 - 1.0) / (2.0 - 1.0)
    g = no.rot_frequencies({"dims": 2, "base": 1.0, "scaling": sc})                               # base 1: frequency 1, wavelength 6.3: kept
    assert g == [1.0] and abs(((1 - s) * mid / 10.0 + s * mid) / mid - (0.1 + 0.9 * s)) < 1e-12
    mx = {"heads": 1, "dim": 2, "vdim": 3}
    Wl = {"q": np.eye(2, 4), "v": np.eye(3, 4), "f": np.zeros((2, 4)), "f.b": np.zeros(2), "lower": np.array([1.0, 0.0]), "norm": np.ones(3), "o": np.eye(3)}
    S = np.arange(6.0).reshape(1, 2, 3)
    no.hgrn2_step({"m." + k: v for k, v in Wl.items()}, "m.", mx, np.array([1.0, 2.0, 3.0, 4.0]), S, 1e-5)
    assert np.array_equal(S[0, 0], [0.0, 1.0, 2.0]) and np.allclose(S[0, 1], 0.5 * np.array([3.0, 4.0, 5.0]) + 0.5 * np.array([1.0, 2.0, 3.0]))
    assert np.allclose(no.token_shift(np.array([1.0, 2.0]), np.array([3.0, 6.0]), np.array([0.0, 0.25])), [1.0, 3.0])
    y = no.layer_norm(np.array([1.0, 3.0]), np.array([2.0, 2.0]), np.array([0.5, 0.5]), 0.0)
    assert np.allclose(y, [-1.5, 2.5])
