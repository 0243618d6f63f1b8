"""hybrid_bench.py — prefill and decode throughput of the layer-list family at sizes that resemble a real model's layers.
The Desarax sizes run beside the closest DeepSeek model of the framework (true-MLA blocks, fp16) at equal width / depth /
experts; the Rutulix sizes run beside the closest layer-list model, a Desarax model of latent-attention layers at equal width,
layer runs, heads, mask size and feed-forward matrix elements; the Sakusun sizes run beside a Rutulix model (the framework's other
attention-only design with dense feed-forwards) at equal width, depth, heads, window and feed-forward matrix elements; the
Nalizen sizes run beside a Desarax model (the framework's other design with a recurrence, shared attention caches, routed
feed-forwards and the per-layer token input) at equal width, depth, layer pattern, heads, window and active matrix elements.

Used by `bench.py --hybrid`.  Random weights generated on the GPU (bf16), uploaded through dsk_upload_tensor(src_on_device).
Decode is the device-side greedy loop (CUDA events around the captured step graph); prefill is dsk_forward_chunk over a prompt
longer than the latent window, timed by the host around the (synchronous) call after a warm-up call.  Roofline fractions are
against the measured copy bandwidth (decode: algorithmic weight bytes per token) and the measured cuBLAS bf16 rate (prefill:
2 x active matrix elements per token).
"""
import json
import os
import time

import numpy as np

SIZES = {
    # width, vocab, layer pattern (s = state-space, a = latent attention, A = latent attention reading the previous one's cache)
    "small": dict(width=1024, vocab=32000, pattern="ssassA", heads=32, vdim=64, state=64, groups=4, conv=4, att_heads=8, att_dim=64,
                  att_vdim=64, kv_rank=256, window=512, experts=16, top=2, ff=512, side=32),
    "v2lite_like": dict(width=2048, vocab=102400, pattern="ssassAssassA", heads=64, vdim=64, state=128, groups=8, conv=4, att_heads=16,
                        att_dim=128, att_vdim=128, kv_rank=512, window=1024, experts=64, top=6, ff=1408, side=64),
    # Rutulix: grouped-query attention layers with dense feed-forwards; layers loop[0] .. loop[1]-1 run loop[2] times
    "rutulix_small": dict(design="Rutulix", width=1024, vocab=32000, n_layers=8, loop=(2, 4, 2), att_heads=16, kv_heads=4, att_dim=64, rot=32,
                          window=512, ff=4096, kv_rank=256),
    "rutulix_large": dict(design="Rutulix", width=2048, vocab=102400, n_layers=12, loop=(4, 8, 2), att_heads=16, kv_heads=4, att_dim=128, rot=64,
                          window=1024, ff=8192, kv_rank=512),
    # Sakusun: pattern of latent-attention (L) and grouped-query attention (A) layers, gated feed-forwards of three matrices
    "sakusun_small": dict(design="Sakusun", width=1024, vocab=32000, pattern="LALLLALA", att_heads=16, kv_heads=4, att_dim=64, window=512, keep=4,
                          rel_rows=32, rel_max=1024, lat_dim=64, rot=32, kv_rank=256, q_rank=384, ff=2752, taps=4, buckets=65521),
    "sakusun_large": dict(design="Sakusun", width=2048, vocab=102400, pattern="LALLLALLLALA", att_heads=16, kv_heads=4, att_dim=128, window=1024, keep=4,
                          rel_rows=32, rel_max=2048, lat_dim=128, rot=64, kv_rank=512, q_rank=768, ff=5504, taps=4, buckets=65521),
    # Nalizen: pattern of recurrent (r) and attention layers (a: own keys and values, A: those of the previous a); the first layer's
    # feed-forward is dense, the others are routed (experts of two matrices)
    "nalizen_small": dict(design="Nalizen", width=1024, vocab=32000, pattern="rrarrA", lin_heads=16, lin_dim=64, lin_vdim=64, att_heads=16, kv_heads=4,
                          att_dim=64, rot=32, window=512, experts=16, top=2, ff=768, side=32),
    "nalizen_large": dict(design="Nalizen", width=2048, vocab=102400, pattern="rrarrArrarrA", lin_heads=16, lin_dim=128, lin_vdim=128, att_heads=16,
                          kv_heads=4, att_dim=128, rot=64, window=1024, experts=64, top=6, ff=2112, side=64),
}


def nalizen_config(z):
    layers, last_a = [], None
    for i, ch in enumerate(z["pattern"]):
        # the dense first feed-forward has as many matrix elements as the routed ones have active
        mlp = {"kind": "dense", "ff": z["top"] * z["ff"] * 2 // 3} if i == 0 else \
              {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["ff"]}}
        if ch == "r":
            layers.append({"type": "hgrn2", "mixer": {"heads": z["lin_heads"], "dim": z["lin_dim"], "vdim": z["lin_vdim"]}, "mlp": mlp})
            continue
        mx = {"heads": z["att_heads"], "kv_heads": z["kv_heads"], "dim": z["att_dim"], "vdim": z["att_dim"], "scale": z["att_dim"] ** -0.5,
              "mask": {"size": z["window"]},
              "rot": {"dims": z["rot"], "base": 500000.0, "scaling": {"factor": 32.0, "low": 1.0, "high": 8.0, "original": z["window"]}}}
        if ch == "A" and last_a is not None:
            mx["kv_from"] = last_a
        else:
            last_a = i
        layers.append({"type": "attention", "mixer": mx, "mlp": mlp})
    return {"architecture": "Nalizen", "vocab": z["vocab"], "width": z["width"], "layers": layers, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "token_side": {"dim": z["side"]}}


def closest_desarax_of_nalizen(z):
    """The closest model of the framework to a Nalizen size: Desarax layers in the same pattern (state-space recurrence for the
    gated linear one with as many heads, value channels and state rows; latent attention with a latent as wide as the key
    heads; routed GLU experts of three matrices with as many active elements as the two-matrix experts), same width, window,
    experts and token input."""
    return dict(width=z["width"], vocab=z["vocab"], pattern=z["pattern"].replace("r", "s"), heads=z["lin_heads"], vdim=z["lin_vdim"], state=z["lin_dim"],
                groups=max(1, z["lin_heads"] // 8), conv=4, att_heads=z["att_heads"], att_dim=z["att_dim"], att_vdim=z["att_dim"],
                kv_rank=z["kv_heads"] * z["att_dim"], window=z["window"], experts=z["experts"], top=z["top"], ff=z["ff"] * 2 // 3, side=z["side"])


def mint_nalizen(dsk, torch, cfg, quant, chunk, context, device=0):
    import hashlib
    hc, specs = dsk.nalizen_from_config(cfg, quant=quant, max_seq_len=context, chunk=chunk)
    m = dsk.Model(hc, 0, 1, device, layers=specs)
    dev = torch.device("cuda", device)
    W, V, L = cfg["width"], cfg["vocab"], len(cfg["layers"])
    sd = cfg["token_side"]["dim"]

    def up(name, shape, kind="mat"):
        torch.manual_seed(int(hashlib.md5(name.encode()).hexdigest()[:8], 16))
        if kind == "mat":
            t = torch.randn(*shape, device=dev) * (shape[-1] ** -0.5)
        elif kind == "embed":
            t = torch.randn(*shape, device=dev)
        elif kind == "norm":
            t = 1.0 + 0.1 * torch.randn(*shape, device=dev)
        elif kind == "unit":
            t = torch.empty(*shape, device=dev).uniform_(0.0, 0.9)
        else:
            t = 0.1 * torch.randn(*shape, device=dev)
        t = t.to(torch.bfloat16).contiguous()
        m.upload_device(name, "BF16", shape, t.data_ptr(), t.numel() * 2)
        torch.cuda.synchronize()

    up("embed", (V, W), "embed"); up("final.norm", (W,), "norm"); up("final.norm.b", (W,), "small"); up("side.embed", (V, sd * L), "embed")
    for i, lc in enumerate(cfg["layers"]):
        p, mx, ff = f"l{i}.", lc["mixer"], lc["mlp"]
        for nm in ("norm1", "norm2"):
            up(p + nm, (W,), "norm"); up(p + nm + ".b", (W,), "small")
        up(p + "shift", (W,), "unit")
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        if lc["type"] == "attention":
            G = mx["kv_heads"]
            up(p + "mix.q", (H * D, W)); up(p + "mix.g", (H * Vd, W)); up(p + "mix.o", (W, H * Vd))
            if "kv_from" not in mx:
                up(p + "mix.k", (G * D, W)); up(p + "mix.v", (G * Vd, W))
        else:
            up(p + "mix.q", (H * D, W)); up(p + "mix.f", (H * D, W)); up(p + "mix.f.b", (H * D,), "small"); up(p + "mix.lower", (H * D,), "unit")
            up(p + "mix.v", (H * Vd, W)); up(p + "mix.norm", (Vd,), "norm"); up(p + "mix.o", (W, H * Vd))
        if ff["kind"] == "dense":
            up(p + "mlp.gate", (ff["ff"], W)); up(p + "mlp.up", (ff["ff"], W)); up(p + "mlp.down", (W, ff["ff"]))
        else:
            E, fe = ff["router"]["experts"], ff["expert"]["ff"]
            up(p + "mlp.router", (E, W)); up(p + "mlp.router.b", (E,), "small")
            for e in range(E):
                up(f"{p}mlp.e{e}.up", (fe, W)); up(f"{p}mlp.e{e}.down", (W, fe))
        up(p + "side.gate", (sd, W)); up(p + "side.proj", (W, sd)); up(p + "side.norm", (W,), "norm")
    m.finalize()
    return m


def nalizen_matrix_elements(cfg, z):
    """Matrix elements one token multiplies with (projections, gate, feed-forward, token input, head), and the attention's own
    multiply-adds per token at the mean number of visible keys (half the window)."""
    W, n, att = cfg["width"], cfg["width"] * cfg["vocab"], 0.0
    for lc in cfg["layers"]:
        mx, ff = lc["mixer"], lc["mlp"]
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        if lc["type"] == "attention":
            n += H * D * W + 2 * H * Vd * W + (0 if "kv_from" in mx else mx["kv_heads"] * (D + Vd) * W)
            att += H * (D + Vd) * (z["window"] / 2.0)
        else:
            n += (2 * H * D + H * Vd) * W + W * H * Vd
        n += 3 * ff["ff"] * W if ff["kind"] == "dense" else 2 * ff["router"]["top"] * ff["expert"]["ff"] * W + ff["router"]["experts"] * W
        n += 2 * cfg["token_side"]["dim"] * W
    return n, att


def run_nalizen(dsk, torch, name, hbm, tfl, prompt_len, gen, chunk, log):
    """A Nalizen size and the closest model of the framework (Desarax) at equal size."""
    z = SIZES[name]
    cfg = nalizen_config(z)
    t0 = time.time()
    m = mint_nalizen(dsk, torch, cfg, "bf16", chunk, prompt_len + gen + 8)
    log(f"hybrid/{name}/bf16: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
    mat, att = nalizen_matrix_elements(cfg, z)
    res = [measure_layer_list(m, f"Nalizen {name}", z["vocab"], 2.0 * mat, hbm, tfl, prompt_len, gen, chunk, log,
                              {"layers": len(z["pattern"]), "width": z["width"], "attention_flops_per_token_fp32": 2.0 * att})]
    m.close()
    zd = closest_desarax_of_nalizen(z)
    cfgd = desarax_config(zd)
    t0 = time.time()
    m = mint_desarax(dsk, torch, cfgd, "bf16", chunk, prompt_len + gen + 8)
    log(f"hybrid/{name}/closest Desarax/bf16: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
    res.append(measure_layer_list(m, f"Desarax layers at {name}", z["vocab"], 2.0 * active_matrix_elements(cfgd), hbm, tfl, prompt_len, gen, chunk, log,
                                  {"layers": len(cfgd["layers"]), "width": z["width"]}))
    m.close()
    return res


def sakusun_config(z):
    att = {"heads": z["att_heads"], "kv_heads": z["kv_heads"], "dim": z["att_dim"], "vdim": z["att_dim"], "scale": z["att_dim"] ** -0.5, "softcap": 30.0,
           "bias_max": z["rel_max"], "mask": {"size": z["window"], "keep_first": z["keep"]}, "v_mix": True}
    lat = {"heads": z["att_heads"], "dim": z["lat_dim"], "rot_dim": z["rot"], "vdim": z["lat_dim"], "kv_rank": z["kv_rank"], "q_rank": z["q_rank"],
           "scale": (z["lat_dim"] + z["rot"]) ** -0.5, "rot": {"dims": z["rot"], "base": 10000.0}}
    layers = [{"type": "attention" if ch == "A" else "latent_attention", "mixer": dict(att if ch == "A" else lat), "mlp": {"kind": "dense", "ff": z["ff"]}}
              for ch in z["pattern"]]
    return {"architecture": "Sakusun", "vocab": z["vocab"], "width": z["width"], "layers": layers, "norm": {"eps": 1e-5}, "canon": {"taps": z["taps"]},
            "embedding": {"scale": 0.75, "bigram": {"buckets": z["buckets"], "mul_prev": 53, "mul_cur": 11}}}


def closest_rutulix(z):
    """The closest model of the framework to a Sakusun size: Rutulix layers (grouped-query attention, dense feed-forward of two
    matrices with as many elements as the gated three), as many as the Sakusun model has, same width, heads and mask size."""
    return dict(design="Rutulix", width=z["width"], vocab=z["vocab"], n_layers=len(z["pattern"]), loop=(0, 1, 1), att_heads=z["att_heads"],
                kv_heads=z["kv_heads"], att_dim=z["att_dim"], rot=z["att_dim"] // 2, window=z["window"], ff=z["ff"] * 3 // 2, kv_rank=z["kv_rank"])


def mint_sakusun(dsk, torch, cfg, z, quant, chunk, context, device=0):
    import hashlib
    hc, specs = dsk.sakusun_from_config(cfg, quant=quant, max_seq_len=context, chunk=chunk)
    m = dsk.Model(hc, 0, 1, device, layers=specs)
    dev = torch.device("cuda", device)
    W, V = cfg["width"], cfg["vocab"]

    def up(name, shape, kind="mat"):
        torch.manual_seed(int(hashlib.md5(name.encode()).hexdigest()[:8], 16))
        if kind == "mat":
            t = torch.randn(*shape, device=dev) * (shape[-1] ** -0.5)
        elif kind == "embed":
            t = torch.randn(*shape, device=dev)
        elif kind == "norm":
            t = 1.0 + 0.1 * torch.randn(*shape, device=dev)
        elif kind == "one":
            t = torch.full((1,), 0.8, device=dev)
        else:
            t = 0.1 * torch.randn(*shape, device=dev)
        t = t.to(torch.bfloat16).contiguous()
        m.upload_device(name, "BF16", shape, t.data_ptr(), t.numel() * 2)
        torch.cuda.synchronize()

    up("embed", (V, W), "embed"); up("bigram", (cfg["embedding"]["bigram"]["buckets"] + 1, W), "embed"); up("head", (V, W)); up("final.norm", (), "one")
    taps = cfg["canon"]["taps"]
    for i, lc in enumerate(cfg["layers"]):
        p, mx, ff = f"l{i}.", lc["mixer"], lc["mlp"]["ff"]
        for n in ("1", "2"):
            up(p + "norm" + n, (), "one"); up(p + "ls" + n, (W,), "norm"); up(p + "canon" + n, (W, taps), "small")
            up(p + "rg" + n, (W, W)); up(p + "rg" + n + ".b", (W,), "small")
        if lc["type"] == "attention":
            H, G, D, Vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            up(p + "mix.q", (H * D, W)); up(p + "mix.k", (G * D, W)); up(p + "mix.v", (G * Vd, W))
            up(p + "mix.q.b", (H * D,), "small"); up(p + "mix.k.b", (G * D,), "small"); up(p + "mix.v.b", (G * Vd,), "small")
            up(p + "mix.q.norm", (H * D,), "norm"); up(p + "mix.k.norm", (G * D,), "norm"); up(p + "mix.rel", (z["rel_rows"], H), "small")
            up(p + "mix.sink", (H,), "small"); up(p + "mix.vmix", (), "one"); up(p + "mix.o", (W, H * Vd))
        else:
            H, D, Rd, Vd, R, Q = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            up(p + "mix.dq", (Q, W)); up(p + "mix.dq.norm", (Q,), "norm"); up(p + "mix.uq", (H * (D + Rd), Q)); up(p + "mix.dkv", (R + Rd, W))
            up(p + "mix.dkv.norm", (R,), "norm"); up(p + "mix.uk", (H * D, R)); up(p + "mix.uv", (H * Vd, R)); up(p + "mix.g", (H * Vd, W))
            up(p + "mix.o", (W, H * Vd))
        up(p + "mlp.gate", (ff, W)); up(p + "mlp.up", (ff, W)); up(p + "mlp.down", (W, ff))
    m.finalize()
    return m


def sakusun_matrix_elements(cfg, z):
    """Matrix elements one token multiplies with (projections, gates, feed-forward, head), and the attention's own multiply-adds
    per token at the mean number of visible keys of a prompt of `window` x 2 tokens."""
    W, n, att = cfg["width"], cfg["width"] * cfg["vocab"], 0.0
    for lc in cfg["layers"]:
        mx = lc["mixer"]
        n += 2 * W * W + 3 * lc["mlp"]["ff"] * W
        if lc["type"] == "attention":
            H, G, D, Vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            n += (H * D + G * D + G * Vd) * W + W * H * Vd
            att += H * (D + Vd) * (z["window"] / 2.0)
        else:
            H, D, Rd, Vd, R, Q = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            n += (Q + R + Rd) * W + H * (D + Rd) * Q + H * (D + Vd) * R + 2 * H * Vd * W
            att += H * (D + Rd + Vd) * z["window"]
    return n, att


def run_sakusun(dsk, torch, name, hbm, tfl, prompt_len, gen, chunk, log):
    """A Sakusun size and the closest model of the framework (Rutulix) at equal size."""
    z = SIZES[name]
    cfg = sakusun_config(z)
    t0 = time.time()
    m = mint_sakusun(dsk, torch, cfg, z, "bf16", chunk, prompt_len + gen + 8)
    log(f"hybrid/{name}/bf16: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
    mat, att = sakusun_matrix_elements(cfg, z)
    res = [measure_layer_list(m, f"Sakusun {name}", z["vocab"], 2.0 * mat, hbm, tfl, prompt_len, gen, chunk, log,
                              {"layers": len(z["pattern"]), "width": z["width"], "attention_flops_per_token_fp32": 2.0 * att})]
    m.close()
    zr = closest_rutulix(z)
    cfgr = rutulix_config(zr)
    t0 = time.time()
    m = mint_rutulix(dsk, torch, cfgr, "bf16", chunk, prompt_len + gen + 8)
    log(f"hybrid/{name}/closest Rutulix/bf16: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
    mat, att = rutulix_matrix_elements(cfgr, zr)
    res.append(measure_layer_list(m, f"Rutulix layers at {name}", z["vocab"], 2.0 * mat, hbm, tfl, prompt_len, gen, chunk, log,
                                  {"layer_runs": rutulix_runs(zr), "width": z["width"], "attention_flops_per_token_fp32": 2.0 * att}))
    m.close()
    return res


def rutulix_config(z):
    mx = {"heads": z["att_heads"], "kv_heads": z["kv_heads"], "dim": z["att_dim"], "vdim": z["att_dim"], "scale": z["att_dim"] ** -0.5,
          "mask": {"size": z["window"]},
          "rot": {"dims": z["rot"], "base": 10000.0, "scaling": {"factor": 8.0, "original": z["window"], "fast": 32.0, "slow": 1.0}}}
    layers = [{"type": "attention", "mixer": dict(mx), "mlp": {"kind": "dense", "ff": z["ff"]}} for _ in range(z["n_layers"])]
    return {"architecture": "Rutulix", "vocab": z["vocab"], "width": z["width"], "layers": layers, "norm": {"eps": 1e-5},
            "loop": {"start": z["loop"][0], "stop": z["loop"][1], "times": z["loop"][2]}}


def rutulix_runs(z):
    return z["n_layers"] + (z["loop"][1] - z["loop"][0]) * (z["loop"][2] - 1)


def closest_desarax(z):
    """The closest layer-list model to a Rutulix size: latent-attention layers only, as many as the Rutulix model has layer runs,
    same heads and mask size, routed GLU experts whose active matrices (top 2 x 3 matrices) match the dense pair."""
    ff_e = max(64, (z["ff"] // 3) // 64 * 64)
    return dict(width=z["width"], vocab=z["vocab"], pattern="a" * rutulix_runs(z), att_heads=z["att_heads"], att_dim=z["att_dim"],
                att_vdim=z["att_dim"], kv_rank=z["kv_rank"], window=z["window"], experts=8, top=2, ff=ff_e, side=0,
                heads=0, vdim=0, state=0, groups=1, conv=1)


def mint_rutulix(dsk, torch, cfg, quant, chunk, context, device=0):
    import hashlib
    hc, specs = dsk.rutulix_from_config(cfg, quant=quant, max_seq_len=context, chunk=chunk)
    m = dsk.Model(hc, 0, 1, device, layers=specs)
    dev = torch.device("cuda", device)
    W, V = cfg["width"], cfg["vocab"]

    def up(name, shape, kind="mat"):
        torch.manual_seed(int(hashlib.md5(name.encode()).hexdigest()[:8], 16))
        if kind == "mat":
            t = torch.randn(*shape, device=dev) * (shape[-1] ** -0.5)
        elif kind == "embed":
            t = torch.randn(*shape, device=dev)
        elif kind == "norm":
            t = 1.0 + 0.1 * torch.randn(*shape, device=dev)
        elif kind == "talk":
            t = torch.eye(shape[0], device=dev) + 0.1 * torch.randn(*shape, device=dev)
        else:
            t = 0.1 * torch.randn(*shape, device=dev)
        t = t.to(torch.bfloat16).contiguous()
        m.upload_device(name, "BF16", shape, t.data_ptr(), t.numel() * 2)
        torch.cuda.synchronize()

    up("embed", (V, W), "embed"); up("head", (V, W)); up("final.norm", (W,), "norm")
    if hc.loop_times >= 1:
        up("loop.step", (hc.loop_times, W), "small")
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        HD, GD, ff = mx["heads"] * mx["dim"], mx["kv_heads"] * mx["dim"], lc["mlp"]["ff"]
        for nm in ("norm1", "norm1b", "norm2", "norm2b"):
            up(p + nm, (W,), "norm")
        up(p + "mix.q", (HD, W)); up(p + "mix.k", (GD, W)); up(p + "mix.q.norm", (HD,), "norm"); up(p + "mix.k.norm", (GD,), "norm")
        up(p + "mix.talk", (mx["heads"], mx["heads"]), "talk"); up(p + "mix.o", (W, HD))
        up(p + "mlp.up", (ff, W)); up(p + "mlp.up.b", (ff,), "small"); up(p + "mlp.down", (W, ff)); up(p + "mlp.down.b", (W,), "small")
        up(p + "mlp.act", (2,), "small")
    m.finalize()
    return m


def rutulix_matrix_elements(cfg, z):
    """Matrix elements one token multiplies with, and the attention's own multiply-adds per token at the mean number of visible
    keys (half the mask size): scores and weighted values over all heads."""
    W, mx = cfg["width"], cfg["layers"][0]["mixer"]
    per = (mx["heads"] + mx["kv_heads"]) * mx["dim"] * W + W * mx["heads"] * mx["dim"] + 2 * z["ff"] * W
    att = 2 * mx["heads"] * mx["dim"] * (z["window"] / 2.0)
    return W * cfg["vocab"] + rutulix_runs(z) * per, rutulix_runs(z) * att


def desarax_config(z):
    layers, last_a = [], None
    for i, ch in enumerate(z["pattern"]):
        mlp = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"], "scale": 1.0}, "expert": {"ff": z["ff"], "limit": 7.0}}
        if ch == "s":
            layers.append({"type": "mamba2", "mlp": mlp, "mixer": {"heads": z["heads"], "vdim": z["vdim"], "state": z["state"], "groups": z["groups"],
                                                                    "conv": z["conv"], "norm_groups": z["groups"]}})
        else:
            mx = {"heads": z["att_heads"], "dim": z["att_dim"], "vdim": z["att_vdim"], "kv_rank": z["kv_rank"], "mask": {"size": z["window"]},
                  "scale": z["att_dim"] ** -0.5}
            if ch == "A" and last_a is not None:
                mx["kv_from"] = last_a
            else:
                last_a = i
            layers.append({"type": "latent_attention", "mlp": mlp, "mixer": mx})
    cfg = {"architecture": "Desarax", "vocab": z["vocab"], "width": z["width"], "layers": layers, "norm": {"eps": 1e-5, "groups": 4},
           "residual_mult": 0.5, "logit_scale": 1.0}
    if z["side"]:
        cfg["token_side"] = {"dim": z["side"]}
    return cfg


def mint_desarax(dsk, torch, cfg, quant, chunk, context, device=0):
    import hashlib
    hc, specs = dsk.hybrid_from_config(cfg, quant=quant, max_seq_len=context, chunk=chunk)
    m = dsk.Model(hc, 0, 1, device, layers=specs)
    dev = torch.device("cuda", device)
    W, V, L = cfg["width"], cfg["vocab"], len(cfg["layers"])
    sd = (cfg.get("token_side") or {}).get("dim", 0)

    def up(name, shape, kind="mat"):
        torch.manual_seed(int(hashlib.md5(name.encode()).hexdigest()[:8], 16))
        if kind == "mat":
            t = torch.randn(*shape, device=dev) * (shape[-1] ** -0.5)
        elif kind == "embed":
            t = torch.randn(*shape, device=dev)
        elif kind == "norm":
            t = 1.0 + 0.1 * torch.randn(*shape, device=dev)
        elif kind == "alog":
            t = torch.log(torch.empty(*shape, device=dev).uniform_(0.5, 4.0))
        elif kind == "dtb":
            t = torch.empty(*shape, device=dev).uniform_(-3.0, 0.0)
        else:
            t = 0.1 * torch.randn(*shape, device=dev)
        t = t.to(torch.bfloat16).contiguous()
        m.upload_device(name, "BF16", shape, t.data_ptr(), t.numel() * 2)
        torch.cuda.synchronize()

    up("embed", (V, W), "embed"); up("final.norm", (W,), "norm")
    if sd:
        up("side.embed", (V, sd * L), "embed")
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        up(p + "norm1", (W,), "norm")
        if "state" in mx:
            inner, ch = mx["heads"] * mx["vdim"], mx["heads"] * mx["vdim"] + 2 * mx["groups"] * mx["state"]
            up(p + "mix.in", (inner + ch + mx["heads"], W)); up(p + "mix.conv", (ch, mx["conv"])); up(p + "mix.conv.b", (ch,), "small")
            up(p + "mix.dt_bias", (mx["heads"],), "dtb"); up(p + "mix.A_log", (mx["heads"],), "alog"); up(p + "mix.D", (mx["heads"],), "norm")
            up(p + "mix.norm", (inner,), "norm"); up(p + "mix.o", (W, inner))
        else:
            H, D, Vd, R = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"]
            up(p + "mix.q", (H * D, W)); up(p + "mix.uk", (H * D, R)); up(p + "mix.uv", (H * Vd, R)); up(p + "mix.o", (W, H * Vd))
            if "kv_from" not in mx:
                up(p + "mix.dkv", (R, W)); up(p + "mix.dkv.norm", (R,), "norm")
        E, ff = lc["mlp"]["router"]["experts"], lc["mlp"]["expert"]["ff"]
        up(p + "mlp.router", (E, W)); up(p + "mlp.correction", (E,), "small")
        for e in range(E):
            up(f"{p}mlp.e{e}.gate", (ff, W)); up(f"{p}mlp.e{e}.up", (ff, W)); up(f"{p}mlp.e{e}.down", (W, ff))
        if sd:
            up(p + "side.gate", (sd, W)); up(p + "side.proj", (W, sd)); up(p + "side.norm", (W,), "norm")
    m.finalize()
    return m


def active_matrix_elements(cfg):
    """Matrix elements one token multiplies with (for prefill FLOPs = 2 x this)."""
    W, n = cfg["width"], cfg["width"] * cfg["vocab"]
    for lc in cfg["layers"]:
        mx = lc["mixer"]
        if "state" in mx:
            inner = mx["heads"] * mx["vdim"]
            n += (2 * inner + 2 * mx["groups"] * mx["state"] + mx["heads"]) * W + W * inner
        else:
            H, D, Vd, R = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"]
            n += H * D * W + H * (D + Vd) * R + W * H * Vd + (0 if "kv_from" in mx else R * W)
        n += 3 * lc["mlp"]["router"]["top"] * lc["mlp"]["expert"]["ff"] * W + lc["mlp"]["router"]["experts"] * W
        n += 2 * (cfg.get("token_side") or {}).get("dim", 0) * W
    return n


def peaks(repo):
    try:
        p = json.load(open(os.path.join(repo, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def measure_layer_list(m, label, vocab, flops_per_token, hbm, tfl, prompt_len, gen, chunk, log, extra=None):
    """Prefill (host-timed synchronous call, best of 3 after a warm-up) and decode (device loop, CUDA events) of one model."""
    rng = np.random.RandomState(0)
    prompt = rng.randint(0, vocab, prompt_len).astype(np.int32)
    m.forward_chunk(prompt, 0, [prompt_len - 1])                               # warm-up (also the first-use costs)
    ts = []
    for _ in range(3):
        t0 = time.perf_counter()
        m.forward_chunk(prompt, 0, [prompt_len - 1])
        ts.append(time.perf_counter() - t0)
    pre = prompt_len / min(ts)
    m.decode_greedy(prompt_len, 8)                                             # captures the step graph
    m.forward_chunk(prompt, 0, [prompt_len - 1])
    toks, ms = m.decode_greedy(prompt_len, gen)
    dec = gen / (ms * 1e-3)
    ab = m.active_bytes_per_token()
    r = {"model": label, "quant": "bf16", "resident_gb": m.resident_bytes() / 1e9, "prefill_tok_s": pre, "prefill_tokens": prompt_len, "chunk": chunk,
         "decode_tok_s": dec, "decode_tokens": gen, "active_bytes_per_token": ab, "decode_frac_of_hbm": ab * dec / (hbm * 1e9),
         "prefill_frac_of_bf16": flops_per_token * pre / (tfl * 1e12), "launches_per_token": m.launches_per_forward()}
    r.update(extra or {})
    log(json.dumps(r))
    return r


def run_rutulix(dsk, torch, name, hbm, tfl, prompt_len, gen, chunk, log):
    """A Rutulix size and the closest layer-list model (Desarax, latent-attention layers) at equal size."""
    z = SIZES[name]
    cfg = rutulix_config(z)
    t0 = time.time()
    m = mint_rutulix(dsk, torch, cfg, "bf16", chunk, prompt_len + gen + 8)
    log(f"hybrid/{name}/bf16: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
    mat, att = rutulix_matrix_elements(cfg, z)
    res = [measure_layer_list(m, f"Rutulix {name}", z["vocab"], 2.0 * mat, hbm, tfl, prompt_len, gen, chunk, log,
                              {"layer_runs": rutulix_runs(z), "width": z["width"], "attention_flops_per_token_fp32": 2.0 * att})]
    m.close()
    zd = closest_desarax(z)
    cfgd = desarax_config(zd)
    t0 = time.time()
    m = mint_desarax(dsk, torch, cfgd, "bf16", chunk, prompt_len + gen + 8)
    log(f"hybrid/{name}/closest Desarax/bf16: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
    res.append(measure_layer_list(m, f"Desarax latent-attention layers at {name}", z["vocab"], 2.0 * active_matrix_elements(cfgd), hbm, tfl, prompt_len,
                                  gen, chunk, log, {"layers": len(cfgd["layers"]), "width": z["width"]}))
    m.close()
    return res


def run(dsk, torch, repo, bench_module, sizes=("small", "v2lite_like"), prompt_len=2048, gen=128, chunk=2048, log=print):
    hbm, tfl, src = peaks(repo)
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "source": src}, "results": []}
    for name in sizes:
        z = SIZES[name]
        if z.get("design") == "Rutulix":
            out["results"] += run_rutulix(dsk, torch, name, hbm, tfl, prompt_len, gen, chunk, log)
            continue
        if z.get("design") == "Sakusun":
            out["results"] += run_sakusun(dsk, torch, name, hbm, tfl, prompt_len, gen, chunk, log)
            continue
        if z.get("design") == "Nalizen":
            out["results"] += run_nalizen(dsk, torch, name, hbm, tfl, prompt_len, gen, chunk, log)
            continue
        cfg = desarax_config(z)
        for quant in ("bf16",):
            t0 = time.time()
            m = mint_desarax(dsk, torch, cfg, quant, chunk, prompt_len + gen + 8)
            log(f"hybrid/{name}/{quant}: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
            rng = np.random.RandomState(0)
            prompt = rng.randint(0, z["vocab"], prompt_len).astype(np.int32)
            m.forward_chunk(prompt, 0, [prompt_len - 1])                       # warm-up (also the first-use costs)
            ts = []
            for _ in range(3):
                t0 = time.perf_counter()
                m.forward_chunk(prompt, 0, [prompt_len - 1])
                ts.append(time.perf_counter() - t0)
            pre = prompt_len / min(ts)
            m.decode_greedy(prompt_len, 8)                                     # captures the step graph
            m.forward_chunk(prompt, 0, [prompt_len - 1])
            toks, ms = m.decode_greedy(prompt_len, gen)
            dec = gen / (ms * 1e-3)
            ab = m.active_bytes_per_token()
            flops = 2.0 * active_matrix_elements(cfg)
            r = {"model": f"Desarax {name}", "quant": quant, "layers": len(cfg["layers"]), "width": z["width"], "resident_gb": m.resident_bytes() / 1e9,
                 "prefill_tok_s": pre, "prefill_tokens": prompt_len, "chunk": chunk, "decode_tok_s": dec, "decode_tokens": gen,
                 "active_bytes_per_token": ab, "decode_frac_of_hbm": ab * dec / (hbm * 1e9), "prefill_frac_of_bf16": flops * pre / (tfl * 1e12),
                 "launches_per_token": m.launches_per_forward()}
            log(json.dumps(r))
            out["results"].append(r)
            m.close()
        # the closest DeepSeek model of the framework at equal width / depth / experts: true-MLA blocks, fp16 matrices
        w = dict(bench_module.WORKLOADS["v2lite"])
        w.update(dim=z["width"], hidden_dim=z["ff"] * z["top"], n_layers=len(z["pattern"]), n_heads=z["att_heads"], vocab_size=z["vocab"],
                 qk_nope_head_dim=z["att_dim"], qk_rope_head_dim=64, v_head_dim=z["att_vdim"], kv_lora_rank=z["kv_rank"], q_lora_rank=z["kv_rank"],
                 first_k_dense_replace=0, n_shared_experts=0, n_routed_experts=z["experts"], n_active_routed=z["top"], moe_intermediate_size=z["ff"],
                 max_seq_len=1024, quant="fp16", use_mla=1)
        t0 = time.time()
        m = bench_module.mint_on_gpu(dsk, w, 0, 1, 0)
        log(f"deepseek-mla/{name}/fp16: minted {m.resident_bytes() / 1e9:.2f} GB in {time.time() - t0:.1f} s")
        n_pre = 256
        for i in range(8):
            m.forward(int(i), i, dsk.HYDRATE_KV_CACHE)
        t0 = time.perf_counter()
        for i in range(n_pre):                                                 # its prefill is the hydrate loop: one forward per token
            m.forward(int(i % z["vocab"]), i, dsk.OUTPUT_LOGITS if i == n_pre - 1 else dsk.HYDRATE_KV_CACHE)
        pre = n_pre / (time.perf_counter() - t0)
        m.decode_greedy(n_pre, 8)
        toks, ms = m.decode_greedy(n_pre + 8, gen)
        dec = gen / (ms * 1e-3)
        ab = m.active_bytes_per_token()
        r = {"model": f"DeepSeek true-MLA {name}", "quant": "fp16", "layers": w["n_layers"], "width": z["width"], "resident_gb": m.resident_bytes() / 1e9,
             "prefill_tok_s": pre, "prefill_tokens": n_pre, "decode_tok_s": dec, "decode_tokens": gen, "active_bytes_per_token": ab,
             "decode_frac_of_hbm": ab * dec / (hbm * 1e9), "prefill_frac_of_bf16": None, "launches_per_token": m.launches_per_forward()}
        log(json.dumps(r))
        out["results"].append(r)
        m.close()
    return out
