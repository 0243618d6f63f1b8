"""nalizen_oracle.py — plain, slow float64 statement of the Nalizen design (a layer-list model), for tests only.

One function per mechanism, written from the equations with numpy, token by token, and sharing no code with the CUDA path.
`Sequence.feed` carries what a sequence carries: per layer the previous token's mixer input (token shift), per attention
layer that projects keys and values everything it caches, per recurrent layer its state.

Notation: W x for a stored [out, in] matrix; rms(v) = v / sqrt(mean(v^2) + eps); ln(v) = (v - mean) / sqrt(var + eps) * w + b
with var the mean of the squared deviations; sg = logistic function; gelu = the tanh form.

  embedding:  x = s E[token]
  layer:      h = x + (x_prev - x) * mu        (x_prev: this layer's input at the previous token, zeros at the first one; mixer only)
              x <- x + ln1(mixer(h));  x <- x + ln2(ff(x))  (a layer without a feed-forward skips this);
              token input: g = gelu(W_sg x) * T[token, i*sd:(i+1)*sd];  y = W_sp g;  x <- x + rms(y) * w_s
  attention:  q = W_q h, k = W_k h, v = W_v h;  per head, the first rot.dims entries turn in pairs (i, i + dims/2) by the angle
              pos * f_i, f_i = base^(-2i/dims), optionally rescaled (wavelength l = 2 pi / f: kept below original/high, divided by
              factor above original/low, blended linearly in original/l between);  then q and k are divided by their RMS per head;
              s_j = scale (q_h . k_j[h // (H/G)]) for 0 <= i - j < size;  softmax;  o_h = sum_j p_j v_j[h // (H/G)];
              W_o (concat(o) * sg(W_g h)).  kv_from j: no k / v projections; layer j's cached keys and values are read instead.
  hgrn2:      q = silu(W_q h) [H, D], v = W_v h [H, Vd], f = l + (1 - l) sg(W_f h + b_f) [H, D];
              S <- diag(f) S + (1 - f) v^T per head (S [D, Vd]), o = S^T q;  W_o concat(rms(o_h) * w_n)
  ff dense:   W_down (gelu(W_gate x) * (W_up x))
  ff moe:     z = W_r x + b_r;  the `top` largest z (lower index first on ties);  weights = softmax over the chosen z;
              sum_e w_e W_down,e relu(W_up,e x)^2
  output:     logits = E ln_final(x)
"""
import math

import numpy as np

from hybrid_oracle import bf16_to_f64, to_bf16, write_checkpoint  # noqa: F401  (checkpoint minting helpers)


# ---- mechanisms -------------------------------------------------------------------------------------------------------
def rms(v, eps):
    v = np.asarray(v, dtype=np.float64)
    return v / math.sqrt(float(np.mean(v * v)) + eps)


def layer_norm(v, w, b, eps):
    v = np.asarray(v, dtype=np.float64)
    d = v - v.mean()
    return d / math.sqrt(float(np.mean(d * d)) + eps) * w + b


def logistic(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, dtype=np.float64)))


def silu(z):
    z = np.asarray(z, dtype=np.float64)
    return z * logistic(z)


def gelu_tanh(z):
    z = np.asarray(z, dtype=np.float64)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(x, prev, mu):
    return x + (prev - x) * mu


def rot_frequencies(rot):
    """Angle per position of every pair, after the optional rescaling of long wavelengths."""
    dims, sc = rot["dims"], rot.get("scaling")
    out = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        if sc:
            wl = 2.0 * math.pi / f
            if wl > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif not wl < sc["original"] / sc["high"]:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate_half(v, rot, pos):
    """Entries (i, i + dims/2) of the first rot["dims"] entries of v turn together; the rest pass."""
    out = np.array(v, dtype=np.float64)
    if not rot or not rot.get("dims"):
        return out
    half = rot["dims"] // 2
    for i, f in enumerate(rot_frequencies(rot)):
        a = pos * f
        c, s = math.cos(a), math.sin(a)
        u, w = out[i], out[i + half]
        out[i], out[i + half] = u * c - w * s, w * c + u * s
    return out


def attention_step(W, p, mx, h, pos, cache, eps, own):
    """One token through the attention mixer.  cache: {"k": [...], "v": [...]} over all earlier positions; `own`: this layer
    projects keys and values and appends them (otherwise the cache already holds this position, written by its owner)."""
    H, G, D, Vd = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    q = (W[p + "q"] @ h).reshape(H, D)
    q = np.array([rms(rotate_half(q[a], mx.get("rot"), pos), eps) for a in range(H)])
    if own:
        k = (W[p + "k"] @ h).reshape(G, D)
        cache["k"].append(np.array([rms(rotate_half(k[g], mx.get("rot"), pos), eps) for g in range(G)]))
        cache["v"].append((W[p + "v"] @ h).reshape(G, Vd))
    size = (mx.get("mask") or {}).get("size")
    lo = 0 if size is None else max(0, pos - size + 1)
    keys, vals = np.array(cache["k"][lo:pos + 1]), np.array(cache["v"][lo:pos + 1])
    out = np.zeros((H, Vd))
    for a in range(H):
        g = a // (H // G)
        s = mx["scale"] * (keys[:, g] @ q[a])
        e = np.exp(s - s.max())
        out[a] = (e / e.sum()) @ vals[:, g]
    return W[p + "o"] @ (out.reshape(-1) * logistic(W[p + "g"] @ h))


def hgrn2_step(W, p, mx, h, S, eps):
    """One token through the gated linear recurrence.  S [H, D, Vd] is updated in place."""
    H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
    q = silu(W[p + "q"] @ h).reshape(H, D)
    v = (W[p + "v"] @ h).reshape(H, Vd)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * logistic(W[p + "f"] @ h + W[p + "f.b"])).reshape(H, D)
    out = np.zeros((H, Vd))
    for a in range(H):
        S[a] = f[a][:, None] * S[a] + np.outer(1.0 - f[a], v[a])
        out[a] = rms(S[a].T @ q[a], eps) * W[p + "norm"]
    return W[p + "o"] @ out.reshape(-1)


def dense_ff(W, p, x):
    return W[p + "down"] @ (gelu_tanh(W[p + "gate"] @ x) * (W[p + "up"] @ x))


def route(z, top):
    """The `top` largest logits (lower index first on ties) and the softmax over them."""
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    zs = np.array([z[e] for e in order])
    w = np.exp(zs - zs.max())
    return order, w / w.sum()


def routed_ff(W, p, fc, x):
    z = W[p + "router"] @ x + W[p + "router.b"]
    idx, wt = route(z, fc["router"]["top"])
    out = np.zeros(W[p + "e0.down"].shape[0])
    for e, w in zip(idx, wt):
        out += w * (W[f"{p}e{e}.down"] @ np.maximum(W[f"{p}e{e}.up"] @ x, 0.0) ** 2)
    return out


def token_side(W, p, x, row, eps):
    y = W[p + "proj"] @ (gelu_tanh(W[p + "gate"] @ x) * row)
    return rms(y, eps) * W[p + "norm"]


# ---- a sequence -------------------------------------------------------------------------------------------------------
class Sequence:
    def __init__(self, cfg, W):
        self.cfg, self.W, self.eps = cfg, W, cfg["norm"]["eps"]
        width = cfg["width"]
        self.prev = [np.zeros(width) for _ in cfg["layers"]]
        self.cache, self.S = [], []
        for lc in cfg["layers"]:
            mx = lc["mixer"]
            self.cache.append({"k": [], "v": []} if lc["type"] == "attention" and mx.get("kv_from") is None else None)
            self.S.append(np.zeros((mx["heads"], mx["dim"], mx["vdim"])) if lc["type"] == "hgrn2" else None)
        self.pos = 0

    def feed(self, token, layers_out=None):
        cfg, W, eps = self.cfg, self.W, self.eps
        sd = (cfg.get("token_side") or {}).get("dim", 0)
        x = W["embed"][token] * (cfg.get("embedding") or {}).get("scale", 1.0)
        for i, lc in enumerate(cfg["layers"]):
            p, mx = f"l{i}.", lc["mixer"]
            h = token_shift(x, self.prev[i], W[p + "shift"])
            self.prev[i] = x.copy()
            if lc["type"] == "attention":
                src = mx.get("kv_from")
                y = attention_step(W, p + "mix.", mx, h, self.pos, self.cache[i if src is None else src], eps, src is None)
            elif lc["type"] == "hgrn2":
                y = hgrn2_step(W, p + "mix.", mx, h, self.S[i], eps)
            else:
                raise ValueError(lc["type"])
            x = x + layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps)
            fc = lc.get("mlp")
            if fc:
                y = dense_ff(W, p + "mlp.", x) if fc["kind"] == "dense" else routed_ff(W, p + "mlp.", fc, x)
                x = x + layer_norm(y, W[p + "norm2"], W[p + "norm2.b"], eps)
            if sd:
                x = x + token_side(W, p + "side.", x, W["side.embed"][token, i * sd:(i + 1) * sd], eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        self.pos += 1
        return W["embed"] @ layer_norm(x, W["final.norm"], W["final.norm.b"], eps)


def run(cfg, W, tokens):
    """Logits [n, vocab] and residual traces [layers, n, width] of a whole sequence."""
    seq = Sequence(cfg, W)
    logits, traces = [], []
    for t in tokens:
        lo = []
        logits.append(seq.feed(int(t), lo))
        traces.append(lo)
    return np.array(logits), np.array(traces).transpose(1, 0, 2)


# ---- synthetic checkpoints ------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    Wd, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, Wd), "final.norm": (Wd,), "final.norm.b": (Wd,)}
    sd = (cfg.get("token_side") or {}).get("dim", 0)
    if sd:
        shapes["side.embed"] = (V, sd * len(cfg["layers"]))
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        shapes.update({p + "norm1": (Wd,), p + "norm1.b": (Wd,), p + "shift": (Wd,)})
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        if lc["type"] == "attention":
            G = mx.get("kv_heads", H)
            shapes.update({p + "mix.q": (H * D, Wd), p + "mix.g": (H * Vd, Wd), p + "mix.o": (Wd, H * Vd)})
            if mx.get("kv_from") is None:
                shapes.update({p + "mix.k": (G * D, Wd), p + "mix.v": (G * Vd, Wd)})
        else:
            shapes.update({p + "mix.q": (H * D, Wd), p + "mix.f": (H * D, Wd), p + "mix.f.b": (H * D,), p + "mix.lower": (H * D,),
                           p + "mix.v": (H * Vd, Wd), p + "mix.norm": (Vd,), p + "mix.o": (Wd, H * Vd)})
        fc = lc.get("mlp")
        if fc:
            shapes.update({p + "norm2": (Wd,), p + "norm2.b": (Wd,)})
            if fc["kind"] == "dense":
                shapes.update({p + "mlp.gate": (fc["ff"], Wd), p + "mlp.up": (fc["ff"], Wd), p + "mlp.down": (Wd, fc["ff"])})
            else:
                E, ff = fc["router"]["experts"], fc["expert"]["ff"]
                shapes.update({p + "mlp.router": (E, Wd), p + "mlp.router.b": (E,)})
                for e in range(E):
                    shapes.update({f"{p}mlp.e{e}.up": (ff, Wd), f"{p}mlp.e{e}.down": (Wd, ff)})
        if sd:
            shapes.update({p + "side.gate": (sd, Wd), p + "side.proj": (Wd, sd), p + "side.norm": (Wd,)})
    return shapes


def random_weights(cfg, seed=0):
    """bfloat16-representable random weights (as float64) of a size that keeps activations O(1)."""
    rng = np.random.RandomState(seed)
    W = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm"):
            a = 1.0 + 0.2 * rng.randn(*shp)
        elif leaf == "shift":
            a = rng.uniform(0.0, 1.0, shp)
        elif leaf == "lower":
            a = rng.uniform(0.0, 0.9, shp)
        elif name.endswith("f.b"):
            a = rng.uniform(-1.0, 3.0, shp)
        elif leaf == "b":
            a = 0.2 * rng.randn(*shp)
        elif name in ("embed", "side.embed"):
            a = rng.randn(*shp)
        elif leaf == "router":
            a = 2.0 * rng.randn(*shp) / math.sqrt(shp[1])
        else:
            a = 1.5 * rng.randn(*shp) / math.sqrt(shp[-1])
        W[name] = bf16_to_f64(to_bf16(np.asarray(a, dtype=np.float64))).reshape(shp)
    return W


def write(dirname, cfg, W):
    return write_checkpoint(dirname, cfg, W)


def att(heads=4, kv_heads=None, dim=8, vdim=8, size=6, scale=0.3, dims=None, base=100.0, scaling=None, kv_from=None, ff=None):
    """One attention layer of a config.  size None: plain causal attention; dims 0: no rotation; ff: None, an int (dense) or
    (experts, top, hidden)."""
    mx = {"heads": heads, "kv_heads": kv_heads or heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        mx["mask"] = {"size": size}
    dims = dim if dims is None else dims
    if dims:
        mx["rot"] = {"dims": dims, "base": base}
        if scaling:
            mx["rot"]["scaling"] = scaling
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": ff_config(ff)}


def rec(heads=2, dim=8, vdim=8, ff=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": ff_config(ff)}


def ff_config(ff):
    if ff is None:
        return None
    if isinstance(ff, int):
        return {"kind": "dense", "ff": ff}
    return {"kind": "moe", "router": {"experts": ff[0], "top": ff[1]}, "expert": {"ff": ff[2]}}


def model_config(layers, width=40, vocab=53, eps=1e-5, emb_scale=1.5, side=6):
    cfg = {"architecture": "Nalizen", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}, "embedding": {"scale": emb_scale}}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def small_config():
    """A small model with every mechanism; sizes deliberately unequal from layer to layer and mostly not powers of two."""
    sc = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 40}
    layers = [att(heads=6, kv_heads=2, dim=10, vdim=6, size=7, scale=0.6, dims=6, base=50.0, scaling=sc, ff=28),
              rec(heads=3, dim=5, vdim=7, ff=(5, 2, 12)),
              att(heads=6, kv_heads=2, dim=10, vdim=6, size=4, scale=0.9, dims=6, base=50.0, scaling=sc, kv_from=0, ff=(7, 3, 10)),
              rec(heads=2, dim=12, vdim=4, ff=None),
              att(heads=2, kv_heads=1, dim=12, vdim=14, size=11, scale=0.4, dims=12, base=10000.0, ff=(3, 1, 16))]
    return model_config(layers, width=44, vocab=61, side=5)
