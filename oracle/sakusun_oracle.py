"""sakusun_oracle.py — plain, slow float64 statement of the Sakusun design (a layer-list model), for tests only.

One function per mechanism, written from the equations with numpy, token by token, and sharing no code with the CUDA path.
`Sequence.feed` carries what a sequence carries: the previous token, per layer the last taps - 1 inputs of both input
convolutions, and per attention layer everything it caches (keys and values, or latents and shared rotated keys).

Notation: W x for a stored [out, in] matrix; rms(v) = v / sqrt(mean(v^2) + eps); sg = logistic function.

  embedding:  x = s E[token] + Bg[(m_p prev + m_c token) mod n_b]   (row n_b of Bg for the first token of a sequence)
  layer:      for each sublayer f in (mixer, feed-forward), reading the stream x itself:
                u = x + conv(x);  y = f(u) * sg(W_r x + b_r);  x <- x + g rms(y) * ls       (g one number, ls a vector)
              conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros before the sequence starts
  attention:  q = rms(W_q u + b_q) * w_q over all heads' rows at once, k likewise, v = W_v u + b_v;
              in the 2nd, 3rd, .. layer that mixes values: v <- (1 - lam) v + lam v_first (v_first: the first such layer's v of this token);
              s_j = cap * tanh(scale (q_h . k_j[h // (H/G)]) / cap) + rel[bucket(i - j), h];
              j visible: j <= i and (i - j < size or j < keep_first);
              p_j = e^(s_j) / (sum_visible e^(s) + e^(sink_h));  o_h = sum_j p_j v_j[h // (H/G)];  W_o concat(o)
              bucket(n) = n for n < B//2, else min(B - 1, B//2 + floor(ln(n / (B//2)) / ln(D / (B//2)) * (B - B//2)))
  latent attention:  c_q = rms(W_dq u) * w_dq;  q = W_uq c_q, per head [dim plain | rot_dim rotated];
              [c | kr] = W_dkv u with c <- rms(c) * w_dkv, kr one rotated key part for all heads;
              s_j = scale (q_plain . W_uk[h] c_j + rot(q_rot, i) . rot(kr_j, j)) over all j <= i;  softmax;  o_h = sum_j p_j W_uv[h] c_j;
              W_o (concat(o) * sg(W_g u));  rot turns the pairs (2i, 2i + 1) of the first rot.dims entries by pos * base^(-2i/dims)
  ff:         W_down (gelu_tanh(W_gate u) * (W_up u))
  output:     logits = Hd (g_final rms(x))
"""
import math

import numpy as np

from hybrid_oracle import bf16_to_f64, to_bf16, write_checkpoint  # noqa: F401  (checkpoint minting helpers)


# ---- mechanisms -------------------------------------------------------------------------------------------------------
def rms(v, eps):
    v = np.asarray(v, dtype=np.float64)
    return v / math.sqrt(float(np.mean(v * v)) + eps)


def logistic(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, dtype=np.float64)))


def gelu_tanh(z):
    z = np.asarray(z, dtype=np.float64)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def embedding(W, emb, prev, token):
    bg = emb["bigram"]
    row = bg["buckets"] if prev is None else (prev * bg["mul_prev"] + token * bg["mul_cur"]) % bg["buckets"]
    return W["embed"][token] * emb["scale"] + W["bigram"][row]


def input_conv(w, past, x):
    """x + conv(x): w [width, taps]; past: the taps - 1 earlier inputs, oldest first (zeros before the sequence)."""
    taps = w.shape[1]
    seq = list(past) + [x]
    out = np.array(x, dtype=np.float64)
    for j in range(taps):
        out = out + w[:, j] * seq[j]
    return out


def rel_bucket(n, B, D):
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def sees(mask, i, j):
    if j > i:
        return False
    if not mask or "size" not in mask:
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


def attention_step(W, p, mx, u, pos, cache, eps, v_first, mixes):
    """One token through the attention mixer.  cache: {"k": [...], "v": [...]} over all earlier positions, appended here.
    v_first: this token's values in the first value-mixing layer (None there and in layers that do not mix); mixes: this
    layer blends them in.  Returns (mixer output, the values this layer cached)."""
    H, G, D, Vd = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    q = rms(W[p + "q"] @ u + W[p + "q.b"], eps) * W[p + "q.norm"]
    k = rms(W[p + "k"] @ u + W[p + "k.b"], eps) * W[p + "k.norm"]
    v = W[p + "v"] @ u + W[p + "v.b"]
    if mixes:
        lam = float(W[p + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    cache["k"].append(k.reshape(G, D))
    cache["v"].append(v.reshape(G, Vd))
    q = q.reshape(H, D)
    js = [j for j in range(pos + 1) if sees(mx.get("mask"), pos, j)]
    out = np.zeros((H, Vd))
    cap = mx.get("softcap")
    keys, vals = np.array([cache["k"][j] for j in js]), np.array([cache["v"][j] for j in js])      # [visible, G, .]
    for h in range(H):
        g = h // (H // G)
        s = mx["scale"] * (keys[:, g] @ q[h])
        if cap:
            s = cap * np.tanh(s / cap)
        if "bias_max" in mx:
            rel = W[p + "rel"]
            s = s + np.array([rel[rel_bucket(pos - j, rel.shape[0], mx["bias_max"]), h] for j in js])
        sink = float(W[p + "sink"][h])
        m = max(float(s.max()), sink)
        e = np.exp(s - m)
        pr = e / (e.sum() + math.exp(sink - m))
        out[h] = pr @ vals[:, g]
    return W[p + "o"] @ out.reshape(-1), v


def rotate(v, rot, pos):
    """Pairs (2i, 2i + 1) of the first rot["dims"] entries of v turn by pos * base^(-2i/dims)."""
    out = np.array(v, dtype=np.float64)
    dims = rot["dims"]
    for i in range(dims // 2):
        a = pos * rot["base"] ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        a0, a1 = out[2 * i], out[2 * i + 1]
        out[2 * i], out[2 * i + 1] = a0 * c - a1 * s, a1 * c + a0 * s
    return out


def latent_attention_step(W, p, mx, u, pos, cache, eps):
    """One token through the latent-attention mixer.  cache: {"c": [...], "kr": [...]} (latents and rotated shared key parts)."""
    H, D, Rd, Vd, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    cq = rms(W[p + "dq"] @ u, eps) * W[p + "dq.norm"]
    q = (W[p + "uq"] @ cq).reshape(H, D + Rd)
    dkv = W[p + "dkv"] @ u
    cache["c"].append(rms(dkv[:R], eps) * W[p + "dkv.norm"])
    cache["kr"].append(rotate(dkv[R:], mx["rot"], pos))
    uk, uv = W[p + "uk"].reshape(H, D, R), W[p + "uv"].reshape(H, Vd, R)
    out = np.zeros((H, Vd))
    lat, kr = np.array(cache["c"]), np.array(cache["kr"])               # [pos + 1, R], [pos + 1, Rd]
    for h in range(H):
        qr = rotate(q[h, D:], mx["rot"], pos)
        s = mx["scale"] * ((lat @ uk[h].T) @ q[h, :D] + kr @ qr)           # plain keys of head h: uk[h] c_j
        e = np.exp(s - s.max())
        out[h] = (e / e.sum()) @ (lat @ uv[h].T)
    return W[p + "o"] @ (out.reshape(-1) * logistic(W[p + "g"] @ u))


def glu_ff(W, p, u):
    return W[p + "down"] @ (gelu_tanh(W[p + "gate"] @ u) * (W[p + "up"] @ u))


def close_sublayer(W, p, n, x, y, eps):
    """x + g rms(y sg(W_r x + b_r)) * ls for sublayer n (1: mixer, 2: feed-forward)."""
    y = y * logistic(W[f"{p}rg{n}"] @ x + W[f"{p}rg{n}.b"])
    return x + float(W[f"{p}norm{n}"]) * rms(y, eps) * W[f"{p}ls{n}"]


def first_mixing_layer(cfg):
    for i, lc in enumerate(cfg["layers"]):
        if lc["type"] == "attention" and lc["mixer"].get("v_mix"):
            return i
    return -1


# ---- a sequence -------------------------------------------------------------------------------------------------------
class Sequence:
    def __init__(self, cfg, W):
        self.cfg, self.W, self.eps = cfg, W, cfg["norm"]["eps"]
        n, taps, width = len(cfg["layers"]), cfg["canon"]["taps"], cfg["width"]
        self.past = [[[np.zeros(width) for _ in range(taps - 1)] for _ in range(2)] for _ in range(n)]
        self.cache = [{"k": [], "v": []} if lc["type"] == "attention" else {"c": [], "kr": []} for lc in cfg["layers"]]
        self.prev, self.pos = None, 0

    def feed(self, token, layers_out=None):
        cfg, W, eps = self.cfg, self.W, self.eps
        x = embedding(W, cfg["embedding"], self.prev, token)
        first, v_first = first_mixing_layer(cfg), None
        for i, lc in enumerate(cfg["layers"]):
            p, mx = f"l{i}.", lc["mixer"]
            u = input_conv(W[p + "canon1"], self.past[i][0], x)
            self.past[i][0] = (self.past[i][0] + [x])[1:]
            if lc["type"] == "attention":
                mixes = bool(mx.get("v_mix")) and i != first
                y, v = attention_step(W, p + "mix.", mx, u, self.pos, self.cache[i], eps, v_first, mixes)
                if i == first:
                    v_first = v
            elif lc["type"] == "latent_attention":
                y = latent_attention_step(W, p + "mix.", mx, u, self.pos, self.cache[i], eps)
            else:
                raise ValueError(lc["type"])
            x = close_sublayer(W, p, 1, x, y, eps)
            if lc.get("mlp"):
                u = input_conv(W[p + "canon2"], self.past[i][1], x)
                self.past[i][1] = (self.past[i][1] + [x])[1:]
                x = close_sublayer(W, p, 2, x, glu_ff(W, p + "mlp.", u), eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        self.prev, self.pos = token, self.pos + 1
        return W["head"] @ (float(W["final.norm"]) * rms(x, eps))


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
    Wd, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    shapes = {"embed": (V, Wd), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, Wd), "final.norm": (), "head": (V, Wd)}
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        shapes.update({p + "norm1": (), p + "ls1": (Wd,), p + "canon1": (Wd, taps), p + "rg1": (Wd, Wd), p + "rg1.b": (Wd,)})
        if lc["type"] == "attention":
            H, G, D, Vd = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
            shapes.update({p + "mix.q": (H * D, Wd), p + "mix.q.b": (H * D,), p + "mix.k": (G * D, Wd), p + "mix.k.b": (G * D,),
                           p + "mix.v": (G * Vd, Wd), p + "mix.v.b": (G * Vd,), p + "mix.q.norm": (H * D,), p + "mix.k.norm": (G * D,),
                           p + "mix.sink": (H,), p + "mix.o": (Wd, H * Vd)})
            if "bias_max" in mx:
                shapes[p + "mix.rel"] = (mx["rel_rows"], H)
            if mx.get("v_mix"):
                shapes[p + "mix.vmix"] = ()
        else:
            H, D, Rd, Vd, R, Q = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            shapes.update({p + "mix.dq": (Q, Wd), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (D + Rd), Q), p + "mix.dkv": (R + Rd, Wd),
                           p + "mix.dkv.norm": (R,), p + "mix.uk": (H * D, R), p + "mix.uv": (H * Vd, R), p + "mix.g": (H * Vd, Wd),
                           p + "mix.o": (Wd, H * Vd)})
        if lc.get("mlp"):
            ff = lc["mlp"]["ff"]
            shapes.update({p + "norm2": (), p + "ls2": (Wd,), p + "canon2": (Wd, taps), p + "rg2": (Wd, Wd), p + "rg2.b": (Wd,),
                           p + "mlp.gate": (ff, Wd), p + "mlp.up": (ff, Wd), p + "mlp.down": (Wd, ff)})
    return shapes


def random_weights(cfg, seed=0):
    """bfloat16-representable random weights (as float64)."""
    rng = np.random.RandomState(seed)
    W = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2"):
            a = np.array(0.8 + 0.4 * rng.rand())
        elif name == "final.norm":
            a = np.array(1.0 + 0.5 * rng.rand())
        elif leaf == "norm":
            a = 1.0 + 0.2 * rng.randn(*shp)
        elif leaf in ("ls1", "ls2"):
            a = 0.7 + 0.3 * rng.randn(*shp)
        elif leaf in ("canon1", "canon2"):
            a = 0.4 * rng.randn(*shp)
        elif leaf == "b":
            a = 0.3 * rng.randn(*shp)
        elif leaf == "rel":
            a = 0.8 * rng.randn(*shp)
        elif leaf == "sink":
            a = 0.5 + rng.randn(*shp)
        elif leaf == "vmix":
            a = np.array(0.2 + 0.5 * rng.rand())
        elif name in ("embed", "bigram"):
            a = rng.randn(*shp)
        else:
            a = 1.5 * rng.randn(*shp) / math.sqrt(shp[-1])
        W[name] = bf16_to_f64(to_bf16(np.asarray(a, dtype=np.float64))).reshape(shp)
    return W


def write(dirname, cfg, W):
    return write_checkpoint(dirname, public_config(cfg), W)


def public_config(cfg):
    """The config.json form: without the helper key that only sizes the test's distance table."""
    out = dict(cfg)
    out["layers"] = []
    for lc in cfg["layers"]:
        lc = dict(lc)
        lc["mixer"] = {k: v for k, v in lc["mixer"].items() if k != "rel_rows"}
        out["layers"].append(lc)
    return out


def att(heads=3, kv_heads=None, dim=8, vdim=8, size=6, keep_first=2, scale=0.3, softcap=20.0, bias_max=24, rel_rows=8, v_mix=True, ff=None):
    """One attention layer of a config; None for size / softcap / bias_max leaves that key out (plain causal / no cap / no bias)."""
    mx = {"heads": heads, "kv_heads": kv_heads or heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if size is not None:
        mx["mask"] = {"size": size, "keep_first": keep_first}
    if softcap is not None:
        mx["softcap"] = softcap
    if bias_max is not None:
        mx.update(bias_max=bias_max, rel_rows=rel_rows)
    return {"type": "attention", "mixer": mx, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def lat(heads=3, dim=8, rot_dim=4, vdim=8, kv_rank=12, q_rank=10, scale=0.3, base=100.0, dims=None, ff=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
          "rot": {"dims": rot_dim if dims is None else dims, "base": base}}
    return {"type": "latent_attention", "mixer": mx, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model_config(layers, width=40, vocab=53, taps=3, eps=1e-5, emb_scale=0.75, buckets=37, mul_prev=5, mul_cur=3):
    return {"architecture": "Sakusun", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}, "canon": {"taps": taps},
            "embedding": {"scale": emb_scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}


def small_config():
    """A small model with every mechanism; sizes deliberately unequal from layer to layer and mostly not powers of two."""
    layers = [att(heads=6, kv_heads=2, dim=10, vdim=6, size=7, keep_first=3, scale=0.3, softcap=15.0, bias_max=20, rel_rows=10, ff=28),
              lat(heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=14, q_rank=9, scale=0.25, base=500.0, ff=None),
              att(heads=4, kv_heads=1, dim=6, vdim=12, size=5, keep_first=0, scale=0.4, softcap=8.0, bias_max=9, rel_rows=6, ff=20),
              lat(heads=2, dim=5, rot_dim=8, vdim=7, kv_rank=20, q_rank=16, scale=0.2, base=10000.0, ff=36),
              att(heads=2, kv_heads=2, dim=16, vdim=6, size=11, keep_first=1, scale=0.2, softcap=30.0, bias_max=64, rel_rows=16, v_mix=False, ff=24)]
    return model_config(layers, width=44, vocab=61, taps=4)
