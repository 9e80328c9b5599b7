"""Plain numpy (float64) statement of the Zasorax architecture, one function per mechanism: the yardstick the GPU kernels
and the engine are tested against.  It shares no code with the product path: no paging, no packing of projections, no
expanded bias tables, no grouping of tokens by expert.  Every sequence is walked token by token and every attention
mixer keeps an explicit list of what it caches.

Notation: W x for a weight stored [out, in]; positions start at 0 in every sequence; rms(v) = v / sqrt(mean(v^2) + eps).
  embedding:   x = E[tok] * scale
  layer:       x <- x + rms(mixer(x)) w1;  x <- x + rms(ff(x)) w2     (post-norm only: the sublayers read x itself; the
               second half may be absent)
  attention:   q = rms(Wq x) wq and k = rms(Wk x) wk over the WHOLE projection (all heads at once), v = Wv x, no rotation;
               s_ij = q_i.k_j * scale * temp_h + rel[bucket(i - j), h] for the j <= i of i's chunk (floor(i / size) ==
               floor(j / size), chunks counted from position 0); softmax whose denominator also holds exp(sink_h); Wo.
               bucket(n) = n below half = B / 2, else min(B - 1, half + floor(ln(n / half) / ln(D / half) * (B - half))),
               B = rows of rel, D = bias_max.  A layer with kv_from = j caches nothing and reads the keys and values that
               layer j cached, with its own queries, bias table, temperatures and sinks.
  attention_2: q, k, v = Wq x, Wk x, Wv x; rotary on the first rot.dims values of every q and k head (value i paired with
               i + dims / 2, angle pos * base^(-2i / dims)), then each head divided by its root mean square; the value of
               position j turned by j over all of vdim (pair m with m + vdim / 2, angle j * base^(-2m / vdim)) and cached
               so; s = q.k * scale, causal; p_j = exp(s_j) / (1 + sum_j exp(s_j)); the head's output turned back by -i;
               times sigmoid(Wg x)_head; Wo
  ff dense:    Wd act(Wu x), act(z) = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 else
  ff experts:  z = Wr x + b; the `top` largest z (ties: lowest index) with weights softmax over those alone;
               sum_k w_k Wd_k (silu(Wg_k x) * (Wu_k x))
  output:      logits = Whead (rms(x) w_final)
"""
import math

import numpy as np


def bf16_round(a):
    """Nearest-even rounding of float values to bfloat16, returned as float64."""
    u = np.asarray(a, np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32).astype(np.float64)


def to_bf16_bits(a):
    """bf16-representable float values -> uint16 bit patterns."""
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


# ---- configuration / weights --------------------------------------------------------------------------------------------
def chunk_mixer(heads=4, kv_heads=2, dim=6, vdim=5, chunk=7, scale=0.4, bias_max=20, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "scale": scale, "bias_max": bias_max}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def rotary_mixer(heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4, rot_base=100.0, scale=0.35):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": rot_base, "dims": rot_dims}, "scale": scale}


def dense_mlp(ff=24):
    return {"kind": "dense", "ff": ff}


def expert_mlp(ff=8, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(layers, vocab=80, width=24, eps=1e-5, embed_scale=2.0):
    """layers: list of (type, mixer dict, mlp dict or None)."""
    return {"architecture": "Zasorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}


def tensor_shapes(cfg, rel_rows=8):
    """rel_rows: rows of the distance-bias tables (the tensors decide; an int, or a dict layer -> rows)."""
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    for i, l in enumerate(cfg["layers"]):
        p, m, q = "l%d." % i, l["mixer"], "l%d.mix." % i
        out[p + "norm1"] = (W,)
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[q + "q"] = (H * D, W)
        if "kv_from" not in m:
            out[q + "k"], out[q + "v"] = (G * D, W), (G * V, W)
        if l["type"] == "attention":
            out[q + "q.norm"] = (H * D,)
            if "kv_from" not in m:
                out[q + "k.norm"] = (G * D,)
            out[q + "rel"] = (rel_rows[i] if isinstance(rel_rows, dict) else rel_rows, H)
            out[q + "temp"] = out[q + "sink"] = (H,)
        elif l["type"] == "attention_2":
            out[q + "g"] = (H, W)
        else:
            raise ValueError(l["type"])
        out[q + "o"] = (W, H * V)
        f = l["mlp"]
        if f is not None:
            out[p + "norm2"] = (W,)
            if f["kind"] == "dense":
                out[p + "mlp.up"], out[p + "mlp.down"], out[p + "mlp.act"] = (f["ff"], W), (W, f["ff"]), (2,)
            else:
                E, ff = f["router"]["experts"], f["expert"]["ff"]
                out[p + "mlp.router"], out[p + "mlp.router.b"] = (E, W), (E,)
                for e in range(E):
                    out[p + "mlp.e%d.gate" % e] = out[p + "mlp.e%d.up" % e] = (ff, W)
                    out[p + "mlp.e%d.down" % e] = (W, ff)
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg, rng, std=None, rel_rows=8):
    """bf16-representable float64 arrays."""
    W, out = cfg["width"], {}
    for name, shape in tensor_shapes(cfg, rel_rows).items():
        fan_in = shape[-1] if len(shape) == 2 else W
        s = std if std is not None else 1.0 / np.sqrt(fan_in)
        last = name.split(".")[-1]
        if "norm" in last:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "temp":
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last in ("sink", "rel", "act"):
            a = rng.standard_normal(shape)
        elif last == "b":
            a = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            a = 0.5 * rng.standard_normal(shape)
        else:
            a = s * rng.standard_normal(shape)
        out[name] = bf16_round(a)
    return out


# ---- mechanisms --------------------------------------------------------------------------------------------------------
def rms(v, eps):
    v = np.asarray(v, np.float64)
    return v / np.sqrt(np.mean(v * v) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, np.float64)))


def softplus(z):
    return np.logaddexp(0.0, np.asarray(z, np.float64))


def distance_bucket(n, rows, far):
    """Row of a distance-bias table with `rows` rows for the distance n >= 0: one row per distance below half the table,
    logarithmic steps up to the distance `far` above."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def rotate_halves(x, pos, dims, base):
    """Rotary positions on the first `dims` values of x: value i is paired with i + dims / 2."""
    y = np.array(x, np.float64)
    hf = dims // 2
    for i in range(hf):
        a = pos * float(base) ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        u, v = x[i], x[i + hf]
        y[i], y[i + hf] = u * c - v * s, v * c + u * s
    return y


def sink_softmax(scores, sink):
    """Weights of a softmax whose denominator also holds exp(sink); the sink has no value."""
    s = np.asarray(scores, np.float64)
    mx = max(float(np.max(s)), float(sink))
    e = np.exp(s - mx)
    return e / (np.sum(e) + math.exp(sink - mx))


def xielu(z, p, q):
    z = np.asarray(z, np.float64)
    neg = np.minimum(z, 0.0)
    return np.where(z > 0, softplus(p) * z * z + z / 2, (0.5 + softplus(q)) * (np.expm1(neg) - neg) + z / 2)


def dense_ff(w, p, x):
    a = w[p + "mlp.act"]
    return w[p + "mlp.down"] @ xielu(w[p + "mlp.up"] @ x, a[0], a[1])


def route(z, top):
    """The `top` largest entries of z (ties: lowest index) and the softmax over those entries alone."""
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    e = np.exp(np.array([z[i] for i in order]) - z[order[0]])
    return order, e / np.sum(e)


def expert_ff(w, p, f, x):
    z = w[p + "mlp.router"] @ x + w[p + "mlp.router.b"]
    chosen, wts = route(z, f["router"]["top"])
    y = np.zeros(len(x))
    for e, g in zip(chosen, wts):
        a = w[p + "mlp.e%d.gate" % e] @ x
        y += g * (w[p + "mlp.e%d.down" % e] @ (a * sigmoid(a) * (w[p + "mlp.e%d.up" % e] @ x)))
    return y


class KeyValueList:
    """What an attention layer caches for one sequence: one (keys, values) pair of [kv_heads, *] arrays per position."""

    def __init__(self):
        self.k, self.v = [], []


def chunk_attention_step(w, q_, m, eps, st, x, pos, own_kv):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (rms(w[q_ + "q"] @ x, eps) * w[q_ + "q.norm"]).reshape(H, D)
    if own_kv:
        st.k.append((rms(w[q_ + "k"] @ x, eps) * w[q_ + "k.norm"]).reshape(G, D))
        st.v.append((w[q_ + "v"] @ x).reshape(G, V))
    rel, size = w[q_ + "rel"], m.get("mask", {}).get("size", 0)
    first = pos // size * size if size else 0          # no chunk size: plain causal
    out = np.zeros((H, V))
    for h in range(H):
        g = h // (H // G)
        s = [float(q[h] @ st.k[j][g]) * m["scale"] * w[q_ + "temp"][h] + rel[distance_bucket(pos - j, rel.shape[0], m["bias_max"]), h]
             for j in range(first, pos + 1)]
        pr = sink_softmax(s, w[q_ + "sink"][h])
        for n, j in enumerate(range(first, pos + 1)):
            out[h] += pr[n] * st.v[j][g]
    return w[q_ + "o"] @ out.reshape(-1)


def rotary_attention_step(w, q_, m, eps, st, x, pos):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    q = (w[q_ + "q"] @ x).reshape(H, D)
    k = (w[q_ + "k"] @ x).reshape(G, D)
    v = (w[q_ + "v"] @ x).reshape(G, V)
    q = np.stack([rms(rotate_halves(q[h], pos, dims, base), eps) for h in range(H)])
    st.k.append(np.stack([rms(rotate_halves(k[g], pos, dims, base), eps) for g in range(G)]))
    st.v.append(np.stack([rotate_halves(v[g], pos, V, base) for g in range(G)]))
    gate = sigmoid(w[q_ + "g"] @ x)
    out = np.zeros((H, V))
    for h in range(H):
        g = h // (H // G)
        pr = sink_softmax([float(q[h] @ st.k[j][g]) * m["scale"] for j in range(pos + 1)], 0.0)
        o = np.zeros(V)
        for j in range(pos + 1):
            o += pr[j] * st.v[j][g]
        out[h] = rotate_halves(o, -pos, V, base) * gate[h]
    return w[q_ + "o"] @ out.reshape(-1)


class Sequence:
    """Everything one sequence carries from token to token."""

    def __init__(self, cfg):
        self.pos, self.layers = 0, []
        for l in cfg["layers"]:
            m = l["mixer"]
            self.layers.append(self.layers[m["kv_from"]] if "kv_from" in m else KeyValueList())


def token_step(cfg, w, seq, tok, taps=None):
    """Runs one token; returns the logits.  taps (a list): receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][tok] * cfg["embedding"]["scale"]
    for i, l in enumerate(cfg["layers"]):
        p, q_, m = "l%d." % i, "l%d.mix." % i, l["mixer"]
        if l["type"] == "attention":
            y = chunk_attention_step(w, q_, m, eps, seq.layers[i], x, seq.pos, "kv_from" not in m)
        else:
            y = rotary_attention_step(w, q_, m, eps, seq.layers[i], x, seq.pos)
        x = x + rms(y, eps) * w[p + "norm1"]
        f = l["mlp"]
        if f is not None:
            y = dense_ff(w, p, x) if f["kind"] == "dense" else expert_ff(w, p, f, x)
            x = x + rms(y, eps) * w[p + "norm2"]
        if taps is not None:
            taps.append(x.copy())
    seq.pos += 1
    return w["head"] @ (rms(x, eps) * w["final.norm"])


def run_sequence(cfg, w, tokens, want=None, layer_taps=False):
    """Logits [len(want), vocab] of one sequence walked token by token (want: positions, default all)."""
    seq = Sequence(cfg)
    want = range(len(tokens)) if want is None else want
    wanted, out, taps_all = set(want), {}, []
    for t, tok in enumerate(tokens):
        taps = [] if layer_taps else None
        lg = token_step(cfg, w, seq, int(tok), taps)
        if t in wanted:
            out[t] = lg
        if layer_taps:
            taps_all.append(np.stack(taps))
    logits = np.stack([out[t] for t in want]) if len(out) else np.zeros((0, cfg["vocab"]))
    if layer_taps:
        return logits, np.stack(taps_all, axis=1)          # [layers, tokens, width]
    return logits
