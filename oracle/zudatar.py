"""Plain numpy (float64) statement of the Zudatar architecture, one function per mechanism: the yardstick the GPU kernels
and the engine are tested against.  It shares no code with the product path: no paging, no state slots, no packing of
projections, no folding of the latent maps into the queries.  Every sequence is walked token by token; the attention
mixers keep an explicit list of what they cache, the recurrent mixer keeps its state matrices as arrays.

Notation: W x for a weight stored [out, in]; positions start at 0 in every sequence; rms(v) = v / sqrt(mean(v^2) + eps).
  embedding:  x = E[tok] * scale + B[(prev * mul_prev + tok * mul_cur) mod buckets]; the first token reads row `buckets`
  layer:      x <- x + rms(mixer(rms(x) w1)) w1b;  x <- x + rms(ff(rms(x) w2)) w2b     (the second half may be absent)
  attention:  q = Wq h + bq, k = Wk h + bk, v = k (as projected); rotary on pairs (2i, 2i+1) of the first rot dims of q and k,
              then q and k divided by their root mean square per head; s = q.k * scale over the last `window` positions;
              softmax; head output * sigmoid(Wg h)_head; Wo
  latent:     cq = rms(Wdq h) wq, q = Wuq cq;  c = rms(Wdkv h) wc (the cached latent, or another layer's);  k_h = Uk_h c,
              v_h = Uv_h c;  s = q.k * scale over the last `window` positions;  softmax whose denominator also holds
              exp(sink_h);  head output * sigmoid(Wg h)_head;  Wo
  delta:      q, k, v = silu(causal conv over the last `taps` tokens of Wq h, Wk h, Wv h);  q, k <- unit vectors per head
              (x / sqrt(sum x^2 + 1e-6)), q *= dim^-1/2;  beta = sigmoid(Wb h);  g = exp(-exp(A_log_h) softplus(Wa2 Wa1 h + dt_bias))
              per head and key channel;  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
              Wo (concat_h rms(o_h) w * sigmoid(Wg2 Wg1 h)_h)
  ff dense:   Wd (silu(Wg h) * (Wu h))
  output:     logits = E (rms(x) w_final) * logit_scale                                  (the embedding table, unscaled)
"""
import numpy as np


def bf16_round(a):
    """Nearest-even rounding of float values to bfloat16, returned as float64."""
    u = np.asarray(a, np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32).astype(np.float64)


def to_bf16_bits(a):
    """bf16-representable float values -> uint16 bit patterns (integer arrays pass as int32)."""
    a = np.asarray(a)
    if a.dtype.kind in "iu":
        return a.astype(np.int32)
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


# ---- configuration / weights --------------------------------------------------------------------------------------------
def attention_mixer(heads=4, kv_heads=2, dim=8, window=7, rot_dims=4, rot_base=100.0, scale=0.4):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window},
            "rot": {"base": rot_base, "dims": rot_dims}, "scale": scale}


def latent_mixer(heads=3, dim=6, vdim=10, kv_rank=12, q_rank=9, window=5, scale=0.35, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": window}, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def delta_mixer(heads=4, kv_heads=2, dim=6, vdim=5, taps=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}


def dense_mlp(ff=24):
    return {"kind": "dense", "ff": ff}


def make_config(layers, vocab=80, width=24, eps=1e-5, embed_scale=2.0, buckets=37, mul_prev=13, mul_cur=5, logit_scale=0.8):
    """layers: list of (type, mixer dict, mlp dict or None)."""
    return {"architecture": "Zudatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "embedding": {"scale": embed_scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}


def low_rank(m, W):
    """Inner size of the two-step projections of the delta mixer (decay and gate); any value works, the tensors decide."""
    return m.get("low_rank", max(1, W // 8))


def tensor_shapes(cfg, low=None):
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    for i, l in enumerate(cfg["layers"]):
        p, m, q = "l%d." % i, l["mixer"], "l%d.mix." % i
        out[p + "norm1"] = out[p + "norm1b"] = (W,)
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if l["type"] == "attention":
            G = m["kv_heads"]
            out[q + "q"], out[q + "q.b"] = (H * D, W), (H * D,)
            out[q + "k"], out[q + "k.b"] = (G * D, W), (G * D,)
            out[q + "g"] = (H, W)
            out[q + "o"] = (W, H * V)
        elif l["type"] == "latent_attention":
            out[q + "dq"], out[q + "dq.norm"] = (m["q_rank"], W), (m["q_rank"],)
            out[q + "uq"] = (H * D, m["q_rank"])
            if "kv_from" not in m:
                out[q + "dkv"], out[q + "dkv.norm"] = (m["kv_rank"], W), (m["kv_rank"],)
            out[q + "uk"] = (H * D, m["kv_rank"])
            out[q + "uv"] = (H * V, m["kv_rank"])
            out[q + "sink"] = (H,)
            out[q + "g"] = (H, W)
            out[q + "o"] = (W, H * V)
        elif l["type"] == "channel_delta":
            G, r = m["kv_heads"], (low if low is not None else low_rank(m, W))
            out[q + "q"] = out[q + "k"] = (G * D, W)
            out[q + "q.conv"] = out[q + "k.conv"] = (G * D, m["conv"])
            out[q + "v"], out[q + "v.conv"] = (H * V, W), (H * V, m["conv"])
            out[q + "b"] = (H, W)
            out[q + "A_log"] = (H,)
            out[q + "norm"] = (V,)
            out[q + "a1"], out[q + "a2"], out[q + "dt_bias"] = (r, W), (H * D, r), (H * D,)
            out[q + "g1"], out[q + "g2"] = (r, W), (H * V, r)
            out[q + "o"] = (W, H * V)
        else:
            raise ValueError(l["type"])
        f = l["mlp"]
        if f is not None:
            out[p + "norm2"] = out[p + "norm2b"] = (W,)
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (f["ff"], W)
            out[p + "mlp.down"] = (W, f["ff"])
    out["final.norm"] = (W,)
    return out


def random_weights(cfg, rng, std=None, low=None):
    """bf16-representable float64 arrays."""
    W, out = cfg["width"], {}
    for name, shape in tensor_shapes(cfg, low).items():
        fan_in = shape[-1] if len(shape) == 2 else W
        s = std if std is not None else 1.0 / np.sqrt(fan_in)
        last = name.split(".")[-1]
        if "norm" in last:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "b" and len(shape) == 1:
            a = 0.3 * rng.standard_normal(shape)
        elif last == "conv":
            a = 0.5 * rng.standard_normal(shape)
        elif last == "A_log":
            a = -1.0 + 0.7 * rng.standard_normal(shape)
        elif last == "dt_bias":
            a = -0.5 + rng.standard_normal(shape)
        elif last == "sink":
            a = rng.standard_normal(shape)
        elif name in ("embed", "bigram"):
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
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def bigram_row(prev, tok, bg):
    """Row of the bigram table for `tok` after `prev` (None: the sequence's first token)."""
    if prev is None:
        return bg["buckets"]
    return (prev * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"]


def embed(w, cfg, prev, tok):
    e = cfg["embedding"]
    return w["embed"][tok] * e["scale"] + w["bigram"][bigram_row(prev, tok, e["bigram"])]


def rotate_pairs(x, pos, dims, base):
    """Pairs (2i, 2i+1) of the first `dims` values turn by pos * base^(-2i/dims); the rest passes."""
    y = np.array(x, np.float64)
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        u, v = x[2 * i], x[2 * i + 1]
        y[2 * i] = u * np.cos(a) - v * np.sin(a)
        y[2 * i + 1] = v * np.cos(a) + u * np.sin(a)
    return y


def window_softmax(scores, sink=None):
    """Softmax over the given scores; `sink` adds exp(sink) to the denominator only."""
    s = np.asarray(scores, np.float64)
    m = s.max() if sink is None else max(s.max(), sink)
    e = np.exp(s - m)
    den = e.sum() + (0.0 if sink is None else np.exp(sink - m))
    return e / den


def dense_ff(w, p, h):
    return w[p + "mlp.down"] @ (silu(w[p + "mlp.gate"] @ h) * (w[p + "mlp.up"] @ h))


class AttentionState:
    """What the attention mixer keeps per sequence: the prepared keys and the values of every position."""

    def __init__(self):
        self.k, self.v = [], []


def attention_step(w, q_, m, eps, st, h, pos):
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    dims, base = m.get("rot", {}).get("dims", 0), m.get("rot", {}).get("base", 10000.0)
    q = (w[q_ + "q"] @ h + w[q_ + "q.b"]).reshape(H, D)
    k = (w[q_ + "k"] @ h + w[q_ + "k.b"]).reshape(G, D)
    st.v.append(k.copy())                                  # the values are the keys as projected
    st.k.append(np.stack([rms(rotate_pairs(k[g], pos, dims, base), eps) for g in range(G)]))
    gate = sigmoid(w[q_ + "g"] @ h)
    lo = max(0, pos - m["mask"]["size"] + 1)
    out = np.zeros((H, D))
    for hh in range(H):
        g = hh // (H // G)
        qh = rms(rotate_pairs(q[hh], pos, dims, base), eps)
        s = np.array([qh @ st.k[j][g] for j in range(lo, pos + 1)]) * m["scale"]
        p = window_softmax(s)
        out[hh] = sum(p[j - lo] * st.v[j][g] for j in range(lo, pos + 1)) * gate[hh]
    return w[q_ + "o"] @ out.reshape(-1)


class LatentState:
    """The cached latents of every position (shared with the layers that name this one as `kv_from`)."""

    def __init__(self):
        self.c = []


def latent_step(w, q_, m, eps, st, h, pos, own_latent):
    H, D, V, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    if own_latent:
        st.c.append(rms(w[q_ + "dkv"] @ h, eps) * w[q_ + "dkv.norm"])
    cq = rms(w[q_ + "dq"] @ h, eps) * w[q_ + "dq.norm"]
    q = (w[q_ + "uq"] @ cq).reshape(H, D)
    uk, uv = w[q_ + "uk"].reshape(H, D, R), w[q_ + "uv"].reshape(H, V, R)
    gate = sigmoid(w[q_ + "g"] @ h)
    lo = max(0, pos - m["mask"]["size"] + 1)
    out = np.zeros((H, V))
    for hh in range(H):
        s = np.array([q[hh] @ (uk[hh] @ st.c[j]) for j in range(lo, pos + 1)]) * m["scale"]
        p = window_softmax(s, sink=w[q_ + "sink"][hh])
        out[hh] = sum(p[j - lo] * (uv[hh] @ st.c[j]) for j in range(lo, pos + 1)) * gate[hh]
    return w[q_ + "o"] @ out.reshape(-1)


class DeltaState:
    """The state matrices [heads, dim, vdim] and the last taps - 1 inputs of the three convolutions."""

    def __init__(self, m):
        H, G, D, V, T = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        self.S = np.zeros((H, D, V))
        self.hist = {n: np.zeros((T - 1, c)) for n, c in (("q", G * D), ("k", G * D), ("v", H * V))}


def short_conv(w_conv, hist, x):
    """Causal convolution over the last taps tokens (last column: the current one); returns (output, new history)."""
    win = np.vstack([hist, x[None, :]])                     # [taps, channels], oldest first
    y = np.einsum("tc,ct->c", win, w_conv)
    return y, win[1:]


def delta_rule_step(S, q, k, v, beta, g):
    """One token of the gated delta rule for one head.  S: [dim, vdim]; g: decay per key channel."""
    S = g[:, None] * S
    u = beta * (v - S.T @ k)
    S = S + np.outer(k, u)
    return S, S.T @ q


def delta_step(w, q_, m, eps, st, h):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    x = {}
    for n in ("q", "k", "v"):
        y, st.hist[n] = short_conv(w[q_ + n + ".conv"], st.hist[n], w[q_ + n] @ h)
        x[n] = silu(y)
    q, k, v = x["q"].reshape(G, D), x["k"].reshape(G, D), x["v"].reshape(H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(w[q_ + "b"] @ h)
    dt = softplus(w[q_ + "a2"] @ (w[q_ + "a1"] @ h) + w[q_ + "dt_bias"]).reshape(H, D)
    g = np.exp(-np.exp(w[q_ + "A_log"])[:, None] * dt)
    gate = sigmoid(w[q_ + "g2"] @ (w[q_ + "g1"] @ h)).reshape(H, V)
    out = np.zeros((H, V))
    for hh in range(H):
        gg = hh // (H // G)
        st.S[hh], o = delta_rule_step(st.S[hh], q[gg], k[gg], v[hh], beta[hh], g[hh])
        out[hh] = rms(o, eps) * w[q_ + "norm"] * gate[hh]
    return w[q_ + "o"] @ out.reshape(-1)


# ---- the model ---------------------------------------------------------------------------------------------------------
class Sequence:
    """Everything one sequence carries from token to token."""

    def __init__(self, cfg):
        self.pos, self.prev, self.layers = 0, None, []
        for l in cfg["layers"]:
            t, m = l["type"], l["mixer"]
            if t == "attention":
                self.layers.append(AttentionState())
            elif t == "latent_attention":
                self.layers.append(self.layers[m["kv_from"]] if "kv_from" in m else LatentState())
            else:
                self.layers.append(DeltaState(m))


def token_step(cfg, w, seq, tok, taps=None):
    """Runs one token; returns the logits.  taps (a list): receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = embed(w, cfg, seq.prev, tok)
    for i, l in enumerate(cfg["layers"]):
        p, q_, m = "l%d." % i, "l%d.mix." % i, l["mixer"]
        h = rms(x, eps) * w[p + "norm1"]
        if l["type"] == "attention":
            y = attention_step(w, q_, m, eps, seq.layers[i], h, seq.pos)
        elif l["type"] == "latent_attention":
            y = latent_step(w, q_, m, eps, seq.layers[i], h, seq.pos, "kv_from" not in m)
        else:
            y = delta_step(w, q_, m, eps, seq.layers[i], h)
        x = x + rms(y, eps) * w[p + "norm1b"]
        if l["mlp"] is not None:
            h = rms(x, eps) * w[p + "norm2"]
            x = x + rms(dense_ff(w, p, h), eps) * w[p + "norm2b"]
        if taps is not None:
            taps.append(x.copy())
    seq.pos += 1
    seq.prev = tok
    return (w["embed"] @ (rms(x, eps) * w["final.norm"])) * cfg["logit_scale"]


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
