"""Plain, slow restatement of the Nogatar design in float64 numpy: one function per mechanism, token by token where
the design is recurrent.  It is the yardstick of the GPU tests and shares no code with the library.

Notation: x is the residual stream [T, width]; a layer computes x += m * LN1(mixer(x)); x += m * LN2(ff(x)) where
the sublayers read x itself (the norm sits on the sublayer's OUTPUT).  Weights are [out, in] and applied as W @ h.
"""
import math

import numpy as np


def layer_norm(y, w, eps):
    mu = y.mean(-1, keepdims=True)
    var = ((y - mu) ** 2).mean(-1, keepdims=True)
    return (y - mu) / np.sqrt(var + eps) * w


def rms_unit(y, eps):
    return y / np.sqrt((y * y).mean(-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def softmax(z):
    z = z - z.max(-1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(-1, keepdims=True)


# ----------------------------------------------------------------------------- rotary positions
def rotary_frequencies(rot):
    """per-pair frequencies and the factor on cos/sin; `rot` = {base, dims, scaling?}"""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def corr(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(corr(float(sc["fast"]))), 0)
    hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(v, pos, rot):
    """v [..., T, n] with n >= rot dims; the first rot dims are rotated pairwise (2i, 2i+1), the rest pass"""
    f, mag = rotary_frequencies(rot)
    dims = int(rot["dims"])
    a = np.asarray(pos, np.float64)[:, None] * f[None, :]
    c, s = np.cos(a) * mag, np.sin(a) * mag
    out = v.copy()
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


# ----------------------------------------------------------------------------- mixers
def latent_attention(h, pos0, cache, W, mx, eps):
    """h [T, width] = new tokens at positions pos0..; cache = {"c": [n, rank], "kr": [n, rot_dim]} of earlier tokens
    (extended in place).  Non-absorbed form: keys and values are up-projected from the latent for every key."""
    H, d, r, vd, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    pos = np.arange(pos0, pos0 + T)
    q = (h @ W["q"].T).reshape(T, H, d + r)
    q_n, q_r = q[..., :d], q[..., d:]
    dkv = h @ W["dkv"].T
    c = rms_unit(dkv[:, :rank], eps) * W["dkv.norm"]
    kr = dkv[:, rank:]
    rot = dict(mx["rot"])
    q_r = rotate_interleaved(q_r.transpose(1, 0, 2), pos, rot).transpose(1, 0, 2)
    kr = rotate_interleaved(kr, pos, rot)
    cache["c"] = np.concatenate([cache["c"], c], 0)
    cache["kr"] = np.concatenate([cache["kr"], kr], 0)
    C, KR = cache["c"], cache["kr"]
    k_n = (C @ W["uk"].T).reshape(-1, H, d)
    val = (C @ W["uv"].T).reshape(-1, H, vd)
    window = mx.get("mask", {}).get("size") if mx.get("mask") else None
    out = np.zeros((T, H, vd))
    for t in range(T):
        i = pos0 + t
        j0 = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            s = (k_n[j0:i + 1, hh] @ q_n[t, hh] + KR[j0:i + 1] @ q_r[t, hh]) * mx["scale"]
            sink = W.get("sink")
            m = max(s.max(), sink[hh]) if sink is not None else s.max()
            e = np.exp(s - m)
            den = e.sum() + (math.exp(sink[hh] - m) if sink is not None else 0.0)
            out[t, hh] = (e / den) @ val[j0:i + 1, hh]
    return out.reshape(T, H * vd) @ W["o"].T


def mlstm(h, state, W, mx, eps):
    """matrix-memory recurrence, one token at a time; state = {"S": [H, dim, vdim], "n": [H, dim], "m": [H]}"""
    H, d, vd, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W["k"].T).reshape(T, H, d)
    v = (h @ W["v"].T).reshape(T, H, vd)
    ig = cap * np.tanh((h @ W["i"].T + W["i.b"]) / cap)
    fg = log_sigmoid(cap * np.tanh((h @ W["f"].T + W["f.b"]) / cap))
    o = np.zeros((T, H, vd))
    for t in range(T):
        for hh in range(H):
            m_old = state["m"][hh]
            m_new = max(fg[t, hh] + m_old, ig[t, hh])
            a, b = math.exp(fg[t, hh] + m_old - m_new), math.exp(ig[t, hh] - m_new)
            state["S"][hh] = a * state["S"][hh] + b * np.outer(k[t, hh], v[t, hh])
            state["n"][hh] = a * state["n"][hh] + b * k[t, hh]
            state["m"][hh] = m_new
            den = max(abs(state["n"][hh] @ q[t, hh]), math.exp(-m_new)) + 1e-6
            o[t, hh] = state["S"][hh].T @ q[t, hh] / den
    o = rms_unit(o, eps).reshape(T, H * vd) * W["norm"]
    return (o * sigmoid(h @ W["g"].T)) @ W["o"].T


def mlstm_zero_state(mx):
    H, d, vd = mx["heads"], mx["dim"], mx["vdim"]
    return {"S": np.zeros((H, d, vd)), "n": np.zeros((H, d)), "m": np.zeros(H)}


# ----------------------------------------------------------------------------- feed-forward
def expert(h, up, down):
    return (np.maximum(h @ up.T, 0.0) ** 2) @ down.T


def moe(h, W, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = softmax(h @ W["router"].T)
    out = np.zeros((h.shape[0], W["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        idx = np.argsort(-s[t], kind="stable")[:top]
        wsum = s[t, idx].sum() + 1e-20
        for e in idx:
            out[t] += s[t, e] / wsum * expert(h[t], W[f"e{e}.up"], W[f"e{e}.down"])
    if mlp.get("shared") and "shared.up" in W:
        g = sigmoid(h @ W["shared.sg"].T)  # [T, 1]
        out += g * expert(h, W["shared.up"], W["shared.down"])
    assert E == s.shape[1]
    return out


# ----------------------------------------------------------------------------- the model
def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


class Model:
    """weights: name -> float64 array (names as in the checkpoint: embed, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*,
    final.norm, head)."""

    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, {k: np.asarray(v, np.float64) for k, v in weights.items()}

    def new_state(self):
        st = []
        for ly in self.cfg["layers"]:
            if ly["type"] == "mlstm":
                st.append(mlstm_zero_state(ly["mixer"]))
            else:
                mx = ly["mixer"]
                st.append({"c": np.zeros((0, mx["kv_rank"])), "kr": np.zeros((0, mx["rot_dim"]))})
        return {"layers": st, "len": 0}

    def forward(self, tokens, state, want_layers=False):
        """feeds `tokens` after what `state` already holds; returns logits [T, vocab] (and the stream after each layer)"""
        cfg, w = self.cfg, self.w
        eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
        x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
        pos0 = state["len"]
        streams = []
        for i, ly in enumerate(cfg["layers"]):
            W = sub(w, f"l{i}.mix.")
            if ly["type"] == "mlstm":
                y = mlstm(x, state["layers"][i], W, ly["mixer"], eps)
            elif ly["type"] == "latent_attention":
                y = latent_attention(x, pos0, state["layers"][i], W, ly["mixer"], eps)
            else:
                raise ValueError(ly["type"])
            x = x + m * layer_norm(y, w[f"l{i}.norm1"], eps)
            if ly.get("mlp"):
                y = moe(x, sub(w, f"l{i}.mlp."), ly["mlp"])
                x = x + m * layer_norm(y, w[f"l{i}.norm2"], eps)
            streams.append(x.copy())
        state["len"] += len(tokens)
        z = layer_norm(x, w["final.norm"], eps) @ w["head"].T
        cap = cfg.get("logit_softcap")
        if cap:
            z = cap * np.tanh(z / cap)
        return (z, np.stack(streams)) if want_layers else z
