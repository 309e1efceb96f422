"""Plain, slow restatement of the Fosavik design in float64 numpy: one function per mechanism, token by token where
the design is recurrent.  It is the yardstick of the GPU tests and shares no code with the library.

Notation: the model carries `streams` copies X[s] of the residual (hyper-connections).  Sublayer f with vectors a (in),
b (out) and matrix M (mix, indexed [from, to]) does  u = sum_s a[s] X[s];  y = f(rmsnorm(u) * w);
X'[t] = sum_s M[s, t] X[s] + b[t] y.  Weights are [out, in] and applied as W @ h.
"""
import math

import numpy as np


def rms_unit(y, eps):
    return y / np.sqrt((y * y).mean(-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


# ----------------------------------------------------------------------------- hyper-connections
def hc_read(X, a):
    """X [S, T, W], a [S] -> u [T, W]"""
    return np.tensordot(a, X, axes=(0, 0))


def hc_write(X, M, b, y):
    """all streams at once from the old ones"""
    return np.einsum("st,snw->tnw", M, X) + b[:, None, None] * y[None]


# ----------------------------------------------------------------------------- causal convolution with a carried tail
def causal_conv(x, tail, w, b):
    """x [T, C] new inputs, tail [taps-1, C] the inputs before them (oldest first, zeros before the start),
    w [C, taps] with the last column on the current token.  Returns (out [T, C], new tail)."""
    taps = w.shape[1]
    full = np.concatenate([tail, x], 0)
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        win = full[t:t + taps]  # inputs t-(taps-1) .. t
        out[t] = (win * w.T).sum(0) + b
    return out, full[full.shape[0] - (taps - 1):].copy() if taps > 1 else tail


# ----------------------------------------------------------------------------- attention with kept first tokens and a sink
def visible(i, j, window, keep_first):
    if j > i:
        return False
    if window <= 0:
        return True
    return i - j < window or j < keep_first


def attend(q, K, V, pos, scale, window=0, keep_first=0, unit_sink=False):
    """q [T, H, d] at positions pos; K [n, G, d], V [n, G, vd] hold every position 0..n-1 -> [T, H, vd]"""
    T, H, _ = q.shape
    G = K.shape[1]
    out = np.zeros((T, H, V.shape[2]))
    for t in range(T):
        js = [j for j in range(K.shape[0]) if visible(pos[t], j, window, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = (K[js, g] @ q[t, h]) * scale
            m = max(s.max(), 0.0) if unit_sink else s.max()
            e = np.exp(s - m)
            den = e.sum() + (math.exp(-m) if unit_sink else 0.0)  # the sink: exp(0) joins the denominator and nothing joins the sum
            out[t, h] = (e / den) @ V[js, g]
    return out


def gated_window_attention(h, pos0, cache, W, mx, eps):
    """the 'left' half of the parallel mixer: per-head normed queries and keys, the values are the raw keys,
    window with kept first tokens, unit sink, a sigmoid gate per head"""
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, H, d)
    k = (h @ W["k"].T).reshape(T, G, d)
    v = k.copy()
    q = rms_unit(q, eps) * W["q.norm"]
    k = rms_unit(k, eps) * W["k.norm"]
    cache["k"] = np.concatenate([cache["k"], k], 0) if "k" in cache else k
    cache["v"] = np.concatenate([cache["v"], v], 0) if "v" in cache else v
    mask = mx.get("mask") or {}
    o = attend(q, cache["k"], cache["v"], np.arange(pos0, pos0 + T), mx["scale"], mask.get("size", 0), mask.get("keep_first", 0), True)
    gate = sigmoid(h @ W["g"].T)  # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, -1) @ W["o"].T


def differential_attention(h, pos0, cache, W, mx, eps, shared=None):
    """two score maps over the same values, combined as a1 - lambda a2, unit-normed per head.  `shared` is the cache of
    the layer whose keys and values this layer reads instead of projecting its own."""
    H, G, d, vd, diff = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["diff"]
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, H, 2, d)
    if shared is None:
        k = (h @ W["k"].T).reshape(T, G, 2, d)
        v = (h @ W["v"].T).reshape(T, G, vd)
        cache["k"] = np.concatenate([cache["k"], k], 0) if "k" in cache else k
        cache["v"] = np.concatenate([cache["v"], v], 0) if "v" in cache else v
        shared = cache
    pos = np.arange(pos0, pos0 + T)
    a1 = attend(q[:, :, 0], shared["k"][:, :, 0], shared["v"], pos, mx["scale"])
    a2 = attend(q[:, :, 1], shared["k"][:, :, 1], shared["v"], pos, mx["scale"])
    lam = math.exp((W["lq1"] * W["lk1"]).sum()) - math.exp((W["lq2"] * W["lk2"]).sum()) + diff
    o = rms_unit(a1 - lam * a2, eps) * (1.0 - diff)
    return o.reshape(T, -1) @ W["o"].T


# ----------------------------------------------------------------------------- recurrences
def gated_linear_recurrence(h, state, W, mx):
    """the 'right' half of the parallel mixer: S_t = a_t S_{t-1} + sqrt(1 - a_t^2) i_t u_t with block-diagonal gates"""
    width, blocks = mx["width"], mx["blocks"]
    bw = width // blocks
    T = h.shape[0]
    y = gelu_tanh(h @ W["y"].T + W["y.b"])
    xb = h @ W["x"].T + W["x.b"]
    if "tail" not in state:
        state["tail"] = np.zeros((mx["conv"] - 1, width))
        state["S"] = np.zeros(width)
    u, state["tail"] = causal_conv(xb, state["tail"], W["conv"], W["conv.b"])
    out = np.zeros((T, width))
    sp = softplus(W["lam"])
    for t in range(T):
        ub = u[t].reshape(blocks, bw)
        r = sigmoid(np.einsum("boi,bi->bo", W["ra"], ub) + W["ra.b"]).reshape(-1)
        i = sigmoid(np.einsum("boi,bi->bo", W["ri"], ub) + W["ri.b"]).reshape(-1)
        a = np.exp(-8.0 * r * sp)
        state["S"] = a * state["S"] + np.sqrt(1.0 - a * a) * i * u[t]
        out[t] = state["S"] * y[t]
    return out @ W["o"].T


def state_space_duality(h, state, W, mx, eps):
    """per head S_t = exp(-exp(A) dt_t) S_{t-1} + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t; gate, grouped unit norm, projection"""
    Hh, P, N, G, NG = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["norm_groups"]
    inner = Hh * P
    T = h.shape[0]
    zxbcdt = h @ W["in"].T
    z = zxbcdt[:, :inner]
    xbc = zxbcdt[:, inner:2 * inner + 2 * G * N]
    dt = softplus(zxbcdt[:, 2 * inner + 2 * G * N:] + W["dt_bias"])
    if "tail" not in state:
        state["tail"] = np.zeros((mx["conv"] - 1, inner + 2 * G * N))
        state["S"] = np.zeros((Hh, N, P))
    xbc, state["tail"] = causal_conv(xbc, state["tail"], W["conv"], W["conv.b"])
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(T, Hh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    y = np.zeros((T, Hh, P))
    for t in range(T):
        for hd in range(Hh):
            g = hd // (Hh // G)
            decay = math.exp(-math.exp(W["A_log"][hd]) * dt[t, hd])
            state["S"][hd] = decay * state["S"][hd] + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = state["S"][hd].T @ C[t, g] + W["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.reshape(T, NG, inner // NG), eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


# ----------------------------------------------------------------------------- feed-forward
def clamped_glu(h, W, mlp):
    lim = mlp["limit"]
    g = np.minimum(h @ W["gate"].T, lim)
    u = np.clip(h @ W["up"].T, -lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T


# ----------------------------------------------------------------------------- the model
class Model:
    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: np.asarray(v, np.float64) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]

    def sub(self, prefix):
        n = len(prefix)
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        return {"pos": 0, "layers": [dict() for _ in self.cfg["layers"]]}

    def forward(self, tokens, state, want_layers=False):
        """feeds `tokens` after what `state` holds; returns logits [T, vocab] (and the summed streams after every layer)"""
        cfg, w, eps = self.cfg, self.w, self.eps
        T, p0 = len(tokens), state["pos"]
        x = w["embed"][np.asarray(tokens)] + w["pos"][p0:p0 + T]
        X = np.stack([x] * cfg["streams"])
        dumps = []
        for i, ly in enumerate(cfg["layers"]):
            p = f"l{i}."
            st = state["layers"][i]
            mx = ly["mixer"]
            hn = rms_unit(hc_read(X, w[p + "hc1.in"]), eps) * w[p + "norm1"]
            if ly["type"] == "attention":
                src = None if mx.get("kv_from") is None else state["layers"][mx["kv_from"]]
                y = differential_attention(hn, p0, st, self.sub(p + "mix."), mx, eps, src)
            elif ly["type"] == "parallel":
                left = gated_window_attention(hn, p0, st, self.sub(p + "mix.left."), mx["left"], eps)
                right = gated_linear_recurrence(hn, st, self.sub(p + "mix.right."), mx["right"])
                y = mx["left_scale"] * left + mx["right_scale"] * right
            elif ly["type"] == "mamba2":
                y = state_space_duality(hn, st, self.sub(p + "mix."), mx, eps)
            else:
                raise ValueError(ly["type"])
            X = hc_write(X, w[p + "hc1.mix"], w[p + "hc1.out"], y)
            if ly.get("mlp"):
                hn = rms_unit(hc_read(X, w[p + "hc2.in"]), eps) * w[p + "norm2"]
                X = hc_write(X, w[p + "hc2.mix"], w[p + "hc2.out"], clamped_glu(hn, self.sub(p + "mlp."), ly["mlp"]))
            dumps.append(X.sum(0))
        state["pos"] = p0 + T
        logits = (rms_unit(X.sum(0), eps) * w["final.norm"]) @ w["head"].T
        return (logits, dumps) if want_layers else logits
