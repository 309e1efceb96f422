"""Helpers of the Fosavik tests: small configurations, bf16-exact random weights written as a model folder
(config.json + model.safetensors)."""
import numpy as np

from nogatar_util import bf16_round, rel_err, values, write_model  # noqa: F401  (format helpers, not model code)


def diff_layer(heads=4, kv_heads=2, dim=6, vdim=10, diff=0.3, scale=0.4, kv_from=None, mlp=None):
    mx = {"diff": diff, "dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def parallel_layer(heads=6, kv_heads=3, dim=10, window=7, keep_first=3, scale=0.3, width=24, blocks=3, conv=3, left_scale=0.8,
                   right_scale=1.3, mlp=None):
    left = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"keep_first": keep_first, "size": window}, "scale": scale, "vdim": dim}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right": {"blocks": blocks, "conv": conv, "width": width},
                                          "right_scale": right_scale}, "mlp": mlp}


def mamba_layer(heads=4, vdim=6, state=5, groups=2, norm_groups=2, conv=4, mlp=None):
    return {"type": "mamba2", "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim},
            "mlp": mlp}


def dense(ff=14, limit=0.8):
    return {"ff": ff, "kind": "dense", "limit": limit}


def make_config(layers, width=20, vocab=37, streams=3, eps=1e-5, max_positions=512):
    return {"architecture": "Fosavik", "layers": layers, "max_positions": max_positions, "norm": {"eps": eps}, "streams": streams,
            "vocab": vocab, "width": width}


def tensor_shapes(cfg):
    W, S = cfg["width"], cfg["streams"]
    out = {"embed": (cfg["vocab"], W), "pos": (cfg["max_positions"], W)}
    for i, ly in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", ly["mixer"]
        out[p + "norm1"] = (W,)
        out.update({p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S)})
        if ly["type"] == "attention":
            H, G, d, vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            out[p + "mix.q"] = (H * 2 * d, W)
            if mx.get("kv_from") is None:
                out.update({p + "mix.k": (G * 2 * d, W), p + "mix.v": (G * vd, W)})
            out.update({p + "mix.lq1": (d,), p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,), p + "mix.o": (W, H * vd)})
        elif ly["type"] == "parallel":
            lf, rt = mx["left"], mx["right"]
            H, G, d = lf["heads"], lf["kv_heads"], lf["dim"]
            R, B = rt["width"], rt["blocks"]
            out.update({p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.q.norm": (d,), p + "mix.left.k.norm": (d,),
                        p + "mix.left.g": (H, W), p + "mix.left.o": (W, H * d), p + "mix.right.y": (R, W), p + "mix.right.y.b": (R,),
                        p + "mix.right.x": (R, W), p + "mix.right.x.b": (R,), p + "mix.right.conv": (R, rt["conv"]), p + "mix.right.conv.b": (R,),
                        p + "mix.right.ra": (B, R // B, R // B), p + "mix.right.ra.b": (B, R // B), p + "mix.right.ri": (B, R // B, R // B),
                        p + "mix.right.ri.b": (B, R // B), p + "mix.right.lam": (R,), p + "mix.right.o": (W, R)})
        else:
            inner, GN = mx["heads"] * mx["vdim"], mx["groups"] * mx["state"]
            out.update({p + "mix.in": (2 * inner + 2 * GN + mx["heads"], W), p + "mix.conv": (inner + 2 * GN, mx["conv"]),
                        p + "mix.conv.b": (inner + 2 * GN,), p + "mix.dt_bias": (mx["heads"],), p + "mix.A_log": (mx["heads"],),
                        p + "mix.D": (mx["heads"],), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        if ly.get("mlp"):
            ff = ly["mlp"]["ff"]
            out[p + "norm2"] = (W,)
            out.update({p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
            out.update({p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg, seed=0, gain=1.0):
    """name -> (bf16 bits, float64 values)"""
    rng = np.random.default_rng(seed)
    S = cfg["streams"]
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name.endswith("hc1.mix") or name.endswith("hc2.mix"):
            a = np.eye(S) + 0.3 * rng.standard_normal(shape)
        elif ".hc" in name:
            a = (1.0 if last == "out" else 1.0 / S) + 0.3 * rng.standard_normal(shape)
        elif name == "pos":
            a = 0.5 * rng.standard_normal(shape)
        elif last == "conv":
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif len(shape) >= 2:
            a = rng.standard_normal(shape) * gain / np.sqrt(shape[-1])
        elif "norm" in name:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "A_log":
            a = np.log(rng.uniform(0.5, 4.0, shape))
        elif last == "lam":
            a = rng.uniform(-3.0, 1.0, shape)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            a = 0.4 * rng.standard_normal(shape)
        else:
            a = 0.5 * rng.standard_normal(shape)
        out[name] = bf16_round(np.asarray(a, np.float32))
    return out
