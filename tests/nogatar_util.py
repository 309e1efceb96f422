"""Helpers of the Nogatar tests: small random configurations, bf16-exact random weights written as a model folder
(config.json + model.safetensors), and the error measure."""
import json
import os
import struct

import numpy as np


def bf16_round(a):
    """float32 array -> (uint16 bf16 bits, the float64 values those bits stand for); round to nearest even"""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    bits = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return bits, (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def attn_layer(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=12, window=5, rot_dims=None, scaling=True, scale=0.3, base=100.0, mlp=None):
    rot = {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 3.0, "fast": 8.0, "original": 16, "slow": 1.0}
    mixer = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": rot, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def mlstm_layer(heads=2, dim=6, vdim=10, gate_cap=12.0, mlp=None):
    return {"type": "mlstm", "mixer": {"dim": dim, "gate_cap": gate_cap, "heads": heads, "vdim": vdim}, "mlp": mlp}


def moe(experts=5, top=2, ff=12, shared_ff=10):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def make_config(layers, width=24, vocab=53, embed_scale=3.0, eps=1e-5, res_mult=0.4, softcap=20.0):
    cfg = {"architecture": "Nogatar", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
           "residual_mult": res_mult, "vocab": vocab, "width": width}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def tensor_shapes(cfg):
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}
    for i, ly in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", ly["mixer"]
        H, d, vd = mx["heads"], mx["dim"], mx["vdim"]
        out[p + "norm1"] = (W,)
        if ly["type"] == "latent_attention":
            r, k = mx["rot_dim"], mx["kv_rank"]
            out.update({p + "mix.q": (H * (d + r), W), p + "mix.dkv": (k + r, W), p + "mix.dkv.norm": (k,), p + "mix.uk": (H * d, k),
                        p + "mix.uv": (H * vd, k), p + "mix.sink": (H,), p + "mix.o": (W, H * vd)})
        else:
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * vd, W), p + "mix.g": (H * vd, W),
                        p + "mix.o": (W, H * vd), p + "mix.norm": (H * vd,), p + "mix.i": (H, W), p + "mix.i.b": (H,), p + "mix.f": (H, W),
                        p + "mix.f.b": (H,)})
        mlp = ly.get("mlp")
        if mlp:
            out[p + "norm2"] = (W,)
            for e in range(mlp["router"]["experts"]):
                out[p + f"mlp.e{e}.up"] = (mlp["expert"]["ff"], W)
                out[p + f"mlp.e{e}.down"] = (W, mlp["expert"]["ff"])
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared"):
                out.update({p + "mlp.shared.up": (mlp["shared"]["ff"], W), p + "mlp.shared.down": (W, mlp["shared"]["ff"]),
                            p + "mlp.shared.sg": (1, W)})
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg, seed=0, gain=1.0):
    """name -> (bf16 bits, float64 values).  Matrices ~ N(0, gain^2 / fan_in), norm weights about 1, small vectors."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 2:
            a = rng.standard_normal(shape) * gain / np.sqrt(shape[1])
            if name.endswith("router"):
                a *= 3.0  # a router that prefers some experts clearly
        elif "norm" in name:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith("f.b"):
            a = 2.0 + rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape)
        out[name] = bf16_round(a.astype(np.float32))
    return out


def write_model(folder, cfg, weights):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, (bits, _) in weights.items():
        raw = bits.tobytes()
        header[name] = {"dtype": "BF16", "shape": list(bits.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return folder


def values(weights):
    return {k: v[1] for k, v in weights.items()}


def rel_err(got, want):
    """rms of the difference over the rms of the expected rows, worst row"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = np.sqrt(((got - want) ** 2).mean(-1))
    return float((d / (np.sqrt((want ** 2).mean(-1)) + 1e-30)).max())
