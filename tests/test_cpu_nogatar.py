"""cpu: the plain Nogatar restatement is consistent with itself (a prompt cut into portions, a window that covers
everything against no window), and the model registry names its families and refuses what it does not know."""
import copy
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import nogatar_oracle as O  # noqa: E402
import nogatar_util as U  # noqa: E402


def _cfg():
    return U.make_config([U.attn_layer(mlp=U.moe()), U.mlstm_layer(mlp=U.moe(experts=3, top=1, ff=6, shared_ff=0)),
                          U.attn_layer(heads=2, dim=4, rot_dim=6, vdim=3, kv_rank=5, window=4, rot_dims=2, scaling=False)], width=16, vocab=29)


def test_oracle_portions_equal_whole():
    cfg = _cfg()
    w = U.values(U.random_weights(cfg, seed=1))
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg["vocab"], 26)]
    m = O.Model(cfg, w)
    whole = m.forward(toks, m.new_state())
    st, parts, at = m.new_state(), [], 0
    for c in (3, 1, 9, 2, 11):
        parts.append(m.forward(toks[at:at + c], st))
        at += c
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-9


def test_oracle_window_larger_than_prompt_is_no_window():
    cfg = _cfg()
    w = U.values(U.random_weights(cfg, seed=2))
    toks = list(range(12))
    wide, none = copy.deepcopy(cfg), copy.deepcopy(cfg)
    for c, size in ((wide, 12), (none, None)):
        for ly in c["layers"]:
            if ly["type"] == "latent_attention":
                if size:
                    ly["mixer"]["mask"] = {"size": size}
                else:
                    ly["mixer"].pop("mask", None)
    a, b = O.Model(wide, w), O.Model(none, w)
    assert np.abs(a.forward(toks, a.new_state()) - b.forward(toks, b.new_state())).max() < 1e-12
    narrow = O.Model(cfg, w)
    assert np.abs(narrow.forward(toks, narrow.new_state()) - b.forward(toks, b.new_state())).max() > 1e-3


def test_rotary_scaling_limits():
    # far below `original` turns nothing changes for the fastest pair; the slowest pair is divided by the factor
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "fast": 32.0, "original": 64, "slow": 1.0}}
    f, mag = O.rotary_frequencies(rot)
    plain, one = O.rotary_frequencies({"base": 10000.0, "dims": 16})
    assert one == 1.0 and abs(mag - (0.1 * np.log(4.0) + 1.0)) < 1e-12
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 4.0) < 1e-15
    assert np.all(f <= plain + 1e-18) and np.all(f >= plain / 4.0 - 1e-18)


def test_registry_names_and_refusals(tmp_path):
    import qwen_inference_engine_b200 as q
    L = q.lib()
    names = L.qie_model_families().decode().split(",")
    assert "Nogatar" in names and "Qwen2ForCausalLM" in names
    d = tmp_path / "unknown"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"architecture": "SomethingElse"}))
    with pytest.raises(q.QieError) as ei:
        q.Engine(model_dir=str(d))
    assert ei.value.code == -3 and "not registered" in str(ei.value)
    with pytest.raises(q.QieError) as ei:
        q.Engine(model_dir=str(tmp_path / "missing"))
    assert ei.value.code == -3
