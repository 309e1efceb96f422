"""cpu: the plain restatement of the Fosavik design is consistent with itself (one call, token by token, portions), its
mask and convolution helpers do what their docstrings say, and the model registry knows the family."""
import copy
import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import fosavik_oracle as O  # noqa: E402
import fosavik_util as U  # noqa: E402


def test_oracle_cut_invariance():
    layers = [U.diff_layer(mlp=U.dense()), U.parallel_layer(), U.mamba_layer(), U.diff_layer(kv_from=0)]
    cfg = U.make_config(layers, width=12, vocab=19, streams=2)
    w = U.values(U.random_weights(cfg, seed=1))
    toks = [int(t) for t in np.random.default_rng(0).integers(0, 19, 21)]
    m = O.Model(cfg, w)
    whole = m.forward(toks, m.new_state())
    st, rows = m.new_state(), []
    for c0, c1 in ((0, 5), (5, 7), (7, 8), (8, 21)):
        rows.append(m.forward(toks[c0:c1], st))
    assert np.allclose(np.concatenate(rows), whole, rtol=1e-9, atol=1e-9)


def test_mask_and_convolution_helpers():
    # window 3, two kept tokens: position 6 sees 4, 5, 6 and 0, 1
    assert [j for j in range(9) if O.visible(6, j, 3, 2)] == [0, 1, 4, 5, 6]
    assert [j for j in range(9) if O.visible(2, j, 3, 2)] == [0, 1, 2]
    assert [j for j in range(5) if O.visible(3, j, 0, 0)] == [0, 1, 2, 3]
    x = np.arange(1.0, 6.0)[:, None]
    wt = np.array([[100.0, 10.0, 1.0]])
    out, tail = O.causal_conv(x, np.zeros((2, 1)), wt, np.zeros(1))
    assert out[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0] and tail[:, 0].tolist() == [4.0, 5.0]
    out2, tail2 = O.causal_conv(np.array([[6.0]]), tail, wt, np.zeros(1))
    assert out2[0, 0] == 456.0 and tail2[:, 0].tolist() == [5.0, 6.0]


def test_sink_lowers_the_weights():
    q = np.ones((1, 1, 2))
    K = np.ones((1, 1, 2))
    V = np.full((1, 1, 3), 2.0)
    plain = O.attend(q, K, V, [0], 1.0)
    sunk = O.attend(q, K, V, [0], 1.0, unit_sink=True)
    assert np.allclose(plain, 2.0) and np.allclose(sunk, 2.0 * np.exp(2.0) / (1.0 + np.exp(2.0)))


def test_registry_knows_the_family():
    so = os.path.join(ROOT, "qwen_inference_engine_b200", "libqie_b200.so")
    if not os.path.exists(so):
        pytest.skip("library not built")
    lib = ctypes.CDLL(so)
    lib.qie_model_families.restype = ctypes.c_char_p
    assert "Fosavik" in lib.qie_model_families().decode().split(",")
