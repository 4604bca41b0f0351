"""Access to the committed reference outputs (tests/golden/)."""
import json
import os

import numpy as np
import torch

from oracle.convnn_oracle import ConvNNConfig, make_input, make_layer_weights
from oracle.vit_oracle import ViTConfig, make_images, make_vit_weights

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
W_SEED, X_SEED, RAND_SEED = 7, 11, 123

with open(os.path.join(GOLDEN, "manifest.json")) as _f:
    MANIFEST = json.load(_f)
_ARR = np.load(os.path.join(GOLDEN, "reference_outputs.npz"))

LAYER_NAMES = sorted(MANIFEST["layer"])
VIT_NAMES = sorted(MANIFEST["vit"])


def _sum(t):
    d = t.double()
    return [float(d.sum()), float(d.abs().sum())]


def layer_case(name):
    """-> (cfg, weights, x, reference output, candidate indices or None)."""
    m = MANIFEST["layer"][name]
    cfg = ConvNNConfig(**m["cfg"])
    w = make_layer_weights(cfg, seed=W_SEED)
    x = make_input(m["B"], m["T"], cfg.d_hidden, seed=X_SEED)
    assert np.allclose(_sum(x), m["x_sum"], rtol=1e-9), "seeded input drifted from the fixture"
    tot = [0.0, 0.0]
    for k in sorted(w):
        s = _sum(w[k])
        tot[0] += s[0]
        tot[1] += s[1]
    assert np.allclose(tot, m["w_sum"], rtol=1e-9), "seeded weights drifted from the fixture"
    cand = None
    if cfg.sampling_type == "random":
        # the reference drew torch.randperm(T)[:num_samples] right after manual_seed(RAND_SEED)
        torch.manual_seed(RAND_SEED)
        cand = torch.randperm(m["T"])[: cfg.num_samples]
    return cfg, w, x, torch.from_numpy(_ARR["layer/" + name]), cand


def vit_case(name):
    m = MANIFEST["vit"][name]
    kw = dict(m["cfg"])
    kw["img_size"] = tuple(kw["img_size"])
    cfg = ViTConfig(**kw)
    sd = make_vit_weights(cfg, seed=1)
    img = make_images(m["B"], cfg, seed=2)
    assert np.allclose(_sum(img), m["x_sum"], rtol=1e-9)
    return cfg, sd, img, torch.from_numpy(_ARR["vit/" + name])


def rel_err(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))
