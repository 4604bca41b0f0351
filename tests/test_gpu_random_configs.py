"""Seeded random walk over the layer's option space (shapes, metrics, samplings, conv types,
heads, K, softmax on/off, dtype), every case checked stage by stage against the oracle."""
import random

import pytest
import torch

from convnn_b200 import _capi, ops
from oracle.convnn_oracle import (ConvNNConfig, bf16_round, convnn_attention, from_neighbours, make_input,
                                  make_layer_weights, near_tie_rows, select_neighbours, similarity)
from gpu_util import DEV, heads_to_oracle, pack, rel_err, spec_of

pytestmark = pytest.mark.gpu


def _cases(n, seed):
    rng = random.Random(seed)
    out = []
    while len(out) < n:
        H = rng.choice([1, 1, 2, 3, 4])
        dk = rng.choice([8, 16, 24, 32, 48, 64, 96])
        T = 197 if H > 1 else rng.choice([1, 2, 5, 17, 64, 65, 128, 129, 197, 256, 300])
        sampling = rng.choice(["all", "all", "random", "spatial"])
        K = rng.choice([1, 2, 3, 5, 9, 12, 16, 25, 32])
        conv = rng.choice(["depthwise", "standard", "depthwise-separable"])
        S = T if sampling == "all" else rng.randint(1, T)
        nsel = K if sampling == "all" else K - 1
        if nsel > S:
            continue
        out.append(dict(B=rng.choice([1, 2, 3]), T=T, S=S, H=H, dk=dk, K=K, sampling=sampling, conv=conv,
                        metric=rng.choice(["cosine", "matmul", "euclidean"]), softmax=rng.random() < 0.7,
                        dtype=rng.choice(["fp32", "bf16", "bf16"]), seed=rng.randint(0, 10 ** 6)))
    return out


CASES = _cases(48, seed=20240917)


@pytest.mark.parametrize("c", CASES, ids=[f"{i}-{c['dtype']}-{c['metric'][:3]}-{c['sampling'][:3]}-{c['conv'][:5]}-T{c['T']}-H{c['H']}-dk{c['dk']}-K{c['K']}"
                                         for i, c in enumerate(CASES)])
def test_random_config(c):
    D = c["H"] * c["dk"]
    cfg = ConvNNConfig(d_hidden=D, num_heads=c["H"], K=c["K"], sampling_type=c["sampling"], num_samples=c["S"],
                       magnitude_type=c["metric"], seq_length=197, convolution_type=c["conv"],
                       softmax_topk_val=c["softmax"])
    g = torch.Generator().manual_seed(c["seed"])
    cand = None
    if c["sampling"] == "random":
        cand = torch.randperm(c["T"], generator=g)[: c["S"]]
    elif c["sampling"] == "spatial":
        cand = torch.linspace(0, c["T"] - 1, c["S"]).long()
    w = make_layer_weights(cfg, seed=c["seed"] + 1)
    x = make_input(c["B"], c["T"], D, seed=c["seed"] + 2)
    bf16 = c["dtype"] == "bf16"
    dtype = torch.bfloat16 if bf16 else torch.float32
    if bf16:
        x, w = bf16_round(x), {n: bf16_round(t) for n, t in w.items()}
    spec, packed = spec_of(cfg), pack(cfg, w, dtype)
    xg = x.to(DEV, dtype)
    cg = None if cand is None else cand.to(DEV)
    q, k, v, qs, ks = ops.qkv_proj(spec, xg, packed[0], cg)
    idx, val = ops.sim_topk(spec, q, k, qs, ks, cg)
    o = ops.gather_conv(spec, v, idx, val, packed[1], packed[2], S=q.shape[1])
    out = ops.out_proj(spec, o, packed[3], S=q.shape[1])
    whole = ops.forward(spec, xg, packed, cg)
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    assert torch.equal(whole, out)
    # selection judged on the kernel's own q / k (exact products in both dtypes)
    C = cfg.in_channels
    qo, ko, vo = heads_to_oracle(q, C), heads_to_oracle(k, C), heads_to_oracle(v, C)
    sim = similarity(qo, ko, cfg, cand)
    idx_want, val_want = select_neighbours(sim, cfg, cand)
    ties = near_tie_rows(sim, cfg, cand is not None, 2e-6)
    same = (idx.cpu().long() == idx_want).all(-1)
    finite = torch.isfinite(sim).all(-1)                     # euclidean NaN rows are undefined in the reference
    assert bool((same | ties | ~finite).all())
    ok_rows = same & finite
    if bool(ok_rows.any()):
        dv = (val.cpu() - val_want).abs() / val_want.abs().clamp_min(1.0)
        assert float(dv[ok_rows].max()) < 1e-5
    tol = 2e-2 if bf16 else 1e-4
    if bool(finite.all()):
        assert rel_err(out, from_neighbours(vo, idx.cpu(), val.cpu(), w, cfg)) < tol
    if not bf16:
        tr = convnn_attention(x, w, cfg, cand=cand)
        assert rel_err(heads_to_oracle(q, C), tr.q) < 1e-5
