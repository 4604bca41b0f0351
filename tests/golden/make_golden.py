"""Generate the golden fixtures in this folder from the unmodified reference.

    python tests/golden/make_golden.py --reference /path/to/reference

Each case builds the reference module (``layers.MultiHeadConvNNAttention``, the two
branching wrappers, or ``vit.ViT``), loads seeded weights from the oracle's generators
with ``load_state_dict(strict=True)``, runs one eval forward on a seeded input on CPU in
fp32 and stores the output.  Inputs and weights are not stored: they are regenerated
from the seeds, and a checksum of each guards against generator drift.  The reference
is needed only to (re)generate; the tests replay the stored outputs without it.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.convnn_oracle import ConvNNConfig, make_input, make_layer_weights  # noqa: E402
from oracle.pin_against_reference import load_reference, reference_vit  # noqa: E402
from oracle.vit_oracle import ViTConfig, make_images, make_vit_weights  # noqa: E402

# name -> (B, T, ConvNNConfig kwargs, weight seed, input seed, torch seed for randperm)
LAYER_CASES = {
    "cos_all_dw_h1": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="cosine")),
    "cos_all_dw_h1_k1": (2, 33, dict(d_hidden=32, num_heads=1, K=1, magnitude_type="cosine")),
    "mm_all_std_h1": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="matmul", convolution_type="standard")),
    "euc_all_dws_h1": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="euclidean", convolution_type="depthwise-separable")),
    "cos_all_dw_h1_nosoftmax": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="cosine", softmax_topk_val=False)),
    "euc_all_dw_h1_nosoftmax": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="euclidean", softmax_topk_val=False)),
    "cos_spatial_dw_h1": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="cosine", sampling_type="spatial", num_samples=16)),
    "cos_spatial_pad_dw_h1": (2, 65, dict(d_hidden=48, num_heads=1, K=5, magnitude_type="cosine", sampling_type="spatial", num_samples=16, sample_padding=3)),
    "euc_random_dws_h1": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="euclidean", sampling_type="random", num_samples=24, convolution_type="depthwise-separable")),
    "mm_random_std_h1_nosoftmax": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="matmul", sampling_type="random", num_samples=24, convolution_type="standard", softmax_topk_val=False)),
    "cos_all_dw_h3_t197": (2, 197, dict(d_hidden=96, num_heads=3, K=9, magnitude_type="cosine")),
    "cos_all_std_h12_t197": (1, 197, dict(d_hidden=96, num_heads=12, K=9, magnitude_type="cosine", convolution_type="standard")),
    "euc_spatial_dws_h3_t197": (2, 197, dict(d_hidden=96, num_heads=3, K=9, magnitude_type="euclidean", sampling_type="spatial", num_samples=49, convolution_type="depthwise-separable")),
    "cos_all_std_h1_coord": (2, 65, dict(d_hidden=48, num_heads=1, K=9, magnitude_type="cosine", convolution_type="standard", coordinate_encoding=True)),
    "mm_spatial_dws_h3_t197_coord": (1, 197, dict(d_hidden=96, num_heads=3, K=9, magnitude_type="matmul", sampling_type="spatial", num_samples=49, convolution_type="depthwise-separable", coordinate_encoding=True)),
    "cos_all_dw_h1_d192": (2, 65, dict(d_hidden=192, num_heads=1, K=9, magnitude_type="cosine")),
    "cos_all_dw_h1_k25": (1, 130, dict(d_hidden=64, num_heads=1, K=25, magnitude_type="cosine")),
}
W_SEED, X_SEED, RAND_SEED = 7, 11, 123

VIT_CASES = {
    # cfg-1 architecture of the baseline (ViT-Tiny, 32x32, patch 4, 10 classes), B=4
    "vit_tiny_cifar_convnn": (4, dict(layer="ConvNNAttention", img_size=(3, 32, 32), patch_size=4, num_layers=12,
                                      num_heads=1, d_hidden=192, d_mlp=768, num_classes=10, K=9,
                                      magnitude_type="cosine")),
    "vit_small_branchattn": (2, dict(layer="BranchAttention", img_size=(3, 224, 224), patch_size=16, num_layers=2,
                                     num_heads=3, d_hidden=96, d_mlp=192, num_classes=10, K=9,
                                     magnitude_type="cosine", convolution_type="standard")),
    "vit_small_branchconv": (2, dict(layer="BranchConv", img_size=(3, 224, 224), patch_size=16, num_layers=2,
                                     num_heads=3, d_hidden=96, d_mlp=192, num_classes=10, K=5,
                                     magnitude_type="euclidean", sampling_type="spatial", num_samples=49,
                                     convolution_type="depthwise-separable", kernel_size=5)),
}


def checksum(t: torch.Tensor) -> list:
    d = t.double()
    return [float(d.sum()), float(d.abs().sum())]


def weights_checksum(w: dict) -> list:
    s = [0.0, 0.0]
    for k in sorted(w):
        c = checksum(w[k])
        s[0] += c[0]
        s[1] += c[1]
    return s


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    ref_layers, ref_vit = load_reference(a.reference)
    torch.set_grad_enabled(False)
    manifest = {"torch": torch.__version__, "layer": {}, "vit": {}}
    arrays = {}
    for name, (B, T, kw) in LAYER_CASES.items():
        cfg = ConvNNConfig(**kw)
        w = make_layer_weights(cfg, seed=W_SEED)
        x = make_input(B, T, cfg.d_hidden, seed=X_SEED)
        ref = ref_layers.MultiHeadConvNNAttention(
            cfg.d_hidden, cfg.num_heads, 0.0, cfg.K, cfg.sampling_type, cfg.num_samples, cfg.sample_padding,
            cfg.magnitude_type, cfg.seq_length, cfg.coordinate_encoding, cfg.convolution_type,
            cfg.softmax_topk_val).eval()
        ref.load_state_dict(w, strict=True)
        torch.manual_seed(RAND_SEED)
        y = ref(x)
        arrays["layer/" + name] = y.numpy().astype(np.float32)
        manifest["layer"][name] = {"B": B, "T": T, "cfg": kw, "x_sum": checksum(x), "w_sum": weights_checksum(w)}
        print(name, tuple(y.shape), float(y.abs().mean()))
    for name, (B, kw) in VIT_CASES.items():
        cfg = ViTConfig(**kw)
        sd = make_vit_weights(cfg, seed=1)
        img = make_images(B, cfg, seed=2)
        y = reference_vit(ref_vit, cfg, sd)(img)
        arrays["vit/" + name] = y.numpy().astype(np.float32)
        kwj = dict(kw)
        kwj["img_size"] = list(kw["img_size"])
        manifest["vit"][name] = {"B": B, "cfg": kwj, "x_sum": checksum(img), "w_sum": weights_checksum(sd)}
        print(name, tuple(y.shape), float(y.abs().mean()))
    # state_dict layouts of the reference modules (key -> shape) for the drop-in contract
    L = ref_layers
    sd_cases = {
        "convnn_depthwise": L.MultiHeadConvNNAttention(48, 3, 0.0, 9, "all", -1, 0, "cosine"),
        "convnn_standard_coord": L.MultiHeadConvNNAttention(48, 3, 0.0, 9, "all", -1, 0, "cosine", 197, True, "standard"),
        "convnn_dwsep": L.MultiHeadConvNNAttention(48, 3, 0.0, 9, "all", -1, 0, "cosine", 197, False, "depthwise-separable"),
        "branch_attention": L.MultiHeadBranchingAttention(96, 3, 0.0, 9, "all", -1, 0, "cosine", 197, False, "standard", True, 0.5),
        "branch_conv": L.MultiHeadBranchingConv(96, 3, 0.0, 5, 9, "all", -1, 0, "cosine", 197, False, "depthwise", True, 0.5),
        "vit_tiny_convnn": reference_vit(ref_vit, ViTConfig(**VIT_CASES["vit_tiny_cifar_convnn"][1]),
                                         make_vit_weights(ViTConfig(**VIT_CASES["vit_tiny_cifar_convnn"][1]), seed=1)),
    }
    manifest["state_dict"] = {n: {k: list(v.shape) for k, v in m.state_dict().items()} for n, m in sd_cases.items()}
    np.savez_compressed(os.path.join(HERE, "reference_outputs.npz"), **arrays)
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
