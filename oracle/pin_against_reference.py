"""Pin the oracle against the unmodified reference.  TEST INFRASTRUCTURE ONLY.

Usage (needs a checkout of the reference; it is not needed at test or bench time):

    python -m oracle.pin_against_reference --reference /path/to/reference

Imports the reference's ``layers`` and ``vit`` modules, loads the oracle's seeded weights
into them with ``load_state_dict(strict=True)`` and compares outputs over the grid
{H=1 T=65, H=3 T=197} x 3 metrics x 3 conv types x 3 samplings x softmax on/off,
coordinate encoding, both branching wrappers and the whole ViT.  Exits non-zero on the
first mismatch above 1e-5 relative.
"""
from __future__ import annotations

import argparse
import itertools
import sys
import types

import torch


def load_reference(path: str):
    """Import reference modules.  torchsummary / thop / matplotlib are imported at the
    top of reference files but never called in forward; stub them when absent."""
    for name in ("torchsummary", "thop", "matplotlib", "matplotlib.pyplot", "torchvision",
                 "torchvision.transforms", "torchvision.datasets"):
        try:
            __import__(name)
        except Exception:
            m = types.ModuleType(name)
            m.summary = lambda *a, **k: None
            m.profile = lambda *a, **k: (0, 0)
            sys.modules[name] = m
    if path not in sys.path:
        sys.path.insert(0, path)
    import layers as ref_layers  # noqa: E402
    import vit as ref_vit  # noqa: E402
    return ref_layers, ref_vit


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def check_layers(ref_layers, verbose: bool) -> int:
    from .convnn_oracle import (ConvNNConfig, METRICS, SAMPLINGS, CONV_TYPES, convnn_attention,
                                make_input, make_layer_weights)
    n = 0
    worst = 0.0
    grid = itertools.product(((1, 65, 48), (3, 197, 96)), METRICS, CONV_TYPES, SAMPLINGS, (True, False), (False, True))
    for (H, T, D), metric, conv, samp, soft, coord in grid:
        if coord and conv == "depthwise":
            continue  # the reference raises at construction (groups mismatch)
        ns = -1 if samp == "all" else 24
        cfg = ConvNNConfig(d_hidden=D, num_heads=H, K=5, sampling_type=samp, num_samples=ns,
                           sample_padding=0, magnitude_type=metric, seq_length=197,
                           coordinate_encoding=coord, convolution_type=conv, softmax_topk_val=soft)
        w = make_layer_weights(cfg, seed=7)
        x = make_input(2, T, D, seed=11)
        ref = ref_layers.MultiHeadConvNNAttention(D, H, 0.0, 5, samp, ns, 0, metric, 197, coord, conv, soft).eval()
        ref.load_state_dict(w, strict=True)
        with torch.no_grad():
            torch.manual_seed(123)
            y_ref = ref(x)
            torch.manual_seed(123)      # same randperm draw as the reference consumed
            tr = convnn_attention(x, w, cfg)
        e = rel_err(tr.out, y_ref)
        worst = max(worst, e)
        n += 1
        if verbose:
            print(f"H={H} T={T} {metric:9s} {conv:20s} {samp:7s} softmax={soft} coord={coord}: {e:.2e}")
        if not (e < 1e-5):
            print("MISMATCH", H, T, metric, conv, samp, soft, coord, e)
            return 1
    print(f"layer grid: {n} combinations, worst relative error {worst:.2e}")
    return 0


def check_branching(ref_layers) -> int:
    from .convnn_oracle import ConvNNConfig, branching_attention, branching_conv, make_input
    from .vit_oracle import ViTConfig, attention_weight_shapes
    import math
    for layer, conv in (("BranchAttention", "standard"), ("BranchConv", "depthwise-separable")):
        vc = ViTConfig(layer=layer, d_hidden=96, num_heads=3, K=5, convolution_type=conv, kernel_size=5)
        g = torch.Generator().manual_seed(3)
        w = {k: (torch.rand(s, generator=g) * 2 - 1) / math.sqrt(8) for k, s in attention_weight_shapes(vc).items()}
        x = make_input(2, 197, 96, seed=5)
        c = vc.convnn_cfg()
        if layer == "BranchAttention":
            ref = ref_layers.MultiHeadBranchingAttention(96, 3, 0.0, 5, "all", -1, 0, "cosine", 197, False, conv, True, 0.5).eval()
            got = branching_attention(x, w, c, 96, 0.5)
        else:
            ref = ref_layers.MultiHeadBranchingConv(96, 3, 0.0, 5, 5, "all", -1, 0, "cosine", 197, False, conv, True, 0.5).eval()
            got = branching_conv(x, w, c, 96, 0.5, 5)
        ref.load_state_dict(w, strict=True)
        with torch.no_grad():
            want = ref(x)
        e = rel_err(got, want)
        print(f"{layer}: {e:.2e}")
        if not (e < 1e-5):
            return 1
    return 0


def reference_vit(ref_vit, cfg, sd):
    """Build the reference ViT for an oracle ViTConfig and load oracle weights."""
    args = types.SimpleNamespace(**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__})
    args.device = "cpu"
    model = ref_vit.ViT(args).eval()
    model.load_state_dict(sd, strict=True)
    return model


def check_vit(ref_vit) -> int:
    from .vit_oracle import ViTConfig, make_images, make_vit_weights, vit_forward
    cases = [
        ViTConfig(layer="ConvNNAttention", img_size=(3, 32, 32), patch_size=4, num_layers=3, num_heads=1,
                  d_hidden=48, d_mlp=96, num_classes=10, K=9, magnitude_type="cosine"),
        ViTConfig(layer="BranchAttention", img_size=(3, 224, 224), patch_size=16, num_layers=2, num_heads=3,
                  d_hidden=96, d_mlp=192, num_classes=10, K=9, magnitude_type="cosine", convolution_type="standard"),
        ViTConfig(layer="BranchConv", img_size=(3, 224, 224), patch_size=16, num_layers=2, num_heads=3,
                  d_hidden=96, d_mlp=192, num_classes=10, K=5, magnitude_type="euclidean",
                  sampling_type="spatial", num_samples=49, convolution_type="depthwise-separable", kernel_size=5),
    ]
    for cfg in cases:
        sd = make_vit_weights(cfg, seed=1)
        img = make_images(2, cfg, seed=2)
        model = reference_vit(ref_vit, cfg, sd)
        with torch.no_grad():
            want = model(img)
            got = vit_forward(img, sd, cfg)
        e = rel_err(got, want)
        print(f"ViT {cfg.layer}: {e:.2e}")
        if not (e < 1e-5):
            return 1
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    ref_layers, ref_vit = load_reference(a.reference)
    torch.set_grad_enabled(False)
    rc = check_layers(ref_layers, a.verbose) or check_branching(ref_layers) or check_vit(ref_vit)
    print("PINNED" if rc == 0 else "FAILED")
    return rc


if __name__ == "__main__":
    sys.exit(main())
