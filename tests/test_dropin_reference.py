"""Drop-in against the reference's own vit.py, when a reference checkout is available
(environment variable CONVNN_REF_PATH, default ../reference beside the repository).  Skipped otherwise: the golden
fixtures carry the same contract (state_dict layouts) without the checkout."""
import os
import sys

import pytest
import torch

import convnn_b200

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("CONVNN_REF_PATH", os.path.join(os.path.dirname(_ROOT), "reference"))
pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(REF, "vit.py")), reason="no reference checkout")


@pytest.fixture()
def reference_modules():
    from oracle.pin_against_reference import load_reference
    saved = {k: sys.modules.get(k) for k in ("layers", "vit", "utils")}
    ref_layers, ref_vit = load_reference(REF)
    yield ref_layers, ref_vit
    convnn_b200.uninstall()
    for k, v in saved.items():
        if v is None:
            sys.modules.pop(k, None)
        else:
            sys.modules[k] = v
    if REF in sys.path:
        sys.path.remove(REF)


@pytest.mark.parametrize("layer", ["ConvNNAttention", "BranchAttention", "BranchConv"])
def test_reference_vit_constructs_our_layers_and_shares_checkpoints(reference_modules, layer):
    import types
    ref_layers, ref_vit = reference_modules
    args = dict(layer=layer, patch_size=16, num_layers=2, num_heads=3, d_hidden=96, d_mlp=192, dropout=0.0,
                attention_dropout=0.0, convolution_type="standard", softmax_topk_val=True, K=9, sampling_type="all",
                num_samples=-1, sample_padding=0, magnitude_type="cosine", coordinate_encoding=False,
                branch_ratio=0.5, kernel_size=9, device="cpu", img_size=(3, 224, 224), num_classes=10)
    stock = ref_vit.ViT(types.SimpleNamespace(**args))               # the reference's own layers
    convnn_b200.install(ref_layers, ref_vit)
    ours = ref_vit.ViT(types.SimpleNamespace(**args))                # same vit.py, our layers
    attn = ours.transformer_encoder[0].attention
    assert type(attn).__module__.startswith("convolutional-nearest-neighbor-attention_b200")
    assert {k: tuple(v.shape) for k, v in ours.state_dict().items()} == \
           {k: tuple(v.shape) for k, v in stock.state_dict().items()}
    ours.load_state_dict(stock.state_dict(), strict=True)            # reference checkpoint -> drop-in
    stock.load_state_dict(ours.state_dict(), strict=True)            # and back
    mirror = convnn_b200.ViT(convnn_b200.make_args(**args))
    mirror.load_state_dict(stock.state_dict(), strict=True)          # our ViT mirror takes it too
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU path"):
        ours(torch.randn(1, 3, 224, 224))


@pytest.mark.gpu
def test_reference_vit_runs_our_layers_on_the_gpu(reference_modules):
    """install() + the reference's own vit.ViT, built and run on CUDA exactly as main.py builds
    it (vit.py:189-197 constructs the layer, vit.py:263 calls it): the logits must equal the
    stored outputs of the unmodified reference."""
    import types
    from golden_util import vit_case
    ref_layers, ref_vit = reference_modules
    cfg, sd, img, want = vit_case("vit_tiny_cifar_convnn")
    args = {f: getattr(cfg, f) for f in cfg.__dataclass_fields__}
    args.update(device="cuda", img_size=tuple(cfg.img_size))
    convnn_b200.install(ref_layers, ref_vit)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    model = ref_vit.ViT(types.SimpleNamespace(**args)).eval()
    assert type(model.transformer_encoder[0].attention).__module__.startswith(
        "convolutional-nearest-neighbor-attention_b200")
    model.load_state_dict(sd, strict=True)
    with torch.no_grad():
        got = model(img.to("cuda")).float().cpu()
    err = float((got.double() - want.double()).norm() / want.double().norm())
    assert err < 2e-3, err
    assert torch.equal(got.argmax(-1), want.argmax(-1))
