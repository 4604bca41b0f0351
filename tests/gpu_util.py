"""Helpers shared by the GPU parity tests: every CUDA result is obtained through the C ABI
(convnn_b200.ops / the nn.Modules) and compared with the CPU oracle."""
import torch

import convnn_b200
from convnn_b200 import ops
from oracle.convnn_oracle import ConvNNConfig

DEV = "cuda"


def spec_of(cfg: ConvNNConfig) -> ops.LayerSpec:
    return ops.LayerSpec(cfg.d_hidden, cfg.num_heads, cfg.K, cfg.sampling_type, cfg.magnitude_type,
                         cfg.convolution_type, cfg.softmax_topk_val, cfg.coordinate_encoding, cfg.seq_length)


def conv_params(cfg, w):
    if cfg.convolution_type == "depthwise-separable":
        return (w["conv.0.weight"], w["conv.1.weight"])
    return (w["conv.weight"],)


def pack(cfg, w, dtype):
    return ops.pack_weights(spec_of(cfg), w["W_q.weight"], w["W_k.weight"], w["W_v.weight"], w["W_o.weight"],
                            conv_params(cfg, w), dtype, torch.device(DEV))


def module_of(cfg: ConvNNConfig, w, dtype):
    m = convnn_b200.MultiHeadConvNNAttention(
        cfg.d_hidden, cfg.num_heads, 0.0, cfg.K, cfg.sampling_type, cfg.num_samples, cfg.sample_padding,
        cfg.magnitude_type, cfg.seq_length, cfg.coordinate_encoding, cfg.convolution_type, cfg.softmax_topk_val)
    m.load_state_dict(w, strict=True)
    return m.eval().to(DEV, dtype)


def heads_to_oracle(t, C):
    """(B, R, H, Cp) device tensor -> (B, H, R, C) float32 CPU (oracle layout)."""
    return t[..., :C].permute(0, 2, 1, 3).float().cpu().contiguous()


def rel_err(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
