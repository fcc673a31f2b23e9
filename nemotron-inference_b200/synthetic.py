"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (the real NVFP4 checkpoint is not available): bf16 activations
~N(0,1), N(0,0.02) FP32 weights quantised to NVFP4 with a global scale of
amax/(6*448), bf16 gate ~N(0,0.02), correction bias ~U(-0.01,0.01).

The weight quantiser below is harness code, not part of the operator (the
reference only consumes checkpoint-quantised weights): block scale =
E4M3(amax_b / (6*global)), code = E2M1_RNE(w / (global * decoded block scale)).
It is written with torch so that it runs on the GPU for the full-size
configurations; tests pin it bit for bit to the CPU oracle's quantiser.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from . import (DenseLinear, ExpertLayerBindings, ExpertLayerConfig, ExpertWeightPair,
               Nvfp4Matrix)

HIDDEN = 2688
ROUTED_INTERMEDIATE = 1856
SHARED_INTERMEDIATE = 3712
EXPERTS = 128
TOP_K = 6
ROUTED_SCALING = 2.5


def baseline_config(max_tokens: int, experts: int = EXPERTS, hidden: int = HIDDEN,
                    routed: int = ROUTED_INTERMEDIATE, shared: int = SHARED_INTERMEDIATE,
                    top_k: int = TOP_K, latent: int = 0) -> ExpertLayerConfig:
    return ExpertLayerConfig(layer_index=0, hidden_size=hidden, moe_latent_size=latent or hidden,
                             routed_expert_intermediate_size=routed,
                             shared_expert_intermediate_size=shared, n_routed_experts=experts,
                             top_k=top_k, n_group=1, topk_group=1, rms_epsilon=1e-5,
                             routed_scaling_factor=ROUTED_SCALING, norm_topk_prob=True,
                             max_tokens=max_tokens)


def encode_e2m1(q: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even E2M1 codes (uint8 0..15) of a float tensor, saturating."""
    a = q.abs()
    code = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
            + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8)
            + (a >= 3.5).to(torch.uint8) + (a > 5.0).to(torch.uint8))
    return code | (torch.signbit(q).to(torch.uint8) << 3)


def quantize_weight(w: torch.Tensor):
    """[..., N, K] FP32 -> (packed [..., N, K/2] uint8, scales [..., N, K/16] uint8,
    tensor_scale [...] FP32), one global scale per matrix."""
    *lead, n, k = w.shape
    assert k % 16 == 0
    w = w.to(torch.float32)
    amax = w.abs().amax(dim=(-2, -1), keepdim=True)
    global_scale = amax / (6.0 * 448.0)
    global_scale = torch.where(global_scale > 0, global_scale, torch.ones_like(global_scale))
    blocks = w.reshape(*lead, n, k // 16, 16)
    block_max = blocks.abs().amax(dim=-1)
    ratio = block_max / (6.0 * global_scale)
    codes = ratio.to(torch.float8_e4m3fn)
    decoded = codes.to(torch.float32)
    zero = ~(decoded > 0)
    one = torch.tensor(1.0, dtype=torch.float32, device=w.device).to(torch.float8_e4m3fn)
    codes = torch.where(zero, one, codes)
    decoded = torch.where(zero, torch.ones_like(decoded), decoded)
    scale = (global_scale * decoded).unsqueeze(-1)
    nibbles = encode_e2m1(blocks / scale).reshape(*lead, n, k // 2, 2)
    packed = nibbles[..., 0] | (nibbles[..., 1] << 4)
    return packed.contiguous(), codes.view(torch.uint8).contiguous(), global_scale.reshape(tuple(lead))


@dataclass
class SyntheticLayer:
    config: ExpertLayerConfig
    bindings: ExpertLayerBindings
    # stacked copies, convenient for the oracle: [E, ...]
    up_packed: torch.Tensor
    up_scales: torch.Tensor
    up_ts: torch.Tensor
    down_packed: torch.Tensor
    down_scales: torch.Tensor
    down_ts: torch.Tensor


def _normal(shape, std, generator, device):
    return torch.randn(shape, generator=generator, device=device, dtype=torch.float32) * std


def zipf_logit_offset(experts: int, seed: int, head: float = 0.2, tail: float = 2.5,
                      s: float = 1.1) -> torch.Tensor:
    """Per-expert gate-logit offset that skews the expert load (configs[2]).  A seeded
    random ranking gives each expert a Zipf(s) popularity p ~ rank^-s; the offset is
    log p centred on its mean, with the popular side scaled by `head` and the unpopular
    side by `tail`.  With ~N(0,1) logits and top-6 of 128 the defaults give a hottest
    expert near 5x the mean load and a handful of experts with no tokens at T=8192."""
    g = torch.Generator().manual_seed(seed)
    ranks = torch.randperm(experts, generator=g).to(torch.float32) + 1.0
    logp = -s * torch.log(ranks)
    centred = logp - logp.mean()
    return torch.where(centred > 0, head * centred, tail * centred).to(torch.float32)


def checkpoint_shape_config(max_tokens: int) -> ExpertLayerConfig:
    """The latent-MoE shape of the reference's checkpoint
    (runtime/src/api/single_token_forward_model.cpp:116-126)."""
    return ExpertLayerConfig(layer_index=0, hidden_size=4096, moe_latent_size=1024,
                             routed_expert_intermediate_size=2688,
                             shared_expert_intermediate_size=5376, n_routed_experts=512,
                             top_k=22, n_group=1, topk_group=1, rms_epsilon=1e-5,
                             routed_scaling_factor=5.0, norm_topk_prob=True,
                             max_tokens=max_tokens)


def quantize_fp8(w: torch.Tensor):
    """Per-tensor E4M3 weight of the scaled-FP8 family: (codes uint8, weight_scale)."""
    scale = float(w.abs().max().item()) / 448.0
    codes = (w.to(torch.float32) / scale).to(torch.float8_e4m3fn).view(torch.uint8)
    return codes.contiguous(), scale


def _make_linear(shape, family: str, generator, device) -> DenseLinear:
    w = _normal(shape, 0.02, generator, device)
    if family == "fp8":
        codes, scale = quantize_fp8(w)
        return DenseLinear(codes, weight_scale=scale, input_scale=8.0 / 448.0)
    if family == "fp32":
        return DenseLinear(w)
    return DenseLinear(w.to(torch.bfloat16))


def make_layer(config: ExpertLayerConfig, seed: int, device="cpu", norm_weight_uniform=False,
               skewed: bool = False, chunk: int = 16, latent_family: str = "bf16",
               shared_up_family: str = "nvfp4", shared_down_family: str = "nvfp4"
               ) -> SyntheticLayer:
    """Seeded layer weights.  Generation runs on `device` (the stream of random
    numbers depends on the device type); the quantised bytes stay there.
    With config.moe_latent_size != hidden_size the layer gets fc1_latent / fc2_latent
    (fc1 in `latent_family`: "bf16", "fp32" or "fp8"; fc2 dense); the shared expert's
    projections are "nvfp4", "bf16", "fp32" or "fp8"."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    H, I, S, E = (config.moe_latent_size, config.routed_expert_intermediate_size,
                  config.shared_expert_intermediate_size, config.n_routed_experts)
    full_hidden = config.hidden_size
    latent_mode = H != full_hidden
    return _make_layer(config, g, dev, H, full_hidden, I, S, E, latent_mode, norm_weight_uniform,
                       skewed, chunk, seed, latent_family, shared_up_family, shared_down_family)


def _make_layer(config, g, dev, H, full_hidden, I, S, E, latent_mode, norm_weight_uniform, skewed,
                chunk, seed, latent_family, shared_up_family, shared_down_family):
    # H is the row length the routed experts see (the latent size, or the hidden size)
    gate = _normal((E, full_hidden), 0.02, g, dev).to(torch.bfloat16)
    bias = (torch.rand((E,), generator=g, device=dev) * 0.02 - 0.01).to(torch.float32)
    if norm_weight_uniform:
        norm = (torch.rand((full_hidden,), generator=g, device=dev) * 0.2 + 0.9).to(torch.float32)
    else:
        norm = torch.ones((full_hidden,), dtype=torch.float32, device=dev)
    ups, downs = [], []
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        ups.append(quantize_weight(_normal((n, I, H), 0.02, g, dev)))
        downs.append(quantize_weight(_normal((n, H, I), 0.02, g, dev)))
    up_p, up_s, up_t = (torch.cat([u[i] for u in ups]) for i in range(3))
    dn_p, dn_s, dn_t = (torch.cat([d[i] for d in downs]) for i in range(3))
    su = quantize_weight(_normal((S, full_hidden), 0.02, g, dev))
    sd = quantize_weight(_normal((full_hidden, S), 0.02, g, dev))
    up_t_host, dn_t_host = up_t.cpu(), dn_t.cpu()
    routed = [ExpertWeightPair(Nvfp4Matrix(up_p[e], up_s[e], float(up_t_host[e])),
                               Nvfp4Matrix(dn_p[e], dn_s[e], float(dn_t_host[e])))
              for e in range(E)]
    offset = None
    if skewed:
        offset = zipf_logit_offset(E, seed + 7).to(dev)
    bindings = ExpertLayerBindings(
        input_norm_weight=norm, gate_weight=gate, gate_score_correction_bias=bias,
        shared_up=Nvfp4Matrix(su[0], su[1], float(su[2])),
        shared_down=Nvfp4Matrix(sd[0], sd[1], float(sd[2])),
        routed_experts=routed, gate_logit_offset=offset)
    # drawn after everything else so that the layers without them keep their weights
    if latent_mode:
        bindings.fc1_latent = _make_linear((H, full_hidden), latent_family, g, dev)
        bindings.fc2_latent = _make_linear((full_hidden, H), "bf16", g, dev)
    if shared_up_family != "nvfp4":
        bindings.shared_up_linear = _make_linear((S, full_hidden), shared_up_family, g, dev)
        bindings.shared_up = None
    if shared_down_family != "nvfp4":
        bindings.shared_down_linear = _make_linear((full_hidden, S), shared_down_family, g, dev)
        bindings.shared_down = None
    return SyntheticLayer(config, bindings, up_p, up_s, up_t, dn_p, dn_s, dn_t)


def make_tokens(tokens: int, hidden: int, seed: int, device="cpu") -> torch.Tensor:
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn((tokens, hidden), generator=g, device=dev,
                       dtype=torch.float32).to(torch.bfloat16)


def make_ffn_weights(hidden: int, intermediate: int, seed: int, device="cpu"):
    """configs[0]: one routed expert, W_up [I, H] and W_down [H, I] ~N(0, 0.02)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    up = quantize_weight(_normal((intermediate, hidden), 0.02, g, dev))
    down = quantize_weight(_normal((hidden, intermediate), 0.02, g, dev))
    return (Nvfp4Matrix(up[0], up[1], float(up[2])), Nvfp4Matrix(down[0], down[1], float(down[2])))
