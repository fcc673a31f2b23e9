"""Bindings of one expert layer from checkpoint tensors, by the reference's tensor names.

The reference resolves a layer's tensors by exact local name under
`backbone.layers.<i>.` (BuildExpertLayerBindings, runtime/src/backend/expert_layer.cpp:427-492)
and takes an NVFP4 matrix from three checkpoint tensors: `<name>.weight` (packed E2M1,
uint8 [N, K/2]), `<name>.weight_scale` (E4M3 block scales [N, K/16]) and, as the FP32 tensor
scale, `<name>.weight_scale_2` or else `<name>.input_scale`
(tools/manifest/generate_forward_manifest.py:344-400).  A scaled-FP8 linear is `<name>.weight`
in E4M3 with scalar `<name>.weight_scale` and `<name>.input_scale`
(expert_layer.cpp:84-105); anything else is a dense FP32 / bf16 matrix.

`bindings_from_tensors` does the same over a name -> tensor mapping (a loaded safetensors
shard, a state dict), hands the tensors to `ExpertLayerSlice.create` without repacking them,
and can take one rank's slice of the routed experts for expert parallelism.  Tensors may
live on the host or on the device: the library copies them once, expert by expert, into its
own layout in HBM.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from . import DenseLinear, ExpertLayerBindings, ExpertWeightPair, Nvfp4Matrix

_FP8 = getattr(torch, "float8_e4m3fn", None)


def _bytes(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.uint8) if t.dtype != torch.uint8 else t


def _scalar(t: torch.Tensor) -> float:
    return float(t.to(torch.float32).reshape(-1)[0].item())


def _is_fp8(t: torch.Tensor) -> bool:
    return _FP8 is not None and t.dtype == _FP8


def nvfp4_matrix(tensors: Mapping[str, torch.Tensor], name: str) -> Optional[Nvfp4Matrix]:
    """`name` without the trailing `.weight`.  None when the NVFP4 triple is not there."""
    weight = tensors.get(name + ".weight")
    scales = tensors.get(name + ".weight_scale")
    tensor_scale = tensors.get(name + ".weight_scale_2")
    if tensor_scale is None:
        tensor_scale = tensors.get(name + ".input_scale")
    if weight is None or scales is None or tensor_scale is None:
        return None
    if weight.dtype != torch.uint8 or scales.dim() != 2 or scales.numel() == 1:
        return None  # not packed E2M1 with per-block scales
    if weight.shape[0] != scales.shape[0] or weight.shape[1] * 2 != scales.shape[1] * 16:
        return None
    return Nvfp4Matrix(weight, _bytes(scales), _scalar(tensor_scale))


def dense_linear(tensors: Mapping[str, torch.Tensor], name: str) -> Optional[DenseLinear]:
    """The scaled-FP8 family when its three tensors are there, else the dense family."""
    weight = tensors.get(name + ".weight")
    if weight is None or weight.dim() != 2:
        return None
    weight_scale = tensors.get(name + ".weight_scale")
    input_scale = tensors.get(name + ".input_scale")
    if _is_fp8(weight) and weight_scale is not None and input_scale is not None and \
            weight_scale.numel() == 1 and input_scale.numel() == 1:
        return DenseLinear(_bytes(weight), weight_scale=_scalar(weight_scale),
                           input_scale=_scalar(input_scale))
    if weight.dtype in (torch.float32, torch.bfloat16):
        return DenseLinear(weight)
    return None


def bindings_from_tensors(tensors: Mapping[str, torch.Tensor], layer_index: int,
                          n_routed_experts: int, rank: int = 0, world: int = 1,
                          prefix: str = "backbone.layers.") -> Optional[ExpertLayerBindings]:
    """The layer's bindings, or None when a required tensor is missing (the reference
    returns std::nullopt, expert_layer.cpp:473-490).  With world > 1 only the routed
    experts of `rank` are bound (and need be present)."""
    base = f"{prefix}{layer_index}."
    norm = tensors.get(base + "norm.weight")
    gate = tensors.get(base + "mixer.gate.weight")
    bias = tensors.get(base + "mixer.gate.e_score_correction_bias")
    if norm is None or gate is None or bias is None or n_routed_experts % world != 0:
        return None
    per_rank = n_routed_experts // world
    routed = []
    for expert in range(rank * per_rank, (rank + 1) * per_rank):
        up = nvfp4_matrix(tensors, f"{base}mixer.experts.{expert}.up_proj")
        down = nvfp4_matrix(tensors, f"{base}mixer.experts.{expert}.down_proj")
        if up is None or down is None:
            return None
        routed.append(ExpertWeightPair(up, down))
    bindings = ExpertLayerBindings(
        input_norm_weight=norm, gate_weight=gate, gate_score_correction_bias=bias.to(torch.float32),
        shared_up=None, shared_down=None, routed_experts=routed,
        first_local_expert=rank * per_rank)
    # shared expert: NVFP4 where the checkpoint has the triple, else scaled FP8 or dense
    for which in ("up", "down"):
        name = f"{base}mixer.shared_experts.{which}_proj"
        matrix = nvfp4_matrix(tensors, name)
        linear = None if matrix is not None else dense_linear(tensors, name)
        if matrix is None and linear is None:
            return None
        setattr(bindings, f"shared_{which}", matrix)
        setattr(bindings, f"shared_{which}_linear", linear)
    # latent projections: both or neither
    fc1 = dense_linear(tensors, base + "mixer.fc1_latent_proj")
    fc2 = dense_linear(tensors, base + "mixer.fc2_latent_proj")
    if (fc1 is None) != (fc2 is None) or (fc2 is not None and fc2.is_fp8):
        return None
    bindings.fc1_latent, bindings.fc2_latent = fc1, fc2
    return bindings


def tensors_from_bindings(bindings: ExpertLayerBindings, layer_index: int,
                          prefix: str = "backbone.layers.") -> dict:
    """The inverse mapping (what a checkpoint of this layer would contain): used by the
    tests and to write synthetic layers out in the reference's naming."""
    base = f"{prefix}{layer_index}."
    out = {base + "norm.weight": bindings.input_norm_weight,
           base + "mixer.gate.weight": bindings.gate_weight,
           base + "mixer.gate.e_score_correction_bias": bindings.gate_score_correction_bias}

    def put_nvfp4(name, m: Nvfp4Matrix):
        out[name + ".weight"] = m.packed
        out[name + ".weight_scale"] = m.block_scales.view(_FP8) if _FP8 is not None \
            else m.block_scales
        out[name + ".weight_scale_2"] = torch.tensor([m.tensor_scale], dtype=torch.float32)

    def put_linear(name, l: DenseLinear):
        if l.is_fp8:
            out[name + ".weight"] = l.weight.view(_FP8)
            out[name + ".weight_scale"] = torch.tensor(l.weight_scale, dtype=torch.float32)
            out[name + ".input_scale"] = torch.tensor(l.input_scale, dtype=torch.float32)
        else:
            out[name + ".weight"] = l.weight

    for offset, pair in enumerate(bindings.routed_experts):
        expert = bindings.first_local_expert + offset
        put_nvfp4(f"{base}mixer.experts.{expert}.up_proj", pair.up_proj)
        put_nvfp4(f"{base}mixer.experts.{expert}.down_proj", pair.down_proj)
    for which in ("up", "down"):
        name = f"{base}mixer.shared_experts.{which}_proj"
        matrix = getattr(bindings, f"shared_{which}")
        if matrix is not None:
            put_nvfp4(name, matrix)
        else:
            put_linear(name, getattr(bindings, f"shared_{which}_linear"))
    if bindings.fc1_latent is not None:
        put_linear(base + "mixer.fc1_latent_proj", bindings.fc1_latent)
        put_linear(base + "mixer.fc2_latent_proj", bindings.fc2_latent)
    return out
