"""Shared test helpers: conversion of synthetic layers to oracle inputs and the
layer parity report used by the GPU tests, smoke() and bench.py."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

import __graft_entry__ as entry

MAX_ABS_TOL = 2e-2      # north-star tolerance on the layer output
COSINE_TOL = 0.9995
# An intermediate FP4 code or scale byte of the device may differ from the oracle's only
# where a shift of the up-projection's pre-activation by at most this many accumulation-
# noise units (2^-24 * sum_c |a_c w_c|, see apply_override in oracle/nmoe_oracle.c) makes
# the reference packer emit the device's byte.  A sequential FP32 sum has an rms error of
# about half a unit; the largest shift measured on B200 over 1.2e8 codes is reported by
# every parity run as `max_noise_units`.
OVERRIDE_LIMIT = 6.0
ADOPTED_FRACTION_MAX = 1e-5   # adopted bytes / intermediate codes: ties are rare


def oracle_config(cfg):
    oracle = entry.load_oracle()
    return oracle.LayerConfig(
        hidden=cfg.hidden_size, routed_intermediate=cfg.routed_expert_intermediate_size,
        shared_intermediate=cfg.shared_expert_intermediate_size, experts=cfg.n_routed_experts,
        top_k=cfg.top_k, n_group=cfg.n_group, topk_group=cfg.topk_group,
        norm_topk_prob=cfg.norm_topk_prob, rms_eps=cfg.rms_epsilon,
        routed_scaling=cfg.routed_scaling_factor,
        latent=0 if cfg.moe_latent_size == cfg.hidden_size else cfg.moe_latent_size)


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        t = t.to(torch.float32)
    return t.detach().cpu().numpy()


def _dense_matrix(linear):
    """(FP32 matrix the reference multiplies with, input scale or 0) of a DenseLinear."""
    if linear is None:
        return None, 0.0
    oracle = entry.load_oracle()
    if linear.is_fp8:
        # DecodeFp8(byte) * weight_scale in FP32 (scaled_fp8_linear.cu:121-139)
        values = oracle.decode_e4m3_array(_np(linear.weight)) * np.float32(linear.weight_scale)
        return values.astype(np.float32), float(linear.input_scale)
    return _np(linear.weight).astype(np.float32), 0.0


def oracle_weights(layer_data):
    oracle = entry.load_oracle()
    b = layer_data.bindings
    fc1, fc1_scale = _dense_matrix(b.fc1_latent)
    fc2, _ = _dense_matrix(b.fc2_latent)
    sup, sup_scale = _dense_matrix(b.shared_up_linear)
    sdown, sdown_scale = _dense_matrix(b.shared_down_linear)
    up_p, up_s, up_t = _np(layer_data.up_packed), _np(layer_data.up_scales), _np(layer_data.up_ts)
    dn_p, dn_s, dn_t = (_np(layer_data.down_packed), _np(layer_data.down_scales),
                        _np(layer_data.down_ts))
    E = up_p.shape[0]
    return oracle.LayerWeights(
        norm_weight=_np(b.input_norm_weight), gate=_np(b.gate_weight),
        bias=_np(b.gate_score_correction_bias),
        up=[oracle.Nvfp4Weight(up_p[e], up_s[e], float(up_t[e])) for e in range(E)],
        down=[oracle.Nvfp4Weight(dn_p[e], dn_s[e], float(dn_t[e])) for e in range(E)],
        shared_up=None if b.shared_up is None else oracle.Nvfp4Weight(
            _np(b.shared_up.packed), _np(b.shared_up.block_scales), b.shared_up.tensor_scale),
        shared_down=None if b.shared_down is None else oracle.Nvfp4Weight(
            _np(b.shared_down.packed), _np(b.shared_down.block_scales),
            b.shared_down.tensor_scale),
        logit_offset=None if b.gate_logit_offset is None else _np(b.gate_logit_offset),
        fc1=fc1, fc1_input_scale=fc1_scale, fc2=fc2, shared_up_dense=sup,
        shared_up_input_scale=sup_scale, shared_down_dense=sdown,
        shared_down_input_scale=sdown_scale)


def max_abs_and_cosine(a: np.ndarray, b: np.ndarray):
    a64, b64 = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    denom = np.linalg.norm(a64) * np.linalg.norm(b64)
    cosine = float(a64 @ b64 / denom) if denom > 0 else 1.0
    return float(np.max(np.abs(a64 - b64))), cosine


def nibble_mismatches(a: np.ndarray, b: np.ndarray) -> int:
    x = np.bitwise_xor(a, b)
    return int(np.count_nonzero(x & 0x0f) + np.count_nonzero(x & 0xf0))


@dataclass
class ParityReport:
    tokens: int = 0
    index_set_mismatches: int = 0
    index_order_mismatches: int = 0
    min_margin: float = 0.0
    norm_max_diff: float = 0.0
    latent_max_diff: float = 0.0   # fc1_latent output (0 when the layer has no projection)
    logits_max_diff: float = 0.0
    weight_max_diff: float = 0.0
    act_code_mismatches: int = 0
    act_scale_mismatches: int = 0
    hidden_code_mismatches: int = 0
    hidden_scale_mismatches: int = 0
    hidden_codes_total: int = 0
    adopted_codes: int = 0
    adopted_scales: int = 0
    inadmissible_codes: int = 0
    inadmissible_scales: int = 0
    max_noise_units: float = 0.0   # largest pre-activation shift among the adopted bytes
    max_rel_shift: float = 0.0     # the same, relative to the pre-activation
    raw_max_abs: float = 0.0
    raw_cosine: float = 0.0
    raw_tokens_over_tol: int = 0           # tokens whose raw error exceeds the tolerance
    raw_tokens_over_tol_without_tie: int = 0  # ... and that own no adopted byte
    max_abs: float = 0.0      # against the oracle run with admissible device codes adopted
    cosine: float = 0.0
    out_is_bf16: bool = False
    bf16_excess: float = 0.0  # worst (|err| - half ulp of bf16 at the reference value)
    notes: list = field(default_factory=list)

    def ok(self) -> bool:
        exact = (self.index_set_mismatches == 0 and self.act_code_mismatches == 0 and
                 self.act_scale_mismatches == 0 and self.inadmissible_codes == 0 and
                 self.inadmissible_scales == 0 and self.latent_max_diff == 0.0)
        if self.out_is_bf16:
            close = self.bf16_excess <= MAX_ABS_TOL
        else:
            close = self.max_abs <= MAX_ABS_TOL
        # non-candidate logits of the two-pass router come from the tensor-core pass;
        # its error must stay far inside the tie margin (2e-4 on scores = 8e-4 on logits)
        router = self.logits_max_diff <= 1e-4 and self.weight_max_diff <= 1e-6
        # ties are rare and close: a systematic error would flip codes everywhere
        adopted = self.adopted_codes + self.adopted_scales
        rare = adopted <= max(4, int(ADOPTED_FRACTION_MAX * self.hidden_codes_total))
        # against the oracle as it is: every token off by more than the tolerance owns a tie
        raw = self.raw_tokens_over_tol_without_tie == 0 and self.raw_cosine >= COSINE_TOL
        return (exact and close and router and rare and raw and self.cosine >= COSINE_TOL and
                self.max_noise_units <= OVERRIDE_LIMIT)

    def summary(self) -> str:
        return (f"T={self.tokens} idx_set_mismatch={self.index_set_mismatches} "
                f"min_margin={self.min_margin:.3g} act_code_mismatch={self.act_code_mismatches} "
                f"hidden_code_mismatch={self.hidden_code_mismatches}/{self.hidden_codes_total} "
                f"hidden_scale_mismatch={self.hidden_scale_mismatches} "
                f"adopted={self.adopted_codes}+{self.adopted_scales} "
                f"inadmissible={self.inadmissible_codes}+{self.inadmissible_scales} "
                f"tie_distance={self.max_noise_units:.3g} noise units "
                f"(rel {self.max_rel_shift:.3g}) "
                f"raw_max_abs={self.raw_max_abs:.3g} raw_cos={self.raw_cosine:.6f} "
                f"raw_tokens_over_tol={self.raw_tokens_over_tol} "
                f"(without a tie: {self.raw_tokens_over_tol_without_tie}) "
                f"max_abs={self.max_abs:.3g} cos={self.cosine:.6f} "
                f"norm_diff={self.norm_max_diff:.3g} latent_diff={self.latent_max_diff:.3g} "
                f"logits_diff={self.logits_max_diff:.3g} "
                f"weight_diff={self.weight_max_diff:.3g}"
                + (f" bf16_excess={self.bf16_excess:.3g}" if self.out_is_bf16 else ""))


def bf16_half_ulp(reference: np.ndarray) -> np.ndarray:
    """Half the bf16 spacing at |reference| (8 significant bits)."""
    mag = np.maximum(np.abs(reference.astype(np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(mag)) - 8)


def compare_layer_with_oracle(layer, layer_data, x: torch.Tensor, out: torch.Tensor,
                              raw_run: bool = True) -> ParityReport:
    """Runs the CPU oracle on the same inputs and compares every stage with the
    intermediates of the layer's last run."""
    oracle = entry.load_oracle()
    cfg = layer.config()
    T = x.shape[0]
    ocfg, ow = oracle_config(cfg), oracle_weights(layer_data)
    x_np = _np(x).astype(np.float32)
    out_np = _np(out).astype(np.float32)
    trace = layer.trace(T)

    rep = ParityReport(tokens=T, out_is_bf16=out.dtype == torch.bfloat16)
    cands = (_np(trace.routed_hidden_packed), _np(trace.routed_hidden_scales),
             _np(trace.shared_hidden_packed), _np(trace.shared_hidden_scales))
    b = layer_data.bindings
    shared_up_dense = b.shared_up_linear is not None
    shared_down_dense = b.shared_down_linear is not None
    forced = oracle.layer_forward(ocfg, ow, x_np, candidates=cands,
                                  override_limit=OVERRIDE_LIMIT)
    raw = oracle.layer_forward(ocfg, ow, x_np) if raw_run else forced

    gi, oi = _np(trace.selected_index), raw.top_index
    rep.index_set_mismatches = int(np.count_nonzero(
        np.any(np.sort(gi, axis=1) != np.sort(oi, axis=1), axis=1)))
    rep.index_order_mismatches = int(np.count_nonzero(np.any(gi != oi, axis=1)))
    rep.min_margin = float(np.min(oracle.selection_margins(raw.logits, ow.bias, cfg.top_k)))
    rep.norm_max_diff = float(np.max(np.abs(_np(trace.normalized_input) - raw.normalized)))
    rep.logits_max_diff = float(np.max(np.abs(_np(trace.router_logits) - raw.logits)))
    rep.weight_max_diff = float(np.max(np.abs(_np(trace.selected_weight) - raw.top_weight)))
    rep.act_code_mismatches = nibble_mismatches(_np(trace.act_packed), raw.act_packed)
    rep.act_scale_mismatches = int(np.count_nonzero(_np(trace.act_scales) != raw.act_scales))
    if trace.latent_output is not None:
        rep.latent_max_diff = float(np.max(np.abs(_np(trace.latent_output) - raw.latent)))
    rep.hidden_code_mismatches = nibble_mismatches(cands[0], raw.hid_packed)
    rep.hidden_scale_mismatches = int(np.count_nonzero(cands[1] != raw.hid_scales))
    rep.hidden_codes_total = int(cands[0].size * 2)
    rep.adopted_codes, rep.adopted_scales = forced.adopted_codes, forced.adopted_scales
    rep.inadmissible_codes = forced.inadmissible_codes
    rep.inadmissible_scales = forced.inadmissible_scales
    if not shared_down_dense:
        # the quantised relu^2 rows of the shared expert; behind a dense or scaled-FP8
        # shared_up both sides accumulate in FP64, so there are no ties to adopt there
        shared_codes = nibble_mismatches(cands[2], raw.shid_packed)
        shared_scales = int(np.count_nonzero(cands[3] != raw.shid_scales))
        rep.hidden_code_mismatches += shared_codes
        rep.hidden_scale_mismatches += shared_scales
        rep.hidden_codes_total += int(cands[2].size * 2)
        if shared_up_dense:
            rep.inadmissible_codes += shared_codes
            rep.inadmissible_scales += shared_scales
    rep.max_noise_units, rep.max_rel_shift = forced.max_noise_units, forced.max_rel_shift
    rep.raw_max_abs, rep.raw_cosine = max_abs_and_cosine(out_np, raw.out)
    rep.max_abs, rep.cosine = max_abs_and_cosine(out_np, forced.out)
    raw_err = np.abs(out_np.astype(np.float64) - raw.out.astype(np.float64))
    if rep.out_is_bf16:
        err = np.abs(out_np.astype(np.float64) - forced.out.astype(np.float64))
        rep.bf16_excess = float(np.max(err - bf16_half_ulp(forced.out)))
        raw_err = raw_err - bf16_half_ulp(raw.out)
    over = raw_err.max(axis=1) > MAX_ABS_TOL
    rep.raw_tokens_over_tol = int(np.count_nonzero(over))
    rep.raw_tokens_over_tol_without_tie = int(np.count_nonzero(over & ~forced.adopted_token))
    return rep
