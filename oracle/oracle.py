"""ctypes/numpy front end of the CPU oracle (oracle/nmoe_oracle.c) and of the
reference driver (oracle/_ref/ref_driver).  TEST INFRASTRUCTURE ONLY: imported by
tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline / reference
arm, never by the shipped package.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import tempfile
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_LIB = os.path.join(HERE, "libnmoe_oracle.so")
REF_BIN = os.path.join(HERE, "_ref", "ref_driver")

_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int32)


class _Nvfp4Weight(ctypes.Structure):
    _fields_ = [("packed", _u8p), ("scales", _u8p), ("tensor_scale", ctypes.c_float)]


class _LayerConfig(ctypes.Structure):
    _fields_ = [("hidden", ctypes.c_int32), ("routed_intermediate", ctypes.c_int32),
                ("shared_intermediate", ctypes.c_int32), ("experts", ctypes.c_int32),
                ("top_k", ctypes.c_int32), ("n_group", ctypes.c_int32),
                ("topk_group", ctypes.c_int32), ("norm_topk_prob", ctypes.c_int32),
                ("rms_eps", ctypes.c_float), ("routed_scaling", ctypes.c_float),
                ("latent", ctypes.c_int32)]


class _LayerWeights(ctypes.Structure):
    _fields_ = [("norm_weight", _f32p), ("gate", _f32p), ("bias", _f32p),
                ("up", ctypes.POINTER(_Nvfp4Weight)), ("down", ctypes.POINTER(_Nvfp4Weight)),
                ("shared_up", _Nvfp4Weight), ("shared_down", _Nvfp4Weight),
                ("logit_offset", _f32p),
                ("fc1", _f32p), ("fc1_input_scale", ctypes.c_float), ("fc2", _f32p),
                ("shared_up_dense", _f32p), ("shared_up_input_scale", ctypes.c_float),
                ("shared_down_dense", _f32p), ("shared_down_input_scale", ctypes.c_float)]


class _OverrideStats(ctypes.Structure):
    _fields_ = [("adopted_codes", ctypes.c_int64), ("adopted_scales", ctypes.c_int64),
                ("inadmissible_codes", ctypes.c_int64), ("inadmissible_scales", ctypes.c_int64),
                ("max_noise_units", ctypes.c_double), ("max_rel_shift", ctypes.c_double)]


class _LayerTrace(ctypes.Structure):
    _fields_ = [("normalized", _f32p), ("logits", _f32p), ("top_index", _i32p),
                ("top_weight", _f32p), ("act_packed", _u8p), ("act_scales", _u8p),
                ("act_tensor_scale", _f32p), ("hid_packed", _u8p), ("hid_scales", _u8p),
                ("routed_out", _f32p), ("shid_packed", _u8p), ("shid_scales", _u8p),
                ("shared_out", _f32p), ("cand_hid_packed", _u8p), ("cand_hid_scales", _u8p),
                ("cand_shid_packed", _u8p), ("cand_shid_scales", _u8p),
                ("override_limit", ctypes.c_float), ("stats", _OverrideStats),
                ("adopted_token", _u8p), ("latent", _f32p), ("routed_latent", _f32p),
                ("projected", _f32p), ("hid_values", _f32p), ("shid_values", _f32p)]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(PORT_LIB):
            import sys
            sys.path.insert(0, HERE)
            import build_oracle
            build_oracle.build_port()
        L = ctypes.CDLL(PORT_LIB)
        L.nmo_decode_e2m1.restype = ctypes.c_float
        L.nmo_decode_e2m1.argtypes = [ctypes.c_uint8]
        L.nmo_decode_e4m3.restype = ctypes.c_float
        L.nmo_decode_e4m3.argtypes = [ctypes.c_uint8]
        L.nmo_encode_e2m1.restype = ctypes.c_uint8
        L.nmo_encode_e2m1.argtypes = [ctypes.c_float]
        L.nmo_encode_e4m3.restype = ctypes.c_uint8
        L.nmo_encode_e4m3.argtypes = [ctypes.c_float]
        L.nmo_sigmoid.restype = ctypes.c_float
        L.nmo_sigmoid.argtypes = [ctypes.c_float]
        L.nmo_pack_nvfp4.argtypes = [_f32p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float,
                                     _u8p, _u8p, _f32p]
        L.nmo_dequant_nvfp4.argtypes = [_u8p, _u8p, ctypes.c_float, ctypes.c_size_t,
                                        ctypes.c_size_t, _f32p]
        L.nmo_swizzled_scale_bytes.restype = ctypes.c_size_t
        L.nmo_swizzled_scale_bytes.argtypes = [ctypes.c_size_t, ctypes.c_size_t]
        L.nmo_swizzle_scales.argtypes = [_u8p, ctypes.c_size_t, ctypes.c_size_t, _u8p]
        L.nmo_quantize_weight.argtypes = [_f32p, ctypes.c_size_t, ctypes.c_size_t, _u8p, _u8p,
                                          _f32p]
        L.nmo_rmsnorm.restype = None
        L.nmo_rmsnorm.argtypes = [_f32p, _f32p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float,
                                  _f32p]
        L.nmo_router_logits.restype = None
        L.nmo_router_logits.argtypes = [_f32p, _f32p, ctypes.c_size_t, ctypes.c_size_t,
                                        ctypes.c_size_t, _f32p]
        L.nmo_select_top_experts.argtypes = [_f32p, _f32p, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_float, _i32p, _f32p]
        L.nmo_selection_margin.restype = ctypes.c_float
        L.nmo_selection_margin.argtypes = [_f32p, _f32p, ctypes.c_int, ctypes.c_int]
        L.nmo_nvfp4_linear_row_literal.argtypes = [_f32p, ctypes.c_size_t, ctypes.c_size_t, _u8p,
                                                   _u8p, ctypes.c_float, _f32p]
        L.nmo_layer_forward.argtypes = [ctypes.POINTER(_LayerConfig),
                                        ctypes.POINTER(_LayerWeights), _f32p, ctypes.c_int64,
                                        _f32p, ctypes.POINTER(_LayerTrace)]
        L.nmo_layer_forward_literal.argtypes = [ctypes.POINTER(_LayerConfig),
                                                ctypes.POINTER(_LayerWeights), _f32p,
                                                ctypes.c_int64, _f32p]
        L.nmo_expert_ffn_forward.argtypes = [
            _f32p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(_Nvfp4Weight),
            ctypes.POINTER(_Nvfp4Weight), _f32p, _u8p, _u8p, _u8p, _u8p, ctypes.c_float,
            ctypes.POINTER(_OverrideStats), _u8p]
        L.nmo_num_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


# ---------------------------------------------------------------------------
# scalar codecs and unit operators
# ---------------------------------------------------------------------------

def decode_e2m1_table() -> np.ndarray:
    return np.array([lib().nmo_decode_e2m1(i) for i in range(16)], dtype=np.float32)


def decode_e4m3_table() -> np.ndarray:
    return np.array([lib().nmo_decode_e4m3(i) for i in range(256)], dtype=np.float32)


def encode_e2m1(values) -> np.ndarray:
    L = lib()
    return np.array([L.nmo_encode_e2m1(float(v)) for v in _f32(values).ravel()], dtype=np.uint8)


def encode_e4m3(values) -> np.ndarray:
    L = lib()
    return np.array([L.nmo_encode_e4m3(float(v)) for v in _f32(values).ravel()], dtype=np.uint8)


def sigmoid(values) -> np.ndarray:
    L = lib()
    return np.array([L.nmo_sigmoid(float(v)) for v in _f32(values).ravel()], dtype=np.float32)


def pack_nvfp4(x, fixed_tensor_scale: float = 0.0):
    """PackRowMajorFp32ToNvfp4 on the whole [rows, cols] matrix (one tensor scale).
    Returns (packed [rows, cols/2], scales [rows, cols/16], tensor_scale) or None when
    the reference would reject the input."""
    x = _f32(x)
    rows, cols = x.shape
    if cols % 16 != 0 or rows == 0:
        return None
    packed = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, cols // 16), dtype=np.uint8)
    ts = ctypes.c_float(0.0)
    rc = lib().nmo_pack_nvfp4(_p(x, _f32p), rows, cols, fixed_tensor_scale, _p(packed, _u8p),
                              _p(scales, _u8p), ctypes.byref(ts))
    if rc != 0:
        return None
    return packed, scales, float(ts.value)


def pack_nvfp4_per_row(x):
    """The layer's usage: every row is its own call (rows == 1)."""
    x = _f32(x)
    rows, cols = x.shape
    packed = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, cols // 16), dtype=np.uint8)
    ts = np.zeros((rows,), dtype=np.float32)
    for r in range(rows):
        p, s, t = pack_nvfp4(x[r:r + 1])
        packed[r], scales[r], ts[r] = p[0], s[0], t
    return packed, scales, ts


def dequant_nvfp4(packed, scales, tensor_scale: float) -> np.ndarray:
    packed, scales = _u8(packed), _u8(scales)
    rows, cols = packed.shape[0], packed.shape[1] * 2
    out = np.zeros((rows, cols), dtype=np.float32)
    lib().nmo_dequant_nvfp4(_p(packed, _u8p), _p(scales, _u8p), tensor_scale, rows, cols,
                            _p(out, _f32p))
    return out


def swizzle_scales(scales, cols: int) -> np.ndarray:
    scales = _u8(scales)
    rows = scales.shape[0]
    out = np.zeros((lib().nmo_swizzled_scale_bytes(rows, cols),), dtype=np.uint8)
    lib().nmo_swizzle_scales(_p(scales, _u8p), rows, cols, _p(out, _u8p))
    return out


def quantize_weight(w):
    """Seeded-harness weight quantiser (global = amax/(6*448)); not in the reference."""
    w = _f32(w)
    rows, cols = w.shape
    packed = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, cols // 16), dtype=np.uint8)
    ts = ctypes.c_float(0.0)
    lib().nmo_quantize_weight(_p(w, _f32p), rows, cols, _p(packed, _u8p), _p(scales, _u8p),
                              ctypes.byref(ts))
    return packed, scales, float(ts.value)


def rmsnorm(x, weight, eps: float) -> np.ndarray:
    x, weight = _f32(x), _f32(weight)
    out = np.zeros_like(x)
    lib().nmo_rmsnorm(_p(x, _f32p), _p(weight, _f32p), x.shape[0], x.shape[1], eps,
                      _p(out, _f32p))
    return out


def router_logits(y, gate) -> np.ndarray:
    y, gate = _f32(y), _f32(gate)
    out = np.zeros((y.shape[0], gate.shape[0]), dtype=np.float32)
    lib().nmo_router_logits(_p(y, _f32p), _p(gate, _f32p), y.shape[0], gate.shape[0], y.shape[1],
                            _p(out, _f32p))
    return out


def select_top_experts(logits, bias, top_k: int, n_group: int = 1, topk_group: int = 1,
                       norm_topk_prob: bool = True, routed_scaling: float = 1.0):
    logits, bias = _f32(logits), _f32(bias)
    rows, experts = logits.shape
    idx = np.zeros((rows, top_k), dtype=np.int32)
    wt = np.zeros((rows, top_k), dtype=np.float32)
    L = lib()
    for r in range(rows):
        row = logits[r]
        L.nmo_select_top_experts(_p(row, _f32p), _p(bias, _f32p), experts, top_k, n_group,
                                 topk_group, 1 if norm_topk_prob else 0, routed_scaling,
                                 _p(idx[r], _i32p), _p(wt[r], _f32p))
    return idx, wt


def selection_margins(logits, bias, top_k: int) -> np.ndarray:
    logits, bias = _f32(logits), _f32(bias)
    L = lib()
    return np.array([L.nmo_selection_margin(_p(logits[r], _f32p), _p(bias, _f32p),
                                            logits.shape[1], top_k)
                     for r in range(logits.shape[0])], dtype=np.float32)


def nvfp4_linear_literal(x, w_packed, w_scales, w_tensor_scale: float) -> np.ndarray:
    """RunNvfp4LinearHost applied row by row."""
    x, w_packed, w_scales = _f32(x), _u8(w_packed), _u8(w_scales)
    rows, k = x.shape
    n = w_packed.shape[0]
    out = np.zeros((rows, n), dtype=np.float32)
    for r in range(rows):
        lib().nmo_nvfp4_linear_row_literal(_p(x[r], _f32p), n, k, _p(w_packed, _u8p),
                                           _p(w_scales, _u8p), w_tensor_scale, _p(out[r], _f32p))
    return out


# ---------------------------------------------------------------------------
# the layer
# ---------------------------------------------------------------------------

@dataclass
class Nvfp4Weight:
    packed: np.ndarray   # [N, K/2] uint8
    scales: np.ndarray   # [N, K/16] uint8
    tensor_scale: float


@dataclass
class LayerWeights:
    norm_weight: np.ndarray          # [H] fp32
    gate: np.ndarray                 # [E, H] fp32 (bf16 values widened)
    bias: np.ndarray                 # [E]
    up: List[Nvfp4Weight]
    down: List[Nvfp4Weight]
    shared_up: Optional[Nvfp4Weight]
    shared_down: Optional[Nvfp4Weight]
    logit_offset: Optional[np.ndarray] = None
    # dense / scaled-FP8 linears as the FP32 matrices the reference multiplies with; an
    # input scale > 0 selects the scaled-FP8 family's activation round trip
    fc1: Optional[np.ndarray] = None               # [latent, H]
    fc1_input_scale: float = 0.0
    fc2: Optional[np.ndarray] = None               # [H, latent]
    shared_up_dense: Optional[np.ndarray] = None   # [S, H]
    shared_up_input_scale: float = 0.0
    shared_down_dense: Optional[np.ndarray] = None  # [H, S]
    shared_down_input_scale: float = 0.0


@dataclass
class LayerConfig:
    hidden: int
    routed_intermediate: int
    shared_intermediate: int
    experts: int
    top_k: int
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = True
    rms_eps: float = 1e-5
    routed_scaling: float = 1.0
    latent: int = 0   # moe_latent_size; 0 = hidden (no latent projections)


def _cw(w: Nvfp4Weight, keep: list) -> _Nvfp4Weight:
    p, s = _u8(w.packed), _u8(w.scales)
    keep.extend([p, s])
    return _Nvfp4Weight(_p(p, _u8p), _p(s, _u8p), w.tensor_scale)


def _c_args(cfg: LayerConfig, w: LayerWeights, keep: list):
    c = _LayerConfig(cfg.hidden, cfg.routed_intermediate, cfg.shared_intermediate, cfg.experts,
                     cfg.top_k, cfg.n_group, cfg.topk_group, 1 if cfg.norm_topk_prob else 0,
                     cfg.rms_eps, cfg.routed_scaling, cfg.latent)
    ups = (_Nvfp4Weight * cfg.experts)(*[_cw(x, keep) for x in w.up])
    downs = (_Nvfp4Weight * cfg.experts)(*[_cw(x, keep) for x in w.down])
    norm, gate, bias = _f32(w.norm_weight), _f32(w.gate), _f32(w.bias)
    keep.extend([norm, gate, bias, ups, downs])
    cw = _LayerWeights()
    cw.norm_weight = _p(norm, _f32p)
    cw.gate = _p(gate, _f32p)
    cw.bias = _p(bias, _f32p)
    cw.up = ups
    cw.down = downs
    if w.shared_up is not None:
        cw.shared_up = _cw(w.shared_up, keep)
    if w.shared_down is not None:
        cw.shared_down = _cw(w.shared_down, keep)
    for name in ("fc1", "fc2", "shared_up_dense", "shared_down_dense"):
        matrix = getattr(w, name)
        if matrix is not None:
            matrix = _f32(matrix)
            keep.append(matrix)
            setattr(cw, name, _p(matrix, _f32p))
    cw.fc1_input_scale = w.fc1_input_scale
    cw.shared_up_input_scale = w.shared_up_input_scale
    cw.shared_down_input_scale = w.shared_down_input_scale
    if w.logit_offset is not None:
        off = _f32(w.logit_offset)
        keep.append(off)
        cw.logit_offset = _p(off, _f32p)
    return c, cw


@dataclass
class LayerResult:
    out: np.ndarray
    normalized: np.ndarray
    logits: np.ndarray
    top_index: np.ndarray
    top_weight: np.ndarray
    act_packed: np.ndarray
    act_scales: np.ndarray
    act_tensor_scale: np.ndarray
    hid_packed: np.ndarray
    hid_scales: np.ndarray
    shid_packed: np.ndarray
    shid_scales: np.ndarray
    routed_out: Optional[np.ndarray]
    shared_out: np.ndarray
    adopted_codes: int = 0
    adopted_scales: int = 0
    inadmissible_codes: int = 0
    inadmissible_scales: int = 0
    max_noise_units: float = 0.0       # largest adopted pre-activation shift, in noise units
    max_rel_shift: float = 0.0         # the same shift relative to the pre-activation
    adopted_token: Optional[np.ndarray] = None  # [T] bool: the token owns an adopted byte
    latent: Optional[np.ndarray] = None         # [T, latent] fc1_latent output
    routed_latent: Optional[np.ndarray] = None  # [T, latent] routed sum
    projected: Optional[np.ndarray] = None      # [T, H] fc2_latent of it
    hid_values: Optional[np.ndarray] = None     # [T, k, I] relu^2(up_proj) before quantisation
    shid_values: Optional[np.ndarray] = None    # [T, S]


DEFAULT_OVERRIDE_LIMIT = 6.0


def layer_forward(cfg: LayerConfig, w: LayerWeights, x, candidates=None,
                  override_limit: float = DEFAULT_OVERRIDE_LIMIT,
                  want_routed_out: bool = False) -> LayerResult:
    """The whole layer on FP32 input [T, H].  `candidates` = (hid_packed [T,k,I/2],
    hid_scales [T,k,I/16], shid_packed [T,S/2], shid_scales [T,S/16]) from the device
    turns on the admissible-code override: a differing intermediate byte is adopted when
    a shift of the pre-activation by at most `override_limit` accumulation-noise units
    (2^-24 * sum |a_c w_c|) makes the reference packer emit it."""
    x = _f32(x)
    T = x.shape[0]
    H, I, S, E, K = (cfg.hidden, cfg.routed_intermediate, cfg.shared_intermediate, cfg.experts,
                     cfg.top_k)
    L = cfg.latent or H
    keep: list = []
    c, cw = _c_args(cfg, w, keep)
    out = np.zeros((T, H), dtype=np.float32)
    r = LayerResult(
        out=out, normalized=np.zeros((T, H), np.float32), logits=np.zeros((T, E), np.float32),
        top_index=np.zeros((T, K), np.int32), top_weight=np.zeros((T, K), np.float32),
        act_packed=np.zeros((T, L // 2), np.uint8), act_scales=np.zeros((T, L // 16), np.uint8),
        act_tensor_scale=np.zeros((T,), np.float32),
        hid_packed=np.zeros((T, K, I // 2), np.uint8), hid_scales=np.zeros((T, K, I // 16), np.uint8),
        shid_packed=np.zeros((T, S // 2), np.uint8), shid_scales=np.zeros((T, S // 16), np.uint8),
        routed_out=np.zeros((T, K, L), np.float32) if want_routed_out else None,
        shared_out=np.zeros((T, H), np.float32), latent=np.zeros((T, L), np.float32),
        routed_latent=np.zeros((T, L), np.float32), projected=np.zeros((T, H), np.float32))
    tr = _LayerTrace()
    tr.normalized = _p(r.normalized, _f32p)
    tr.logits = _p(r.logits, _f32p)
    tr.top_index = _p(r.top_index, _i32p)
    tr.top_weight = _p(r.top_weight, _f32p)
    tr.act_packed = _p(r.act_packed, _u8p)
    tr.act_scales = _p(r.act_scales, _u8p)
    tr.act_tensor_scale = _p(r.act_tensor_scale, _f32p)
    tr.hid_packed = _p(r.hid_packed, _u8p)
    tr.hid_scales = _p(r.hid_scales, _u8p)
    tr.shid_packed = _p(r.shid_packed, _u8p)
    tr.shid_scales = _p(r.shid_scales, _u8p)
    if want_routed_out:
        tr.routed_out = _p(r.routed_out, _f32p)
    tr.shared_out = _p(r.shared_out, _f32p)
    tr.latent = _p(r.latent, _f32p)
    tr.routed_latent = _p(r.routed_latent, _f32p)
    tr.projected = _p(r.projected, _f32p)
    if want_routed_out:
        r.hid_values = np.zeros((T, K, I), np.float32)
        r.shid_values = np.zeros((T, S), np.float32)
        tr.hid_values = _p(r.hid_values, _f32p)
        tr.shid_values = _p(r.shid_values, _f32p)
    tr.override_limit = override_limit
    adopted_token = np.zeros((T,), np.uint8)
    tr.adopted_token = _p(adopted_token, _u8p)
    if candidates is not None:
        cands = [_u8(a) for a in candidates]
        keep.extend(cands)
        tr.cand_hid_packed = _p(cands[0], _u8p)
        tr.cand_hid_scales = _p(cands[1], _u8p)
        tr.cand_shid_packed = _p(cands[2], _u8p)
        tr.cand_shid_scales = _p(cands[3], _u8p)
    rc = lib().nmo_layer_forward(ctypes.byref(c), ctypes.byref(cw), _p(x, _f32p), T,
                                 _p(out, _f32p), ctypes.byref(tr))
    if rc != 0:
        raise RuntimeError(f"nmo_layer_forward failed with {rc}")
    r.adopted_codes = tr.stats.adopted_codes
    r.adopted_scales = tr.stats.adopted_scales
    r.inadmissible_codes = tr.stats.inadmissible_codes
    r.inadmissible_scales = tr.stats.inadmissible_scales
    r.max_noise_units = tr.stats.max_noise_units
    r.max_rel_shift = tr.stats.max_rel_shift
    r.adopted_token = adopted_token.astype(bool)
    return r


def fp8_round_trip(x, input_scale: float) -> np.ndarray:
    """The scaled-FP8 family's activation round trip (scaled_fp8_linear.cu:231-236)."""
    x = _f32(x)
    out = np.zeros_like(x)
    L = lib()
    L.nmo_fp8_round_trip.argtypes = [_f32p, ctypes.c_size_t, ctypes.c_float, _f32p]
    L.nmo_fp8_round_trip.restype = None
    L.nmo_fp8_round_trip(_p(x, _f32p), x.size, ctypes.c_float(input_scale), _p(out, _f32p))
    return out


def decode_e4m3_array(codes) -> np.ndarray:
    """E4M3 bytes -> FP32 values (DecodeFp8, scaled_fp8_linear.cu:35-39)."""
    return decode_e4m3_table()[np.asarray(codes, dtype=np.uint8)]


def layer_forward_literal(cfg: LayerConfig, w: LayerWeights, x) -> np.ndarray:
    x = _f32(x)
    keep: list = []
    c, cw = _c_args(cfg, w, keep)
    out = np.zeros((x.shape[0], cfg.hidden), dtype=np.float32)
    rc = lib().nmo_layer_forward_literal(ctypes.byref(c), ctypes.byref(cw), _p(x, _f32p),
                                         x.shape[0], _p(out, _f32p))
    if rc != 0:
        raise RuntimeError(f"nmo_layer_forward_literal failed with {rc}")
    return out


@dataclass
class FfnResult:
    out: np.ndarray
    hid_packed: np.ndarray
    hid_scales: np.ndarray
    adopted_codes: int = 0
    adopted_scales: int = 0
    inadmissible_codes: int = 0
    inadmissible_scales: int = 0
    max_noise_units: float = 0.0
    max_rel_shift: float = 0.0
    adopted_row: Optional[np.ndarray] = None


def expert_ffn_forward(x, up: Nvfp4Weight, down: Nvfp4Weight, candidates=None,
                       override_limit: float = DEFAULT_OVERRIDE_LIMIT) -> FfnResult:
    """down(relu^2(up(x))) per row, both projections through the NVFP4 host linear with
    the weights dequantised once (bit-equal to `expert_ffn`, fast).  `candidates` =
    (hid_packed [R, I/2], hid_scales [R, I/16]) from the device turns on the
    admissible-code override of `layer_forward`."""
    x = _f32(x)
    R, H = x.shape
    I = up.packed.shape[0]
    keep: list = []
    cup, cdown = _cw(up, keep), _cw(down, keep)
    res = FfnResult(out=np.zeros((R, H), np.float32), hid_packed=np.zeros((R, I // 2), np.uint8),
                    hid_scales=np.zeros((R, I // 16), np.uint8))
    stats = _OverrideStats()
    adopted = np.zeros((R,), np.uint8)
    cq = cs = None
    if candidates is not None:
        cq, cs = _u8(candidates[0]), _u8(candidates[1])
    rc = lib().nmo_expert_ffn_forward(
        _p(x, _f32p), R, H, I, ctypes.byref(cup), ctypes.byref(cdown), _p(res.out, _f32p),
        _p(res.hid_packed, _u8p), _p(res.hid_scales, _u8p),
        _p(cq, _u8p) if cq is not None else None, _p(cs, _u8p) if cs is not None else None,
        ctypes.c_float(override_limit), ctypes.byref(stats), _p(adopted, _u8p))
    if rc != 0:
        raise RuntimeError(f"nmo_expert_ffn_forward failed with {rc}")
    for name in ("adopted_codes", "adopted_scales", "inadmissible_codes", "inadmissible_scales",
                 "max_noise_units", "max_rel_shift"):
        setattr(res, name, getattr(stats, name))
    res.adopted_row = adopted.astype(bool)
    return res


def expert_ffn(x, up: Nvfp4Weight, down: Nvfp4Weight):
    """down(relu^2(up(x))) per row composed from the literal row linear (re-dequantises
    the weight for every row: slow, small shapes only).  Returns (hidden, out)."""
    x = _f32(x)
    h = nvfp4_linear_literal(x, up.packed, up.scales, up.tensor_scale)
    h = np.where(h > 0, h * h, 0).astype(np.float32)
    return h, nvfp4_linear_literal(h, down.packed, down.scales, down.tensor_scale)


def num_threads() -> int:
    return int(lib().nmo_num_threads())


# ---------------------------------------------------------------------------
# reference driver
# ---------------------------------------------------------------------------

def have_reference() -> bool:
    return os.path.exists(REF_BIN) and os.access(REF_BIN, os.X_OK)


def ref_run(command: str, args: list, inputs: dict, outputs: dict) -> dict:
    """Runs oracle/_ref/ref_driver.  `inputs` maps placeholder -> ndarray, `outputs`
    maps placeholder -> dtype; `args` may contain the placeholders."""
    with tempfile.TemporaryDirectory() as tmp:
        paths = {}
        for name, array in inputs.items():
            paths[name] = os.path.join(tmp, name + ".bin")
            np.ascontiguousarray(array).tofile(paths[name])
        for name in outputs:
            paths[name] = os.path.join(tmp, name + ".out")
        argv = [REF_BIN, command] + [paths.get(a, str(a)) for a in args]
        subprocess.run(argv, check=True)
        return {name: np.fromfile(paths[name], dtype=dt) for name, dt in outputs.items()}
