"""B200 NVFP4 mixture-of-experts expert layer: Python host side over the C ABI.

The classes mirror the reference operator's interface
(`nemotron::ExpertLayerConfig`, `ExpertLayerBindings`, `ExpertLayerSlice`,
runtime/include/nemotron/expert_layer.h:18-105) so that a test written against
the reference reads the same here.  torch is used for device memory and streams
only; every computation goes through `libnmoe_b200.so` (include/nmoe.h).  There
is no CPU path: without the built library, or without a CUDA device, the
operators raise.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libnmoe_b200.so")

NMOE_OK = 0
NMOE_F32 = 0
NMOE_BF16 = 1
NMOE_F16 = 2   # only for the rows expert-parallel ranks return

STATUS_NAMES = {
    0: "NMOE_OK", 1: "NMOE_ERR_INVALID_ARGUMENT", 2: "NMOE_ERR_CUDA", 3: "NMOE_ERR_UNSUPPORTED",
    4: "NMOE_ERR_DEVICE_TIMEOUT", 5: "NMOE_ERR_ACTIVATION_RANGE", 6: "NMOE_ERR_CAPACITY",
}

# Every symbol include/nmoe.h declares.
EXPORTED_SYMBOLS = (
    "nmoe_status_string", "nmoe_layer_create", "nmoe_layer_destroy", "nmoe_layer_run",
    "nmoe_layer_sync_status", "nmoe_layer_last_error", "nmoe_layer_trace_view",
    "nmoe_layer_copy_trace_field", "nmoe_layer_enable_stage_timing", "nmoe_layer_stage_times",
    "nmoe_layer_export_hidden", "nmoe_ffn_create", "nmoe_ffn_destroy", "nmoe_ffn_run",
    "nmoe_ffn_sync_status", "nmoe_ffn_export_hidden", "nmoe_quantize_nvfp4",
    "nmoe_dequant_nvfp4", "nmoe_swizzled_scale_bytes", "nmoe_swizzle_scales", "nmoe_rmsnorm",
    "nmoe_router_logits", "nmoe_router_topk", "nmoe_route_tokens_noalloc",
    "nmoe_ep_record_bytes", "nmoe_ep_dispatch", "nmoe_ep_experts", "nmoe_ep_shared",
    "nmoe_ep_combine", "nmoe_layer_reserve_sms", "nmoe_ep_window_create",
    "nmoe_ep_window_attach", "nmoe_ep_window_detach", "nmoe_ep_window_dispatch",
    "nmoe_ep_window_experts", "nmoe_ep_window_combine", "nmoe_ep_window_fork_shared",
    "nmoe_layer_set_wait_limit_ms", "nmoe_layer_wait_flag", "nmoe_layer_reserve_tokens",
    "nmoe_layer_set_unfused_activation", "nmoe_layer_export_unfused", "nmoe_layer_keep_trace",
)


class NmoeError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        name = STATUS_NAMES.get(status, str(status))
        super().__init__(f"{where}: {name}" + (f" ({detail})" if detail else ""))


class _Config(ctypes.Structure):
    _fields_ = [("layer_index", ctypes.c_int32), ("hidden_size", ctypes.c_int32),
                ("moe_latent_size", ctypes.c_int32),
                ("routed_expert_intermediate_size", ctypes.c_int32),
                ("shared_expert_intermediate_size", ctypes.c_int32),
                ("n_routed_experts", ctypes.c_int32), ("top_k", ctypes.c_int32),
                ("n_group", ctypes.c_int32), ("topk_group", ctypes.c_int32),
                ("norm_topk_prob", ctypes.c_int32), ("rms_epsilon", ctypes.c_float),
                ("routed_scaling_factor", ctypes.c_float), ("max_tokens", ctypes.c_int32),
                ("max_recv_pairs", ctypes.c_int32)]


class _Nvfp4Matrix(ctypes.Structure):
    _fields_ = [("output_rows", ctypes.c_size_t), ("input_cols", ctypes.c_size_t),
                ("packed_data", ctypes.c_void_p), ("packed_nbytes", ctypes.c_size_t),
                ("block_scales_data", ctypes.c_void_p), ("block_scales_nbytes", ctypes.c_size_t),
                ("tensor_scale_data", ctypes.c_void_p), ("tensor_scale_nbytes", ctypes.c_size_t)]


class _DenseTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("nbytes", ctypes.c_size_t),
                ("dtype", ctypes.c_int), ("rows", ctypes.c_size_t), ("cols", ctypes.c_size_t)]


class _Linear(ctypes.Structure):
    _fields_ = [("family", ctypes.c_int), ("weight", _DenseTensor),
                ("weight_scale", ctypes.c_float), ("input_scale", ctypes.c_float)]


class _Weights(ctypes.Structure):
    _fields_ = [("input_norm_weight", _DenseTensor), ("gate_weight", _DenseTensor),
                ("gate_score_correction_bias", _DenseTensor),
                ("routed_up", ctypes.POINTER(_Nvfp4Matrix)),
                ("routed_down", ctypes.POINTER(_Nvfp4Matrix)),
                ("n_local_experts", ctypes.c_int32), ("first_local_expert", ctypes.c_int32),
                ("shared_up", _Nvfp4Matrix), ("shared_down", _Nvfp4Matrix),
                ("gate_logit_offset", ctypes.c_void_p),
                ("fc1_latent", _Linear), ("fc2_latent", _Linear),
                ("shared_up_linear", _Linear), ("shared_down_linear", _Linear)]


class _TraceView(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in (
        "normalized_input", "router_logits", "selected_index", "selected_weight", "act_packed",
        "act_scales", "act_tensor_scale", "parts", "latent_output", "routed_latent_output",
        "projected_routed_output", "shared_output")]


_lib = None


def load_library() -> ctypes.CDLL:
    """Loads the C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIBRARY_PATH):
        raise FileNotFoundError(
            f"{LIBRARY_PATH} is missing: run __graft_entry__.build() (there is no fallback path)")
    lib = ctypes.CDLL(LIBRARY_PATH)
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float
    lib.nmoe_status_string.restype = ctypes.c_char_p
    lib.nmoe_status_string.argtypes = [ctypes.c_int]
    lib.nmoe_layer_create.argtypes = [ctypes.POINTER(_Config), ctypes.POINTER(_Weights),
                                      ctypes.POINTER(vp)]
    lib.nmoe_layer_destroy.argtypes = [vp]
    lib.nmoe_layer_destroy.restype = None
    lib.nmoe_layer_run.argtypes = [vp, vp, vp, ctypes.c_int, i64, vp, ctypes.c_int]
    lib.nmoe_layer_sync_status.argtypes = [vp, vp]
    lib.nmoe_layer_last_error.argtypes = [vp]
    lib.nmoe_layer_last_error.restype = ctypes.c_char_p
    lib.nmoe_layer_trace_view.argtypes = [vp, ctypes.POINTER(_TraceView)]
    lib.nmoe_layer_copy_trace_field.argtypes = [vp, vp, i32, vp, ctypes.c_size_t]
    lib.nmoe_layer_export_hidden.argtypes = [vp, vp, vp, vp, vp, vp]
    lib.nmoe_layer_enable_stage_timing.argtypes = [vp, i32]
    lib.nmoe_layer_reserve_sms.argtypes = [vp, i32]
    lib.nmoe_layer_keep_trace.argtypes = [vp, i32]
    lib.nmoe_layer_reserve_tokens.argtypes = [vp, i32]
    lib.nmoe_layer_set_unfused_activation.argtypes = [vp, i32]
    lib.nmoe_layer_export_unfused.argtypes = [vp, vp, vp, vp, vp]
    lib.nmoe_layer_set_wait_limit_ms.argtypes = [vp, ctypes.c_double]
    lib.nmoe_layer_wait_flag.argtypes = [vp, vp, vp, ctypes.c_uint32]
    lib.nmoe_layer_stage_times.argtypes = [vp, ctypes.POINTER(ctypes.c_float), i32]
    lib.nmoe_ffn_create.argtypes = [ctypes.POINTER(_Nvfp4Matrix), ctypes.POINTER(_Nvfp4Matrix),
                                    i32, ctypes.POINTER(vp)]
    lib.nmoe_ffn_destroy.argtypes = [vp]
    lib.nmoe_ffn_destroy.restype = None
    lib.nmoe_ffn_run.argtypes = [vp, vp, vp, ctypes.c_int, i64, vp, i32]
    lib.nmoe_ffn_sync_status.argtypes = [vp, vp]
    lib.nmoe_ffn_export_hidden.argtypes = [vp, vp, vp, vp]
    lib.nmoe_quantize_nvfp4.argtypes = [vp, vp, ctypes.c_int, i64, i64, i32, vp, vp, vp, vp]
    lib.nmoe_dequant_nvfp4.argtypes = [vp, vp, vp, vp, i32, i64, i64, vp]
    lib.nmoe_swizzled_scale_bytes.argtypes = [i64, i64]
    lib.nmoe_swizzled_scale_bytes.restype = ctypes.c_size_t
    lib.nmoe_swizzle_scales.argtypes = [vp, vp, i64, i64, vp]
    lib.nmoe_rmsnorm.argtypes = [vp, vp, ctypes.c_int, i64, i64, vp, f32, vp]
    lib.nmoe_router_logits.argtypes = [vp, vp, vp, i64, i32, i32, vp]
    lib.nmoe_router_topk.argtypes = [vp, vp, vp, i64, i32, i32, i32, i32, i32, f32, vp, vp]
    lib.nmoe_ep_record_bytes.argtypes = [vp]
    lib.nmoe_ep_record_bytes.restype = ctypes.c_size_t
    lib.nmoe_ep_dispatch.argtypes = [vp, vp, vp, ctypes.c_int, i64, i64, ctypes.POINTER(vp),
                                     ctypes.POINTER(vp)]
    lib.nmoe_ep_experts.argtypes = [vp, vp, vp, i64, vp, i64, vp, ctypes.c_int]
    lib.nmoe_ep_shared.argtypes = [vp, vp]
    lib.nmoe_ep_combine.argtypes = [vp, vp, vp, ctypes.c_int, vp, ctypes.c_int, vp, ctypes.c_int]
    lib.nmoe_ep_window_create.argtypes = [vp, i64, ctypes.c_int, vp]
    lib.nmoe_ep_window_attach.argtypes = [vp, vp]
    lib.nmoe_ep_window_detach.argtypes = [vp]
    lib.nmoe_ep_window_fork_shared.argtypes = [vp, i32]
    lib.nmoe_ep_window_dispatch.argtypes = [vp, vp, vp, ctypes.c_int, i64]
    lib.nmoe_ep_window_experts.argtypes = [vp, vp, i32, i32]
    lib.nmoe_ep_window_combine.argtypes = [vp, vp, vp, ctypes.c_int, vp, ctypes.c_int]
    lib.nmoe_route_tokens_noalloc.argtypes = [vp, vp, ctypes.c_int, i64, i32, vp, f32, vp, vp, i32,
                                              i32, i32, i32, i32, f32, vp, vp]
    _lib = lib
    return lib


def _check(status: int, where: str, detail: str = "") -> None:
    if status != NMOE_OK:
        raise NmoeError(status, where, detail)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: this library has no CPU path")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return NMOE_F32
    if t.dtype == torch.bfloat16:
        return NMOE_BF16
    if t.dtype == torch.float16:
        return NMOE_F16
    raise ValueError(f"unsupported dtype {t.dtype}: expected float32 or bfloat16")


# ---------------------------------------------------------------------------
# Reference-shaped types
# ---------------------------------------------------------------------------

@dataclass
class ExpertLayerConfig:
    """Field for field `nemotron::ExpertLayerConfig` (expert_layer.h:18-31), plus the
    token capacity the device scratch is sized for."""
    layer_index: int = 0
    hidden_size: int = 0
    moe_latent_size: int = 0
    routed_expert_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    n_routed_experts: int = 0
    top_k: int = 0
    n_group: int = 1
    topk_group: int = 1
    rms_epsilon: float = 1.0e-5
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = True
    max_tokens: int = 8192
    max_recv_pairs: int = 0  # expert parallelism only (0 = 2 * max_tokens * top_k)


@dataclass
class Nvfp4Matrix:
    """The byte fields of an NVFP4 `GemmDescriptor` (gemm_catalog.h:20-42):
    packed [N, K/2] uint8 (column 2j in the low nibble), block_scales [N, K/16]
    uint8 E4M3 row-major, tensor_scale FP32.  Tensors may live on host or device."""
    packed: torch.Tensor
    block_scales: torch.Tensor
    tensor_scale: float

    @property
    def output_rows(self) -> int:
        return self.packed.shape[0]

    @property
    def input_cols(self) -> int:
        return self.packed.shape[1] * 2

    def _as_c(self, keep: list) -> _Nvfp4Matrix:
        packed = self.packed.contiguous()
        scales = self.block_scales.contiguous()
        ts = torch.tensor([self.tensor_scale], dtype=torch.float32)
        keep.extend([packed, scales, ts])
        return _Nvfp4Matrix(packed.shape[0], packed.shape[1] * 2, packed.data_ptr(),
                            packed.numel(), scales.data_ptr(), scales.numel(), ts.data_ptr(), 4)


@dataclass
class DenseLinear:
    """A linear of the dense family (`weight` FP32 / bf16 [out, in], DOUBLE accumulation:
    UploadedLinearOp, linear_op.cpp:97-118) or of the scaled-FP8 family (`weight` uint8
    E4M3 codes [out, in] with per-tensor `weight_scale` and `input_scale`:
    ScaledFp8LinearOp, scaled_fp8_linear.cu:121-139, :222-283)."""
    weight: torch.Tensor
    weight_scale: Optional[float] = None
    input_scale: Optional[float] = None

    @property
    def is_fp8(self) -> bool:
        return self.weight.dtype == torch.uint8

    def _as_c(self, keep: list) -> _Linear:
        w = self.weight.contiguous()
        keep.append(w)
        out = _Linear()
        if self.is_fp8:
            out.family = 2
            out.weight = _DenseTensor(w.data_ptr(), w.numel(), NMOE_F32, w.shape[0], w.shape[1])
            out.weight_scale = float(self.weight_scale)
            out.input_scale = float(self.input_scale)
        else:
            out.family = 1
            out.weight = _dense(w, keep)
        return out


@dataclass
class ExpertWeightPair:
    up_proj: Nvfp4Matrix
    down_proj: Nvfp4Matrix


@dataclass
class ExpertLayerBindings:
    """`nemotron::ExpertLayerBindings` (expert_layer.h:38-56).  The latent projections
    may be absent (identity, moe_latent_size == hidden_size); the shared expert's
    projections are NVFP4 (`shared_up` / `shared_down`) unless a dense / scaled-FP8
    `shared_up_linear` / `shared_down_linear` replaces them."""
    input_norm_weight: torch.Tensor            # [hidden] fp32 / bf16
    gate_weight: torch.Tensor                  # [experts, hidden] fp32 / bf16
    gate_score_correction_bias: torch.Tensor   # [experts]
    shared_up: Optional[Nvfp4Matrix]
    shared_down: Optional[Nvfp4Matrix]
    routed_experts: List[ExpertWeightPair] = field(default_factory=list)
    gate_logit_offset: Optional[torch.Tensor] = None  # [experts] fp32, synthetic-skew hook
    first_local_expert: int = 0  # expert parallelism: global index of routed_experts[0]
    fc1_latent: Optional["DenseLinear"] = None   # [latent, hidden]
    fc2_latent: Optional["DenseLinear"] = None   # [hidden, latent], dense
    shared_up_linear: Optional["DenseLinear"] = None
    shared_down_linear: Optional["DenseLinear"] = None


def _dense(t: torch.Tensor, keep: list) -> _DenseTensor:
    t = t.contiguous()
    keep.append(t)
    rows, cols = (t.shape[0], t.shape[1]) if t.dim() == 2 else (1, t.numel())
    return _DenseTensor(t.data_ptr(), t.numel() * t.element_size(), _dtype_code(t), rows, cols)


@dataclass
class ExpertLayerTrace:
    """Device views of the intermediates of the last run (`ExpertLayerRunTrace`,
    expert_layer.h:63-76, for any token count)."""
    normalized_input: Optional[torch.Tensor]  # None after a large batch with keep_trace off
    router_logits: torch.Tensor
    selected_index: torch.Tensor
    selected_weight: torch.Tensor
    act_packed: torch.Tensor
    act_scales: torch.Tensor
    act_tensor_scale: torch.Tensor
    parts: Optional[torch.Tensor]  # FP32 [tokens, top_k + 1, hidden]; None after a bf16-output run
    latent_output: Optional[torch.Tensor]            # [tokens, latent]; None without fc1_latent
    routed_latent_output: Optional[torch.Tensor]     # [tokens, latent]
    projected_routed_output: Optional[torch.Tensor]  # [tokens, hidden]
    shared_output: Optional[torch.Tensor]            # [tokens, hidden]
    routed_hidden_packed: torch.Tensor
    routed_hidden_scales: torch.Tensor
    shared_hidden_packed: torch.Tensor
    shared_hidden_scales: torch.Tensor


class ExpertLayerSlice:
    """`nemotron::ExpertLayerSlice` (expert_layer.h:84-105).  `create` returns None
    on invalid configuration or bindings, `run` returns False on failure, as the
    reference does; `last_error` says why."""

    def __init__(self, handle: int, config: ExpertLayerConfig):
        self._handle = ctypes.c_void_p(handle)
        self._config = config
        self._has_latent = False
        self.last_error = ""

    @staticmethod
    def create(config: ExpertLayerConfig, bindings: ExpertLayerBindings
               ) -> Optional["ExpertLayerSlice"]:
        lib = load_library()
        if not torch.cuda.is_available():
            raise RuntimeError("ExpertLayerSlice needs a CUDA device: there is no CPU path")
        keep: list = []
        c = _Config(config.layer_index, config.hidden_size, config.moe_latent_size,
                    config.routed_expert_intermediate_size,
                    config.shared_expert_intermediate_size, config.n_routed_experts,
                    config.top_k, config.n_group, config.topk_group,
                    1 if config.norm_topk_prob else 0, config.rms_epsilon,
                    config.routed_scaling_factor, config.max_tokens, config.max_recv_pairs)
        n = len(bindings.routed_experts)
        ups = (_Nvfp4Matrix * max(n, 1))()
        downs = (_Nvfp4Matrix * max(n, 1))()
        for i, pair in enumerate(bindings.routed_experts):
            ups[i] = pair.up_proj._as_c(keep)
            downs[i] = pair.down_proj._as_c(keep)
        w = _Weights()
        w.input_norm_weight = _dense(bindings.input_norm_weight, keep)
        w.gate_weight = _dense(bindings.gate_weight, keep)
        w.gate_score_correction_bias = _dense(bindings.gate_score_correction_bias, keep)
        w.routed_up = ups
        w.routed_down = downs
        w.n_local_experts = n
        w.first_local_expert = bindings.first_local_expert
        if bindings.shared_up is not None:
            w.shared_up = bindings.shared_up._as_c(keep)
        if bindings.shared_down is not None:
            w.shared_down = bindings.shared_down._as_c(keep)
        for name in ("fc1_latent", "fc2_latent", "shared_up_linear", "shared_down_linear"):
            linear = getattr(bindings, name)
            if linear is not None:
                setattr(w, name, linear._as_c(keep))
        w.gate_logit_offset = None
        if bindings.gate_logit_offset is not None:
            offset = bindings.gate_logit_offset.to(torch.float32).contiguous()
            keep.append(offset)
            w.gate_logit_offset = offset.data_ptr()
        handle = ctypes.c_void_p()
        status = lib.nmoe_layer_create(ctypes.byref(c), ctypes.byref(w), ctypes.byref(handle))
        if status != NMOE_OK or not handle.value:
            ExpertLayerSlice.create_error = STATUS_NAMES.get(status, str(status))
            return None
        layer = ExpertLayerSlice(handle.value, config)
        layer._has_latent = bindings.fc1_latent is not None
        return layer

    create_error = ""

    def valid(self) -> bool:
        return bool(self._handle and self._handle.value)

    def config(self) -> ExpertLayerConfig:
        return self._config

    def run_async(self, input: torch.Tensor, output: torch.Tensor) -> None:
        """Enqueues the layer on the current stream; raises on a host-side error."""
        _require_cuda(input, "input")
        _require_cuda(output, "output")
        if input.dim() != 2 or input.shape[1] != self._config.hidden_size or \
                output.shape != input.shape:
            raise NmoeError(1, "ExpertLayerSlice.run", "shape must be [tokens, hidden] for both")
        lib = load_library()
        _check(lib.nmoe_layer_run(self._handle, _stream(), input.data_ptr(), _dtype_code(input),
                                  input.shape[0], output.data_ptr(), _dtype_code(output)),
               "nmoe_layer_run", self._last_error())

    def sync_status(self) -> int:
        return load_library().nmoe_layer_sync_status(self._handle, _stream())

    def run(self, input: torch.Tensor, output: torch.Tensor) -> bool:
        """Synchronous, boolean, like ExpertLayerSlice::Run (expert_layer.cpp:752)."""
        try:
            self.run_async(input, output)
        except (NmoeError, ValueError) as error:
            self.last_error = str(error)
            return False
        status = self.sync_status()
        if status != NMOE_OK:
            self.last_error = STATUS_NAMES.get(status, str(status))
            return False
        return True

    STAGES = ("norm_quant", "router_logits", "router_topk", "route_plan", "permute",
              "routed_up_gemm", "routed_down_gemm", "shared_up_gemm", "shared_down_gemm", "combine")

    def enable_stage_timing(self, enable: bool = True) -> None:
        _check(load_library().nmoe_layer_enable_stage_timing(self._handle, 1 if enable else 0),
               "nmoe_layer_enable_stage_timing")

    def reserve_sms(self, reserved: int) -> None:
        """Keep `reserved` SMs free of the persistent GEMM CTAs (for kernels of other streams)."""
        _check(load_library().nmoe_layer_reserve_sms(self._handle, int(reserved)),
               "nmoe_layer_reserve_sms")

    def keep_trace(self, enable: bool) -> None:
        """False: stop writing intermediates that only `trace` reads (the FP32 normalised
        rows of large batches); `trace` then returns None for them."""
        _check(load_library().nmoe_layer_keep_trace(self._handle, 1 if enable else 0),
               "nmoe_layer_keep_trace")

    def reserve_tokens(self, max_tokens: int) -> None:
        """Grows the scratch to `max_tokens` rows per run (synchronises the device)."""
        _check(load_library().nmoe_layer_reserve_tokens(self._handle, int(max_tokens)),
               "nmoe_layer_reserve_tokens", self._last_error())
        self._config.max_tokens = max(self._config.max_tokens, int(max_tokens))

    def set_unfused_activation(self, enable: bool = True) -> None:
        """Two-pass activation path: the activated rows stay FP32 and are quantised with
        their own tensor scale, as the reference's host linear does; handles activated
        values beyond 6*448 and keeps what `unfused_trace` returns."""
        _check(load_library().nmoe_layer_set_unfused_activation(self._handle, 1 if enable else 0),
               "nmoe_layer_set_unfused_activation", self._last_error())

    def unfused_trace(self, tokens: int):
        """(routed_activated [tokens, top_k, I], routed_outputs [tokens, top_k, latent],
        shared_activated [tokens, S]) of the last run, which must have used the unfused path."""
        cfg = self._config
        dev = torch.device("cuda", torch.cuda.current_device())
        ra = torch.empty((tokens, cfg.top_k, cfg.routed_expert_intermediate_size),
                         dtype=torch.float32, device=dev)
        ro = torch.empty((tokens, cfg.top_k, cfg.moe_latent_size), dtype=torch.float32, device=dev)
        sa = torch.empty((tokens, cfg.shared_expert_intermediate_size), dtype=torch.float32,
                         device=dev)
        _check(load_library().nmoe_layer_export_unfused(self._handle, _stream(), ra.data_ptr(),
                                                        ro.data_ptr(), sa.data_ptr()),
               "nmoe_layer_export_unfused", self._last_error())
        torch.cuda.current_stream().synchronize()
        return ra, ro, sa

    def set_wait_limit_ms(self, milliseconds: float) -> None:
        """How long a kernel of this layer waits for a flag another GPU raises before it
        gives up with NMOE_ERR_DEVICE_TIMEOUT."""
        _check(load_library().nmoe_layer_set_wait_limit_ms(self._handle, float(milliseconds)),
               "nmoe_layer_set_wait_limit_ms")

    def wait_flag(self, flag: torch.Tensor, expected: int) -> None:
        """Enqueues the bounded wait of the peer-window stages on a caller-owned 32-bit
        device word: returns (on the device) when flag >= expected or at the limit."""
        _require_cuda(flag, "flag")
        if flag.element_size() != 4:
            raise ValueError("flag must be a 32-bit device word")
        _check(load_library().nmoe_layer_wait_flag(self._handle, _stream(), flag.data_ptr(),
                                                   int(expected)), "nmoe_layer_wait_flag")

    def stage_times_ms(self) -> dict:
        """Device time of every stage of the last run (waits for it)."""
        buf = (ctypes.c_float * len(self.STAGES))()
        _check(load_library().nmoe_layer_stage_times(self._handle, buf, len(self.STAGES)),
               "nmoe_layer_stage_times")
        return dict(zip(self.STAGES, [float(v) for v in buf]))

    def _last_error(self) -> str:
        raw = load_library().nmoe_layer_last_error(self._handle)
        return raw.decode() if raw else ""

    def trace(self, tokens: int) -> ExpertLayerTrace:
        """Copies the intermediates of the last run (which had `tokens` rows)."""
        lib = load_library()
        cfg = self._config
        dev = torch.device("cuda", torch.cuda.current_device())
        H, E, K = cfg.hidden_size, cfg.n_routed_experts, cfg.top_k
        I, S = cfg.routed_expert_intermediate_size, cfg.shared_expert_intermediate_size

        fields = ("normalized_input", "router_logits", "selected_index", "selected_weight",
                  "act_packed", "act_scales", "act_tensor_scale", "parts", "latent_output",
                  "routed_latent_output", "projected_routed_output", "shared_output")
        L = cfg.moe_latent_size
        latent = L != H or self._has_latent

        def grab(name, shape, dtype, optional=False):
            out = torch.empty(shape, dtype=dtype, device=dev)
            status = lib.nmoe_layer_copy_trace_field(self._handle, _stream(), fields.index(name),
                                                     out.data_ptr(),
                                                     out.numel() * out.element_size())
            if optional and status != NMOE_OK:
                return None  # the layer does not hold this field for the last run
            _check(status, "nmoe_layer_copy_trace_field")
            return out

        rp = torch.empty((tokens, K, I // 2), dtype=torch.uint8, device=dev)
        rs = torch.empty((tokens, K, I // 16), dtype=torch.uint8, device=dev)
        sp = torch.empty((tokens, S // 2), dtype=torch.uint8, device=dev)
        ss = torch.empty((tokens, S // 16), dtype=torch.uint8, device=dev)
        _check(lib.nmoe_layer_export_hidden(self._handle, _stream(), rp.data_ptr(), rs.data_ptr(),
                                            sp.data_ptr(), ss.data_ptr()),
               "nmoe_layer_export_hidden")
        trace = ExpertLayerTrace(
            normalized_input=grab("normalized_input", (tokens, H), torch.float32, optional=True),
            router_logits=grab("router_logits", (tokens, E), torch.float32),
            selected_index=grab("selected_index", (tokens, K), torch.int32),
            selected_weight=grab("selected_weight", (tokens, K), torch.float32),
            act_packed=grab("act_packed", (tokens, L // 2), torch.uint8),
            act_scales=grab("act_scales", (tokens, L // 16), torch.uint8),
            act_tensor_scale=grab("act_tensor_scale", (tokens,), torch.float32),
            parts=grab("parts", (tokens, K, L) if latent else (tokens, K + 1, H), torch.float32,
                       optional=True),
            latent_output=grab("latent_output", (tokens, L), torch.float32, optional=True),
            routed_latent_output=grab("routed_latent_output", (tokens, L), torch.float32,
                                      optional=True),
            projected_routed_output=grab("projected_routed_output", (tokens, H), torch.float32,
                                         optional=True),
            shared_output=grab("shared_output", (tokens, H), torch.float32, optional=True),
            routed_hidden_packed=rp, routed_hidden_scales=rs,
            shared_hidden_packed=sp, shared_hidden_scales=ss)
        torch.cuda.current_stream().synchronize()
        return trace

    def close(self) -> None:
        if self._handle and self._handle.value:
            load_library().nmoe_layer_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ExpertFfn:
    """One NVFP4 expert FFN down(relu^2(up(x))): the per-(token, expert) composition
    of expert_layer.cpp:913-922."""

    def __init__(self, up: Nvfp4Matrix, down: Nvfp4Matrix, max_rows: int):
        lib = load_library()
        if not torch.cuda.is_available():
            raise RuntimeError("ExpertFfn needs a CUDA device: there is no CPU path")
        keep: list = []
        cu, cd = up._as_c(keep), down._as_c(keep)
        handle = ctypes.c_void_p()
        _check(lib.nmoe_ffn_create(ctypes.byref(cu), ctypes.byref(cd), max_rows,
                                   ctypes.byref(handle)), "nmoe_ffn_create")
        self._handle = handle
        self.hidden = up.input_cols
        self.intermediate = up.output_rows

    def run(self, x: torch.Tensor, variant: int = 0) -> torch.Tensor:
        _require_cuda(x, "x")
        out = torch.empty((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        lib = load_library()
        _check(lib.nmoe_ffn_run(self._handle, _stream(), x.data_ptr(), _dtype_code(x), x.shape[0],
                                out.data_ptr(), variant), "nmoe_ffn_run")
        _check(lib.nmoe_ffn_sync_status(self._handle, _stream()), "nmoe_ffn_sync_status")
        return out

    def hidden_codes(self, rows: int):
        dev = torch.device("cuda", torch.cuda.current_device())
        packed = torch.empty((rows, self.intermediate // 2), dtype=torch.uint8, device=dev)
        scales = torch.empty((rows, self.intermediate // 16), dtype=torch.uint8, device=dev)
        _check(load_library().nmoe_ffn_export_hidden(self._handle, _stream(), packed.data_ptr(),
                                                     scales.data_ptr()), "nmoe_ffn_export_hidden")
        torch.cuda.current_stream().synchronize()
        return packed, scales

    def close(self) -> None:
        if self._handle and self._handle.value:
            load_library().nmoe_ffn_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------
# Unit operators
# ---------------------------------------------------------------------------

def quantize_nvfp4(x: torch.Tensor, per_row: bool = True, swizzled: bool = False):
    """PackRowMajorFp32ToNvfp4 on the device.  Returns (packed, scales, tensor_scale[,
    swizzled_scales])."""
    _require_cuda(x, "x")
    lib = load_library()
    rows, cols = x.shape
    packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, cols // 16), dtype=torch.uint8, device=x.device)
    ts = torch.empty((rows if per_row else 1,), dtype=torch.float32, device=x.device)
    sw = None
    if swizzled:
        sw = torch.empty((lib.nmoe_swizzled_scale_bytes(rows, cols),), dtype=torch.uint8,
                         device=x.device)
    _check(lib.nmoe_quantize_nvfp4(_stream(), x.data_ptr(), _dtype_code(x), rows, cols,
                                   1 if per_row else 0, packed.data_ptr(), scales.data_ptr(),
                                   sw.data_ptr() if sw is not None else None, ts.data_ptr()),
           "nmoe_quantize_nvfp4")
    return (packed, scales, ts, sw) if swizzled else (packed, scales, ts)


def dequant_nvfp4(packed: torch.Tensor, scales: torch.Tensor, tensor_scale: torch.Tensor,
                  per_row: bool = True) -> torch.Tensor:
    _require_cuda(packed, "packed")
    rows, cols = packed.shape[0], packed.shape[1] * 2
    out = torch.empty((rows, cols), dtype=torch.float32, device=packed.device)
    _check(load_library().nmoe_dequant_nvfp4(_stream(), packed.data_ptr(), scales.data_ptr(),
                                             tensor_scale.data_ptr(), 1 if per_row else 0, rows,
                                             cols, out.data_ptr()), "nmoe_dequant_nvfp4")
    return out


def swizzle_scales(scales: torch.Tensor, cols: int) -> torch.Tensor:
    _require_cuda(scales, "scales")
    lib = load_library()
    rows = scales.shape[0]
    out = torch.empty((lib.nmoe_swizzled_scale_bytes(rows, cols),), dtype=torch.uint8,
                      device=scales.device)
    _check(lib.nmoe_swizzle_scales(_stream(), scales.data_ptr(), rows, cols, out.data_ptr()),
           "nmoe_swizzle_scales")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _require_cuda(x, "x")
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _check(load_library().nmoe_rmsnorm(_stream(), x.data_ptr(), _dtype_code(x), x.shape[0],
                                       x.shape[1], weight.data_ptr(), eps, out.data_ptr()),
           "nmoe_rmsnorm")
    return out


def router_logits(normalized: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    _require_cuda(normalized, "normalized")
    rows, hidden = normalized.shape
    experts = gate.shape[0]
    out = torch.empty((rows, experts), dtype=torch.float32, device=normalized.device)
    _check(load_library().nmoe_router_logits(_stream(), normalized.data_ptr(), gate.data_ptr(),
                                             rows, experts, hidden, out.data_ptr()),
           "nmoe_router_logits")
    return out


def router_topk(logits: torch.Tensor, bias: torch.Tensor, top_k: int, n_group: int = 1,
                topk_group: int = 1, norm_topk_prob: bool = True, routed_scaling: float = 1.0):
    _require_cuda(logits, "logits")
    rows, experts = logits.shape
    idx = torch.empty((rows, top_k), dtype=torch.int32, device=logits.device)
    wt = torch.empty((rows, top_k), dtype=torch.float32, device=logits.device)
    _check(load_library().nmoe_router_topk(_stream(), logits.data_ptr(), bias.data_ptr(), rows,
                                           experts, top_k, n_group, topk_group,
                                           1 if norm_topk_prob else 0, routed_scaling,
                                           idx.data_ptr(), wt.data_ptr()), "nmoe_router_topk")
    return idx, wt


def route_tokens_noalloc(x: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                         gate: torch.Tensor, bias: torch.Tensor, top_k: int, n_group: int = 1,
                         topk_group: int = 1, norm_topk_prob: bool = True,
                         routed_scaling: float = 1.0):
    """RMSNorm -> gate logits -> top-k in one call that allocates nothing inside the
    library (the intermediates live in a fixed array of the library image; see
    nmoe_route_tokens_noalloc in include/nmoe.h for who needs that and for the limits).
    The two result tensors are allocated here, by the caller, before the call."""
    _require_cuda(x, "x")
    rows, hidden = x.shape
    experts = gate.shape[0]
    idx = torch.empty((rows, top_k), dtype=torch.int32, device=x.device)
    wt = torch.empty((rows, top_k), dtype=torch.float32, device=x.device)
    _check(load_library().nmoe_route_tokens_noalloc(
        _stream(), x.data_ptr(), _dtype_code(x), rows, hidden, norm_weight.data_ptr(), eps,
        gate.data_ptr(), bias.data_ptr(), experts, top_k, n_group, topk_group,
        1 if norm_topk_prob else 0, routed_scaling, idx.data_ptr(), wt.data_ptr()),
        "nmoe_route_tokens_noalloc")
    return idx, wt
