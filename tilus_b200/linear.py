"""QuantizedLinear: the reference's operator surface
(examples/quantization/matmul_a16wx.py:408-548) over the sm_100a kernels.

Same constructor arguments, parameters and methods as the reference class:

    QuantizedLinear(x_dtype, w_dtype, group_size, in_features, out_features)
      .quantized_weight : uint8[out_features * in_features * nbits / 8]
      .scales           : x_dtype[in_features / group_size, out_features]
      .load_and_quantize(weight[out_features, in_features])
      .forward(x[M, in_features]) -> [M, out_features]

``quantized_weight`` holds this library's interleaved layout (packing.LAYOUT_VERSION),
not the reference's mma-fragment tiling; ``load_packed`` converts from the reference's
formats.  The forward pass always runs the CUDA library; there is no CPU path.
"""
from __future__ import annotations

import torch
from torch import nn

from . import ops, packing, quantize
from .dtypes import KIND_UINT, act_dtype, weight_dtype

_TORCH_ACT = {"float16": torch.float16, "bfloat16": torch.bfloat16}


class QuantizedLinear(nn.Module):
    def __init__(self, x_dtype, w_dtype, group_size: int, in_features: int, out_features: int,
                 zero_point: int | None = None):
        super().__init__()
        x_dtype = act_dtype(x_dtype)
        w_dtype = weight_dtype(w_dtype)
        self.act_torch_dtype = _TORCH_ACT[x_dtype.name]  # float16 or bfloat16, as the reference (matmul_a16wx.py:418-419)
        # The reference class demands float or signed types ("symmetric quantization",
        # matmul_a16wx.py:421-423) while its kernel takes any 1-8 bit type (:163-165).
        # Unsigned types are accepted here with an explicit zero point.
        if zero_point is None:
            zero_point = 0
        if w_dtype.kind != KIND_UINT and zero_point != 0:
            raise ValueError("a zero point is only meaningful for unsigned weight types")
        assert in_features % group_size == 0, "in_features must be divisible by group_size"
        assert in_features * out_features * w_dtype.nbits % 8 == 0
        packing.check_shape(in_features, out_features)
        if group_size % 32 != 0:
            raise ValueError("group_size must be a multiple of 32")

        self.x_dtype = x_dtype
        self.w_dtype = w_dtype
        self.group_size = group_size
        self.in_features = in_features
        self.out_features = out_features
        self.zero_point = int(zero_point)

        self.quantized_weight = nn.Parameter(
            torch.empty(out_features * in_features * w_dtype.nbits // 8, dtype=torch.uint8), requires_grad=False
        )
        self.scales = nn.Parameter(
            torch.empty(in_features // group_size, out_features, dtype=self.act_torch_dtype), requires_grad=False
        )
        self.register_buffer("layout_version", torch.tensor(packing.LAYOUT_VERSION, dtype=torch.int32))
        self._ws_need = {}  # workspace bytes per batch size M (filled on first use)
        self._host_calls = {}  # prepared b200q_gemm_host calls per (buffers, stream), see ops.linear_forward_host

    # -- loading ---------------------------------------------------------------------
    def load_and_quantize(self, weight: torch.Tensor):
        """Quantize a dense weight[out_features, in_features] and store it packed."""
        assert (self.out_features, self.in_features) == tuple(weight.shape), "weight shape mismatch"
        if self.w_dtype.kind == KIND_UINT:
            raise ValueError("load_and_quantize is symmetric: use a signed or float weight type "
                             "(unsigned codes come in through load_codes / load_packed)")
        dev = self.quantized_weight.device
        if dev.type == "cuda":  # one fused pass on the GPU: scales, codes, packing
            packed, scales = quantize.quantize_and_pack(weight.to(dev), self.w_dtype, self.group_size,
                                                        self.act_torch_dtype)
            self.load_packed(packed, scales, layout="b200")
            return
        codes, scales = quantize.quantize_weight(weight.to(dev), self.w_dtype, self.group_size, self.act_torch_dtype)
        self.load_codes(codes, scales)

    def load_codes(self, codes: torch.Tensor, scales: torch.Tensor):
        """codes uint8[in_features, out_features] (type-native codes), scales [K/group, N]."""
        dev = self.quantized_weight.device
        packed = packing.interleave(codes.to(dev), self.w_dtype)
        with torch.no_grad():
            self.quantized_weight.copy_(packed)
            self.scales.copy_(scales.to(dev).reshape(self.scales.shape))

    def load_packed(self, storage: torch.Tensor, scales: torch.Tensor, layout: str = "canonical"):
        """Load weights packed by the reference: ``canonical`` (tilus.Tensor storage of the
        [K, N] matrix), ``ref_tiled`` (the reference QuantizedLinear's quantized_weight) or
        ``k_major`` (bit-dense along K per column)."""
        K, N, b = self.in_features, self.out_features, self.w_dtype.nbits
        if layout == "canonical":
            codes = packing.unpack_canonical(storage, b, K, N)
        elif layout == "ref_tiled":
            codes = packing.unpack_ref_tiled(storage, b, K, N)
        elif layout == "k_major":
            codes = packing.unpack_canonical(storage, b, N, K).t().contiguous()
        elif layout == "b200":
            with torch.no_grad():
                self.quantized_weight.copy_(storage.reshape(-1))
                self.scales.copy_(scales.reshape(self.scales.shape))
            return
        else:
            raise ValueError(f"unknown layout {layout!r}")
        self.load_codes(codes, scales)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        """Checkpoints carry ``layout_version``.  A state dict without it was written by the
        reference's QuantizedLinear (parameters ``quantized_weight`` + ``scales`` only,
        examples/quantization/matmul_a16wx.py:455-468): its ``quantized_weight`` is the
        [K/16, N/16, 32*b] tiling of QuantizedMatmulChangeLayout (:64-98) and is re-packed here,
        so reference checkpoints load directly.  Any other version is refused."""
        key_w, key_v = prefix + "quantized_weight", prefix + "layout_version"
        if key_w in state_dict and key_v not in state_dict:
            K, N, b = self.in_features, self.out_features, self.w_dtype.nbits
            stored = state_dict[key_w]
            if stored.numel() != K * N * b // 8:
                error_msgs.append(f"{key_w}: expected {K * N * b // 8} bytes, got {stored.numel()}")
            else:
                codes = packing.unpack_ref_tiled(stored.detach().cpu().reshape(-1), b, K, N)
                state_dict = dict(state_dict)
                state_dict[key_w] = packing.interleave(codes, self.w_dtype)
                state_dict[key_v] = torch.tensor(packing.LAYOUT_VERSION, dtype=torch.int32)
        elif key_v in state_dict and int(state_dict[key_v]) != packing.LAYOUT_VERSION:
            error_msgs.append(f"{key_v}: checkpoint has packed-weight layout version {int(state_dict[key_v])}, "
                              f"this library reads version {packing.LAYOUT_VERSION}")
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)

    def codes(self) -> torch.Tensor:
        """Type-native codes uint8[in_features, out_features] (inverse of load_codes)."""
        return packing.deinterleave(self.quantized_weight.data, self.w_dtype, self.in_features, self.out_features)

    def dequantized_weight(self) -> torch.Tensor:
        """[in_features, out_features] in the activation dtype: the weights forward() multiplies by."""
        return ops.dequantize(self.quantized_weight.data, self.scales.data, self.w_dtype, self.group_size,
                              self.zero_point)

    # -- compute ---------------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x if x.dim() == 2 else x.reshape(-1, self.in_features)
        if x2.shape[1] != self.in_features:
            raise ValueError(f"expected {self.in_features} input features, got {x2.shape[1]}")
        out = ops.linear_forward(x2, self.quantized_weight.data, self.scales.data, self.w_dtype.code, self.zero_point,
                                 self.group_size, self.in_features, self.out_features, self._ws_need)
        return out if x.dim() == 2 else out.reshape(*x.shape[:-1], self.out_features)

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor | None = None) -> torch.Tensor:
        """forward() for activations kept in host memory: ``x_host`` [M, in_features] fp16 (pinned
        for an asynchronous copy) in, ``out_host`` [M, out_features] fp16 out (allocated pinned when
        not given).  Copy-in, GEMM and copy-out are queued on the layer's current stream by one
        library call (b200q_gemm_host); synchronise the stream before reading the result."""
        if out_host is None:
            out_host = torch.empty(x_host.shape[0], self.out_features, dtype=self.act_torch_dtype).pin_memory()
        return ops.linear_forward_host(x_host, out_host, self.quantized_weight.data, self.scales.data,
                                       self.w_dtype.code, self.zero_point, self.group_size, self.in_features,
                                       self.out_features, self._ws_need, self._host_calls)

    def forward_swiglu_cast(self, x: torch.Tensor, num_per_channels: int = 128, swiglu_clamp_value=None):
        """For a gate_up projection (out_features = 2 * hidden, gate columns first): this layer's GEMM
        followed by SwiGLU and the per-token FP8 cast, queued by one library call
        (b200q_gemm_swiglu_cast).  Returns (out float8_e4m3fn [M, hidden], out_sf float32
        [M, hidden / num_per_channels], gate_up [M, out_features])."""
        from . import _lib

        x2 = x if x.dim() == 2 else x.reshape(-1, self.in_features)
        if not x2.is_cuda or x2.dtype != self.act_torch_dtype or x2.stride(1) != 1:
            raise ValueError(f"activations must be CUDA {self.act_torch_dtype} with unit inner stride")
        M, N, K = x2.shape[0], self.out_features, self.in_features
        H = N // 2
        dev = x2.device
        gate_up = torch.empty(M, N, dtype=x2.dtype, device=dev)
        out = torch.empty(M, H, dtype=torch.float8_e4m3fn, device=dev)
        sf = torch.empty(M, H // num_per_channels, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            ws = ops.get_workspace(dev, ops.workspace_bytes(M, N, K, self.w_dtype, self.zero_point, self.group_size))
            st = _lib.load().b200q_gemm_swiglu_cast(
                x2.data_ptr(), x2.stride(0), self.quantized_weight.data_ptr(), self.scales.data_ptr(),
                gate_up.data_ptr(), N, out.data_ptr(), H, sf.data_ptr(), M, N, K, self.w_dtype.code, self.zero_point,
                self.group_size, ops.act_code(x2.dtype), num_per_channels, 0 if swiglu_clamp_value is None else 1,
                0.0 if swiglu_clamp_value is None else float(swiglu_clamp_value), ws.data_ptr(), ws.numel(),
                torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(st)
        return out, sf, gate_up

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, x_dtype={self.x_dtype.name}, "
                f"w_dtype={self.w_dtype.name}, "
                f"group_size={self.group_size}, zero_point={self.zero_point}")
