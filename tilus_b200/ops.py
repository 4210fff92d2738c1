"""Low-level operators over the C ABI: quantized_matmul, dequantize, plan.

Tensors are torch CUDA tensors used only as device memory; the stream is torch's
current stream.  Mirrors the reference's kernel call
``kernel(m_size, n_size, k_size, a_ptr, b_ptr, scale_ptr, c_ptr)``
(examples/quantization/matmul_a16wx.py:539-547) with the dtype / group arguments that
the reference fixes at JIT time made explicit.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .dtypes import weight_dtype
from .packing import BLOCK_K, BLOCK_N

_workspaces = {}


def act_code(dtype: torch.dtype) -> int:
    """Activation dtype tag of the C ABI (B200Q_F16 / B200Q_BF16)."""
    if dtype == torch.float16:
        return _lib.ACT_F16
    if dtype == torch.bfloat16:
        return _lib.ACT_BF16
    raise TypeError(f"activations, scales and outputs are float16 or bfloat16, got {dtype}")


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def workspace_bytes(M: int, N: int, K: int, w_dtype, zero_point: int = 0, group_size: int = 128) -> int:
    dt = weight_dtype(w_dtype)
    n = _lib.load().b200q_workspace_bytes(M, N, K, dt.code, zero_point, group_size)
    if n == 0:
        raise _lib.B200QError(_lib.ST_UNSUPPORTED, f"no kernel for M={M} N={N} K={K} {dt.name} zp={zero_point} g={group_size}")
    return int(n)


def get_workspace(device, nbytes: int) -> torch.Tensor:
    """Per (device, stream) zero-initialised workspace, grown on demand.  The kernels
    leave it zeroed, so it is cleared only when (re)allocated."""
    key = (torch.device(device).index, _stream_ptr(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def plan(M: int, N: int, K: int, w_dtype, zero_point: int = 0, group_size: int = 128) -> dict:
    dt = weight_dtype(w_dtype)
    pl = _lib.Plan()
    _lib.check(_lib.load().b200q_plan(M, N, K, dt.code, zero_point, group_size, ctypes.byref(pl)))
    return pl.as_dict()


def quantized_matmul(a: torch.Tensor, bq: torch.Tensor, scales: torch.Tensor, w_dtype, group_size: int,
                     zero_point: int = 0, out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                     plan_override: dict | None = None) -> torch.Tensor:
    """C[M, N] = A[M, K] x dequant(Bq).  ``bq`` is the b200-packed weight (packing.interleave),
    ``scales`` is fp16 [K/group, N]."""
    lib = _lib.load()
    dt = weight_dtype(w_dtype)
    if not (a.is_cuda and bq.is_cuda and scales.is_cuda):
        raise ValueError("quantized_matmul needs CUDA tensors (there is no CPU path)")
    act = act_code(a.dtype)
    if scales.dtype != a.dtype:
        raise TypeError("activations and scales must have the same dtype (float16 or bfloat16)")
    if a.dim() != 2 or a.stride(1) != 1:
        raise ValueError("a must be a 2-D tensor with unit inner stride")
    M, K = a.shape
    G, N = scales.shape
    if G * group_size != K or not scales.is_contiguous():
        raise ValueError("scales must be a contiguous [K/group_size, N] tensor")
    if bq.dtype != torch.uint8 or bq.numel() * 8 != K * N * dt.nbits or not bq.is_contiguous():
        raise ValueError("bq must be a contiguous uint8 tensor of K*N*nbits/8 bytes")
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    if M == 0:
        return out
    with torch.cuda.device(a.device):
        if workspace is None:
            workspace = get_workspace(a.device, workspace_bytes(M, N, K, dt, zero_point, group_size))
        args = (a.data_ptr(), a.stride(0), bq.data_ptr(), scales.data_ptr(), out.data_ptr(), out.stride(0),
                M, N, K, dt.code, zero_point, group_size, act, workspace.data_ptr(), workspace.numel(),
                _stream_ptr(a.device))
        if plan_override is None:
            st = lib.b200q_gemm(*args)
        else:
            pl = _lib.Plan()
            _lib.check(lib.b200q_plan(M, N, K, dt.code, zero_point, group_size, ctypes.byref(pl)))
            for k, v in plan_override.items():
                setattr(pl, k, v)
            st = lib.b200q_gemm_planned(*args, ctypes.byref(pl))
    _lib.check(st)
    return out


def linear_forward(x2: torch.Tensor, bq: torch.Tensor, scales: torch.Tensor, code: int, zero_point: int,
                   group_size: int, K: int, N: int, ws_need: dict) -> torch.Tensor:
    """The call QuantizedLinear.forward makes: same kernel launch as quantized_matmul, with the
    layer's constants already validated at construction and the workspace size cached per M
    (``ws_need``), so that a decode step spends its host time in the launch, not in checks."""
    if not x2.is_cuda:
        raise ValueError("QuantizedLinear needs CUDA tensors (there is no CPU path)")
    if x2.dtype != scales.dtype or x2.stride(1) != 1:
        raise TypeError(f"activations must be {scales.dtype} with unit inner stride")
    act = act_code(x2.dtype)
    lib = _lib.load()
    M = x2.shape[0]
    out = torch.empty(M, N, dtype=x2.dtype, device=x2.device)
    if M == 0:
        return out
    dev = x2.device
    need = ws_need.get(M)
    if need is None:
        need = lib.b200q_workspace_bytes(M, N, K, code, zero_point, group_size)
        if need == 0:
            raise _lib.B200QError(_lib.ST_UNSUPPORTED, f"no kernel for M={M} N={N} K={K}")
        ws_need[M] = need
    switch = torch.cuda.current_device() != dev.index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        stream = torch.cuda.current_stream(dev).cuda_stream
        key = (dev.index, stream)
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)
            _workspaces[key] = ws
        st = lib.b200q_gemm(x2.data_ptr(), x2.stride(0), bq.data_ptr(), scales.data_ptr(), out.data_ptr(), N, M, N, K,
                            code, zero_point, group_size, act, ws.data_ptr(), ws.numel(), stream)
    finally:
        if switch:
            torch.cuda.set_device(prev)
    if st != 0:
        _lib.check(st)
    return out


_host_staging: dict = {}


def linear_forward_host(x_host: torch.Tensor, out_host: torch.Tensor, bq: torch.Tensor, scales: torch.Tensor,
                        code: int, zero_point: int, group_size: int, K: int, N: int, ws_need: dict,
                        prepared: dict) -> torch.Tensor:
    """QuantizedLinear.forward_host: activations and result live in host memory (pinned, so that the
    copies are asynchronous).  One library call queues copy-in, GEMM and copy-out on the current
    stream of the layer's device; the caller synchronises that stream before reading ``out_host``."""
    # A serving loop calls this with the same pinned buffers over and over: everything the checks
    # below depend on is in the key, and a hit goes straight to the library call with the
    # arguments prepared the first time (the checks and conversions cost more than the call).
    dev = bq.device
    stream = torch._C._cuda_getCurrentRawStream(dev.index)
    key = (x_host.data_ptr(), out_host.data_ptr(), x_host.shape, x_host.stride(), out_host.stride(), x_host.dtype,
           out_host.dtype, stream, bq.data_ptr(), scales.data_ptr())
    hit = prepared.get(key)
    if hit is not None:
        if torch._C._cuda_getDevice() == dev.index:
            st = hit[0](*hit[1])
        else:
            with torch.cuda.device(dev):
                st = hit[0](*hit[1])
        if st != 0:
            _lib.check(st)
        return out_host
    if x_host.is_cuda or out_host.is_cuda:
        raise ValueError("forward_host takes host tensors (use forward for device tensors)")
    if x_host.dtype != scales.dtype or out_host.dtype != scales.dtype:
        raise TypeError(f"activations and result must be {scales.dtype}")
    act = act_code(x_host.dtype)
    if x_host.dim() != 2 or x_host.stride(1) != 1 or x_host.shape[1] != K:
        raise ValueError(f"x_host must be [M, {K}] with unit inner stride")
    M = x_host.shape[0]
    if out_host.dim() != 2 or out_host.stride(1) != 1 or tuple(out_host.shape) != (M, N):
        raise ValueError(f"out_host must be [{M}, {N}] with unit inner stride")
    if M == 0:
        return out_host
    lib = _lib.load()
    need = ws_need.get(M)
    if need is None:
        need = lib.b200q_workspace_bytes(M, N, K, code, zero_point, group_size)
        if need == 0:
            raise _lib.B200QError(_lib.ST_UNSUPPORTED, f"no kernel for M={M} N={N} K={K}")
        ws_need[M] = need
    with torch.cuda.device(dev):
        wkey = (dev.index, stream)
        ws = _workspaces.get(wkey)
        if ws is None or ws.numel() < need:
            ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)
            _workspaces[wkey] = ws
        # Decode batches (the kernel's own CTAs fetch the activations and consecutive calls overlap) keep
        # staging buffers of their own, so that a call for a larger batch in between does not make the
        # next decode call wait for it (the library only lets a call start early behind a call of its kind).
        skey = wkey + (M <= 16,)
        stage = _host_staging.get(skey)
        if stage is None or stage[0].numel() < M * K or stage[1].numel() < M * N:
            stage = (torch.empty(M * K, dtype=torch.int16, device=dev), torch.empty(M * N, dtype=torch.int16, device=dev))
            _host_staging[skey] = stage
        args = (x_host.data_ptr(), x_host.stride(0), bq.data_ptr(), scales.data_ptr(), out_host.data_ptr(),
                out_host.stride(0), M, N, K, code, zero_point, group_size, act, stage[0].data_ptr(),
                stage[1].data_ptr(), ws.data_ptr(), ws.numel(), stream)
        st = lib.b200q_gemm_host(*args)
    if st != 0:
        _lib.check(st)
    if len(prepared) > 256:  # a caller that keeps changing buffers: start over rather than grow
        prepared.clear()
    # the entry keeps the device buffers it names alive (a later, larger request replaces them in the pools)
    prepared[key] = (lib.b200q_gemm_host, args, ws, stage)
    return out_host


def dequantize(bq: torch.Tensor, scales: torch.Tensor, w_dtype, group_size: int, zero_point: int = 0) -> torch.Tensor:
    """W[K, N] in the dtype of ``scales`` (float16 or bfloat16): the weights the GEMM multiplies by
    (bit-exact with the reference's cast-then-scale)."""
    lib = _lib.load()
    dt = weight_dtype(w_dtype)
    G, N = scales.shape
    K = G * group_size
    if not (bq.is_cuda and scales.is_cuda):
        raise ValueError("dequantize needs CUDA tensors (there is no CPU path)")
    if bq.dtype != torch.uint8 or bq.numel() * 8 != K * N * dt.nbits:
        raise ValueError("bq must be a uint8 tensor of K*N*nbits/8 bytes")
    w = torch.empty(K, N, dtype=scales.dtype, device=bq.device)
    with torch.cuda.device(bq.device):
        _lib.check(lib.b200q_dequantize(bq.data_ptr(), scales.contiguous().data_ptr(), w.data_ptr(), N, K, dt.code,
                                        zero_point, group_size, act_code(scales.dtype), _stream_ptr(bq.device)))
    return w


def device_status(workspace: torch.Tensor | None, device=None) -> list:
    """Status header of a workspace ([0, 0, 0, 0] when no bounded device-side wait gave up); clears
    it.  ``workspace=None`` reads the library's built-in scratch (b200q_gemm_static_ws) of ``device``."""
    arr = (ctypes.c_int32 * 4)()
    dev = workspace.device if workspace is not None else torch.device(device if device is not None else "cuda")
    with torch.cuda.device(dev):
        st = _lib.load().b200q_device_status(workspace.data_ptr() if workspace is not None else None,
                                             ctypes.byref(arr), _stream_ptr(dev))
    if st not in (_lib.ST_OK, _lib.ST_DEVICE_TIMEOUT):
        _lib.check(st)
    return list(arr)


# ---- the step behind the gate_up projection: SwiGLU and the per-token FP8 cast ----------------------
def per_token_cast(x: torch.Tensor, num_per_channels: int = 128):
    """x [tokens, hidden] (float16 / bfloat16, CUDA) -> (out float8_e4m3fn [tokens, hidden],
    out_sf float32 [tokens, hidden / num_per_channels]): the reference's PerTokenCast
    (examples/quantization/per_token_cast.py:22-97)."""
    if not x.is_cuda:
        raise ValueError("per_token_cast needs a CUDA tensor (there is no CPU path)")
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a 2-D tensor with unit inner stride")
    T, H = x.shape
    out = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=x.device)
    sf = torch.empty(T, H // num_per_channels, dtype=torch.float32, device=x.device)
    if T == 0:
        return out, sf
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().b200q_per_token_cast(x.data_ptr(), x.stride(0), out.data_ptr(), H, sf.data_ptr(), T, H,
                                                    num_per_channels, act_code(x.dtype), _stream_ptr(x.device)))
    return out, sf


def swiglu_forward_and_per_token_cast(x: torch.Tensor, num_per_channels: int = 128, pos_to_token_topk=None,
                                      topk_weights=None, pos_to_expert=None, swiglu_clamp_value=None):
    """x [tokens, 2 * hidden] -> (out float8_e4m3fn [tokens, hidden], out_sf float32 [tokens, hidden / g]):
    silu(x[:, :hidden]) * x[:, hidden:], optional clamp, routing weight and expert mask, then the
    per-token cast - the reference's SwiGLUForwardAndPerTokenCast
    (examples/quantization/swiglu_forward_and_per_token_cast.py:28-166).  Rows whose pos_to_expert
    entry is negative are left unwritten."""
    if not x.is_cuda:
        raise ValueError("swiglu_forward_and_per_token_cast needs a CUDA tensor (there is no CPU path)")
    if x.dim() != 2 or x.stride(1) != 1 or x.shape[1] % 2:
        raise ValueError("x must be [tokens, 2 * hidden] with unit inner stride")
    T, H = x.shape[0], x.shape[1] // 2
    out = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=x.device)
    sf = torch.empty(T, H // num_per_channels, dtype=torch.float32, device=x.device)
    if T == 0:
        return out, sf

    def ptr(t, dtype):
        if t is None:
            return None
        if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
            raise ValueError(f"index / weight tensors must be contiguous CUDA tensors of {dtype}")
        return t.data_ptr()

    with torch.cuda.device(x.device):
        _lib.check(_lib.load().b200q_swiglu_per_token_cast(
            x.data_ptr(), x.stride(0), out.data_ptr(), H, sf.data_ptr(), T, H, num_per_channels, act_code(x.dtype),
            ptr(pos_to_token_topk, torch.int32), ptr(topk_weights, torch.float32), ptr(pos_to_expert, torch.int32),
            0 if swiglu_clamp_value is None else 1, 0.0 if swiglu_clamp_value is None else float(swiglu_clamp_value),
            _stream_ptr(x.device)))
    return out, sf
