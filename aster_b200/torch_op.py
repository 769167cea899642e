"""PyTorch front door: ``torch.ops.aster_b200.gemm_nt`` runs the CUDA GEMM on torch tensors.

The step above the operator surface in the reference is a linalg.matmul front end
(contrib/mlir-air/README.md); for a PyTorch user the equivalent is an operator that takes
CUDA tensors.  The tensors only lend their storage: the op passes ``data_ptr()`` and torch's
current stream to the C ABI (``b200_gemm_run``), there is no copy and no fallback to
``torch.matmul``.

    import aster_b200.torch_op            # registers the op
    c = torch.ops.aster_b200.gemm_nt(a, b, bias, relu=True, out_dtype=torch.bfloat16)
    c = aster_b200.torch_op.gemm_nt_direct(a, b, bias, relu=True)   # same, without the dispatcher

``a`` is ``[M, K]``, ``b`` is ``[N, K]`` (both contiguous, K fastest: ``c = a @ b.T``), dtype
float16, bfloat16 or float8_e4m3fn; ``bias`` is an optional float32 ``[N]``; ``scale_a`` /
``scale_b`` are optional one-element float32 CUDA tensors (per-tensor dequantisation scales).
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _native as nat
from .gemm import GemmPlan

_DTYPES = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float8_e4m3fn: "e4m3"}
_OUT_DTYPES = {torch.float32: "f32", torch.bfloat16: "bf16"}

# (device, M, N, K, dtype_ab, dtype_c, epilogue) -> (plan, workspace tensor or None)
_plans: dict = {}


def _plan_for(device: torch.device, M: int, N: int, K: int, dtype_ab: str, dtype_c: str, epilogue: str):
    key = (device.index, M, N, K, dtype_ab, dtype_c, epilogue)
    hit = _plans.get(key)
    if hit is None:
        plan = GemmPlan(M, N, K, dtype_ab, dtype_c, epilogue=epilogue)
        res = plan.resources()
        ws_bytes = res.workspace_bytes or res.optional_workspace_bytes
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device) if ws_bytes else None
        hit = _plans[key] = (plan, ws)
    return hit


_run_fn = None


def _gemm_run():
    global _run_fn
    if _run_fn is None:
        _run_fn = nat.lib().b200_gemm_run
    return _run_fn


def _raw_stream(device: torch.device) -> int:
    """Handle of torch's current stream on ``device`` (0 = the default stream)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return raw(device.index) or None
    return torch.cuda.current_stream(device).cuda_stream or None


_EPILOGUES = {(False, False): "none", (True, True): "bias_relu", (True, False): "bias", (False, True): "relu"}
_ready_devices: set = set()


def gemm_nt_direct(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, relu: bool = False,
                   out_dtype: torch.dtype = torch.float32, scale_a: Optional[torch.Tensor] = None,
                   scale_b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The operator's implementation as a plain function: same checks and result as
    ``torch.ops.aster_b200.gemm_nt`` without the dispatcher's per-call cost (tens of
    microseconds for a Python custom op), for eager callers with small problems."""
    if not (a.is_cuda and b.is_cuda) or a.device != b.device:
        raise RuntimeError("aster_b200::gemm_nt needs both operands on the same CUDA device (there is no CPU path)")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise RuntimeError(f"expected a [M,K] and b [N,K], got {tuple(a.shape)} and {tuple(b.shape)}")
    if a.dtype != b.dtype or a.dtype not in _DTYPES or out_dtype not in _OUT_DTYPES:
        raise RuntimeError(f"unsupported dtypes {a.dtype}, {b.dtype} -> {out_dtype}")
    for name, t in (("bias", bias), ("scale_a", scale_a), ("scale_b", scale_b)):
        if t is not None and (t.dtype != torch.float32 or t.device != a.device):
            raise RuntimeError(f"{name} must be a float32 tensor on the operands' device")
    if not a.is_contiguous():
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    if bias is not None and bias.numel() != N:
        raise RuntimeError(f"bias has {bias.numel()} elements, expected N={N}")
    device = a.device
    out = torch.empty((M, N), dtype=out_dtype, device=device)

    def launch() -> None:
        if device.index not in _ready_devices:
            nat.init_current()
            _ready_devices.add(device.index)
        plan, ws = _plan_for(device, M, N, K, _DTYPES[a.dtype], _OUT_DTYPES[out_dtype], _EPILOGUES[(bias is not None, relu)])
        # Straight to the entry point with plain integers (its argument types are declared, so
        # ctypes converts them): the wrapper objects of GemmPlan.run cost more host time than a
        # small problem's kernel runs for.
        nat.check(_gemm_run()(
            plan.handle, a.data_ptr(), b.data_ptr(), out.data_ptr(), None if bias is None else bias.contiguous().data_ptr(),
            None if scale_a is None else scale_a.data_ptr(), None if scale_b is None else scale_b.data_ptr(),
            None if ws is None else ws.data_ptr(), 0 if ws is None else ws.numel(), _raw_stream(device)))

    if torch.cuda.current_device() == device.index:  # the C ABI works on the current device, like torch
        launch()
    else:
        with torch.cuda.device(device):
            launch()
    return out


@torch.library.custom_op("aster_b200::gemm_nt", mutates_args=())
def gemm_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, relu: bool = False,
            out_dtype: torch.dtype = torch.float32, scale_a: Optional[torch.Tensor] = None,
            scale_b: Optional[torch.Tensor] = None) -> torch.Tensor:
    return gemm_nt_direct(a, b, bias, relu, out_dtype, scale_a, scale_b)


@gemm_nt.register_fake
def _(a, b, bias=None, relu=False, out_dtype=torch.float32, scale_a=None, scale_b=None):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=out_dtype)


def clear_plan_cache() -> None:
    for plan, _ in _plans.values():
        plan.destroy()
    _plans.clear()
