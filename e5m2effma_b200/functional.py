"""torch-facing wrappers over the C interface, with the argument meaning and error behaviour of
the reference binding (binds/python/csrc/e5m2effma_torch.cpp:127-274): row-major `a @ b` is
issued as the column-major product D^T = b^T a^T (its lines 179-198), statuses map to
NotImplementedError / ValueError / RuntimeError (its lines 82-88)."""
import os
from typing import Optional

import torch

from . import capi

_DT = {torch.float8_e4m3fn: capi.E4M3, torch.bfloat16: capi.BF16, torch.float16: capi.FP16,
       torch.float32: capi.FP32, torch.float8_e5m2: capi.E5M2}
_FP8 = (torch.float8_e5m2, torch.float8_e4m3fn)
_OPERANDS = (torch.float8_e5m2, torch.float8_e4m3fn, torch.bfloat16, torch.float32)


def get_include():
    """Directory holding e5m2effma.h, for C / C++ callers that link the library directly."""
    return [os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")]


def _check(status, what):
    if status == capi.OK:
        return
    msg = f"{what} failed ({capi.status_string(status)}): {capi.last_error()}"
    if status == capi.NOT_SUPPORTED:
        raise NotImplementedError(msg)
    if status == capi.INVALID_VALUE:
        raise ValueError(msg)
    raise RuntimeError(msg)


def _dtype(t, what):
    if t not in _DT:
        raise TypeError(f"{what} must be float8_e5m2, float8_e4m3fn, bfloat16, float16 or float32, got {t}")
    return _DT[t]


def _scalar(t, dev, what):
    if t is None:
        return None
    if t.device != dev:
        raise ValueError(f"{what} must be on {dev}, got {t.device}")
    if t.dtype != torch.float32:
        raise TypeError(f"{what} must be torch.float32, got {t.dtype}")
    if t.numel() != 1:
        raise ValueError(f"{what} must have exactly one element, got shape {tuple(t.shape)}")
    return t.data_ptr()


def _operand_scale(t, dev, what, outer):
    """(pointer, is_vector, holder): one float32 or one per outer index."""
    if t is None:
        return None, False, None
    if t.device != dev:
        raise ValueError(f"{what} must be on {dev}, got {t.device}")
    if t.dtype != torch.float32:
        raise TypeError(f"{what} must be torch.float32, got {t.dtype}")
    if t.numel() == 1:
        return t.data_ptr(), False, t
    if t.numel() != outer or t.dim() > 2:
        raise ValueError(f"{what} must have one element or {outer} elements, got shape {tuple(t.shape)}")
    h = t.contiguous().view(-1)
    return h.data_ptr(), True, h


def _layout(t):
    """(ok, row_major, ld) of a 2-D operand as the column-major interface sees it."""
    r, c = t.shape
    if t.stride(1) == 1 and (r <= 1 or t.stride(0) >= c):
        return True, True, (c if r <= 1 else t.stride(0))
    if t.stride(0) == 1 and (c <= 1 or t.stride(1) >= r):
        return True, False, (r if c <= 1 else t.stride(1))
    return False, False, 0


def _qualified(t, k_is_dim1):
    ok, row, ld = _layout(t)
    if ok and ld % 16 == 0 and t.data_ptr() % 16 == 0:
        return t, row, ld
    c = t.contiguous() if k_is_dim1 else t.t().contiguous().t()
    ok, row, ld = _layout(c)
    return c, row, ld


def matmul(a, b, *, out_dtype: Optional[torch.dtype] = None, bias=None, out=None, alpha: float = 1.0,
           beta: float = 0.0, scale_a=None, scale_b=None, scale_out=None, amax_out=None):
    """out = alpha * (scale_a * scale_b) * (a @ b) + bias + beta * out for a [M, K], b [K, N]."""
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError(f"a and b must be 2-D, got shapes {tuple(a.shape)} and {tuple(b.shape)}")
    for t, nm in ((a, "a"), (b, "b")):
        if t.dtype not in _OPERANDS:
            raise TypeError(f"{nm} must be float8_e5m2, float8_e4m3fn, bfloat16 or float32, got {t.dtype}")
    if not a.is_cuda:
        raise ValueError(f"a must be a CUDA tensor, got a tensor on {a.device}")
    dev = a.device
    if b.device != dev:
        raise ValueError(f"b must be on {dev}, got {b.device}")
    M, K = a.shape
    N = b.shape[1]
    if b.shape[0] != K:
        raise ValueError(f"shapes do not match for a @ b: {tuple(a.shape)} and {tuple(b.shape)}")
    if K % 16:
        raise ValueError(f"K = {K} must be a multiple of 16 (pad the reduction dimension with zeros)")
    if scale_a is not None and a.dtype not in _FP8:
        raise ValueError("scale_a is only meaningful for an FP8 a (it is the dequantization factor)")
    if scale_b is not None and b.dtype not in _FP8:
        raise ValueError("scale_b is only meaningful for an FP8 b (it is the dequantization factor)")
    if beta != 0.0 and out is None:
        raise ValueError("beta != 0 accumulates into out, so out must be given")
    if out is not None:
        if out.device != dev:
            raise ValueError(f"out must be on {dev}, got {out.device}")
        _dtype(out.dtype, "out")
        if out_dtype is not None and out_dtype != out.dtype:
            raise ValueError(f"out_dtype {out_dtype} does not match out.dtype {out.dtype}")
        if out.dim() != 2 or tuple(out.shape) != (M, N):
            raise ValueError(f"out must have shape [{M}, {N}], got {tuple(out.shape)}")
        if out.stride(1) != 1 or (M > 1 and out.stride(0) < N):
            raise ValueError(f"out must be row-contiguous (stride(1) == 1), got strides {out.stride()}")
    else:
        out = torch.empty((M, N), device=dev, dtype=out_dtype or torch.bfloat16)
    dt = _dtype(out.dtype, "out")
    if scale_out is not None and out.dtype not in _FP8:
        raise ValueError("scale_out is only meaningful for an FP8 output (it is the quantization factor)")
    if bias is not None:
        if bias.device != dev:
            raise ValueError(f"bias must be on {dev}, got {bias.device}")
        _dtype(bias.dtype, "bias")
        if bias.dim() != 1 or bias.shape[0] != N or bias.stride(0) != 1:
            raise ValueError(f"bias must be a contiguous vector of length N = {N}, got shape {tuple(bias.shape)}")
    if M == 0 or N == 0:
        return out
    qa, a_row, lda = _qualified(a, True)
    qb, b_row, ldb = _qualified(b, False)
    # column-major view: out^T (N x M) = b^T (N x K) * a^T (K x M)
    transa = capi.OP_N if b_row else capi.OP_T
    transb = capi.OP_N if a_row else capi.OP_T
    sa_ptr, sa_vec, _ha = _operand_scale(scale_a, dev, "scale_a", M)
    sb_ptr, sb_vec, _hb = _operand_scale(scale_b, dev, "scale_b", N)
    A = capi.tensor(qb.data_ptr(), _DT[b.dtype], sb_ptr, None, None, capi.SCALING_OUTER if sb_vec else 0)
    B = capi.tensor(qa.data_ptr(), _DT[a.dtype], sa_ptr, None, None, capi.SCALING_OUTER if sa_vec else 0)
    D = capi.tensor(out.data_ptr(), dt, None, _scalar(scale_out, dev, "scale_out"), _scalar(amax_out, dev, "amax_out"))
    BIAS = None if bias is None else capi.tensor(bias.data_ptr(), _DT[bias.dtype])
    ldd = N if M <= 1 else out.stride(0)
    with torch.cuda.device(dev):
        st = capi.gemm(transa, transb, N, M, K, float(alpha), A, ldb, B, lda, float(beta), None, 0, D, ldd, BIAS,
                       torch.cuda.current_stream().cuda_stream)
    _check(st, "e5ma_gemm")
    return out


def linear(x, weight, bias=None, *, out_dtype=None, scale_x=None, scale_w=None, scale_out=None, amax_out=None):
    """x @ weight.t() + bias; x [..., K], weight [N, K] (both K-contiguous: the FP8 layout)."""
    if weight.dim() != 2:
        raise ValueError(f"weight must be 2-D [out_features, in_features], got shape {tuple(weight.shape)}")
    if x.dim() < 1 or x.shape[-1] != weight.shape[1]:
        raise ValueError(f"x must have shape [..., {weight.shape[1]}], got {tuple(x.shape)}")
    x2 = x.reshape(-1, x.shape[-1])
    if scale_x is not None and scale_x.numel() > 1:
        scale_x = scale_x.reshape(-1)
    y = matmul(x2, weight.t(), out_dtype=out_dtype, bias=bias, scale_a=scale_x, scale_b=scale_w,
               scale_out=scale_out, amax_out=amax_out)
    return y.reshape(*x.shape[:-1], weight.shape[0])


def cast(x, dtype, *, scale_inv=None, scale=None, amax=None):
    """Element-wise conversion between the five dtypes; returns a new contiguous tensor."""
    if not x.is_cuda:
        raise ValueError(f"x must be a CUDA tensor, got a tensor on {x.device}")
    dev = x.device
    st, dt = _dtype(x.dtype, "x"), _dtype(dtype, "dtype")
    if scale_inv is not None and x.dtype not in _FP8:
        raise ValueError("scale_inv is only meaningful for an FP8 x")
    if scale is not None and dtype not in _FP8:
        raise ValueError("scale is only meaningful for an FP8 result")
    xc = x.contiguous()
    y = torch.empty(xc.shape, device=dev, dtype=dtype)
    if xc.numel() == 0:
        return y
    S = capi.tensor(xc.data_ptr(), st, _scalar(scale_inv, dev, "scale_inv"))
    D = capi.tensor(y.data_ptr(), dt, None, _scalar(scale, dev, "scale"), _scalar(amax, dev, "amax"))
    with torch.cuda.device(dev):
        _check(capi.cast(S, D, xc.numel(), torch.cuda.current_stream().cuda_stream), "e5ma_cast")
    return y


def adam_step(param, grad, exp_avg, exp_avg_sq, *, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, step,
              adamw=True, bias_correction=True, grad_scale=1.0, param_fp8=None, fp8_scale=None, fp8_amax=None):
    """One fused in-place Adam / AdamW step (step counts from 1)."""
    if not param.is_cuda:
        raise ValueError(f"param must be a CUDA tensor, got a tensor on {param.device}")
    dev = param.device
    n = param.numel()
    for t, nm in ((grad, "grad"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        if t.device != dev:
            raise ValueError(f"{nm} must be on {dev}, got {t.device}")
        if t.numel() != n:
            raise ValueError(f"{nm} has {t.numel()} elements, param has {n}")
    for t, nm in ((param, "param"), (grad, "grad"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        if not t.is_contiguous():
            raise ValueError(f"{nm} must be contiguous")
    if param.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"param must be torch.float32 or torch.bfloat16, got {param.dtype}")
    if grad.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise TypeError(f"grad must be torch.float32, torch.bfloat16 or torch.float16, got {grad.dtype}")
    if exp_avg.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"exp_avg must be torch.float32 or torch.bfloat16, got {exp_avg.dtype}")
    if exp_avg_sq.dtype != exp_avg.dtype:
        raise TypeError(f"exp_avg_sq must have the dtype of exp_avg ({exp_avg.dtype}), got {exp_avg_sq.dtype}")
    if step < 1:
        raise ValueError(f"step must be >= 1 (1-based), got {step}")
    if lr < 0.0 or eps < 0.0 or weight_decay < 0.0:
        raise ValueError("lr, eps and weight_decay must be non-negative")
    b1, b2 = betas
    if not (0.0 <= b1 < 1.0 and 0.0 <= b2 < 1.0):
        raise ValueError(f"betas must be in [0, 1), got ({b1}, {b2})")
    Q = None
    if param_fp8 is not None:
        if param_fp8.device != dev:
            raise ValueError(f"param_fp8 must be on {dev}, got {param_fp8.device}")
        if param_fp8.dtype not in _FP8:
            raise TypeError(f"param_fp8 must be torch.float8_e5m2 or torch.float8_e4m3fn, got {param_fp8.dtype}")
        if param_fp8.numel() != n or not param_fp8.is_contiguous():
            raise ValueError(f"param_fp8 must be contiguous with the element count of param ({n})")
        Q = capi.tensor(param_fp8.data_ptr(), _DT[param_fp8.dtype], None, _scalar(fp8_scale, dev, "fp8_scale"),
                        _scalar(fp8_amax, dev, "fp8_amax"))
    elif fp8_scale is not None or fp8_amax is not None:
        raise ValueError("fp8_scale / fp8_amax need param_fp8")
    if n == 0:
        return
    cfg = capi.AdamConfig(lr, b1, b2, eps, weight_decay, int(step), int(bool(adamw)), int(bool(bias_correction)),
                          grad_scale)
    P = capi.tensor(param.data_ptr(), _DT[param.dtype])
    G = capi.tensor(grad.data_ptr(), _DT[grad.dtype])
    M = capi.tensor(exp_avg.data_ptr(), _DT[exp_avg.dtype])
    V = capi.tensor(exp_avg_sq.data_ptr(), _DT[exp_avg_sq.dtype])
    with torch.cuda.device(dev):
        _check(capi.adam(cfg, n, P, G, M, V, Q, torch.cuda.current_stream().cuda_stream), "e5ma_adam")


def adam_step_multi(params, grads, exp_avgs, exp_avg_sqs, *, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, step,
                    adamw=True, bias_correction=True, grad_scale=1.0):
    """One Adam / AdamW step over lists of tensors that share a device and their dtypes, in as few kernel
    launches as possible (e5b_adam_multi); same arithmetic as adam_step on each tensor."""
    if not params:
        return
    dev = params[0].device
    for lst, nm in ((params, "params"), (grads, "grads"), (exp_avgs, "exp_avgs"), (exp_avg_sqs, "exp_avg_sqs")):
        if len(lst) != len(params):
            raise ValueError(f"{nm} has {len(lst)} tensors, params has {len(params)}")
        for t in lst:
            if t.device != dev or not t.is_cuda:
                raise ValueError(f"every tensor must be on {dev}")
            if not t.is_contiguous():
                raise ValueError(f"{nm} must be contiguous")
    for p, g, m, v in zip(params, grads, exp_avgs, exp_avg_sqs):
        if not (p.numel() == g.numel() == m.numel() == v.numel()):
            raise ValueError("param, grad and moments of one entry must have the same number of elements")
    if step < 1:
        raise ValueError(f"step must be >= 1 (1-based), got {step}")
    b1, b2 = betas
    cfg = capi.AdamConfig(lr, b1, b2, eps, weight_decay, int(step), int(bool(adamw)), int(bool(bias_correction)), grad_scale)
    T = lambda t: capi.tensor(t.data_ptr(), _dtype(t.dtype, "tensor"))
    with torch.cuda.device(dev):
        st = capi.adam_multi(cfg, [p.numel() for p in params], [T(p) for p in params], [T(g) for g in grads],
                             [T(m) for m in exp_avgs], [T(v) for v in exp_avg_sqs], None,
                             torch.cuda.current_stream().cuda_stream)
    _check(st, "e5b_adam_multi")


class AdamW(torch.optim.Optimizer):
    """torch.optim-style AdamW (Adam with adamw=False) on the fused kernel; same hyper-parameters and
    state as the reference's optimizer (binds/python/e5m2effma/optim.py:31-53), but parameters that share a
    device, dtypes and step count are updated by shared launches (e5b_adam_multi) instead of one each."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, *, adamw=True,
                 state_dtype=None):
        if lr < 0.0 or eps < 0.0 or weight_decay < 0.0:
            raise ValueError(f"lr, eps and weight_decay must be non-negative (got {lr}, {eps}, {weight_decay})")
        if not (0.0 <= betas[0] < 1.0 and 0.0 <= betas[1] < 1.0):
            raise ValueError(f"betas must be in [0, 1), got {betas}")
        if state_dtype not in (None, torch.float32, torch.bfloat16):
            raise TypeError(f"state_dtype must be torch.float32 or torch.bfloat16, got {state_dtype}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adamw=adamw,
                                      state_dtype=state_dtype or torch.float32))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            buckets = {}   # (device, param dtype, grad dtype, step) -> tensors that can share launches
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise ValueError("AdamW does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=group["state_dtype"], memory_format=torch.contiguous_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=group["state_dtype"], memory_format=torch.contiguous_format)
                st["step"] += 1
                if not (p.is_contiguous() and p.grad.is_contiguous()):
                    raise ValueError("parameters and gradients must be contiguous")
                b = buckets.setdefault((p.device, p.dtype, p.grad.dtype, st["step"]), ([], [], [], []))
                b[0].append(p); b[1].append(p.grad); b[2].append(st["exp_avg"]); b[3].append(st["exp_avg_sq"])
            for (_, _, _, stp), (ps, gs, ms, vs) in buckets.items():
                adam_step_multi(ps, gs, ms, vs, lr=group["lr"], betas=group["betas"], eps=group["eps"],
                                weight_decay=group["weight_decay"], step=stp, adamw=group["adamw"])
        return loss
