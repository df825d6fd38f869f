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


def _byte_range(t):
    """[first, last) byte addresses a strided tensor can touch."""
    if t.numel() == 0:
        return 0, 0
    span = 1 + sum((n - 1) * abs(st) for n, st in zip(t.shape, t.stride()))
    return t.data_ptr(), t.data_ptr() + span * t.element_size()


def _overlap(x, y):
    (x0, x1), (y0, y1) = _byte_range(x), _byte_range(y)
    return x0 < y1 and y0 < x1


class _Product:
    """Validation and lowering of one row-major product out[M, N] = a[M, K] @ b[K, N] onto the column-major C
    interface.  In column-major terms the same bytes are out^T[N, M] = b^T[N, K] a^T[K, M], so b plays the
    interface's A and a plays its B (the reference binding lowers the same way, csrc/e5m2effma_torch.cpp:179-198);
    a row-major operand is "not transposed" on that side, a column-major one "transposed"."""

    def __init__(self, a, b):
        if a.dim() != 2 or b.dim() != 2:
            raise ValueError(f"matmul takes 2-D operands; got shapes {tuple(a.shape)} and {tuple(b.shape)}")
        for label, t in (("a", a), ("b", b)):
            if t.dtype not in _OPERANDS:
                raise TypeError(f"operand {label}: dtype must be float8_e5m2, float8_e4m3fn, bfloat16 or float32, not {t.dtype}")
        if not a.is_cuda:
            raise ValueError(f"operand a lives on {a.device}; a CUDA tensor is required (there is no host path)")
        if b.device != a.device:
            raise ValueError(f"operand b lives on {b.device} but a on {a.device}")
        if a.shape[1] != b.shape[0]:
            raise ValueError(f"inner shapes disagree in a @ b: {tuple(a.shape)} x {tuple(b.shape)}")
        if a.shape[1] % 16:
            raise ValueError(f"the reduction length K = {a.shape[1]} is not a multiple of 16; zero-pad K")
        self.a, self.b, self.dev = a, b, a.device
        self.M, self.K, self.N = a.shape[0], a.shape[1], b.shape[1]

    def scales(self, scale_a, scale_b, scale_out, out_dtype):
        if scale_a is not None and self.a.dtype not in _FP8:
            raise ValueError("scale_a dequantises an FP8 a; a is not FP8")
        if scale_b is not None and self.b.dtype not in _FP8:
            raise ValueError("scale_b dequantises an FP8 b; b is not FP8")
        if scale_out is not None and out_dtype not in _FP8:
            raise ValueError("scale_out quantises an FP8 result; the output is not FP8")
        self.sa = _operand_scale(scale_a, self.dev, "scale_a", self.M)
        self.sb = _operand_scale(scale_b, self.dev, "scale_b", self.N)

    def output(self, out, out_dtype, beta):
        M, N = self.M, self.N
        if out is None:
            if beta != 0.0:
                raise ValueError("a non-zero beta adds to the previous content of out: out must be given")
            return torch.empty((M, N), device=self.dev, dtype=out_dtype or torch.bfloat16)
        if out.device != self.dev:
            raise ValueError(f"out lives on {out.device} but the operands on {self.dev}")
        _dtype(out.dtype, "out")
        if out_dtype is not None and out_dtype != out.dtype:
            raise ValueError(f"out_dtype = {out_dtype} contradicts out.dtype = {out.dtype}")
        if tuple(out.shape) != (M, N):
            raise ValueError(f"out has shape {tuple(out.shape)}; the product has shape ({M}, {N})")
        if out.stride(1) != 1 or (M > 1 and out.stride(0) < N):
            raise ValueError(f"out must be row-contiguous without overlapping rows; its strides are {out.stride()}")
        for label, t in (("a", self.a), ("b", self.b)):
            if _overlap(out, t):
                raise ValueError(f"out and {label} share memory; the kernels read operands while they write the result")
        return out

    def bias(self, bias):
        if bias is None:
            return None
        if bias.device != self.dev:
            raise ValueError(f"bias lives on {bias.device} but the operands on {self.dev}")
        _dtype(bias.dtype, "bias")
        if bias.dim() != 1 or bias.shape[0] != self.N or bias.stride(0) != 1:
            raise ValueError(f"bias must be a dense vector with one entry per output column ({self.N}); got shape {tuple(bias.shape)}")
        return capi.tensor(bias.data_ptr(), _DT[bias.dtype])

    def run(self, out, bias_t, alpha, beta, scale_out, amax_out):
        qa, a_rowmajor, lda = _qualified(self.a, True)
        qb, b_rowmajor, ldb = _qualified(self.b, False)
        (pa, a_vec, _keep_a), (pb, b_vec, _keep_b) = self.sa, self.sb
        first = capi.tensor(qb.data_ptr(), _DT[self.b.dtype], pb, None, None, capi.SCALING_OUTER if b_vec else 0)
        second = capi.tensor(qa.data_ptr(), _DT[self.a.dtype], pa, None, None, capi.SCALING_OUTER if a_vec else 0)
        result = capi.tensor(out.data_ptr(), _DT[out.dtype], None, _scalar(scale_out, self.dev, "scale_out"),
                             _scalar(amax_out, self.dev, "amax_out"))
        ld_out = self.N if self.M <= 1 else out.stride(0)
        with torch.cuda.device(self.dev):
            st = capi.gemm(capi.OP_N if b_rowmajor else capi.OP_T, capi.OP_N if a_rowmajor else capi.OP_T, self.N, self.M, self.K,
                           float(alpha), first, ldb, second, lda, float(beta), None, 0, result, ld_out, bias_t,
                           torch.cuda.current_stream().cuda_stream)
        _check(st, "e5ma_gemm")


def matmul(a, b, *, out_dtype: Optional[torch.dtype] = None, bias=None, out=None, alpha: float = 1.0,
           beta: float = 0.0, scale_a=None, scale_b=None, scale_out=None, amax_out=None):
    """out = alpha * (scale_a * scale_b) * (a @ b) + bias + beta * out for a [M, K], b [K, N]."""
    prod = _Product(a, b)
    out = prod.output(out, out_dtype, beta)
    prod.scales(scale_a, scale_b, scale_out, out.dtype)
    bias_t = prod.bias(bias)
    if prod.M and prod.N:
        prod.run(out, bias_t, alpha, beta, scale_out, amax_out)
    return out


def linear(x, weight, bias=None, *, out_dtype=None, scale_x=None, scale_w=None, scale_out=None, amax_out=None):
    """x @ weight.t() + bias; x [..., K], weight [N, K] (both K-contiguous: the FP8 layout)."""
    if weight.dim() != 2:
        raise ValueError(f"weight is [out_features, in_features]; got shape {tuple(weight.shape)}")
    out_features, in_features = weight.shape
    if x.dim() == 0 or x.shape[-1] != in_features:
        raise ValueError(f"the last dimension of x must be in_features = {in_features}; got shape {tuple(x.shape)}")
    lead = x.shape[:-1]
    rows = x.reshape(-1, in_features)
    per_row = scale_x.reshape(-1) if scale_x is not None and scale_x.numel() > 1 else scale_x
    flat = matmul(rows, weight.t(), out_dtype=out_dtype, bias=bias, scale_a=per_row, scale_b=scale_w, scale_out=scale_out,
                  amax_out=amax_out)
    return flat.reshape(*lead, out_features)


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


def _hyper(lr, betas, eps, weight_decay, step=1):
    """Range checks shared by the optimizer entry points; returns the two betas."""
    if step < 1:
        raise ValueError(f"step counts from 1; got step = {step}")
    for label, v in (("lr", lr), ("eps", eps), ("weight_decay", weight_decay)):
        if v < 0.0:
            raise ValueError(f"{label} = {v} is negative")
    b1, b2 = betas
    if not (0.0 <= b1 < 1.0 and 0.0 <= b2 < 1.0):
        raise ValueError(f"betas must lie in [0, 1); got ({b1}, {b2})")
    return b1, b2


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
    state = (("param", param), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq))
    for i, (na, ta) in enumerate(state):        # the three arrays are rewritten in place, element by element
        for nb, tb in state[i + 1:] + (("grad", grad),):
            if _overlap(ta, tb):
                raise ValueError(f"{na} and {nb} share memory")
    if param.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"param must be torch.float32 or torch.bfloat16, got {param.dtype}")
    if grad.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise TypeError(f"grad must be torch.float32, torch.bfloat16 or torch.float16, got {grad.dtype}")
    if exp_avg.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"exp_avg must be torch.float32 or torch.bfloat16, got {exp_avg.dtype}")
    if exp_avg_sq.dtype != exp_avg.dtype:
        raise TypeError(f"exp_avg_sq must have the dtype of exp_avg ({exp_avg.dtype}), got {exp_avg_sq.dtype}")
    b1, b2 = _hyper(lr, betas, eps, weight_decay, step)
    Q = None
    if param_fp8 is not None:
        if param_fp8.device != dev:
            raise ValueError(f"param_fp8 must be on {dev}, got {param_fp8.device}")
        if param_fp8.dtype not in _FP8:
            raise TypeError(f"param_fp8 must be torch.float8_e5m2 or torch.float8_e4m3fn, got {param_fp8.dtype}")
        if param_fp8.numel() != n or not param_fp8.is_contiguous():
            raise ValueError(f"param_fp8 must be contiguous with the element count of param ({n})")
        for nb, tb in state + (("grad", grad),):
            if _overlap(param_fp8, tb):
                raise ValueError(f"param_fp8 and {nb} share memory")
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
    b1, b2 = _hyper(lr, betas, eps, weight_decay, step)
    live = [i for i, p in enumerate(params) if p.numel() > 0]      # empty tensors have no address to pass on
    if not live:
        return
    params, grads, exp_avgs, exp_avg_sqs = ([lst[i] for i in live] for lst in (params, grads, exp_avgs, exp_avg_sqs))
    cfg = capi.AdamConfig(lr, b1, b2, eps, weight_decay, int(step), int(bool(adamw)), int(bool(bias_correction)), grad_scale)
    T = lambda t: capi.tensor(t.data_ptr(), _dtype(t.dtype, "tensor"))
    with torch.cuda.device(dev):
        st = capi.adam_multi(cfg, [p.numel() for p in params], [T(p) for p in params], [T(g) for g in grads],
                             [T(m) for m in exp_avgs], [T(v) for v in exp_avg_sqs], None,
                             torch.cuda.current_stream().cuda_stream)
    _check(st, "e5b_adam_multi")


class AdamW(torch.optim.Optimizer):
    """AdamW (or Adam with L2 regularisation when adamw=False) as a torch.optim optimizer on the fused kernel.
    Hyper-parameters and per-parameter state ("step", "exp_avg", "exp_avg_sq") are those of the reference's
    optimizer (binds/python/e5m2effma/optim.py:31-53), so checkpoints carry over; unlike it, parameters that agree
    in device, dtypes and step count are updated by shared launches (e5b_adam_multi) instead of one launch each."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, *, adamw=True,
                 state_dtype=None):
        _hyper(lr, betas, eps, weight_decay)
        if state_dtype is None:
            state_dtype = torch.float32
        if state_dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"moments are kept in float32 or bfloat16; got state_dtype = {state_dtype}")
        defaults = {"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay, "adamw": adamw, "state_dtype": state_dtype}
        super().__init__(params, defaults)

    def _moments(self, p, dtype):
        """State of parameter p, created on first use; returns (exp_avg, exp_avg_sq, step after this update)."""
        st = self.state[p]
        if "step" not in st:
            st["step"] = 0
            for key in ("exp_avg", "exp_avg_sq"):
                st[key] = torch.zeros_like(p, dtype=dtype, memory_format=torch.contiguous_format)
        st["step"] += 1
        return st["exp_avg"], st["exp_avg_sq"], st["step"]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            launches = {}      # (device, param dtype, grad dtype, step) -> four parallel lists for one multi-tensor call
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                if g.is_sparse:
                    raise ValueError("sparse gradients are not supported by the fused kernel")
                if not (p.is_contiguous() and g.is_contiguous()):
                    raise ValueError("the fused kernel needs contiguous parameters and gradients")
                m, v, t = self._moments(p, group["state_dtype"])
                lists = launches.setdefault((p.device, p.dtype, g.dtype, t), ([], [], [], []))
                for lst, x in zip(lists, (p, g, m, v)):
                    lst.append(x)
            for (_dev, _pt, _gt, t), (ps, gs, ms, vs) in launches.items():
                adam_step_multi(ps, gs, ms, vs, lr=group["lr"], betas=group["betas"], eps=group["eps"],
                                weight_decay=group["weight_decay"], step=t, adamw=group["adamw"])
        return loss
