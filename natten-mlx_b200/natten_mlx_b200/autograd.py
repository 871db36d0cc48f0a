"""``torch.autograd.Function`` wrappers binding each forward to its backward.

They take the place of the reference's ``mx.custom_function`` / ``.vjp``
wrappers (src/natten_mlx/autograd/na2d.py:12-99, src/natten_mlx/autograd/split.py:12-261):
tensors first, then the normalised tuples, ``None`` gradients for everything
that is not a tensor.  The fused function saves its output and log-sum-exp, so
the backward recomputes nothing but the softmax weights.
"""

from __future__ import annotations

import torch

from ._core import ops
from ._core import cuda as _cuda


class _FusedNA(torch.autograd.Function):
    """(out, lse) = attention over the window (and extra tokens)."""

    @staticmethod
    def forward(ctx, q, k, v, k_extra, v_extra, sizes, ks, st, dl, ca, scale, host_sizes=None):
        backend = ops._backend_module()
        out, lse = backend.fused_forward(q, k, v, ks, st, dl, ca, scale, k_extra=k_extra, v_extra=v_extra,
                                         sizes=sizes, host_sizes=host_sizes)
        ctx.save_for_backward(q, k, v, k_extra, v_extra, out, lse)
        ctx.sizes = sizes
        ctx.host_sizes = host_sizes
        ctx.params = (ks, st, dl, ca, scale)
        ctx.mark_non_differentiable()
        return out, lse

    @staticmethod
    def backward(ctx, grad_out, grad_lse):
        q, k, v, k_extra, v_extra, out, lse = ctx.saved_tensors
        ks, st, dl, ca, scale = ctx.params
        backend = ops._backend_module()
        if grad_out is None:
            grad_out = torch.zeros_like(out)
        dq, dk, dv, dke, dve = backend.fused_backward(
            q, k, v, out, lse, grad_out, grad_lse, ks, st, dl, ca, scale, k_extra=k_extra, v_extra=v_extra,
            sizes=ctx.sizes, host_sizes=ctx.host_sizes)
        return dq, dk, dv, dke, dve, None, None, None, None, None, None, None


class _QK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, rank, ks, st, dl, ca, scale):
        ctx.save_for_backward(q, k)
        ctx.params = (rank, ks, st, dl, ca, scale)
        return getattr(ops, f"na{rank}d_qk_forward")(q, k, ks, st, dl, ca, scale)

    @staticmethod
    def backward(ctx, grad_attn):
        q, k = ctx.saved_tensors
        rank, ks, st, dl, ca, scale = ctx.params
        dq, dk = getattr(ops, f"na{rank}d_qk_backward")(q, k, grad_attn, ks, st, dl, ca, scale)
        return dq, dk, None, None, None, None, None, None


class _AV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, attn, v, rank, ks, st, dl, ca):
        ctx.save_for_backward(attn, v)
        ctx.params = (rank, ks, st, dl, ca)
        return getattr(ops, f"na{rank}d_av_forward")(attn, v, ks, st, dl, ca)

    @staticmethod
    def backward(ctx, grad_out):
        attn, v = ctx.saved_tensors
        rank, ks, st, dl, ca = ctx.params
        dattn, dv = getattr(ops, f"na{rank}d_av_backward")(attn, v, grad_out, ks, st, dl, ca)
        return dattn, dv, None, None, None, None, None


class _QKBias(torch.autograd.Function):
    """QK logits with a relative position bias (the allin1 ops)."""

    @staticmethod
    def forward(ctx, q, k, rpb, ks, dl, scale):
        rank = q.dim() - 3
        one, no = (1,) * rank, (False,) * rank
        ctx.save_for_backward(q, k)
        ctx.params = (ks, dl, scale, None if rpb is None else tuple(rpb.shape), one, no)
        return _cuda.qk_forward(q, k, ks, one, dl, no, scale, bias=rpb)

    @staticmethod
    def backward(ctx, grad_attn):
        q, k = ctx.saved_tensors
        ks, dl, scale, rpb_shape, one, no = ctx.params
        res = _cuda.qk_backward(q, k, grad_attn, ks, one, dl, no, scale, want_dbias_shape=rpb_shape)
        drpb = res[2] if rpb_shape is not None else None
        return res[0], res[1], drpb, None, None, None


class _Merge(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o0, l0, o1, l1):
        ctx.save_for_backward(o0, l0, o1, l1)
        return _cuda.merge_forward(o0, l0, o1, l1)

    @staticmethod
    def backward(ctx, grad_out, grad_lse):
        o0, l0, o1, l1 = ctx.saved_tensors
        if grad_out is None:
            grad_out = torch.zeros_like(o0)
        do0, dl0, do1, dl1 = _cuda.merge_backward(o0, l0, o1, l1, grad_out, grad_lse)
        return do0, dl0.to(l0.dtype), do1, dl1.to(l1.dtype)


def fused_with_grad(q, k, v, ks, st, dl, ca, scale, k_extra=None, v_extra=None, sizes=None, host_sizes=None):
    """(out, lse) with gradients for q, k, v and the extra tokens.  ``host_sizes`` is a host copy of the per-sample
    ``sizes`` (it lets a variable-size batch run on the tensor-core kernels without a device-to-host copy)."""
    return _FusedNA.apply(q, k, v, k_extra, v_extra, sizes, ks, st, dl, ca, scale, host_sizes)


def _named(rank):
    def fused(q, k, v, kernel_size, stride, dilation, is_causal, scale):
        return fused_with_grad(q, k, v, kernel_size, stride, dilation, is_causal, scale)[0]

    def qk(q, k, kernel_size, stride, dilation, is_causal, scale):
        return _QK.apply(q, k, rank, kernel_size, stride, dilation, is_causal, scale)

    def av(attn, v, kernel_size, stride, dilation, is_causal):
        return _AV.apply(attn, v, rank, kernel_size, stride, dilation, is_causal)

    def varlen(q, k, v, sizes, kernel_size, dilation, scale):
        one, no = (1,) * rank, (False,) * rank
        return fused_with_grad(q, k, v, kernel_size, one, dilation, no, scale, sizes=sizes)[0]

    return fused, qk, av, varlen


na1d_with_grad, na1d_qk_with_grad, na1d_av_with_grad, na1d_varlen_with_grad = _named(1)
na2d_with_grad, na2d_qk_with_grad, na2d_av_with_grad, na2d_varlen_with_grad = _named(2)
na3d_with_grad, na3d_qk_with_grad, na3d_av_with_grad, na3d_varlen_with_grad = _named(3)


def qk_bias_with_grad(q, k, rpb, ks, dl, scale):
    return _QKBias.apply(q, k, rpb, ks, dl, scale)


def merge_pair_with_grad(o0, l0, o1, l1):
    return _Merge.apply(o0, l0, o1, l1)
