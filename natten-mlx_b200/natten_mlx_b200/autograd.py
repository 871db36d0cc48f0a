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
    def forward(ctx, q, k, v, k_extra, v_extra, sizes, ks, st, dl, ca, scale):
        backend = ops._backend_module()
        out, lse = backend.fused_forward(q, k, v, ks, st, dl, ca, scale, k_extra=k_extra, v_extra=v_extra,
                                         sizes=sizes)
        ctx.save_for_backward(q, k, v, k_extra, v_extra, out, lse)
        ctx.sizes = sizes
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
            sizes=ctx.sizes)
        return dq, dk, dv, dke, dve, None, None, None, None, None, None


class _PerSampleNA(torch.autograd.Function):
    """(out, lse) of a variable-size batch, one tensor-core call per sample; zeros in the padding."""

    @staticmethod
    def forward(ctx, q, k, v, host_sizes, ks, dl, scale):
        backend = ops._backend_module()
        out, lse = backend.fused_forward_per_sample(q, k, v, host_sizes, ks, dl, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.params = (host_sizes, ks, dl, scale)
        return out, lse

    @staticmethod
    def backward(ctx, grad_out, grad_lse):
        q, k, v, out, lse = ctx.saved_tensors
        host_sizes, ks, dl, scale = ctx.params
        backend = ops._backend_module()
        if grad_out is None:
            grad_out = torch.zeros_like(out)
        dq, dk, dv = backend.fused_backward_per_sample(q, k, v, out, lse, grad_out, grad_lse, host_sizes, ks, dl,
                                                       scale)
        return dq, dk, dv, None, None, None, None


class _DenseExtra(torch.autograd.Function):
    """Dense attention of every query over a few extra tokens, returning (out, lse) with gradients
    through both: torch's flash scaled-dot-product kernel (a library kernel for a plain dense
    attention, as the reference's ``mx.fast.scaled_dot_product_attention``, functional.py:176).
    The library's backward knows nothing of a gradient on the log-sum-exp; that term is
    ``dq += dlse * scale * softmax(S) K`` (one more forward with V := K) and
    ``dK += scale * softmax(S)^T (dlse * q)`` (the value gradient of one more backward)."""

    @staticmethod
    def forward(ctx, q, ak, av, scale):
        rep = q.shape[-2] // ak.shape[-2]
        qt = q.transpose(1, 2)                                            # [B, Hq, N, D]
        kk = ak.repeat_interleave(rep, dim=2).transpose(1, 2).contiguous()  # [B, Hq, X, D]
        vv = av.repeat_interleave(rep, dim=2).transpose(1, 2).contiguous()
        res = torch.ops.aten._scaled_dot_product_flash_attention(qt, kk, vv, 0.0, False, False, scale=scale)
        ctx.save_for_backward(qt, kk, vv, res[0], res[1], res[2], res[3], res[6], res[7])
        ctx.meta = (res[4], res[5], float(scale), rep)
        return res[0].transpose(1, 2), res[1].transpose(1, 2)

    @staticmethod
    def backward(ctx, grad_out, grad_lse):
        qt, kk, vv, out, lse, cq, ck, seed, offset = ctx.saved_tensors
        max_q, max_k, scale, rep = ctx.meta
        op_f = torch.ops.aten._scaled_dot_product_flash_attention
        op_b = torch.ops.aten._scaled_dot_product_flash_attention_backward
        go = torch.zeros_like(out) if grad_out is None else grad_out.transpose(1, 2)   # strided view: no copy
        dq, dk, dv = op_b(go, qt, kk, vv, out, lse, cq, ck, max_q, max_k, 0.0, False, seed, offset, scale=scale)
        if grad_lse is not None:
            gl = (grad_lse.transpose(1, 2) * scale).to(qt.dtype)[..., None]           # [B, Hq, N, 1]
            res = op_f(qt, kk, kk, 0.0, False, False, scale=scale)
            dq.addcmul_(gl, res[0])
            _, _, dk_l = op_b(gl * qt, qt, kk, kk, res[0], res[1], res[2], res[3], res[4], res[5],
                              0.0, False, res[6], res[7], scale=scale)
            dk = dk + dk_l
        b, hq, x, d = dk.shape
        fold = lambda t: t.view(b, hq // rep, rep, x, d).float().sum(2).to(t.dtype).transpose(1, 2)   # [B, X, Hkv, D]
        return dq.transpose(1, 2), fold(dk), fold(dv), None


def dense_extra_with_grad(q, ak, av, scale):
    """(out [B, N, Hq, D], lse [B, N, Hq]) of dense attention over the extra tokens."""
    return _DenseExtra.apply(q, ak, av, scale)


def per_sample_with_grad(q, k, v, host_sizes, ks, dl, scale):
    return _PerSampleNA.apply(q, k, v, host_sizes, ks, dl, scale)


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


def fused_with_grad(q, k, v, ks, st, dl, ca, scale, k_extra=None, v_extra=None, sizes=None):
    """(out, lse) with gradients for q, k, v and the extra tokens."""
    return _FusedNA.apply(q, k, v, k_extra, v_extra, sizes, ks, st, dl, ca, scale)


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
