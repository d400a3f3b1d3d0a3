"""``torch.autograd.Function`` wrappers of the two SORF stages under the upstream class names
(features/SORF.py:15-80), over ``qml_lightning_b200.cuda.sorf_gpu``.  Only the first argument is differentiable."""
import torch

from ..cuda import sorf_gpu as _ops


class SORFTransformCuda(torch.autograd.Function):
    """``apply(u [n,N], d [T,S,N], coeff_normalisation, ntransforms) -> [n,S,N]`` (features/SORF.py:15-39)."""

    @staticmethod
    def forward(ctx, u, d, coeff_normalisation, ntransforms):
        ctx.scalars = (float(coeff_normalisation), int(ntransforms))
        ctx.save_for_backward(d)
        return _ops.hadamard_transform_gpu(u, d, *ctx.scalars)

    @staticmethod
    def backward(ctx, grad_coefficients):
        (d,) = ctx.saved_tensors
        return _ops.hadamard_transform_backwards_gpu(grad_coefficients.contiguous(), d, *ctx.scalars), None, None, None


class CosFeatures(torch.autograd.Function):
    """``apply(coeffs [n,F], b [F], nmol, batch_indexes i32[n]) -> [nmol,F]`` (features/SORF.py:42-80)."""

    @staticmethod
    def forward(ctx, coeffs, b, nmol, batch_indexes):
        ctx.nmol = int(nmol)
        ctx.save_for_backward(coeffs, b, batch_indexes)
        return _ops.CosFeaturesCUDA(coeffs, b, ctx.nmol, batch_indexes)

    @staticmethod
    def backward(ctx, grad_features):
        return _ops.CosDerivativeFeaturesCUDA(grad_features.contiguous(), *ctx.saved_tensors[:2], ctx.nmol,
                                              ctx.saved_tensors[2]), None, None, None
