"""``sorf_gpu`` of the upstream project (cuda/hadamard_cuda.cpp:23-126)."""
import torch

from .. import cabi


def hadamard_transform_gpu(input, dmatrix, normalisation, ntransforms):
    """``[n,N], [T,S,N] -> [n,S,N]`` (hadamard_cuda.cpp:47-60)."""
    if not input.is_cuda:
        raise RuntimeError("input must be a CUDA tensor")
    if not dmatrix.is_cuda:
        raise RuntimeError("dmatrix must be a CUDA tensor")
    return cabi.sorf_coefficients(input, dmatrix, float(normalisation), int(ntransforms))


def hadamard_transform_backwards_gpu(input, dmatrix, normalisation, ntransforms):
    """``[n,S,N] -> [n,N]`` (hadamard_cuda.cpp:62-75)."""
    if not input.is_cuda:
        raise RuntimeError("input must be a CUDA tensor")
    if not dmatrix.is_cuda:
        raise RuntimeError("dmatrix must be a CUDA tensor")
    return cabi.sorf_coefficients_backward(input, dmatrix, float(normalisation), int(ntransforms))


def CosFeaturesCUDA(coeffs, b, nmol, batch_indexes):
    """``f32[nmol,F]`` (hadamard_cuda.cpp:23-32)."""
    return cabi.cos_features(coeffs, b, int(nmol), batch_indexes)


def CosDerivativeFeaturesCUDA(grads, coeffs, b, nmol, batch_indexes):
    """``f32[n,F]`` (hadamard_cuda.cpp:34-43)."""
    return cabi.cos_features_backward(grads, coeffs, b, batch_indexes)


def sorf_matrix_gpu(input, scaling):
    """``[n,N], [T,S,N] -> f32[n, S*N]``: the stacked ``N^(-T/2) (HD)^T x`` without further normalisation
    (hadamard_cuda.cpp:77-91)."""
    if not input.is_cuda:
        raise RuntimeError("input must be a CUDA tensor")
    T, S, N = scaling.shape
    return cabi.sorf_coefficients(input, scaling, 1.0, T).view(input.shape[0], S * N)


def compute_hadamard_features(sorf_matrix, bias, ordering, features):
    """``features f64[nmol,F] += sqrt(2/F) cos(sorf_matrix + bias)`` (in place; hadamard_cuda.cpp:93-97)."""
    if not sorf_matrix.is_cuda:
        raise RuntimeError("sorf_matrix must be a CUDA tensor")
    cabi.hadamard_features_accumulate(sorf_matrix, bias, ordering, features)


def compute_partial_feature_derivatives(sorf_matrix, bias, sin_coeffs):
    """``sin_coeffs f64[n,F] = sqrt(2/F) sin(sorf_matrix + bias)`` (in place)."""
    cabi.partial_feature_derivatives(sorf_matrix, bias, sin_coeffs)


def compute_molecular_featurization_derivative(partial_feature_derivatives, normalisation, scaling, input_derivatives,
                                               ordering, feature_derivatives):
    """``feature_derivatives f64[nmol,A,3,F] +=`` the chain-rule product (in place)."""
    cabi.featurization_derivative_accumulate(partial_feature_derivatives, normalisation, scaling, input_derivatives, ordering,
                                             feature_derivatives)


def compute_hadamard_derivative_features(sorf_matrix, normalisation, bias, scaling, input_derivatives, ordering,
                                         feature_derivatives):
    """Both steps of the derivative features at once (hadamard_cuda.cpp:99-109)."""
    partial = torch.empty(sorf_matrix.shape, dtype=torch.float64, device=sorf_matrix.device)
    compute_partial_feature_derivatives(sorf_matrix, bias, partial)
    compute_molecular_featurization_derivative(partial, normalisation, scaling, input_derivatives, ordering, feature_derivatives)
