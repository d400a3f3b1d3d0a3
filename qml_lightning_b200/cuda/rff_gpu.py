"""``rff_gpu`` of the upstream project (cuda/random_features.cpp:11-39): in-place accumulation of the RFF training
features of the rows of one element."""
import torch

from .. import cabi


def _counts(nmol, A, device):
    return torch.full((nmol,), A, dtype=torch.int32, device=device)


def _check(**tensors):
    for name, t in tensors.items():
        if not t.is_cuda:
            raise RuntimeError(f"{name.replace('_', ' ')} must be a CUDA tensor")     # wording of random_features.cpp:13-17


def get_rff(input, sampling_matrix, bias, ordering, features):
    """``features f64[nmol,D] += sqrt(2/D) cos(input @ sampling_matrix + bias)`` summed per molecule
    (random_features.cpp:11-20; kernel cuda/random_features_kernel.cu:5-41).  ``input f32[n,K]``, ``sampling_matrix [K,D]``
    and ``bias [D]`` in float64 as upstream passes them (float32 is accepted too)."""
    _check(input=input, sampling_matrix=sampling_matrix, bias=bias, ordering=ordering, features=features)
    if input.shape[0] == 0:
        return
    g, A = cabi.grouping_from_ordering(ordering, features.shape[0])
    Z, _ = cabi.rff_train_features(cabi.pad_rows(input.float(), g.rows_cap), None, sampling_matrix[None].float(), bias[None].float(), g,
                                   _counts(features.shape[0], A, input.device), features.shape[0], A)
    features += Z


def get_rff_derivatives(input, grad, sampling_matrix, bias, ordering, feature_derivatives):
    """``feature_derivatives f64[nmol,A,3,D] += sqrt(2/D) sin(input @ W + b) * (grad @ W)`` summed per molecule
    (random_features.cpp:22-33; kernel cuda/random_features_kernel.cu:43-94).  ``grad f32[n,A,3,K]``."""
    _check(input=input, grad=grad, sampling_matrix=sampling_matrix, bias=bias, ordering=ordering,
           feature_derivatives=feature_derivatives)
    if input.shape[0] == 0:
        return
    nmol = feature_derivatives.shape[0]
    g, A = cabi.grouping_from_ordering(ordering, nmol, int(grad.shape[1]))
    _, G = cabi.rff_train_features(cabi.pad_rows(input.float(), g.rows_cap), cabi.pad_rows(grad.float(), g.rows_cap),
                                   sampling_matrix[None].float(), bias[None].float(), g, _counts(nmol, A, input.device), nmol, A)
    feature_derivatives += G
