"""PCA helpers with the upstream function names (upstream representations/dimensionality_reduction.py).

``get_reductors`` is the one-off SVD set-up step and stays a library call; the projections used on the hot path
run inside the grouped-GEMM kernel (``qmlb_pca_project``) and are exposed here for rows of a single element.
"""
import torch


def get_reductors(gto, charges, npcas, species, print_info=False):
    """Per element: SVD of up to 512 randomly chosen atom representations, first ``npcas`` left singular vectors."""
    reductors = {}
    for e in species:
        rows = gto[charges == e]
        if rows.shape[0] == 0:
            continue
        pick = torch.randperm(rows.size(0))[:512]
        u, s, _ = torch.linalg.svd(rows[pick].T, full_matrices=False)
        if print_info:
            cev = 100 - (s.sum() - s[:npcas].sum()) / s.sum() * 100
            print(f"{u.shape[0]} -> {npcas}  Cumulative Explained Feature Variance = {cev:6.2f} %")
        reductors[e] = u[:, :npcas]
    return reductors


def project_representation(X, reductor):
    """``[nsamples, repsize] -> [nsamples, npcas]``."""
    return torch.matmul(X, reductor)


def project_derivative(dX, reductor):
    """``[nsamples, natoms, 3, repsize] -> [nsamples, natoms, 3, npcas]``."""
    return torch.matmul(dX, reductor)
