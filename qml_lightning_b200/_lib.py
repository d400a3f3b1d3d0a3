"""ctypes binding of ``libqmlb200.so`` (the C ABI declared in ``include/qmlb200.h``).

The library is built in-tree by ``qml_lightning_b200.build``.  There is no CPU or PyTorch fallback: if the library is
missing, loading raises, and every wrapper refuses non-CUDA tensors.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get('QMLB200_LIB', os.path.join(HERE, 'lib', 'libqmlb200.so'))

c_int, c_float, c_size_t, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_void_p


class FchlParamsC(ctypes.Structure):
    """Mirror of ``qmlb_fchl_params``."""
    _fields_ = [('species', c_void_p), ('nspecies', c_int), ('Rs2', c_void_p), ('nRs2', c_int), ('Rs3', c_void_p),
                ('nRs3', c_int), ('eta2', c_float), ('eta3', c_float), ('two_body_decay', c_float),
                ('three_body_weight', c_float), ('three_body_decay', c_float), ('rcut', c_float)]


P = ctypes.POINTER(FchlParamsC)

# name -> (restype, argtypes); must list every symbol declared in include/qmlb200.h
SIGNATURES = {
    'qmlb_last_error': (ctypes.c_char_p, []),
    'qmlb_version': (c_int, []),
    'qmlb_fchl19_repsize': (c_int, [c_int, c_int, c_int]),
    'qmlb_element_types': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_num_neighbours': (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    'qmlb_neighbour_list': (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    'qmlb_fchl19_forward': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, P, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    'qmlb_fchl19_backward': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, P, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    'qmlb_fchl19_forward_jacobian': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, P, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    'qmlb_rows_capacity': (c_size_t, [c_size_t, c_int]),
    'qmlb_group_scratch_bytes': (c_size_t, [c_int, c_int]),
    'qmlb_group_by_element': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    'qmlb_group_by_element_noalloc': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    'qmlb_pca_project': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_pca_project_tc': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_tc_timeouts': (c_int, []),
    'qmlb_pca_pack_bytes': (c_size_t, [c_int, c_int, c_int, c_int]),
    'qmlb_pca_pack': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    'qmlb_pca_project_packed': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_sorf_coefficients': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    'qmlb_sorf_coefficients_backward': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    'qmlb_cos_features': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_cos_features_backward': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_sorf_pack_bytes': (c_size_t, [c_int, c_int, c_int, c_int]),
    'qmlb_sorf_pack': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_sorf_energy_grad': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    'qmlb_predict_workspace_bytes': (c_size_t, [c_int, c_int, c_size_t, c_int, c_int, c_int]),
    'qmlb_pca_pair_pack_bytes': (c_size_t, [c_int, c_int, c_int]),
    'qmlb_pca_pair_pack': (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    'qmlb_sorf_predict': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, P, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                  c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_size_t, c_void_p, c_size_t, c_void_p,
                                  c_void_p, c_void_p]),
    'qmlb_rff_energy_grad': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                     c_int, c_void_p, c_void_p, c_void_p]),
    'qmlb_rff_pack_bytes': (c_size_t, [c_int, c_int, c_int]),
    'qmlb_rff_pack': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    'qmlb_rff_energy_grad_tc': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p]),
    'qmlb_rff_predict': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, P, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                 c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_size_t, c_void_p, c_size_t, c_void_p,
                                 c_void_p, c_void_p]),
    'qmlb_rff_predict_packed': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, P, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                        c_void_p, c_int, c_void_p, c_int, c_size_t, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]),
    'qmlb_pca_project_jacobian': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_sorf_train_features': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_size_t, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p,
                                         c_void_p]),
    'qmlb_rff_train_features': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                        c_int, c_size_t, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    'qmlb_hadamard_features_accumulate': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_partial_feature_derivatives': (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_featurization_derivative_accumulate': (c_int, [c_void_p, ctypes.c_double, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                         c_int, c_int, c_void_p, c_void_p]),
    'qmlb_normal_equations_accumulate': (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    'qmlb_normal_equations_accumulate_cublas': (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    'qmlb_syrk_f64': (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_gemm_tn_f64': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    'qmlb_gemv_t_f64': (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    'qmlb_symmetrize_upper': (c_int, [c_void_p, c_int, c_void_p]),
    'qmlb_packed_upper_elements': (c_size_t, [c_int]),
    'qmlb_pack_upper': (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    'qmlb_unpack_upper': (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
}

_lib = None


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} not found: build it with `python qml_lightning_b200/build.py` "
                               "(there is no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc, what=''):
    if rc != 0:
        msg = load().qmlb_last_error().decode(errors='replace')
        raise RuntimeError(f"{what or 'qmlb200'} failed (code {rc}): {msg}")
