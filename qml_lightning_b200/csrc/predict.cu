// Whole-batch energy + gradient prediction for the SORF model: the six stages chained on one stream with a
// caller-provided workspace, no allocation and no host synchronisation.
//
// Replaces HadamardFeaturesModel.forward followed by autograd.grad (models/hadamard_features.py:82-123, 157-162):
//   group atoms by element -> FCHL19 rows -> PCA -> fused SORF energy/gradient -> PCA^T -> FCHL19 VJP + molecule sums.
#include "common.cuh"

namespace {

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Workspace {
    size_t rows_cap;
    size_t off_row_of_slot, off_slot_of_row, off_group_start, off_scratch, off_rep, off_x, off_gx, off_energy, off_pca_fwd, off_pca_bwd, total;
    size_t pca_fwd_bytes, pca_bwd_bytes;
    Workspace(int nb, int A, size_t n_atoms_upper, int nel, int repsize, int width) {
        const size_t slots = (size_t)nb * A;
        rows_cap = qmlb_rows_capacity(n_atoms_upper < slots ? n_atoms_upper : slots, nel);
        size_t o = 0;
        off_row_of_slot = o; o = align256(o + sizeof(int) * slots);
        off_slot_of_row = o; o = align256(o + sizeof(int) * rows_cap);
        off_group_start = o; o = align256(o + sizeof(int) * (nel + 1));
        off_scratch = o;     o = align256(o + qmlb_group_scratch_bytes(nb, nel));
        off_rep = o;         o = align256(o + sizeof(float) * rows_cap * repsize);
        off_x = o;           o = align256(o + sizeof(float) * rows_cap * width);
        off_gx = o;          o = align256(o + sizeof(float) * rows_cap * width);
        off_energy = o;      o = align256(o + sizeof(float) * rows_cap);
        // projection matrices split and tiled for the tensor-core kernel, one image per direction
        pca_fwd_bytes = qmlb_pca_pack_bytes(nel, repsize, width, 0);
        pca_bwd_bytes = qmlb_pca_pack_bytes(nel, repsize, width, 1);
        off_pca_fwd = o;     o = align256(o + pca_fwd_bytes);
        off_pca_bwd = o;     o = align256(o + pca_bwd_bytes);
        total = o;
    }
};

}  // namespace

extern "C" size_t qmlb_predict_workspace_bytes(int nb, int A, size_t n_atoms_upper, int nelements, int repsize, int npcas) {
    if (nb <= 0 || A <= 0 || nelements <= 0 || repsize <= 0 || npcas <= 0) return 0;
    return Workspace(nb, A, n_atoms_upper, nelements, repsize, npcas).total;
}

namespace {

// Stages shared by the SORF and RFF models; `features` maps projected rows to per-atom energies and gradients.
template <typename FeatureStage>
int predict_pipeline(const float *X, const float *Z, const int *atom_counts, int nb, int A, const qmlb_fchl_params *p,
                     const float *cell, const float *inv_cell, const float *elements, int nelements,
                     const float *reductors, const void *pca_packed, int npcas, size_t n_atoms_upper, void *workspace,
                     size_t workspace_bytes, float *energy, float *grad_X, qmlb_stream_t stream, const char *who,
                     FeatureStage features) {
    QMLB_REQUIRE(nb >= 0 && A > 0 && nelements > 0 && npcas > 0, "%s: bad sizes", who);
    if (nb == 0) return QMLB_OK;  // empty batch: nothing to launch (its tensors have no storage to point at)
    QMLB_REQUIRE(X && Z && atom_counts && p && elements && (reductors || pca_packed) && workspace && energy && grad_X, "%s: null argument", who);
    const int repsize = qmlb_fchl19_repsize(p->nspecies, p->nRs2, p->nRs3);
    const Workspace W(nb, A, n_atoms_upper, nelements, repsize, npcas);
    QMLB_REQUIRE(workspace_bytes >= W.total, "%s: workspace of %zu bytes given, %zu needed", who, workspace_bytes, W.total);
    QMLB_REQUIRE(((uintptr_t)workspace & 255) == 0, "%s: workspace must be 256-byte aligned", who);
    char *base = static_cast<char *>(workspace);
    int *row_of_slot = reinterpret_cast<int *>(base + W.off_row_of_slot);
    int *slot_of_row = reinterpret_cast<int *>(base + W.off_slot_of_row);
    int *group_start = reinterpret_cast<int *>(base + W.off_group_start);
    float *rep = reinterpret_cast<float *>(base + W.off_rep);
    float *x = reinterpret_cast<float *>(base + W.off_x);
    float *gx = reinterpret_cast<float *>(base + W.off_gx);
    float *atom_energy = reinterpret_cast<float *>(base + W.off_energy);
    int rc;
    if ((rc = qmlb_group_by_element(Z, atom_counts, elements, nelements, nb, A, row_of_slot, slot_of_row, group_start,
                                    W.rows_cap, base + W.off_scratch, stream))) return rc;
    if ((rc = qmlb_fchl19_forward(X, Z, atom_counts, nb, A, p, cell, inv_cell, row_of_slot, rep, stream))) return rc;
    // both projections run on the tensor cores (tcgen05, 3xTF32 split: fp32-accurate) on split and tiled images of the
    // projection matrices: the caller's (qmlb_pca_pair_pack, once per model) or, without them, built here on every call
    const void *pca_fwd, *pca_bwd;
    if (pca_packed) {
        QMLB_REQUIRE(((uintptr_t)pca_packed & 255) == 0, "%s: pca_packed must be 256-byte aligned", who);
        pca_fwd = pca_packed;
        pca_bwd = static_cast<const char *>(pca_packed) + align256(W.pca_fwd_bytes);
    } else {
        if ((rc = qmlb_pca_pack(reductors, nelements, repsize, npcas, 0, base + W.off_pca_fwd, W.pca_fwd_bytes, stream))) return rc;
        if ((rc = qmlb_pca_pack(reductors, nelements, repsize, npcas, 1, base + W.off_pca_bwd, W.pca_bwd_bytes, stream))) return rc;
        pca_fwd = base + W.off_pca_fwd;
        pca_bwd = base + W.off_pca_bwd;
    }
    if ((rc = qmlb_pca_project_packed(rep, pca_fwd, group_start, nelements, W.rows_cap, repsize, npcas, 0, x, stream))) return rc;
    if ((rc = features(x, group_start, slot_of_row, W.rows_cap, atom_energy, gx))) return rc;
    // the representation buffer is reused for d(energy)/d(representation)
    if ((rc = qmlb_pca_project_packed(gx, pca_bwd, group_start, nelements, W.rows_cap, repsize, npcas, 1, rep, stream))) return rc;
    return qmlb_fchl19_backward(X, Z, atom_counts, nb, A, p, cell, inv_cell, row_of_slot, rep, grad_X, atom_energy, energy,
                                stream);
}

}  // namespace

extern "C" size_t qmlb_pca_pair_pack_bytes(int nelements, int repsize, int npcas) {
    const size_t f = qmlb_pca_pack_bytes(nelements, repsize, npcas, 0), b = qmlb_pca_pack_bytes(nelements, repsize, npcas, 1);
    return (f && b) ? align256(f) + align256(b) : 0;
}

extern "C" int qmlb_pca_pair_pack(const float *reductors, int nelements, int repsize, int npcas, void *pca_packed,
                                  size_t packed_bytes, qmlb_stream_t stream) {
    const size_t f = qmlb_pca_pack_bytes(nelements, repsize, npcas, 0), b = qmlb_pca_pack_bytes(nelements, repsize, npcas, 1);
    QMLB_REQUIRE(reductors && pca_packed && f && b, "qmlb_pca_pair_pack: bad arguments");
    QMLB_REQUIRE(packed_bytes >= align256(f) + align256(b) && ((uintptr_t)pca_packed & 255) == 0,
                 "qmlb_pca_pair_pack: buffer too small or not 256-byte aligned");
    if (int rc = qmlb_pca_pack(reductors, nelements, repsize, npcas, 0, pca_packed, f, stream)) return rc;
    return qmlb_pca_pack(reductors, nelements, repsize, npcas, 1, static_cast<char *>(pca_packed) + align256(f), b, stream);
}

extern "C" int qmlb_sorf_predict(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                                 const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                                 const float *elements, int nelements, const float *reductors, const void *pca_packed, int npcas,
                                 const void *packed, int S, int T, float sigma, int fast_math, size_t n_atoms_upper,
                                 void *workspace, size_t workspace_bytes, float *energy, float *grad_X,
                                 qmlb_stream_t stream) {
    QMLB_REQUIRE(packed || nb == 0, "qmlb_sorf_predict: null argument");
    return predict_pipeline(X, Z, atom_counts, nb, A, p, cell, inv_cell, elements, nelements, reductors, pca_packed, npcas,
                            n_atoms_upper, workspace, workspace_bytes, energy, grad_X, stream, "qmlb_sorf_predict",
                            [&](const float *x, const int *group_start, const int *slot_of_row, size_t rows_cap,
                                float *atom_energy, float *gx) {
                                return qmlb_sorf_energy_grad(x, group_start, slot_of_row, nelements, rows_cap, npcas, S, T,
                                                             sigma, packed, fast_math, atom_energy, gx, stream);
                            });
}

extern "C" int qmlb_rff_predict(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                                const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                                const float *elements, int nelements, const float *reductors, const void *pca_packed, int npcas,
                                const float *W, const float *b, const float *alpha, int nfeatures, int fast_math, size_t n_atoms_upper,
                                void *workspace, size_t workspace_bytes, float *energy, float *grad_X,
                                qmlb_stream_t stream) {
    QMLB_REQUIRE((W && b && alpha) || nb == 0, "qmlb_rff_predict: null argument");
    return predict_pipeline(X, Z, atom_counts, nb, A, p, cell, inv_cell, elements, nelements, reductors, pca_packed, npcas,
                            n_atoms_upper, workspace, workspace_bytes, energy, grad_X, stream, "qmlb_rff_predict",
                            [&](const float *x, const int *group_start, const int *slot_of_row, size_t rows_cap,
                                float *atom_energy, float *gx) {
                                return qmlb_rff_energy_grad(x, group_start, slot_of_row, nelements, rows_cap, npcas,
                                                            nfeatures, W, b, alpha, fast_math, atom_energy, gx, stream);
                            });
}

extern "C" int qmlb_rff_predict_packed(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                                       const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                                       const float *elements, int nelements, const float *reductors, const void *pca_packed,
                                       int npcas, const void *packed, int fast_math, size_t n_atoms_upper, void *workspace,
                                       size_t workspace_bytes, float *energy, float *grad_X, qmlb_stream_t stream) {
    QMLB_REQUIRE(packed || nb == 0, "qmlb_rff_predict_packed: null argument");
    return predict_pipeline(X, Z, atom_counts, nb, A, p, cell, inv_cell, elements, nelements, reductors, pca_packed, npcas,
                            n_atoms_upper, workspace, workspace_bytes, energy, grad_X, stream, "qmlb_rff_predict_packed",
                            [&](const float *x, const int *group_start, const int *slot_of_row, size_t rows_cap,
                                float *atom_energy, float *gx) {
                                return qmlb_rff_energy_grad_tc(x, group_start, slot_of_row, nelements, rows_cap, npcas, packed,
                                                               fast_math, atom_energy, gx, stream);
                            });
}
