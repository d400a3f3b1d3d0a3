/*
 * qmlb200 -- C ABI of the B200 (sm_100a) kernels for the qml-lightning
 * inference/training hot path: FCHL19 representation (forward, vector-Jacobian
 * product, explicit Jacobian), per-element PCA projection, SORF / RFF feature
 * maps with the per-molecule sum, the dot with the regression weights and the
 * force back-propagation, and the normal-equation accumulation.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless its comment says "host";
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *    nothing here synchronises the device or allocates device memory;
 *  - every function returns QMLB_OK (0) or an error code; qmlb_last_error()
 *    returns a thread-local message for the last non-zero return;
 *  - tensors are dense row-major with the shapes given in the comments;
 *  - `X  f32[nb, A, 3]` coordinates, `Z f32[nb, A]` nuclear charges (0 = padding),
 *    `atom_counts i32[nb]`: the tensor contract of the upstream project
 *    (README.md:69-75); atoms a >= atom_counts[m] of molecule m are padding;
 *  - `cell` / `inv_cell` f32[nb,3,3] or NULL for non-periodic input
 *    (upstream passes an empty [0,3,3] tensor).
 *
 * Each declaration names the upstream interface it replaces (paths inside the
 * upstream qml-lightning tree).
 */
#ifndef QMLB200_H
#define QMLB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QMLB_OK 0
#define QMLB_ERR_INVALID 1     /* bad argument (null pointer, size, unsupported shape) */
#define QMLB_ERR_CUDA 2        /* a CUDA runtime call or launch failed */
#define QMLB_ERR_UNSUPPORTED 3 /* valid request outside the implemented range */

typedef void *qmlb_stream_t;

/* FCHL19 hyper-parameters at kernel level.  `three_body_weight` is the value
 * AFTER the constructor scaling sqrt(eta3/pi)*w (representations/FCHL.py:35);
 * Rs2/Rs3 are the radial grids of FCHL.py:39-40. */
typedef struct qmlb_fchl_params {
    const float *species; /* f32[nspecies] charges defining the element index */
    int nspecies;
    const float *Rs2;     /* f32[nRs2] */
    int nRs2;
    const float *Rs3;     /* f32[nRs3] */
    int nRs3;
    float eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut;
} qmlb_fchl_params;

const char *qmlb_last_error(void);
int qmlb_version(void);

/* repsize = nspecies*nRs2 + nspecies*(nspecies+1)*nRs3  (FCHL.py:42) */
int qmlb_fchl19_repsize(int nspecies, int nRs2, int nRs3);

/* ---- element typing and neighbour lists ------------------------------------------------- */

/* get_element_types_kernel / getElementTypesCUDA (cuda/fchl_cuda_kernel.cu:1716-1757),
 * op qml_lightning_fchl::get_element_types (cuda/torchscript/FCHL19.cpp:38-64).
 * out i32[nb, A]: index of Z in species, -1 when absent; padded atoms get 0 as upstream's zero-init. */
int qmlb_element_types(const float *Z, const int *atom_counts, const float *species, int nspecies, int nb, int A,
                       int *element_types, qmlb_stream_t stream);

/* get_num_neighbours_kernel / getNumNeighboursCUDA (cuda/pairlist_kernel.cu:145-224, 462-480),
 * op qml_lightning_fchl::get_num_neighbours (FCHL19.cpp:66-86).
 * out i32[nb, A_out] (A_out = max(atom_counts) upstream; columns >= atom_counts[m] are zero). */
int qmlb_num_neighbours(const float *X, const int *atom_counts, int nb, int A, float rcut, const float *cell,
                        const float *inv_cell, int *num_neighbours, int A_out, qmlb_stream_t stream);

/* get_neighbour_list_kernel / getNeighbourListCUDA (cuda/pairlist_kernel.cu:326-391, 508-526),
 * op qml_lightning_fchl::get_neighbour_list (FCHL19.cpp:88-112).
 * out i32[nb, A_out, max_neighbours]: ascending j, padded with -1 (filled here). */
int qmlb_neighbour_list(const float *X, const int *atom_counts, int nb, int A, float rcut, const float *cell,
                        const float *inv_cell, int max_neighbours, int *neighbour_list, int A_out,
                        qmlb_stream_t stream);

/* ---- FCHL19 ----------------------------------------------------------------------------- */

/* fchl19_representation_cuda / FCHLCuda (cuda/fchl_cuda_kernel.cu:476-674, 1804-1846),
 * get_fchl_representation (cuda/fchl_cuda.cpp:56-90, torchscript/FCHL19.cpp:114-150), the forward of op
 * qml_lightning_fchl::fchl_forwards (FCHL19.cpp:244-277).  Neighbours are found inside the kernel
 * (rule 0 < r^2 < rcut^2, pairlist_kernel.cu:386), so no neighbour list is passed.
 * rep f32[*, repsize]: row of atom (m,a) is  row_of_slot[m*A+a]  when row_of_slot != NULL (rows < 0 are
 * skipped), else m*A+a; in the latter case padded atoms are written as zero rows. */
int qmlb_fchl19_forward(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                        const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                        const int *row_of_slot, float *rep, qmlb_stream_t stream);

/* fchl19_backwards_cuda / FCHLBackwardsCuda (cuda/fchl_cuda_kernel.cu:1325-1714, 1885-1926),
 * fchl_backwards (fchl_cuda.cpp:119-155, FCHL19.cpp:210-239), the backward of fchl_forwards (FCHL19.cpp:279-315):
 * grad_X[m,a,:] = sum_i sum_c grad_rep[row(m,i), c] * d rep[m,i,c] / d r_a.
 * grad_X f32[nb, A, 3] is fully overwritten (padded atoms get zeros).
 * atom_energy (optional, f32 per row) is summed per molecule into mol_energy f32[nb] when both are non-NULL. */
int qmlb_fchl19_backward(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                         const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                         const int *row_of_slot, const float *grad_rep, float *grad_X, const float *atom_energy,
                         float *mol_energy, qmlb_stream_t stream);

/* fchl19_representation_and_derivative_cuda / FCHLRepresentationAndDerivativeCuda
 * (cuda/fchl_cuda_kernel.cu:676-1005, 1928-1964), get_fchl_and_derivative (fchl_cuda.cpp:157-202,
 * FCHL19.cpp:152-208).  rep f32[nb,A,repsize]; jac f32[nb,A,A,3,repsize] with
 * jac[m,i,a,x,c] = d rep[m,i,c] / d r_{a,x}.  Both are fully overwritten.  With row_of_slot != NULL the row of
 * centre atom (m,i) is row_of_slot[m*A+i] in both outputs (rep f32[rows,repsize], jac f32[rows,A,3,repsize]) and
 * rows < 0 are skipped. */
int qmlb_fchl19_forward_jacobian(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                                 const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                                 const int *row_of_slot, float *rep, float *jac, qmlb_stream_t stream);

/* ---- element grouping (replaces the boolean-mask gathers and torch.where host syncs of
 *      models/hadamard_features.py:99-107 and models/kernel.py:141-150) -------------------- */

/* Rows of the per-atom work arrays are ordered by model element, each element group padded to a multiple of
 * QMLB_ROW_TILE rows.  Given Z and the model's `elements` (f32[nelements] charges) this writes
 *   row_of_slot i32[nb*A]        row of atom (m,a), -1 (padding / element not in `elements`) or
 *                                QMLB_ROW_OVERFLOW (a real atom for which rows_cap had no row left)
 *   slot_of_row i32[rows_cap]    m*A+a of a row, -1 for padding rows
 *   group_start i32[nelements+1] first row of each element group (group_start[nelements] = rows in use)
 * Within a group rows follow (m,a) order, so the result is deterministic.
 * rows_cap must be >= qmlb_rows_capacity(n_atoms_upper, nelements) with n_atoms_upper >= the number of real
 * atoms.  The host cannot check that bound without waiting for the device, so the device does: atoms beyond the
 * capacity are marked QMLB_ROW_OVERFLOW, nothing is written out of bounds, and qmlb_fchl19_backward (hence
 * qmlb_sorf_predict / qmlb_rff_predict*) returns NaN energies and gradients for every molecule that holds such an
 * atom.  `scratch` is qmlb_group_scratch_bytes(nb, nelements) bytes of device memory. */
#define QMLB_ROW_TILE 128
#define QMLB_ROW_OVERFLOW (-2)
size_t qmlb_rows_capacity(size_t n_atoms_upper, int nelements);
size_t qmlb_group_scratch_bytes(int nb, int nelements);
int qmlb_group_by_element(const float *Z, const int *atom_counts, const float *elements, int nelements, int nb,
                          int A, int *row_of_slot, int *slot_of_row, int *group_start, size_t rows_cap,
                          void *scratch, qmlb_stream_t stream);

/* Allocation-free variant of qmlb_group_by_element: identical outputs, but the scratch counters live in a fixed
 * QMLB_GROUP_STATIC_SCRATCH_BYTES array inside the library instead of caller memory.  It has no counterpart in the
 * upstream project.  It is meant for callers that receive their buffers from a host application and must not
 * allocate device memory themselves (a simulation engine's force plug-in working inside the engine's memory
 * budget; a latency-critical thread that must stay out of cudaMalloc/cudaFree, which serialise against all streams).
 *  - Limit: qmlb_group_scratch_bytes(nb, nelements) <= QMLB_GROUP_STATIC_SCRATCH_BYTES, i.e. about
 *    32 * 262,000 / nelements molecules per call; larger batches are rejected with QMLB_ERR_INVALID.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current); make that first call before starting any stream capture.  No call allocates or frees memory.
 *  - All calls on a device share the one array: calls whose kernels may overlap on the GPU (different streams,
 *    different host threads) race on it and must be ordered by the caller.  The array keeps the previous call's
 *    counters; none of them needs clearing because every counter is rewritten before it is read.
 *  - Every GPU that loads the library carries the array (1 MiB) until the process exits. */
#define QMLB_GROUP_STATIC_SCRATCH_BYTES (1u << 20)
int qmlb_group_by_element_noalloc(const float *Z, const int *atom_counts, const float *elements, int nelements, int nb,
                                  int A, int *row_of_slot, int *slot_of_row, int *group_start, size_t rows_cap,
                                  qmlb_stream_t stream);

/* ---- PCA projection ----------------------------------------------------------------------- */

/* project_representation = torch.matmul(X, reductor) per element (representations/dimensionality_reduction.py:47-58;
 * call sites models/hadamard_features.py:111, models/random_features.py:96, models/kernel.py:154).
 * in f32[rows_cap, K], reductors f32[nelements, K, N], out f32[rows_cap, N]; rows are element-grouped as above.
 * transpose = 0: out = in . P_e            (K = repsize, N = npcas)
 * transpose = 1: out = in . P_e^T          (the autograd backward: in is [rows, npcas], out [rows, repsize]) */
int qmlb_pca_project(const float *in, const float *reductors, const int *group_start, int nelements, size_t rows_cap,
                     int repsize, int npcas, int transpose, float *out, qmlb_stream_t stream);

/* SUPERSEDED by qmlb_pca_pack / qmlb_pca_project_packed below (same arithmetic, pre-split projection matrices, wider
 * tiles); kept as an independent tensor-core implementation that the tests cross-check the newer one against.
 * The same contraction on the 5th-generation tensor cores: tcgen05.mma kind::tf32 with the accumulator in tensor
 * memory and a 3xTF32 operand split (fp32-accurate result).  sub_rows = matrix rows per grouped row (1 for
 * representations and gradients, 3*A for Jacobians).  qmlb_tc_timeouts() returns how many blocks ever gave up on a
 * bounded wait (0 in a healthy run; it synchronises the device). */
int qmlb_pca_project_tc(const float *in, const float *reductors, const int *group_start, int nelements, size_t rows_cap,
                        int sub_rows, int repsize, int npcas, int transpose, float *out, qmlb_stream_t stream);
int qmlb_tc_timeouts(void);

/* The same projection with the projection matrices split (hi + lo TF32) and tiled once per call into the shared-memory
 * image of every (element, column tile, 32-k chunk), so that the kernel fetches its B operand with bulk copies and a
 * block covers up to 256 output columns (dimensionality_reduction.py:47-58 and its autograd transpose).  This is what
 * qmlb_sorf_predict / qmlb_rff_predict_packed use.  Usage: qmlb_pca_pack_bytes -> buffer (128-byte aligned) ->
 * qmlb_pca_pack (one direction per buffer: transpose = 0 projection, 1 transposed product) -> qmlb_pca_project_packed. */
size_t qmlb_pca_pack_bytes(int nelements, int repsize, int npcas, int transpose);
int qmlb_pca_pack(const float *reductors, int nelements, int repsize, int npcas, int transpose, void *packed,
                  size_t packed_bytes, qmlb_stream_t stream);
int qmlb_pca_project_packed(const float *in, const void *packed, const int *group_start, int nelements, size_t rows_cap,
                            int repsize, int npcas, int transpose, float *out, qmlb_stream_t stream);

/* ---- SORF ----------------------------------------------------------------------------------- */

/* hadamard_kernel / hadamard_gpu (cuda/hadamard_kernel.cu:5-102, 719-737), hadamard_transform_gpu
 * (torchscript/SORF.cpp:24-36), forward of op qml_lightning_sorf::get_SORF_coefficients (SORF.cpp:76-87).
 * u f32[n,N], D f32[T,S,N] (+-1), out f32[n,S,N] = normalisation * N^(-T/2) * (H D_{T-1} ... H D_0) u. */
int qmlb_sorf_coefficients(const float *u, const float *D, int n, int N, int S, int T, float normalisation,
                           float *out, qmlb_stream_t stream);

/* hadamard_kernel_backwards / hadamard_backwards_gpu (hadamard_kernel.cu:204-312, 758-776), backward of
 * get_SORF_coefficients (SORF.cpp:89-101).  grad f32[n,S,N] -> out f32[n,N]. */
int qmlb_sorf_coefficients_backward(const float *grad, const float *D, int n, int N, int S, int T,
                                    float normalisation, float *out, qmlb_stream_t stream);

/* compute_cos_features_kernel / cos_features_gpu (hadamard_kernel.cu:778-814), CosFeaturesCUDA (SORF.cpp:52-61),
 * forward of op qml_lightning_sorf::get_cos_features (SORF.cpp:106-119).
 * coeffs f32[n,F], bias f32[F], batch_indexes i32[n] (molecule of each row, non-decreasing or arbitrary),
 * out f32[nmol,F] = sum over rows of sqrt(2/F) cos(coeffs + bias); fully overwritten. */
int qmlb_cos_features(const float *coeffs, const float *bias, const int *batch_indexes, int n, int F, int nmol,
                      float *out, qmlb_stream_t stream);

/* compute_cos_derivative_features_kernel / cos_derivative_features_gpu (hadamard_kernel.cu:816-854),
 * backward of get_cos_features (SORF.cpp:121-133): out[a,f] = grads[mol(a),f] * -sin(coeffs+bias) * sqrt(2/F). */
int qmlb_cos_features_backward(const float *grads, const float *coeffs, const float *bias, const int *batch_indexes,
                               int n, int F, float *out, qmlb_stream_t stream);

/* Packed SORF parameters for the fused kernel below: sign diagonals, bias and pre-scaled weights re-ordered to
 * the register layout of the in-register/shared-memory FWHT.  Source tensors are the model attributes
 * Dmat f32[nelements,T,S,N], bias f32[nelements,S*N], alpha f32[S*N] (models/hadamard_features.py:34-41,119-121).
 * `packed` is qmlb_sorf_pack_bytes(...) bytes of device memory, written by qmlb_sorf_pack. */
size_t qmlb_sorf_pack_bytes(int nelements, int N, int S, int T);
int qmlb_sorf_pack(const float *Dmat, const float *bias, const float *alpha, int nelements, int N, int S, int T,
                   void *packed, qmlb_stream_t stream);

/* Fused replacement of the chain get_SORF_coefficients -> get_cos_features -> matmul(Ztest, alpha) and of its
 * autograd backward (models/hadamard_features.py:113-121; SORF.cpp:89-101,121-133): per row a
 *   atom_energy[a] = sum_f alpha_f sqrt(2/F) cos(c_af + b_f),   c = (sqrt(N)/sigma) N^(-T/2) (H D)^T x_a
 *   grad_x[a,:]    = d atom_energy[a] / d x_a
 * without materialising c.  x f32[rows_cap,N] element-grouped; fast_math != 0 uses the SFU sin/cos. */
int qmlb_sorf_energy_grad(const float *x, const int *group_start, const int *slot_of_row, int nelements,
                          size_t rows_cap, int N, int S, int T, float sigma, const void *packed, int fast_math,
                          float *atom_energy, float *grad_x, qmlb_stream_t stream);

/* ---- whole-batch prediction ----------------------------------------------------------------- */

/* HadamardFeaturesModel.forward + torch.autograd.grad(-E.sum(), X) (models/hadamard_features.py:82-123, 157-162;
 * predict_opt :125-179) as one call: energy f32[nb] (without self energies, like upstream forward) and
 * grad_X f32[nb,A,3] = dE/dX (forces are -grad_X).  All six stages run on `stream` inside `workspace`
 * (qmlb_predict_workspace_bytes bytes, 256-byte aligned device memory); nothing is allocated and the host never
 * waits for the device.  n_atoms_upper is an upper bound of the number of real atoms (nb*A if unknown; the length
 * of upstream's atomIDs tensor when available).  elements f32[nelements] are the model's elements,
 * reductors f32[nelements, repsize, npcas], packed from qmlb_sorf_pack.  pca_packed (optional, NULL = build the images
 * inside the workspace on every call) are the split and tiled images of the projection matrices for both directions,
 * made once per model by qmlb_pca_pair_pack into qmlb_pca_pair_pack_bytes bytes of 256-byte aligned device memory; with
 * it `reductors` is not read. */
size_t qmlb_pca_pair_pack_bytes(int nelements, int repsize, int npcas);
int qmlb_pca_pair_pack(const float *reductors, int nelements, int repsize, int npcas, void *pca_packed, size_t packed_bytes,
                       qmlb_stream_t stream);
size_t qmlb_predict_workspace_bytes(int nb, int A, size_t n_atoms_upper, int nelements, int repsize, int npcas);
int qmlb_sorf_predict(const float *X, const float *Z, const int *atom_counts, int nb, int A, const qmlb_fchl_params *p,
                      const float *cell, const float *inv_cell, const float *elements, int nelements,
                      const float *reductors, const void *pca_packed, int npcas, const void *packed, int S, int T, float sigma,
                      int fast_math,
                      size_t n_atoms_upper, void *workspace, size_t workspace_bytes, float *energy, float *grad_X,
                      qmlb_stream_t stream);

/* ---- RFF ------------------------------------------------------------------------------------ */

/* Fused replacement of the RFF model's feature stage and its autograd backward
 * (models/random_features.py:98-100: index_add_ of sqrt(2/D) cos(x @ W_e + b_e), then matmul with alpha): per row a
 *   atom_energy[a] = sum_f alpha_f sqrt(2/D) cos((x_a W_e)_f + b_ef),   grad_x[a,:] = d atom_energy[a] / d x_a
 * x f32[rows_cap, npcas] element-grouped, W f32[nelements, npcas, D], b f32[nelements, D], alpha f32[D].
 * npcas in {32, 64, 128, 256}. */
int qmlb_rff_energy_grad(const float *x, const int *group_start, const int *slot_of_row, int nelements, size_t rows_cap,
                         int npcas, int nfeatures, const float *W, const float *b, const float *alpha, int fast_math,
                         float *atom_energy, float *grad_x, qmlb_stream_t stream);

/* Tensor-core version of qmlb_rff_energy_grad (same upstream lines; tcgen05.mma on fp16 hi/lo operand pairs with fp32
 * accumulation, results within fp32 rounding of the FFMA version).  The model parameters are re-packed once:
 *   qmlb_rff_pack_bytes -> allocate (256-byte aligned) -> qmlb_rff_pack(W, b, alpha) -> qmlb_rff_energy_grad_tc per batch.
 * qmlb_rff_pack must be called again whenever W, b or alpha change.  Feature counts are padded to a multiple of 32
 * inside the packed buffer (padding features carry zero weight).  qmlb_rff_pack_bytes returns 0 for unsupported
 * sizes.  Operands larger than 2^41 in magnitude are outside the supported range.  A kernel that is handed parameters
 * packed for another npcas or element count, or a block that gives up on one of its bounded waits, fills its rows of
 * atom_energy and grad_x with NaN and reports through qmlb_tc_timeouts(). */
size_t qmlb_rff_pack_bytes(int nelements, int npcas, int nfeatures);
int qmlb_rff_pack(const float *W, const float *b, const float *alpha, int nelements, int npcas, int nfeatures, void *packed,
                  size_t packed_bytes, qmlb_stream_t stream);
int qmlb_rff_energy_grad_tc(const float *x, const int *group_start, const int *slot_of_row, int nelements, size_t rows_cap,
                            int npcas, const void *packed, int fast_math, float *atom_energy, float *grad_x,
                            qmlb_stream_t stream);

/* RandomFourrierFeaturesModel.forward + autograd.grad (models/random_features.py:69-102, 104-158) as one call;
 * same conventions and workspace as qmlb_sorf_predict. */
int qmlb_rff_predict(const float *X, const float *Z, const int *atom_counts, int nb, int A, const qmlb_fchl_params *p,
                     const float *cell, const float *inv_cell, const float *elements, int nelements,
                     const float *reductors, const void *pca_packed, int npcas, const float *W, const float *b,
                     const float *alpha, int nfeatures,
                     int fast_math, size_t n_atoms_upper, void *workspace, size_t workspace_bytes, float *energy,
                     float *grad_X, qmlb_stream_t stream);

/* qmlb_rff_predict on parameters packed by qmlb_rff_pack: the feature stage runs on the tensor cores
 * (qmlb_rff_energy_grad_tc).  This is the path RandomFourrierFeaturesModel uses. */
int qmlb_rff_predict_packed(const float *X, const float *Z, const int *atom_counts, int nb, int A, const qmlb_fchl_params *p,
                            const float *cell, const float *inv_cell, const float *elements, int nelements,
                            const float *reductors, const void *pca_packed, int npcas, const void *packed, int fast_math,
                            size_t n_atoms_upper,
                            void *workspace, size_t workspace_bytes, float *energy, float *grad_X, qmlb_stream_t stream);

/* Projection of an element-grouped explicit Jacobian: project_derivative = einsum('jmnk,kl->jmnl')
 * (representations/dimensionality_reduction.py:61-72; call site models/kernel.py:160).
 * jac_rows f32[rows_cap, sub_rows, repsize] (sub_rows = 3*A), out f32[rows_cap, sub_rows, npcas]. */
int qmlb_pca_project_jacobian(const float *jac_rows, const float *reductors, const int *group_start, int nelements,
                              size_t rows_cap, int sub_rows, int repsize, int npcas, float *out, qmlb_stream_t stream);

/* ---- training rows and normal equations ------------------------------------------------------ */

/* SORF training features of one batch: sorf_matrix_kernel, compute_featurisation_kernel, compute_sin_coeffs_kernel,
 * compute_featurisation_derivative_kernel (cuda/hadamard_kernel.cu:424-717) as driven by calculate_features
 * (models/hadamard_features.py:66-80) and build_Z_components (models/kernel.py:134-170), for all elements at once.
 * x f32[rows_cap,N] and dx f32[rows_cap,A,3,N] are element-grouped; Dmat f32[nel,T,S,N], bias f32[nel,S*N] unpacked.
 * Zout f64[nb,F] (overwritten) = per-molecule features; G f64[nb,A,3,F] (overwritten) = -dZ/dr, the force features
 * (dx and G may both be NULL for energy-only training).  sinc_scratch: rows_cap*F floats.  N in [32, 512]. */
int qmlb_sorf_train_features(const float *x, const float *dx, const float *Dmat, const float *bias, const int *group_start,
                             const int *slot_of_row, const int *row_of_slot, const int *atom_counts, int nelements, int nb,
                             int A, size_t rows_cap, int N, int S, int T, float sigma, double *Zout, double *G,
                             float *sinc_scratch, qmlb_stream_t stream);

/* The fine-grained SORF training operators of the upstream extension module sorf_gpu (cuda/hadamard_cuda.cpp:77-126),
 * for scripts that drive upstream's per-element calculate_features themselves (models/hadamard_features.py:66-80).
 * They work on the n rows of ONE element, take the molecule of every row from ordering i32[n] and ACCUMULATE into
 * caller-owned float64 tensors (float64 atomics, like upstream), which must therefore be initialised by the caller.
 *   qmlb_hadamard_features_accumulate: compute_hadamard_features / compute_featurisation_kernel
 *     (cuda/hadamard_kernel.cu:541-563): features f64[nmol,F] += sqrt(2/F) cos(coeffs f32[n,F] + bias f32[F]).
 *   qmlb_partial_feature_derivatives: compute_partial_feature_derivatives / compute_sin_coeffs_kernel (:565-585):
 *     out f64[n,F] = sqrt(2/F) sin(coeffs + bias)  (overwritten).
 *   qmlb_featurization_derivative_accumulate: compute_molecular_featurization_derivative /
 *     compute_featurisation_derivative_kernel (:587-717): feature_derivatives f64[nmol,A,3,F] +=
 *     normalisation * partial_derivatives[a,f] * [N^(-T/2) (H D_{T-1} ... H D_0) input_derivatives[a,j,x,:]]_f,
 *     D f32[T,S,N], input_derivatives f32[n,A,3,N]. */
int qmlb_hadamard_features_accumulate(const float *coeffs, const float *bias, const int *ordering, int n, int F,
                                      double *features, qmlb_stream_t stream);
int qmlb_partial_feature_derivatives(const float *coeffs, const float *bias, int n, int F, double *out, qmlb_stream_t stream);
int qmlb_featurization_derivative_accumulate(const double *partial_derivatives, double normalisation, const float *D,
                                             const float *input_derivatives, const int *ordering, int n, int A, int N, int S,
                                             int T, double *feature_derivatives, qmlb_stream_t stream);

/* RFF training features of one batch: random_fourrier_features_kernel / _derivative
 * (cuda/random_features_kernel.cu:5-94) via get_rff / get_rff_derivatives (cuda/random_features.cpp:11-33), as
 * driven by RandomFourrierFeaturesModel.calculate_features (models/random_features.py:60-67), for all elements
 * at once and with upstream's arithmetic: float32 inputs, float64 products, sums and sin/cos (upstream passes
 * W.double(), b.double()).  x f32[rows_cap,K], dx f32[rows_cap,A,3,K] element-grouped; W f32[nel,K,D], b f32[nel,D].
 * Zout f64[nb,D] and G f64[nb,A,3,D] (= -dZ/dr) are overwritten, every element written once (dx and G may both be
 * NULL for energy-only training).  One fused kernel (float64 tensor-core products with the sin/cos scaling and the
 * per-molecule sum in registers); no scratch memory.  K must be a multiple of 4. */
int qmlb_rff_train_features(const float *x, const float *dx, const float *W, const float *b, const int *group_start,
                            const int *slot_of_row, const int *row_of_slot, const int *atom_counts, int nelements, int nb,
                            int A, size_t rows_cap, int K, int D, double *Zout, double *G, qmlb_stream_t stream);

/* ZTZ += M^T M (row-major UPPER triangle only) and ZTy += M^T y for a row block M f64[rows,F]:
 * torch.matmul(Ztrain.T, Ztrain) / torch.matmul(Ztrain.T, targets) in build_Z_components (models/kernel.py:172-192).
 * In-tree float64 kernels: qmlb_syrk_f64 (mma.sync.m8n8k4.f64 tiles of the upper triangle) and qmlb_gemv_t_f64
 * (float64 atomics over row splits: ZTy is reproducible to rounding, not bitwise).  qmlb_symmetrize_upper mirrors the
 * triangle before the solve.  qmlb_normal_equations_accumulate_cublas is the same update through cuBLAS DSYRK + DGEMV,
 * kept so that the in-tree kernel can be timed against the library in the same process. */
int qmlb_normal_equations_accumulate(const double *M, int rows, int F, const double *y, double *ZTZ, double *ZTy,
                                     qmlb_stream_t stream);
int qmlb_normal_equations_accumulate_cublas(const double *M, int rows, int F, const double *y, double *ZTZ, double *ZTy,
                                            qmlb_stream_t stream);
int qmlb_syrk_f64(const double *M, int rows, int F, double *ZTZ, qmlb_stream_t stream);

/* C f64[Fi,Fj] += P^T Q for P f64[rows,Fi], Q f64[rows,Fj] (all row-major), every entry of C: the product behind
 * matmul_and_reduce (cuda/utils_cuda.cpp:26-33, kernel cuda/utils_kernel.cu:70-129: C += A B with A = P^T, B = Q),
 * which upstream selects with use_specialized_matmul (models/kernel.py:176-188) and feeds with float32 copies of the
 * rows.  Here the float32-rounded rows are promoted and multiplied on the float64 tensor-core path (the same kernel
 * as qmlb_syrk_f64), so every product is exact and the sums carry float64 rounding only: closer to the exact
 * product than upstream's compensated float32 sum. */
int qmlb_gemm_tn_f64(const double *P, const double *Q, int rows, int Fi, int Fj, double *C, qmlb_stream_t stream);
int qmlb_gemv_t_f64(const double *M, int rows, int F, const double *y, double *ZTy, qmlb_stream_t stream);
int qmlb_symmetrize_upper(double *ZTZ, int F, qmlb_stream_t stream);

/* Packed form of the accumulated upper triangle for the exchange between ranks: the sum of the per-rank partial
 * matrices (one all-reduce where upstream has a single device, models/kernel.py:46-217) needs only the F(F+1)/2
 * entries that were accumulated, half the bytes of the square matrix.  packed f64[qmlb_packed_upper_elements(F)]:
 * row i holds columns i..F-1 and starts at i*F - i*(i-1)/2.  qmlb_unpack_upper writes the triangle back and mirrors
 * it (the matrix is symmetric again afterwards).  F <= 65535. */
size_t qmlb_packed_upper_elements(int F);
int qmlb_pack_upper(const double *ZTZ, int F, double *packed, qmlb_stream_t stream);
int qmlb_unpack_upper(const double *packed, int F, double *ZTZ, qmlb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* QMLB200_H */
