// TorchScript operator shim over the qmlb200 C ABI.
//
// Registers the operator names that saved upstream models resolve at load time, with the upstream argument lists
// (all tensors; scalars as 0-dim tensors, usually on the CPU):
//   qml_lightning_fchl::{fchl_forwards, get_fchl_and_derivative, get_element_types, get_neighbour_list,
//                        get_num_neighbours}                       (upstream cuda/torchscript/FCHL19.cpp:318-333)
//   qml_lightning_sorf::{get_SORF_coefficients, get_cos_features}   (upstream cuda/torchscript/SORF.cpp:138-150)
// and one new operator, qml_lightning_b200::sorf_energy, that the rebuilt HadamardFeaturesModel.forward calls: the
// whole FCHL19 -> PCA -> SORF -> energy chain with the coordinate gradient computed in the same pass (and its RFF
// twin qml_lightning_b200::rff_energy for RandomFourrierFeaturesModel.forward).
//
// This file contains no device code: it only allocates tensors, picks the current stream and device, and forwards
// raw pointers to libqmlb200.so.  Unlike upstream it honours the current CUDA stream and device of the inputs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/script.h>

#include <vector>

#include "qmlb200.h"

using torch::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

namespace {

void check(int rc, const char *what) {
    TORCH_CHECK(rc == QMLB_OK, what, " failed (code ", rc, "): ", qmlb_last_error());
}

qmlb_stream_t current_stream() { return (qmlb_stream_t)at::cuda::getCurrentCUDAStream().stream(); }

Tensor f32c(const Tensor &t) { return t.to(torch::kFloat32).contiguous(); }
Tensor i32c(const Tensor &t) { return t.to(torch::kInt32).contiguous(); }

const float *cell_ptr(const Tensor &c) { return c.numel() == 0 ? nullptr : c.data_ptr<float>(); }

struct Fchl {
    Tensor species, Rs2, Rs3;
    qmlb_fchl_params p;
    Fchl(const Tensor &species_, const Tensor &Rs2_, const Tensor &Rs3_, double eta2, double eta3, double d2, double w3,
         double d3, double rcut, const torch::Device &dev) {
        species = f32c(species_.to(dev));
        Rs2 = f32c(Rs2_.to(dev));
        Rs3 = f32c(Rs3_.to(dev));
        p.species = species.data_ptr<float>();
        p.nspecies = (int)species.numel();
        p.Rs2 = Rs2.data_ptr<float>();
        p.nRs2 = (int)Rs2.numel();
        p.Rs3 = Rs3.data_ptr<float>();
        p.nRs3 = (int)Rs3.numel();
        p.eta2 = (float)eta2;
        p.eta3 = (float)eta3;
        p.two_body_decay = (float)d2;
        p.three_body_weight = (float)w3;
        p.three_body_decay = (float)d3;
        p.rcut = (float)rcut;
    }
    int repsize() const { return qmlb_fchl19_repsize(p.nspecies, p.nRs2, p.nRs3); }
};

struct Batch {
    Tensor X, Z, counts, cell, inv_cell;
    int nb, A;
    Batch(Tensor X_, Tensor Z_, const Tensor &counts_, const Tensor &cell_, const Tensor &inv_cell_) {
        TORCH_CHECK(X_.device().type() == torch::kCUDA, "coordinates must be a CUDA tensor");
        TORCH_CHECK(Z_.device().type() == torch::kCUDA, "charges must be a CUDA tensor");
        TORCH_CHECK(counts_.device().type() == torch::kCUDA, "atom_counts must be a CUDA tensor");
        if (X_.dim() == 2) X_ = X_.unsqueeze(0);
        if (Z_.dim() == 1) Z_ = Z_.unsqueeze(0);
        X = f32c(X_);
        Z = f32c(Z_);
        counts = i32c(counts_);
        cell = f32c(cell_.to(X.device()));
        inv_cell = f32c(inv_cell_.to(X.device()));
        nb = (int)Z.size(0);
        A = (int)Z.size(1);
        TORCH_CHECK(X.size(0) == nb && X.size(1) == A && X.size(2) == 3, "coordinates must be [nbatch, natoms, 3]");
        TORCH_CHECK(counts.numel() == nb, "atom_counts must have one entry per molecule");
    }
};

// ---- qml_lightning_fchl ---------------------------------------------------------------------------------------

Tensor get_element_types(Tensor X, Tensor Z, Tensor natom_counts, Tensor species) {
    TORCH_CHECK(X.device().type() == torch::kCUDA, "coordinates must be a CUDA tensor");
    TORCH_CHECK(Z.device().type() == torch::kCUDA, "charges must be a CUDA tensor");
    TORCH_CHECK(species.device().type() == torch::kCUDA, "species must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(Z.device());
    if (Z.dim() == 1) Z = Z.unsqueeze(0);
    Z = f32c(Z);
    Tensor counts = i32c(natom_counts), sp = f32c(species);
    Tensor out = torch::zeros({Z.size(0), Z.size(1)}, Z.options().dtype(torch::kInt32));
    check(qmlb_element_types(Z.data_ptr<float>(), counts.data_ptr<int>(), sp.data_ptr<float>(), (int)sp.numel(),
                             (int)Z.size(0), (int)Z.size(1), out.data_ptr<int>(), current_stream()),
          "get_element_types");
    return out;
}

Tensor get_num_neighbours(Tensor X, Tensor natoms, Tensor rcut, Tensor cell, Tensor inv_cell) {
    TORCH_CHECK(X.device().type() == torch::kCUDA, "coordinates must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(X.device());
    if (X.dim() == 2) X = X.unsqueeze(0);
    X = f32c(X);
    Tensor counts = i32c(natoms), c = f32c(cell.to(X.device())), ic = f32c(inv_cell.to(X.device()));
    const int A_out = counts.max().item<int>();  // upstream output width (FCHL19.cpp:77)
    Tensor out = torch::zeros({X.size(0), A_out}, X.options().dtype(torch::kInt32));
    check(qmlb_num_neighbours(X.data_ptr<float>(), counts.data_ptr<int>(), (int)X.size(0), (int)X.size(1),
                              rcut.item<float>(), cell_ptr(c), cell_ptr(ic), out.data_ptr<int>(), A_out, current_stream()),
          "get_num_neighbours");
    return out;
}

Tensor get_neighbour_list(Tensor X, Tensor natoms, Tensor max_neighbours, Tensor rcut, Tensor cell, Tensor inv_cell) {
    TORCH_CHECK(X.device().type() == torch::kCUDA, "coordinates must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(X.device());
    if (X.dim() == 2) X = X.unsqueeze(0);
    X = f32c(X);
    Tensor counts = i32c(natoms), c = f32c(cell.to(X.device())), ic = f32c(inv_cell.to(X.device()));
    const int A_out = counts.max().item<int>();
    const int max_nb = max_neighbours.item<int>();
    Tensor out = torch::full({X.size(0), A_out, max_nb}, -1, X.options().dtype(torch::kInt32));
    check(qmlb_neighbour_list(X.data_ptr<float>(), counts.data_ptr<int>(), (int)X.size(0), (int)X.size(1),
                              rcut.item<float>(), cell_ptr(c), cell_ptr(ic), max_nb, out.data_ptr<int>(), A_out,
                              current_stream()),
          "get_neighbour_list");
    return out;
}

class FCHL19Fn : public torch::autograd::Function<FCHL19Fn> {
   public:
    static variable_list forward(AutogradContext *ctx, Tensor X, Tensor Z, Tensor species, Tensor atomIDs, Tensor molIDs,
                                 Tensor atom_counts, Tensor cell, Tensor inv_cell, Tensor Rs2, Tensor Rs3, Tensor eta2,
                                 Tensor eta3, Tensor two_body_decay, Tensor three_body_weight, Tensor three_body_decay,
                                 Tensor rcut) {
        TORCH_CHECK(species.device().type() == torch::kCUDA, "species must be a CUDA tensor");
        TORCH_CHECK(atomIDs.device().type() == torch::kCUDA, "atomIDs must be a CUDA tensor");
        TORCH_CHECK(molIDs.device().type() == torch::kCUDA, "molIDs must be a CUDA tensor");
        TORCH_CHECK(cell.device().type() == torch::kCUDA, "cell must be a CUDA tensor");
        TORCH_CHECK(inv_cell.device().type() == torch::kCUDA, "inv_cell must be a CUDA tensor");
        Batch b(X, Z, atom_counts, cell, inv_cell);
        c10::cuda::CUDAGuard guard(b.X.device());
        Fchl f(species, Rs2, Rs3, eta2.item<double>(), eta3.item<double>(), two_body_decay.item<double>(),
               three_body_weight.item<double>(), three_body_decay.item<double>(), rcut.item<double>(), b.X.device());
        Tensor rep = torch::empty({b.nb, b.A, f.repsize()}, b.X.options());
        check(qmlb_fchl19_forward(b.X.data_ptr<float>(), b.Z.data_ptr<float>(), b.counts.data_ptr<int>(), b.nb, b.A, &f.p,
                                  cell_ptr(b.cell), cell_ptr(b.inv_cell), nullptr, rep.data_ptr<float>(), current_stream()),
              "fchl_forwards");
        ctx->save_for_backward({b.X, b.Z, b.counts, b.cell, b.inv_cell, f.species, f.Rs2, f.Rs3});
        ctx->saved_data["scalars"] = std::vector<double>{f.p.eta2, f.p.eta3, f.p.two_body_decay, f.p.three_body_weight,
                                                         f.p.three_body_decay, f.p.rcut};
        return {rep};
    }

    static variable_list backward(AutogradContext *ctx, variable_list grad_output) {
        auto s = ctx->get_saved_variables();
        auto sc = ctx->saved_data["scalars"].toDoubleVector();
        Tensor X = s[0], Z = s[1], counts = s[2], cell = s[3], inv_cell = s[4];
        c10::cuda::CUDAGuard guard(X.device());
        Fchl f(s[5], s[6], s[7], sc[0], sc[1], sc[2], sc[3], sc[4], sc[5], X.device());
        Tensor g = f32c(grad_output[0]);
        const int nb = (int)Z.size(0), A = (int)Z.size(1);
        Tensor gX = torch::empty({nb, A, 3}, X.options());
        check(qmlb_fchl19_backward(X.data_ptr<float>(), Z.data_ptr<float>(), counts.data_ptr<int>(), nb, A, &f.p,
                                   cell_ptr(cell), cell_ptr(inv_cell), nullptr, g.data_ptr<float>(), gX.data_ptr<float>(),
                                   nullptr, nullptr, current_stream()),
              "fchl_backwards");
        Tensor u;
        return {gX, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u};
    }
};

Tensor fchl_forwards(const Tensor &X, const Tensor &Z, const Tensor &species, const Tensor &atomIDs, const Tensor &molIDs,
                     const Tensor &atom_counts, const Tensor &cell, const Tensor &inv_cell, const Tensor &Rs2,
                     const Tensor &Rs3, const Tensor &eta2, const Tensor &eta3, const Tensor &two_body_decay,
                     const Tensor &three_body_weight, const Tensor &three_body_decay, const Tensor &rcut) {
    return FCHL19Fn::apply(X, Z, species, atomIDs, molIDs, atom_counts, cell, inv_cell, Rs2, Rs3, eta2, eta3,
                           two_body_decay, three_body_weight, three_body_decay, rcut)[0];
}

std::vector<Tensor> get_fchl_and_derivative(Tensor X, Tensor Z, Tensor species, Tensor atomIDs, Tensor molIDs,
                                            Tensor atom_counts, Tensor cell, Tensor inv_cell, Tensor Rs2, Tensor Rs3,
                                            Tensor eta2, Tensor eta3, Tensor two_body_decay, Tensor three_body_weight,
                                            Tensor three_body_decay, Tensor rcut, bool gradients) {
    Batch b(X, Z, atom_counts, cell, inv_cell);
    c10::cuda::CUDAGuard guard(b.X.device());
    Fchl f(species, Rs2, Rs3, eta2.item<double>(), eta3.item<double>(), two_body_decay.item<double>(),
           three_body_weight.item<double>(), three_body_decay.item<double>(), rcut.item<double>(), b.X.device());
    Tensor rep = torch::empty({b.nb, b.A, f.repsize()}, b.X.options());
    if (!gradients) {
        check(qmlb_fchl19_forward(b.X.data_ptr<float>(), b.Z.data_ptr<float>(), b.counts.data_ptr<int>(), b.nb, b.A, &f.p,
                                  cell_ptr(b.cell), cell_ptr(b.inv_cell), nullptr, rep.data_ptr<float>(), current_stream()),
              "get_fchl_and_derivative");
        return {rep};
    }
    Tensor jac = torch::empty({b.nb, b.A, b.A, 3, f.repsize()}, b.X.options());
    check(qmlb_fchl19_forward_jacobian(b.X.data_ptr<float>(), b.Z.data_ptr<float>(), b.counts.data_ptr<int>(), b.nb, b.A,
                                       &f.p, cell_ptr(b.cell), cell_ptr(b.inv_cell), nullptr, rep.data_ptr<float>(),
                                       jac.data_ptr<float>(), current_stream()),
          "get_fchl_and_derivative");
    return {rep, jac};
}

// ---- qml_lightning_sorf ---------------------------------------------------------------------------------------

class SORFFn : public torch::autograd::Function<SORFFn> {
   public:
    static variable_list forward(AutogradContext *ctx, Tensor u, Tensor d, Tensor coeff_normalisation, Tensor ntransforms) {
        TORCH_CHECK(u.device().type() == torch::kCUDA, "u must be a CUDA tensor");
        TORCH_CHECK(d.device().type() == torch::kCUDA, "dmatrix must be a CUDA tensor");
        c10::cuda::CUDAGuard guard(u.device());
        Tensor uc = f32c(u), dc = f32c(d);
        const float norm = coeff_normalisation.item<float>();
        const int T = ntransforms.item<int>();
        TORCH_CHECK(uc.dim() == 2 && dc.dim() == 3 && dc.size(2) == uc.size(1) && T <= dc.size(0), "bad SORF shapes");
        Tensor out = torch::empty({uc.size(0), dc.size(1), uc.size(1)}, uc.options());
        check(qmlb_sorf_coefficients(uc.data_ptr<float>(), dc.data_ptr<float>(), (int)uc.size(0), (int)uc.size(1),
                                     (int)dc.size(1), T, norm, out.data_ptr<float>(), current_stream()),
              "get_SORF_coefficients");
        ctx->save_for_backward({dc});
        ctx->saved_data["norm"] = (double)norm;
        ctx->saved_data["T"] = (int64_t)T;
        return {out};
    }
    static variable_list backward(AutogradContext *ctx, variable_list grad_output) {
        Tensor d = ctx->get_saved_variables()[0];
        c10::cuda::CUDAGuard guard(d.device());
        Tensor g = f32c(grad_output[0]);
        Tensor out = torch::empty({g.size(0), g.size(2)}, g.options());
        check(qmlb_sorf_coefficients_backward(g.data_ptr<float>(), d.data_ptr<float>(), (int)g.size(0), (int)g.size(2),
                                              (int)g.size(1), (int)ctx->saved_data["T"].toInt(),
                                              (float)ctx->saved_data["norm"].toDouble(), out.data_ptr<float>(),
                                              current_stream()),
              "get_SORF_coefficients backward");
        Tensor u;
        return {out, u, u, u};
    }
};

class CosFeaturesFn : public torch::autograd::Function<CosFeaturesFn> {
   public:
    static variable_list forward(AutogradContext *ctx, Tensor coeffs, Tensor b, Tensor nmol, Tensor batch_indexes) {
        TORCH_CHECK(coeffs.device().type() == torch::kCUDA, "coeffs must be a CUDA tensor");
        TORCH_CHECK(b.device().type() == torch::kCUDA, "b must be a CUDA tensor");
        TORCH_CHECK(batch_indexes.device().type() == torch::kCUDA, "batch_indexes must be a CUDA tensor");
        c10::cuda::CUDAGuard guard(coeffs.device());
        Tensor c = f32c(coeffs), bc = f32c(b), idx = i32c(batch_indexes);
        const int n_mol = nmol.item<int>();
        Tensor out = torch::empty({n_mol, c.size(1)}, c.options());
        check(qmlb_cos_features(c.data_ptr<float>(), bc.data_ptr<float>(), idx.data_ptr<int>(), (int)c.size(0),
                                (int)c.size(1), n_mol, out.data_ptr<float>(), current_stream()),
              "get_cos_features");
        ctx->save_for_backward({c, bc, idx});
        return {out};
    }
    static variable_list backward(AutogradContext *ctx, variable_list grad_output) {
        auto s = ctx->get_saved_variables();
        Tensor c = s[0], b = s[1], idx = s[2];
        c10::cuda::CUDAGuard guard(c.device());
        Tensor g = f32c(grad_output[0]);
        Tensor out = torch::empty_like(c);
        check(qmlb_cos_features_backward(g.data_ptr<float>(), c.data_ptr<float>(), b.data_ptr<float>(), idx.data_ptr<int>(),
                                         (int)c.size(0), (int)c.size(1), out.data_ptr<float>(), current_stream()),
              "get_cos_features backward");
        Tensor u;
        return {out, u, u, u};
    }
};

Tensor get_sorf(const Tensor &u, const Tensor &d, const Tensor &coeff_normalisation, const Tensor &ntransforms) {
    return SORFFn::apply(u, d, coeff_normalisation, ntransforms)[0];
}

Tensor get_cos_features(const Tensor &coeffs, const Tensor &b, const Tensor &nmol, const Tensor &batch_indexes) {
    return CosFeaturesFn::apply(coeffs, b, nmol, batch_indexes)[0];
}

// ---- qml_lightning_b200 : fused model forward -----------------------------------------------------------------

Tensor sorf_pack(const Tensor &Dmat, const Tensor &bias, const Tensor &alpha) {
    TORCH_CHECK(Dmat.device().type() == torch::kCUDA, "Dmat must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(Dmat.device());
    Tensor D = f32c(Dmat), b = f32c(bias.to(D.device())), a = f32c(alpha.to(D.device()));
    TORCH_CHECK(D.dim() == 4, "Dmat must be [nelements, ntransforms, nstacks, npcas]");
    const int nel = (int)D.size(0), T = (int)D.size(1), S = (int)D.size(2), N = (int)D.size(3);
    TORCH_CHECK(b.numel() == (int64_t)nel * S * N && a.numel() == (int64_t)S * N, "bias / alpha do not match Dmat");
    Tensor packed = torch::empty({(int64_t)(qmlb_sorf_pack_bytes(nel, N, S, T) / sizeof(float))}, D.options());
    check(qmlb_sorf_pack(D.data_ptr<float>(), b.data_ptr<float>(), a.data_ptr<float>(), nel, N, S, T,
                         packed.data_ptr<float>(), current_stream()),
          "sorf_pack");
    return packed;
}

// E[m] and dE/dX in one pass; the autograd backward scales the stored gradient by the incoming d/dE[m].
class SorfEnergyFn : public torch::autograd::Function<SorfEnergyFn> {
   public:
    static variable_list forward(AutogradContext *ctx, Tensor X, Tensor Z, Tensor atom_counts, Tensor cell, Tensor inv_cell,
                                 Tensor species, Tensor Rs2, Tensor Rs3, Tensor fchl_scalars, Tensor elements,
                                 Tensor reductors, Tensor packed, int64_t nstacks, int64_t ntransforms, double sigma,
                                 int64_t n_atoms_upper, bool fast_math) {
        Batch b(X, Z, atom_counts, cell, inv_cell);
        c10::cuda::CUDAGuard guard(b.X.device());
        Tensor sc = fchl_scalars.to(torch::kCPU).to(torch::kFloat64).contiguous();
        TORCH_CHECK(sc.numel() == 6, "fchl_scalars must hold eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut");
        const double *s = sc.data_ptr<double>();
        Fchl f(species, Rs2, Rs3, s[0], s[1], s[2], s[3], s[4], s[5], b.X.device());
        Tensor el = f32c(elements.to(b.X.device())), red = f32c(reductors), pk = f32c(packed);
        TORCH_CHECK(red.dim() == 3 && red.size(0) == el.numel() && red.size(1) == f.repsize(),
                    "reductors must be [nelements, repsize, npcas]");
        const int nel = (int)el.numel(), npcas = (int)red.size(2);
        const size_t upper = n_atoms_upper > 0 ? (size_t)n_atoms_upper : (size_t)b.nb * b.A;
        const size_t bytes = qmlb_predict_workspace_bytes(b.nb, b.A, upper, nel, f.repsize(), npcas);
        Tensor ws = torch::empty({(int64_t)bytes + 256}, b.X.options().dtype(torch::kUInt8));
        char *wp = reinterpret_cast<char *>(((uintptr_t)ws.data_ptr<uint8_t>() + 255) & ~(uintptr_t)255);
        Tensor E = torch::empty({b.nb}, b.X.options());
        Tensor gX = torch::empty({b.nb, b.A, 3}, b.X.options());
        if (b.nb > 0)
        check(qmlb_sorf_predict(b.X.data_ptr<float>(), b.Z.data_ptr<float>(), b.counts.data_ptr<int>(), b.nb, b.A, &f.p,
                                cell_ptr(b.cell), cell_ptr(b.inv_cell), el.data_ptr<float>(), nel, red.data_ptr<float>(),
                                nullptr, npcas, pk.data_ptr<float>(), (int)nstacks, (int)ntransforms, (float)sigma, fast_math ? 1 : 0,
                                upper, wp, bytes, E.data_ptr<float>(), gX.data_ptr<float>(), current_stream()),
              "sorf_energy");
        ctx->save_for_backward({gX});
        return {E};
    }
    static variable_list backward(AutogradContext *ctx, variable_list grad_output) {
        Tensor gX = ctx->get_saved_variables()[0];
        Tensor g = grad_output[0].to(gX.dtype()).reshape({-1, 1, 1}) * gX;
        Tensor u;
        return {g, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u};
    }
};

Tensor sorf_energy(const Tensor &X, const Tensor &Z, const Tensor &atom_counts, const Tensor &cell, const Tensor &inv_cell,
                   const Tensor &species, const Tensor &Rs2, const Tensor &Rs3, const Tensor &fchl_scalars,
                   const Tensor &elements, const Tensor &reductors, const Tensor &packed, int64_t nstacks,
                   int64_t ntransforms, double sigma, int64_t n_atoms_upper, bool fast_math) {
    return SorfEnergyFn::apply(X, Z, atom_counts, cell, inv_cell, species, Rs2, Rs3, fchl_scalars, elements, reductors,
                               packed, nstacks, ntransforms, sigma, n_atoms_upper, fast_math)[0];
}

// RFF twin of sorf_pack: fp16 hi/lo chunk images of W plus bias and weights for the tensor-core feature kernel.
Tensor rff_pack(const Tensor &W, const Tensor &b, const Tensor &alpha) {
    TORCH_CHECK(W.device().type() == torch::kCUDA, "W must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(W.device());
    Tensor Wc = f32c(W), bc = f32c(b.to(Wc.device())), ac = f32c(alpha.to(Wc.device()));
    TORCH_CHECK(Wc.dim() == 3, "W must be [nelements, npcas, D]");
    const int nel = (int)Wc.size(0), K = (int)Wc.size(1), D = (int)Wc.size(2);
    TORCH_CHECK(bc.numel() == (int64_t)nel * D && ac.numel() == D, "b must be [nelements, D] and alpha [D]");
    const size_t bytes = qmlb_rff_pack_bytes(nel, K, D);
    TORCH_CHECK(bytes > 0, "rff_pack: npcas must be 32, 64, 128 or 256");
    Tensor packed = torch::empty({(int64_t)bytes}, Wc.options().dtype(torch::kUInt8));
    check(qmlb_rff_pack(Wc.data_ptr<float>(), bc.data_ptr<float>(), ac.data_ptr<float>(), nel, K, D, packed.data_ptr<uint8_t>(),
                        bytes, current_stream()),
          "rff_pack");
    return packed;
}

// RFF twin of SorfEnergyFn.
class RffEnergyFn : public torch::autograd::Function<RffEnergyFn> {
   public:
    static variable_list forward(AutogradContext *ctx, Tensor X, Tensor Z, Tensor atom_counts, Tensor cell, Tensor inv_cell,
                                 Tensor species, Tensor Rs2, Tensor Rs3, Tensor fchl_scalars, Tensor elements,
                                 Tensor reductors, Tensor packed, int64_t n_atoms_upper, bool fast_math) {
        Batch bt(X, Z, atom_counts, cell, inv_cell);
        c10::cuda::CUDAGuard guard(bt.X.device());
        Tensor sc = fchl_scalars.to(torch::kCPU).to(torch::kFloat64).contiguous();
        TORCH_CHECK(sc.numel() == 6, "fchl_scalars must hold eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut");
        const double *s = sc.data_ptr<double>();
        Fchl f(species, Rs2, Rs3, s[0], s[1], s[2], s[3], s[4], s[5], bt.X.device());
        Tensor el = f32c(elements.to(bt.X.device())), red = f32c(reductors);
        TORCH_CHECK(red.dim() == 3 && red.size(0) == el.numel() && red.size(1) == f.repsize(),
                    "reductors must be [nelements, repsize, npcas]");
        TORCH_CHECK(packed.device() == bt.X.device() && packed.scalar_type() == torch::kUInt8 && packed.is_contiguous(),
                    "packed must be the uint8 tensor returned by rff_pack, on the device of X");
        const int nel = (int)el.numel(), npcas = (int)red.size(2);
        const size_t upper = n_atoms_upper > 0 ? (size_t)n_atoms_upper : (size_t)bt.nb * bt.A;
        const size_t bytes = qmlb_predict_workspace_bytes(bt.nb, bt.A, upper, nel, f.repsize(), npcas);
        Tensor ws = torch::empty({(int64_t)bytes + 256}, bt.X.options().dtype(torch::kUInt8));
        char *wp = reinterpret_cast<char *>(((uintptr_t)ws.data_ptr<uint8_t>() + 255) & ~(uintptr_t)255);
        Tensor E = torch::empty({bt.nb}, bt.X.options());
        Tensor gX = torch::empty({bt.nb, bt.A, 3}, bt.X.options());
        if (bt.nb > 0)
        check(qmlb_rff_predict_packed(bt.X.data_ptr<float>(), bt.Z.data_ptr<float>(), bt.counts.data_ptr<int>(), bt.nb, bt.A,
                                      &f.p, cell_ptr(bt.cell), cell_ptr(bt.inv_cell), el.data_ptr<float>(), nel,
                                      red.data_ptr<float>(), nullptr, npcas, packed.data_ptr<uint8_t>(), fast_math ? 1 : 0, upper, wp,
                                      bytes, E.data_ptr<float>(), gX.data_ptr<float>(), current_stream()),
              "rff_energy");
        ctx->save_for_backward({gX});
        return {E};
    }
    static variable_list backward(AutogradContext *ctx, variable_list grad_output) {
        Tensor gX = ctx->get_saved_variables()[0];
        Tensor g = grad_output[0].to(gX.dtype()).reshape({-1, 1, 1}) * gX;
        Tensor u;
        return {g, u, u, u, u, u, u, u, u, u, u, u, u, u};
    }
};

Tensor rff_energy(const Tensor &X, const Tensor &Z, const Tensor &atom_counts, const Tensor &cell, const Tensor &inv_cell,
                  const Tensor &species, const Tensor &Rs2, const Tensor &Rs3, const Tensor &fchl_scalars,
                  const Tensor &elements, const Tensor &reductors, const Tensor &packed, int64_t n_atoms_upper,
                  bool fast_math) {
    return RffEnergyFn::apply(X, Z, atom_counts, cell, inv_cell, species, Rs2, Rs3, fchl_scalars, elements, reductors, packed,
                              n_atoms_upper, fast_math)[0];
}

}  // namespace

TORCH_LIBRARY(qml_lightning_fchl, m) {
    m.def("fchl_forwards", fchl_forwards);
    m.def("get_fchl_and_derivative", get_fchl_and_derivative);
    m.def("get_element_types", get_element_types);
    m.def("get_neighbour_list", get_neighbour_list);
    m.def("get_num_neighbours", get_num_neighbours);
}

TORCH_LIBRARY(qml_lightning_sorf, m) {
    m.def("get_SORF_coefficients", get_sorf);
    m.def("get_cos_features", get_cos_features);
}

TORCH_LIBRARY(qml_lightning_b200, m) {
    m.def("sorf_pack", sorf_pack);
    m.def("sorf_energy", sorf_energy);
    m.def("rff_pack", rff_pack);
    m.def("rff_energy", rff_energy);
}
