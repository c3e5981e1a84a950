// TEST INFRASTRUCTURE ONLY -- not part of the product path.
//
// Binding file for the UNMODIFIED reference implementation (MrHuff/F3M, F3M_src/n_tree.cu and
// the files it includes).  The reference sources are not copied: they are compiled from where
// they lie through the include path given by oracle/Makefile.  Besides the reference's public
// entry points (FFM_XY<float,d>, rbf_call<T,d>; F3M_src/pybinder_setup.cu:17-62) this file adds
// two read-only probes that drive the reference's own tree and interaction-list code and return
// its intermediate tensors, so that box assignments and far/small/near lists of the new engine
// can be compared with the reference's:
//   tree_levels  : n_tree_cuda<float,d> constructor + divide() k times   (n_tree.cu:79-179)
//   field_trace  : the level loop of FFM_XY (n_tree.cu:1071-1117) with get_field (n_tree.cu:903-969)
//                  in place of far_field_run, i.e. the same lists but no arithmetic on b.
#include "n_tree.cu"
#include <torch/extension.h>

#ifndef F3M_REF_DIM
#define F3M_REF_DIM 3
#endif

namespace {
constexpr int D = F3M_REF_DIM;
using tree_t = n_tree_cuda<float, D>;

std::vector<torch::Tensor> snapshot(tree_t &t) {
    return {t.sorted_index.clone(), t.unique_counts.clone(), t.unique_counts_cum_reindexed.clone(),
            t.centers.clone(), t.edge.clone()};
}

std::vector<std::vector<torch::Tensor>> tree_levels(torch::Tensor &X, int nlevels, const std::string &dev) {
    torch::Tensor edge, xmin, xmax;
    std::tie(edge, xmin, xmax) = calculate_edge_X<float, D>(X, dev);
    tree_t tree(edge, X, xmin, xmax, dev);
    std::vector<std::vector<torch::Tensor>> out;
    for (int l = 0; l < nlevels; l++) {
        tree.divide();
        out.push_back(snapshot(tree));
    }
    return out;
}

// Returns, per level built: [far, small, keep, X-tree snapshot (5 tensors), Y-tree snapshot (5 tensors)].
std::vector<std::vector<torch::Tensor>> field_trace(torch::Tensor &X, torch::Tensor &Y, const std::string &dev,
                                                    float ls, float min_points, int nr_interp, bool var_comp,
                                                    float eff_var_limit, int small_field_limit) {
    float lcs = 1 / (2 * ls * ls);
    std::vector<std::vector<torch::Tensor>> out;
    torch::Tensor near_field = torch::zeros({1, 2}).toType(torch::kInt32).to(dev);
    torch::Tensor far_field, small_field;
    auto record = [&](tree_t &tx, tree_t &ty) {
        std::vector<torch::Tensor> rec = {far_field.clone(), small_field.clone(), near_field.clone()};
        for (auto &t : snapshot(tx)) rec.push_back(t);
        for (auto &t : snapshot(ty)) rec.push_back(t);
        out.push_back(rec);
    };
    if (X.data_ptr() == Y.data_ptr()) {
        torch::Tensor edge, xmin, xmax;
        std::tie(edge, xmin, xmax) = calculate_edge_X<float, D>(X, dev);
        tree_t tx(edge, X, xmin, xmax, dev);
        while (near_field.numel() > 0 and tx.avg_nr_points > min_points) {
            tx.divide();
            std::tie(far_field, small_field, near_field) =
                get_field<float, D>(near_field, tx, tx, lcs, nr_interp, dev, var_comp, eff_var_limit, small_field_limit);
            record(tx, tx);
        }
    } else {
        torch::Tensor edge, xmin, ymin, xmax, ymax, xe, ye;
        std::tie(edge, xmin, ymin, xmax, ymax, xe, ye) = calculate_edge<float, D>(X, Y, dev);
        tree_t tx(edge, X, xmin, xmax, dev);
        tree_t ty(edge, Y, ymin, ymax, dev);
        while (near_field.numel() > 0 and (tx.avg_nr_points > min_points and ty.avg_nr_points > min_points)) {
            tx.divide();
            ty.divide();
            std::tie(far_field, small_field, near_field) =
                get_field<float, D>(near_field, tx, ty, lcs, nr_interp, dev, var_comp, eff_var_limit, small_field_limit);
            record(tx, ty);
        }
    }
    return out;
}
}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.attr("dim") = D;
    m.def("FFM_XY_FLOAT", &FFM_XY<float, D>, "reference FFM_XY<float,d>");
    m.def("rbf_float", &rbf_call<float, D>, "reference dense product, float");
    m.def("rbf_double", &rbf_call<double, D>, "reference dense product, double tensors");
    m.def("tree_levels", &tree_levels, "reference tree state after each divide()");
    m.def("field_trace", &field_trace, "reference far/small/keep lists per level");
}
