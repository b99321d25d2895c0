// TEST INFRASTRUCTURE ONLY — exposes the reference's own CUDA implementations of the hot path
// as torch ops so that the GPU parity tests can run them next to ours on the same inputs.
//
// This file is ours; the implementations it forwards to are compiled, unmodified, from the
// reference's sources where they lie (see build_ref.py):
//   dynamis_state/src/csrc/graph/radius_graph_kernels.cu      radius_graph_pbc_cuda_impl_ex
//   dynamis_state/src/csrc/partition/sfc_kernels.cu           sfc_partition_cuda_impl
//   dynamis_state/src/csrc/graph/dist_graph_ops_kernels.cu    filter_edges / extract_halo_info
//   dynamis_state/src/csrc/partition/kdtree_kernels.cu        kdtree_bisect_cuda_impl
#include <ATen/ATen.h>
#include <torch/library.h>
#include <tuple>

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor>
radius_graph_pbc_cuda_impl_ex(at::Tensor pos, at::Tensor cell, at::Tensor pbc, float radius,
                              int64_t max_num_neighbors, bool enforce_max_strictly,
                              c10::optional<at::Tensor> target_indices, bool counts_only);
at::Tensor sfc_partition_cuda_impl(at::Tensor pos, at::Tensor weights, int64_t W, int64_t curve_type);
at::Tensor kdtree_bisect_cuda_impl(at::Tensor pos, at::Tensor weights, int64_t W);  // kdtree_kernels.cu
std::tuple<at::Tensor, at::Tensor>
filter_edges_to_radius_cuda_impl(at::Tensor edges, at::Tensor cell_shifts, at::Tensor pos, at::Tensor cell,
                                 double radius);
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
extract_halo_info_cuda_impl(at::Tensor edges, at::Tensor pid_outer, at::Tensor my_outer_atoms, int64_t my_rank,
                            int64_t world_size, int64_t N);

static std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor>
ref_radius_graph(at::Tensor pos, at::Tensor cell, at::Tensor pbc, double radius,
                 c10::optional<at::Tensor> target_indices, bool counts_only)
{
    return radius_graph_pbc_cuda_impl_ex(pos.contiguous(), cell.to(pos.device()).to(at::kFloat).contiguous(),
                                         pbc.to(at::kBool).contiguous(), (float)radius, 0, false, target_indices,
                                         counts_only);
}

static at::Tensor ref_sfc_partition(at::Tensor pos, c10::optional<at::Tensor> weights, int64_t W, int64_t curve)
{
    at::Tensor w;
    if (weights.has_value()) w = weights->to(at::kLong).contiguous();
    return sfc_partition_cuda_impl(pos.contiguous(), w, W, curve);
}

static std::tuple<at::Tensor, at::Tensor>
ref_filter_edges(at::Tensor edges, at::Tensor shifts, at::Tensor pos, at::Tensor cell, double radius)
{
    return filter_edges_to_radius_cuda_impl(edges.contiguous(), shifts.contiguous(), pos.contiguous(),
                                            cell.to(pos.device()).to(at::kFloat).contiguous(), radius);
}

static std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
ref_extract_halo_info(at::Tensor edges, at::Tensor pid, at::Tensor mine, int64_t rank, int64_t W, int64_t N)
{
    return extract_halo_info_cuda_impl(edges.contiguous(), pid.to(at::kLong).contiguous(), mine.contiguous(), rank, W, N);
}

// same argument preparation as kdtree_bisect_cuda (dynamis_state/src/csrc/partition/kdtree.cpp:9-26)
static at::Tensor ref_kdtree_partition(at::Tensor pos, c10::optional<at::Tensor> weights, int64_t W)
{
    at::Tensor w;
    if (weights.has_value() && weights->defined()) w = weights->to(at::kFloat).contiguous();
    return kdtree_bisect_cuda_impl(pos.contiguous(), w, W);
}

TORCH_LIBRARY(dynamis_ref, m)
{
    m.def("radius_graph(Tensor pos, Tensor cell, Tensor pbc, float radius, Tensor? target_indices, bool counts_only)"
          " -> (Tensor, Tensor, Tensor, Tensor)", &ref_radius_graph);
    m.def("sfc_partition(Tensor pos, Tensor? weights, int W, int curve) -> Tensor", &ref_sfc_partition);
    m.def("kdtree_partition(Tensor pos, Tensor? weights, int W) -> Tensor", &ref_kdtree_partition);
    m.def("filter_edges(Tensor edges, Tensor shifts, Tensor pos, Tensor cell, float radius) -> (Tensor, Tensor)",
          &ref_filter_edges);
    m.def("extract_halo_info(Tensor edges, Tensor pid, Tensor mine, int rank, int W, int N)"
          " -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)", &ref_extract_halo_info);
}
