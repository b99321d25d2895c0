/*
 * dynb — C ABI of the B200 (sm_100a) implementation of the Dynamis per-step data-parallel
 * hot path: periodic radius graph, space-filling-curve partition, halo maps, halo exchange.
 *
 * Conventions
 *   - Every pointer named *_dev is device memory of the current CUDA device; *_host is host
 *     memory (pinned where the call copies asynchronously into it).
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and nothing
 *     here synchronises unless the comment says so.
 *   - Functions return 0 on success, a negative DYNB_ERR_* code otherwise;
 *     dynb_last_error() returns a message for the calling thread's last failure.
 *   - Nothing here allocates or frees device memory unless the comment says so: the caller
 *     provides outputs and workspaces (sizes come from the *_workspace_bytes functions).
 *
 * Each entry point cites the reference interface it replaces (path inside the reference
 * project : line).
 */
#ifndef DYNB_H
#define DYNB_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DYNB_OK 0
#define DYNB_ERR_ARG (-1)     /* invalid argument */
#define DYNB_ERR_CUDA (-2)    /* a CUDA runtime call failed */
#define DYNB_ERR_STATE (-3)   /* call order / object state */
#define DYNB_ERR_TIMEOUT (-4) /* a bounded device-side wait expired */

#define DYNB_F32 0
#define DYNB_F64 1

/* Bits of dynb_rg_header.status (set by kernels, read by the host after the plan). */
#define DYNB_RG_SRC_OVERFLOW 1u    /* more periodic images than src_capacity: re-plan with header.M */
#define DYNB_RG_BAD_TARGET 2u      /* a target index outside [0, n_atoms) */
#define DYNB_RG_SHIFT_RANGE 4u     /* an atom lies more than 32767 cells outside the unit cell */
#define DYNB_RG_NONFINITE 8u       /* a position is NaN or Inf */

const char* dynb_last_error(void);
int dynb_version(void);

/* ------------------------------------------------------------------ radius graph
 * Replaces radius_graph_pbc / radius_graph_pbc_ex / radius_graph_pbc_counts_ex
 * (dynamis_state/src/csrc/graph/radius_graph.cpp:7-127) and the implementation behind them
 * (dynamis_state/src/csrc/graph/radius_graph_kernels.cu:479-934).
 *
 * Two phases, because the number of edges is only known after counting:
 *   dynb_rg_plan   wrap -> periodic images -> cell binning -> per-target degrees -> offsets;
 *                  copies a dynb_rg_header into header_host asynchronously.
 *   (caller synchronises the stream, reads header.E, allocates the outputs)
 *   dynb_rg_fill   writes edge_index [2,E] int64 and cell_shifts [E,3] float32.
 * The workspace carries the plan between the two calls and must not be touched in between.
 */
typedef struct dynb_rg_header {
    int64_t E;          /* directed edges (sum of degrees) */
    int64_t M;          /* source images (atoms + periodic copies) */
    uint32_t status;    /* DYNB_RG_* bits */
    uint32_t max_degree;
    int32_t grid[3];    /* cell grid dimensions chosen on the device */
    int32_t group_cells;/* cells per warp work item along x */
    int64_t num_groups;
    int64_t reserved[2];
} dynb_rg_header;

/* Suggested capacities for a system: src_capacity bounds the number of periodic images
 * (exact upper bound n_atoms * prod(2*rep+1) is used when it is small), cell_capacity the
 * number of grid cells.  cell_host: 9 reals of `dtype`, rows = lattice vectors. */
int dynb_rg_suggest_capacity(int64_t n_atoms, const void* cell_host, const uint8_t* pbc_host, double radius,
                             int dtype, int64_t* src_capacity, int64_t* cell_capacity);

int dynb_rg_workspace_bytes(int64_t n_atoms, int64_t n_targets, int64_t src_capacity, int64_t cell_capacity,
                            int dtype, int64_t* bytes);

int dynb_rg_plan(const void* pos_dev, int dtype, int64_t n_atoms, const void* cell_host, const uint8_t* pbc_host,
                 double radius, const int64_t* target_indices_dev /* or NULL = all atoms */, int64_t n_targets,
                 void* workspace_dev, int64_t workspace_bytes, int64_t src_capacity, int64_t cell_capacity,
                 int32_t* neighbor_counts_dev /* [n_targets] caller order, or NULL */,
                 dynb_rg_header* header_host, void* stream);

/* dist_sq_dev (optional, may be NULL): squared edge lengths in the plan's dtype, in the order
 * the edges are written, exactly as the kernel arithmetic produced them (the reference computes
 * them, radius_graph_kernels.cu:299, but does not return them). */
int dynb_rg_fill(const void* workspace_dev, int dtype, int64_t* edge_index_dev /* [2,E] */,
                 float* cell_shifts_dev /* [E,3] */, void* dist_sq_dev /* [E] or NULL */, int64_t E, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DYNB_H */
