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
#define DYNB_RG_SHIFT_RANGE 4u     /* an atom lies more than 511 cells outside the unit cell */
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
    int64_t reserved[2]; /* [0]: 0, or the longest candidate list in 32-record slots when one exceeded the 16 slots the
                          * count pass keeps hit bits for (dynb_rg_fill recomputes the distances of those groups); [1]: unused */
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

/* dynb_rg_fill for the model-side graph glue (dynamis_model/src/dynamis_model/nnp/mace.py:591-608,
 * uma.py:915-948): the models negate the offsets (unit_shifts = -cell_offsets), keep the edges whose
 * destination is an owned atom (edge_index[1] < num_local) and form shifts = unit_shifts @ cell in
 * float32 — three more passes over the edge list.  Here the owned-destination filter is the plan's
 * target subset 0..num_local-1, negate_shifts = 1 writes the offsets negated, and cart_shifts_dev
 * (optional, may be NULL) receives unit_shifts @ cell_host (9 floats, row-major) with the rounding of
 * a K = 3 float32 GEMM.  id_map_dev (optional, may be NULL; n_atoms entries): ids written into
 * edge_index instead of the atom indices — the local -> global mapping DistGraphBuilder applies to both
 * rows after a steady-state build (dynamis_state/src/dynamis_state/dist_graph_builder.py:441-470). */
int dynb_rg_fill_glue(const void* workspace_dev, int dtype, int64_t* edge_index_dev /* [2,E] */,
                      float* unit_shifts_dev /* [E,3] */, float* cart_shifts_dev /* [E,3] or NULL */,
                      const float* cell_host /* [9] */, int negate_shifts, const int64_t* id_map_dev,
                      int64_t E, void* stream);

/* Halo marking over a plan (all atoms as targets, radius = cutoff + ghost buffer): for every edge
 * src -> dst whose endpoints have different owners, sets bit owner[dst] of
 * needed_dev[src * words + ...] (words = ceil(world_size / 32)) and has_foreign_dev[dst] = 1.
 * Both outputs are cleared first.  This is the edge loop of build_halo_maps
 * (dynamis_state/src/csrc/build_halo_maps.cpp:50-58, 127-138) without materialising the graph. */
int dynb_rg_halo_mark(const void* workspace_dev, int dtype, const int64_t* owner_dev, int64_t n_atoms,
                      int64_t world_size, uint32_t* needed_dev, uint8_t* has_foreign_dev, void* stream);

/* ------------------------------------------------------------------ SFC partition
 * Replaces sfc_partition_cuda (dynamis_state/src/csrc/partition/sfc.cpp:9-33,
 * sfc_kernels.cu:178-251): labels_dev[i] in [0, W) for every atom.  curve_type 0 = Morton
 * (21 bits per axis), 1 = the reference's 7-bit "Hilbert" transform.  weights_dev: int64 per-atom
 * cost (non-negative) or NULL (equal counts).  perm_dev (optional): atom indices in curve order.
 * Atoms with equal keys are ordered by ascending index (the reference leaves ties unspecified).
 * With perm_dev == NULL, W <= 1025 and the full workspace, the labels come from a digit-by-digit
 * selection of the W - 1 split points on (key, index) instead of a sort (same labels, about a third of
 * the time); a workspace of the sorted path's size alone selects the sorted path. */
int dynb_sfc_workspace_bytes(int64_t n_atoms, int64_t* bytes);
int dynb_sfc_partition(const float* pos_dev, int64_t n_atoms, const int64_t* weights_dev, int64_t W, int curve_type,
                       int64_t* labels_dev, int64_t* perm_dev, void* workspace_dev, int64_t workspace_bytes,
                       void* stream);
/* Keys alone, in atom order (sfc_kernels.cu:32-109). */
int dynb_sfc_keys(const float* pos_dev, int64_t n_atoms, int curve_type, int64_t* keys_dev, void* workspace_dev,
                  int64_t workspace_bytes, void* stream);
/* The same partition when the atoms are spread over several ranks and no rank holds them all (the
 * reference gathers every atom to every rank first, dynamis/src/dynamis/simulatorState.py:136-199, then
 * calls sfc_partition_cuda): dynb_sfc_minmax gives this rank's coordinate extrema as six floats
 * (min xyz, max xyz) for the caller to min/max-reduce between the ranks; dynb_sfc_keys_from_bounds
 * computes the keys of this rank's atoms against the reduced extrema (sfc_kernels.cu:32-109, same
 * arithmetic); dynb_label_by_splits labels an atom with the number of split points (key, global id) that
 * are <= its own (key, global id) — the split points being the atoms at the sorted positions where the
 * reference's closed form (sfc_kernels.cu:114-137) starts a new label, found by the ranks together.
 * minmax_dev: 32 floats; the first six carry the extrema, the rest is scratch. */
int dynb_sfc_minmax(const float* pos_dev, int64_t n_atoms, float* minmax_dev, void* stream);
int dynb_sfc_keys_from_bounds(const float* pos_dev, int64_t n_atoms, int curve_type, float* minmax_dev, int64_t* keys_dev,
                              void* stream);
int dynb_label_by_splits(const int64_t* keys_dev, const int64_t* ids_dev, int64_t n, const int64_t* split_keys_dev,
                         const int64_t* split_ids_dev, int n_splits, int64_t* labels_dev, void* stream);
/* Stable LSD radix sort of (uint64 key, uint32 value) pairs on key bits [begin_bit, end_bit), in
 * place (replaces the at::sort call at sfc_kernels.cu:224). */
int dynb_radix_sort_workspace_bytes(int64_t n, int64_t* bytes);
int dynb_radix_sort_pairs(uint64_t* keys_dev, uint32_t* vals_dev, int64_t n, int begin_bit, int end_bit,
                          void* workspace_dev, int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ partition bookkeeping
 * atom_counts = bincount(labels) and partition_indices = vertex_numbers[nonzero(labels == R)]
 * (dynamis_state/src/csrc/partition/sfc_partitioner.cpp:166-176).  bad_dev: one uint32, non-zero
 * when a value fell outside [0, W).  dynb_select_eq_i64 writes at most n values to out_dev
 * (ascending positions; gather_src_dev[i] instead of i when given) and the count to count_dev. */
int dynb_bincount_i64(const int64_t* a_dev, int64_t n, int64_t W, int64_t* counts_dev, uint32_t* bad_dev, void* stream);
int dynb_select_workspace_bytes(int64_t n, int64_t* bytes);
int dynb_select_eq_i64(const int64_t* a_dev, int64_t n, int64_t value, const int64_t* gather_src_dev,
                       int64_t* out_dev, int64_t* count_dev, void* workspace_dev, int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ halo maps
 * Per-edge pass of extract_halo_info (dynamis_state/src/csrc/graph/dist_graph_ops_kernels.cu:46-59,
 * 104-188): edges_dev [2,E] with dst owned by my_rank.  Clears and fills
 * recv_mask_dev[src] |= bit pid[src], send_mask_dev[dst] |= bit pid[src], has_remote_dev[dst] = 1 for
 * every edge whose source belongs to another rank (masks are [N, ceil(W/32)] uint32). */
int dynb_halo_mark_from_edges(const int64_t* edges_dev, int64_t E, const int64_t* pid_dev, int64_t N, int64_t my_rank,
                              int64_t world_size, uint32_t* send_mask_dev, uint32_t* recv_mask_dev,
                              uint8_t* has_remote_dev, uint32_t* bad_dev, void* stream);

/* CSR assembly (build_halo_maps.cpp:60-125; dist_graph_ops_kernels.cu:143-177).  Element a in
 * [0, n) carries a set of peer ranks; segment p of the output lists, ascending in a, the elements
 * whose set contains p.  mode 0 (send): owner[a] == R ? mask bits without R : {};
 * mode 1 (recv): owner[a] != R and bit R of mask[a] ? {owner[a]} : {};  mode 2: the mask bits.
 * dynb_csr_plan writes offsets_dev [W+1]; after reading offsets[W] the caller allocates out_dev and
 * calls dynb_csr_fill with the same arguments and workspace (value_map_dev[a] is written instead
 * of a when given). */
int dynb_csr_workspace_bytes(int64_t n, int64_t W, int64_t* bytes);
int dynb_csr_plan(const uint32_t* mask_dev, const int64_t* owner_dev, int64_t n, int64_t R, int mode, int64_t W,
                  int64_t* offsets_dev, void* workspace_dev, int64_t workspace_bytes, void* stream);
int dynb_csr_fill(const uint32_t* mask_dev, const int64_t* owner_dev, int64_t n, int64_t R, int mode, int64_t W,
                  const int64_t* value_map_dev, const int64_t* offsets_dev, int64_t* out_dev,
                  const void* workspace_dev, void* stream);
/* interior_mask[i] = !flags[idx[i]] (build_halo_maps.cpp:138). */
int dynb_gather_not_u8(const uint8_t* flags_dev, const int64_t* idx_dev, int64_t n, uint8_t* out_dev, void* stream);
/* g2l[idx[i]] = i (dist_graph_ops_kernels.cu:143-144). */
int dynb_scatter_iota(const int64_t* idx_dev, int64_t n, int64_t N, int64_t* g2l_dev, uint32_t* bad_dev, void* stream);

/* ------------------------------------------------------------------ edge filter
 * filter_edges_to_radius (dynamis_state/src/csrc/graph/dist_graph_ops.cpp:5-37,
 * dist_graph_ops_kernels.cu:16-43, 62-102): keeps edge e iff
 * |pos[src] + shift @ cell - pos[dst]|^2 <= radius^2 (float32), order preserving.  The plan writes
 * the number kept to count_dev; the fill compacts edges [2,E] -> [2,E_out] and the shift rows of
 * any element size (shift_row_bytes = 3 * element size).  Workspace: dynb_select_workspace_bytes(2*E). */
int dynb_filter_edges_plan(const int64_t* edges_dev, const float* shifts_f32_dev, const float* pos_dev,
                           const float* cell_host, double radius, int64_t E, int64_t* count_dev,
                           void* workspace_dev, int64_t workspace_bytes, void* stream);
int dynb_filter_edges_fill(const int64_t* edges_dev, const void* shifts_raw_dev, int shift_row_bytes, int64_t E,
                           int64_t E_out, int64_t* edges_out_dev, void* shifts_out_dev, const void* workspace_dev,
                           void* stream);

/* ------------------------------------------------------------------ halo exchange
 * Row gather  out[i, :] = input[locs[i], :]  (push_buffer_create,
 * dynamis_model/src/csrc/push_buffer.cu:39-105); rows are row_bytes bytes of any dtype.
 * bad_dev (optional uint32): set non-zero when a loc falls outside [0, n_rows_in); that row is skipped. */
int dynb_pack_rows(const void* input_dev, int64_t n_rows_in, int64_t row_bytes, const int64_t* locs_dev, int64_t n,
                   void* out_dev, uint32_t* bad_dev, void* stream);

/* One peer segment of a push: rows [start, start + count) of the logical send list are stored
 * into remote_ptr (a peer's mapped buffer of remote_rows rows) starting at row remote_row_offset.
 * Same role as the reference's PushTarget (dynamis_model/include/dynamis_model/exchanger.hpp:13-18). */
typedef struct dynb_push_target {
    void* remote_ptr;
    int64_t remote_row_offset;
    int64_t start;
    int64_t count;
    int64_t remote_rows;
} dynb_push_target;

/* Gather + store into peers' memory over NVLink, as a stand-alone launch: IPCExchanger::push_forward /
 * push_backward (gather_and_push_kernel and gather_ghost_grad_and_push_kernel,
 * dynamis_model/src/csrc/exchange/ipc_exchange_kernels.cu:40-122).
 * row_index_dev != NULL: logical row i is x[row_index_dev[i]] (forward push of send_local_indices);
 * NULL: logical row i is x[src_row_base + i] (backward push of the contiguous ghost rows).
 * x has n_rows_in rows.  remote_align: guaranteed byte alignment of every remote row start (16 when the
 * remote buffers and row_bytes are 16-byte multiples).  A row whose source lies outside x or whose
 * destination lies outside the target's remote_rows is skipped and *bad_dev (optional uint32) set. */
int dynb_push_rows(const void* x_dev, int64_t n_rows_in, int64_t row_bytes, const int64_t* row_index_dev,
                   int64_t src_row_base, const dynb_push_target* targets_dev, int n_targets, int64_t total_rows,
                   int remote_align, uint32_t* bad_dev, void* stream);

/* ---- fused halo exchange (FeatureExchanger::feature_push_forward / feature_push_backward,
 * dynamis_model/src/csrc/exchanger.cu:48-120, over IPCExchanger::push_forward / push_backward /
 * record_push_complete / wait_for_pushes, dynamis_model/src/csrc/exchange/ipc_exchanger.cpp:517-828).
 *
 * Every rank owns ONE peer-visible allocation ("exchange allocation") that holds
 *   - result slots [n_local + n_ghost rows] into whose tail the peers store this rank's ghost rows
 *     directly (optional: ring of fwd_ring slots), two staging ghost buffers used when no slot is free,
 *   - two gradient receive buffers [total_send rows] (generation parity),
 *   - handshake records: for each direction (0 forward, 1 reverse, 2 bare handshake), generation
 *     parity and sender a 16-byte record {generation, announced slot, drift word, pad}.
 * A peer only ever receives stores.  Per direction the g-th call of every rank forms generation g; all
 * ranks must issue the same sequence of calls.
 *
 * dynb_halo_peer describes rank k as seen from this rank (entry `rank` itself: remote_base NULL). */
typedef struct dynb_halo_peer {
    void* remote_base;        /* peer's exchange allocation mapped into this process, NULL = not a peer */
    int64_t flags_off;        /* byte offset of the handshake records inside the peer's allocation */
    int64_t fwd_ring_tail;    /* byte offset of the ghost tail of the peer's result slot 0 */
    int64_t fwd_ring_stride;  /* bytes between consecutive result slots of the peer */
    int64_t fwd_stage_off[2]; /* byte offsets of the peer's two staging ghost buffers (generation parity) */
    int64_t fwd_row_offset;   /* first row of this rank's segment inside the peer's ghost region */
    int64_t send_start;       /* segment of this rank's send list that goes to the peer */
    int64_t send_count;
    int64_t bwd_off[2];       /* byte offsets of the peer's two gradient receive buffers */
    int64_t bwd_row_offset;   /* first row of this rank's segment inside the peer's receive buffer */
    int64_t recv_start;       /* segment of this rank's ghost rows owned by the peer */
    int64_t recv_count;
} dynb_halo_peer;

typedef struct dynb_halo_ctx {
    const dynb_halo_peer* peers;  /* device array [world_size] */
    void* local_base;             /* this rank's exchange allocation */
    int64_t local_flags_off;
    uint32_t* done_counter;       /* device word, zero between launches */
    const int32_t* drift_local;   /* device int32 attached to every signal, or NULL (set_watchdog_flags) */
    int32_t* drift_global;        /* device int32 <- OR over all ranks' words after every wait, or NULL */
    uint32_t* status_dev;         /* two device words: [0] 1 + rank whose signal never arrived, [1] bad row index */
    uint32_t* status_host;        /* the same two words in mapped host memory (device address), or NULL */
    int32_t world_size;
    int32_t rank;
} dynb_halo_ctx;

/* Forward, first half (one launch): send-list rows -> peers' ghost regions; x[0:n_local] -> out_head
 * (NULL: no local copy); then the generation signal, carrying announce_slot (0 = "store my next ghost
 * rows into my staging buffer", s + 1 = "into my result slot s") and the drift word.  The destination of
 * this generation's rows is what each peer announced with its previous signal.  flags bit 0: the rows
 * were delivered by other means (copy engine) before this call; only copy and signal.  flags bit 1: walk
 * the send list front to back; by default its block-sized pieces are visited in a scattered order, so that
 * the ranks do not all store into the same peer's segment at the same time. */
int dynb_halo_forward_begin(const dynb_halo_ctx* ctx, const void* x_dev, int64_t n_local, int64_t row_bytes,
                            const int64_t* send_local_dev, int64_t total_send, void* out_head_dev, uint32_t gen,
                            uint32_t announce_slot, int flags, void* stream);
/* Forward, second half (one launch): waits at most timeout_ns for every peer's signal of `gen`, ORs the
 * drift words into drift_global, and copies stage_dev -> out_tail_dev when the rows arrived in staging
 * (out_tail_dev NULL: they are already in place).  On expiry the status words are set and the kernel
 * returns. */
int dynb_halo_forward_end(const dynb_halo_ctx* ctx, uint32_t gen, int64_t timeout_ns, const void* stage_dev,
                          void* out_tail_dev, int64_t tail_bytes, void* stream);
/* Reverse, first half: grad rows [n_local, n_local + n_ghost) -> their owners' receive buffers;
 * grad[0:n_local] -> out (rows with has_recv_dev[row] != 0 may be left to the second half); signal. */
int dynb_halo_backward_begin(const dynb_halo_ctx* ctx, const void* grad_dev, int64_t n_local, int64_t n_ghost,
                             int64_t row_bytes, const uint8_t* has_recv_dev, void* out_dev, uint32_t gen, void* stream);
/* Reverse, second half: bounded wait, drift OR, then out[row] = grad[row] + the received rows naming row
 * (inverse CSR of dynb_inverse_csr, fixed order, no atomics) for the n_rows rows listed in rows_dev.
 * row_first_dev (optional, may be NULL): inv_entries[inv_offsets[rows[r]]] for every listed row r, which
 * shortens the chain of dependent loads in front of the row data. */
int dynb_halo_backward_end(const dynb_halo_ctx* ctx, uint32_t gen, int64_t timeout_ns, const void* grad_dev,
                           const int64_t* rows_dev, const uint32_t* row_first_dev, int64_t n_rows, int64_t feature_dim,
                           int dtype, const void* recv_dev, const int64_t* inv_offsets_dev, const uint32_t* inv_entries_dev,
                           void* out_dev, void* stream);
/* A handshake without rows (record_push_complete / wait_for_pushes as stand-alone calls,
 * ipc_exchanger.cpp:784-828): the signal carries the drift word (flag copied before the counter write,
 * :788-796), the wait ORs all ranks' words into drift_global (watchdog_or_kernel,
 * ipc_exchange_kernels.cu:234-253 — there by remote loads, here from records the peers stored). */
int dynb_halo_signal(const dynb_halo_ctx* ctx, int direction, uint32_t gen, uint32_t announce_slot, void* stream);
int dynb_halo_wait(const dynb_halo_ctx* ctx, int direction, uint32_t gen, int64_t timeout_ns, void* stream);
/* Page-locked host words that kernels can store to (the status words above), and their release. */
int dynb_host_alloc_mapped(int64_t bytes, void** host_ptr_out, void** dev_ptr_out);
int dynb_host_free_mapped(void* host_ptr);

/* Reverse halo: out[i, :] = grad[i, :] + sum of the received rows that name local row i, in fixed
 * peer order (replaces clone + index_add_, dynamis_model/src/csrc/exchanger.cu:111-117, which
 * accumulates with float atomics).  dynb_inverse_csr builds, once per halo plan, for every local
 * row the positions of the send list that name it. */
int dynb_inverse_csr_workspace_bytes(int64_t total_send, int64_t n_local, int64_t* bytes);
int dynb_inverse_csr(const int64_t* send_local_dev, int64_t total_send, int64_t n_local, int64_t* inv_offsets_dev,
                     uint32_t* inv_entries_dev, uint32_t* bad_dev, void* workspace_dev, int64_t workspace_bytes,
                     void* stream);
int dynb_unpack_add_rows(const void* grad_dev, int64_t n_local, int64_t feature_dim, int dtype, const void* recv_dev,
                         const int64_t* inv_offsets_dev, const uint32_t* inv_entries_dev, void* out_dev, void* stream);
/* Peer-visible memory (allocate_ipc_buffer / export_ipc_handle / cudaIpcOpenMemHandle,
 * dynamis_model/src/csrc/exchange/ipc_exchanger.cpp:117-252, 406-430).  These and
 * dynb_host_alloc_mapped are the only calls of the library that allocate, free or map memory;
 * dynb_ipc_alloc zero-fills and synchronises. */
int dynb_ipc_alloc(int64_t bytes, void** ptr_out);
int dynb_ipc_free(void* ptr);
int dynb_ipc_export(void* ptr, uint8_t* handle64_out);
int dynb_ipc_open(const uint8_t* handle64, void** ptr_out);
int dynb_ipc_close(void* ptr);
int dynb_enable_peer_access(int peer_device);
/* Device-to-device copy on the stream (the local rows and ghost rows of the concatenated result), and
 * zero fill (the handshake records when an exchange allocation is kept for a new halo plan). */
int dynb_copy_async(void* dst_dev, const void* src_dev, int64_t bytes, void* stream);
int dynb_fill_zero(void* dst_dev, int64_t bytes, void* stream);

/* ------------------------------------------------------------------ repartition / drift watchdog
 * out[idx[i], :] = rows[i, :] for unique idx: puts rows gathered from all ranks back into canonical
 * atom order (replaces cat + argsort + gather, dynamis/src/dynamis/simulatorState.py:172-183, and the
 * per-rank index_put loop of :238-242).  bad_dev (optional) is set when an index is outside [0, n_out). */
int dynb_scatter_rows(const void* rows_dev, int64_t row_bytes, const int64_t* idx_dev, int64_t n, int64_t n_out,
                      void* out_dev, uint32_t* bad_dev, void* stream);
/* The 2-bit drift word of SimState.write_local_drift_flag (simulatorState.py:257-293) in one kernel:
 * bit 0 when max_i(|x_i - ref_i| + dt (|v_i| + |v_i - vprev_i|)) >= threshold, bit 1 when
 * max_i |x_i - ref_i| > threshold; prev_vel_dev is overwritten with vel_dev.  state_dev: 3 zero-initialised
 * uint32 words owned by the caller (left zero again by every call). */
int dynb_drift_flag(const float* cur_dev, const float* ref_dev, const float* vel_dev, float* prev_vel_dev, int64_t n,
                    double dt, double threshold, uint32_t* state_dev, int32_t* flag_dev, void* stream);

/* ------------------------------------------------------------------ KD-tree partition
 * Replaces kdtree_bisect_cuda (dynamis_state/src/csrc/partition/kdtree.cpp:9-26,
 * kdtree_kernels.cu:264-467): labels_dev[i] in [0, W) by recursive bisection along the widest axis of
 * each segment, ceil(log2 W) levels.  weights_dev: int64 per-atom cost (non-negative) or NULL (equal
 * counts).  Atoms with equal coordinates are ordered by ascending index; weights are summed exactly
 * (the reference uses a float32 cumulative sum, identical while the sums stay below 2^24).
 * method 0: equal-count cuts by selection (no sort), weighted cuts by a stable sort; method 1: sorted
 * cuts for both (same labels; kept so that the two routes can be checked against each other). */
int dynb_kdtree_workspace_bytes(int64_t n_atoms, int64_t W, int64_t* bytes);
int dynb_kdtree_partition(const float* pos_dev, int64_t n_atoms, const int64_t* weights_dev, int64_t W,
                          int64_t* labels_dev, int method, void* workspace_dev, int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ integrator steps
 * Replaces EulerIntegrator::step, VerletIntegrator::halfstep1/2 and LangevinIntegrator::halfstep1/2
 * (dynamis_integrator/src/csrc/euler_integrator.cu:9-75, verlet_integrator.cu:9-116,
 * langevin_integrator.cu:9-150), same per-component arithmetic in float32, in place.
 * kind: 0 Euler step, 1 / 2 Verlet half-steps, 3 / 4 Langevin half-steps (noise_dev, gamma, kT used by
 * 3 and 4 only; pos_dev is not touched by 2 and 4).
 * With drift_flag_dev != NULL (kinds 0, 1, 3) the same launch also produces the drift word of
 * dynb_drift_flag from the new positions and velocities (drift_ref_dev, drift_prev_vel_dev,
 * drift_threshold, drift_state_dev as there), instead of a second pass over the state. */
int dynb_integrator_step(int kind, float* pos_dev, float* vel_dev, const float* frc_dev, const float* mass_dev,
                         const float* noise_dev, int64_t n_atoms, double dt, double gamma, double kT,
                         const float* drift_ref_dev, float* drift_prev_vel_dev, double drift_threshold,
                         uint32_t* drift_state_dev, int32_t* drift_flag_dev, void* stream);

/* ------------------------------------------------------------------ partition without a workspace
 * No counterpart in the reference.  Same result as dynb_sfc_partition, for callers that must not
 * allocate device memory while they run (an engine that gave its whole memory budget to its own
 * pool, a plugin inside another runtime's allocator, a loop that cannot afford the device-wide
 * synchronisation of cudaMalloc): the sort and scan scratch lives in a fixed array inside the
 * library image (6 MiB per GPU that loads the library, held until the process exits) instead of a
 * caller-provided workspace.  Limits and rules:
 *   - n_atoms <= dynb_sfc_static_max_atoms() (131072); larger inputs are rejected with DYNB_ERR_ARG.
 *   - The array is sized for the sorted route of dynb_sfc_partition only, so this entry point always
 *     sorts (also with perm_dev == NULL, where dynb_sfc_partition with its full workspace would select
 *     the split points without a sort); the labels are the same either way.
 *   - The call itself allocates and frees nothing (no cudaMalloc / cudaFree, no allocating library
 *     routine); inputs and outputs are the caller's.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  Make that first call before starting any stream capture.
 *   - All calls on a device share the one array, which still holds the previous call's contents;
 *     nothing in it needs to start at zero (every region is rewritten before it is read).  Two calls
 *     that overlap on the GPU (different streams, or two host threads) race on it: serialise them. */
int64_t dynb_sfc_static_max_atoms(void);
int dynb_sfc_partition_static(const float* pos_dev, int64_t n_atoms, const int64_t* weights_dev, int64_t W,
                              int curve_type, int64_t* labels_dev, int64_t* perm_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DYNB_H */
