/*
 * TEST INFRASTRUCTURE ONLY — CPU oracle for the periodic radius graph.
 *
 * Plain C (OpenMP over targets).  The algorithm text lives in
 * rg_oracle_impl.h, instantiated here for float (pinned against the
 * reference's CUDA build by the GPU parity tests) and double ("parity
 * unpinned": the reference has no float64 path).
 *
 * Build:  make -C oracle      (gcc -O2 -fopenmp -ffp-contract=off -mfma)
 * -ffp-contract=off is required: every fused multiply-add must be one of the
 * explicit FMA() calls, never the compiler's choice.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int64_t E;       /* number of directed edges */
    int64_t Nt;      /* number of target entries */
    int64_t M;       /* number of source images (atoms + periodic copies) */
    int64_t *src;    /* [E] neighbour atom id (edge_index row 0) */
    int64_t *dst;    /* [E] centre atom id   (edge_index row 1) */
    int32_t *shift;  /* [E,3] integer cell shift: pos[src] + shift@cell - pos[dst] */
    int32_t *counts; /* [Nt] degree per target entry, caller order */
    double *d2;      /* [E] squared distance as the kernel arithmetic produced it */
} orc_graph;

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define REAL float
#define FN(name) CAT(name, _f32)
#define FMA(a, b, c) fmaf((a), (b), (c))
#define FLOOR(x) floorf(x)
#define CEIL(x) ceilf(x)
#define SQRT(x) sqrtf(x)
#define FABS(x) fabsf(x)
#include "rg_oracle_impl.h"
#undef REAL
#undef FN
#undef FMA
#undef FLOOR
#undef CEIL
#undef SQRT
#undef FABS

#define REAL double
#define FN(name) CAT(name, _f64)
#define FMA(a, b, c) fma((a), (b), (c))
#define FLOOR(x) floor(x)
#define CEIL(x) ceil(x)
#define SQRT(x) sqrt(x)
#define FABS(x) fabs(x)
#include "rg_oracle_impl.h"

void orc_graph_free(orc_graph *g)
{
    if (!g)
        return;
    free(g->src);
    free(g->dst);
    free(g->shift);
    free(g->counts);
    free(g->d2);
    free(g);
}

int orc_max_threads(void) { return omp_get_max_threads(); }

/* Geometry alone, for host-logic tests: rep[3], cutoff_frac[3], inv[9]. */
void orc_geometry_f32(const float *cell, const uint8_t *pbc, float radius, int *rep,
                      float *cutoff_frac, float *inv)
{
    geom_t_f32 g;
    geometry_f32(cell, pbc, radius, &g);
    for (int d = 0; d < 3; d++) {
        rep[d] = g.rep[d];
        cutoff_frac[d] = g.cutoff_frac[d];
    }
    for (int i = 0; i < 9; i++)
        inv[i] = g.inv[i];
}

/*
 * filter_edges_to_radius restated (dynamis_state/src/csrc/graph/
 * dist_graph_ops_kernels.cu:16-43): keep[e] = |pos[src] + shift@cell - pos[dst]|^2 <= r2,
 * float arithmetic with nvcc's contraction of the two three-term sums.
 */
void orc_edge_keep_mask_f32(const int64_t *src, const int64_t *dst, const float *shifts,
                            const float *pos, const float *cell, float r2, int64_t E,
                            uint8_t *keep)
{
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < E; e++) {
        const int64_t s = src[e], d = dst[e];
        float sx = pos[3 * s], sy = pos[3 * s + 1], sz = pos[3 * s + 2];
        const float dx = pos[3 * d], dy = pos[3 * d + 1], dz = pos[3 * d + 2];
        const float h0 = shifts[3 * e], h1 = shifts[3 * e + 1], h2 = shifts[3 * e + 2];
        sx = sx + dot3_nvcc_f32(h0, cell[0], h1, cell[3], h2, cell[6]);
        sy = sy + dot3_nvcc_f32(h0, cell[1], h1, cell[4], h2, cell[7]);
        sz = sz + dot3_nvcc_f32(h0, cell[2], h1, cell[5], h2, cell[8]);
        const float ax = sx - dx, ay = sy - dy, az = sz - dz;
        keep[e] = dot3_nvcc_f32(ax, ax, ay, ay, az, az) <= r2;
    }
}
