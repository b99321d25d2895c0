/*
 * TEST INFRASTRUCTURE ONLY — CPU restatement of the reference radius graph.
 *
 * This header is included twice by rg_oracle.c, once with REAL=float and once
 * with REAL=double.  It restates, expression by expression, the algorithm of
 * dynamis_state/src/csrc/graph/radius_graph_kernels.cu (reference project
 * paths):
 *   - host cell geometry, replication counts, cutoff fractions, cofactor
 *     inverse ............................................. :516-587
 *   - position wrap  pos - floor(pos @ inv) @ cell ......... :596-605
 *   - selective periodic-image predicate and image position  :34-66, :90-134
 *   - accept predicate d2 <= r2 && d2 > 1e-8 ............... :239-253, :396-400
 *   - edge shift  image_shift + floor(frac_tgt) - floor(frac_src)  :293-302
 *   - empty-input conventions ............................... :499-509
 * The cell grid itself does not influence the edge set (any grid whose scan
 * window covers the cutoff gives the same set), so the grid here is the
 * oracle's own.
 *
 * Rounding: the reference is compiled by nvcc with default FMA contraction and
 * calls cuBLAS for the two K=3 matrix products of the wrap.  The explicit
 * FMA() placement below is the contraction nvcc applies to
 * `a*b + c*d + e*f`  ->  fma(e,f, fma(a,b, c*d)),  and the k-sequential FMA
 * chain of an fp32 GEMM  ->  fma(a2,b2, fma(a1,b1, a0*b0)).
 * The float instantiation is pinned against the reference's own CUDA build by
 * the GPU parity tests; the double instantiation has no reference counterpart
 * (the reference rejects float64 input): "parity unpinned" for double.
 *
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may call
 * this code.  The product never does.
 */

#ifndef REAL
#error "include from rg_oracle.c"
#endif

/* contraction of  a*b + c*d + e*f  as emitted by nvcc (-fmad=true) */
static inline REAL FN(dot3_nvcc)(REAL a, REAL b, REAL c, REAL d, REAL e, REAL f)
{
    return FMA(e, f, FMA(a, b, c * d));
}

/* k-sequential FMA chain of a GEMM inner product with K = 3 */
static inline REAL FN(dot3_gemm)(REAL a0, REAL b0, REAL a1, REAL b1, REAL a2, REAL b2)
{
    return FMA(a2, b2, FMA(a1, b1, a0 * b0));
}

typedef struct {
    int rep[3];
    REAL cutoff_frac[3];
    REAL inv[9];
    REAL cell[9];
    int pbc[3];
} FN(geom_t);

/* radius_graph_kernels.cu:516-587 (plain REAL arithmetic, no contraction) */
static void FN(geometry)(const REAL *cell, const uint8_t *pbc, REAL radius, FN(geom_t) *g)
{
    const REAL *a0 = cell, *a1 = cell + 3, *a2 = cell + 6;
    REAL c12[3] = { a1[1] * a2[2] - a1[2] * a2[1], a1[2] * a2[0] - a1[0] * a2[2],
                    a1[0] * a2[1] - a1[1] * a2[0] };
    REAL vol = a0[0] * c12[0] + a0[1] * c12[1] + a0[2] * c12[2];
    REAL abs_vol = FABS(vol);
    REAL c20[3] = { a2[1] * a0[2] - a2[2] * a0[1], a2[2] * a0[0] - a2[0] * a0[2],
                    a2[0] * a0[1] - a2[1] * a0[0] };
    REAL c01[3] = { a0[1] * a1[2] - a0[2] * a1[1], a0[2] * a1[0] - a0[0] * a1[2],
                    a0[0] * a1[1] - a0[1] * a1[0] };
    REAL n12 = SQRT(c12[0] * c12[0] + c12[1] * c12[1] + c12[2] * c12[2]);
    REAL n20 = SQRT(c20[0] * c20[0] + c20[1] * c20[1] + c20[2] * c20[2]);
    REAL n01 = SQRT(c01[0] * c01[0] + c01[1] * c01[1] + c01[2] * c01[2]);
    REAL d_face[3] = { abs_vol / n12, abs_vol / n20, abs_vol / n01 };
    for (int d = 0; d < 3; d++) {
        g->pbc[d] = pbc[d] ? 1 : 0;
        if (pbc[d]) {
            g->rep[d] = (int)CEIL(radius / d_face[d]);
            g->cutoff_frac[d] = radius / d_face[d];
        } else {
            g->rep[d] = 0;
            g->cutoff_frac[d] = (REAL)0;
        }
    }
    REAL inv_vol = (REAL)1 / vol;
    g->inv[0] = (a1[1] * a2[2] - a1[2] * a2[1]) * inv_vol;
    g->inv[1] = (a0[2] * a2[1] - a0[1] * a2[2]) * inv_vol;
    g->inv[2] = (a0[1] * a1[2] - a0[2] * a1[1]) * inv_vol;
    g->inv[3] = (a1[2] * a2[0] - a1[0] * a2[2]) * inv_vol;
    g->inv[4] = (a0[0] * a2[2] - a0[2] * a2[0]) * inv_vol;
    g->inv[5] = (a0[2] * a1[0] - a0[0] * a1[2]) * inv_vol;
    g->inv[6] = (a1[0] * a2[1] - a1[1] * a2[0]) * inv_vol;
    g->inv[7] = (a0[1] * a2[0] - a0[0] * a2[1]) * inv_vol;
    g->inv[8] = (a0[0] * a1[1] - a0[1] * a1[0]) * inv_vol;
    for (int i = 0; i < 9; i++)
        g->cell[i] = cell[i];
}

/* :34-66 — does atom with fractional coords s need the image (dx,dy,dz)? */
static inline int FN(image_needed)(const FN(geom_t) *g, const REAL *s, const int *dd)
{
    for (int d = 0; d < 3; d++) {
        if (!g->pbc[d] && dd[d] != 0)
            return 0;
        if (dd[d] > 0) {
            if (s[d] >= g->cutoff_frac[d])
                return 0;
        } else if (dd[d] < 0) {
            if (s[d] <= (REAL)1 - g->cutoff_frac[d])
                return 0;
        }
    }
    return 1;
}

typedef struct {
    REAL x, y, z;
    int32_t atom;
    int32_t sh[3]; /* image shift minus floor(frac) of the source atom */
} FN(src_t);

orc_graph *FN(orc_radius_graph)(const REAL *pos, int64_t N, const REAL *cell,
                                const uint8_t *pbc, REAL radius, const int64_t *targets,
                                int64_t Nt_in, int nthreads)
{
    const int64_t Nt = targets ? Nt_in : N;
    orc_graph *out = (orc_graph *)calloc(1, sizeof(orc_graph));
    out->Nt = Nt;
    out->counts = (int32_t *)calloc((size_t)(Nt > 0 ? Nt : 1), sizeof(int32_t));
    if (N == 0 || Nt == 0)
        return out;
    if (nthreads > 0)
        omp_set_num_threads(nthreads);

    FN(geom_t) g;
    FN(geometry)(cell, pbc, radius, &g);

    /* wrap (:596-605): two K=3 GEMMs and a subtraction */
    REAL *pw = (REAL *)malloc(sizeof(REAL) * 3 * (size_t)N);
    int32_t *ff = (int32_t *)malloc(sizeof(int32_t) * 3 * (size_t)N);
    int32_t *nimg = (int32_t *)malloc(sizeof(int32_t) * (size_t)N);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < N; i++) {
        REAL px = pos[3 * i], py = pos[3 * i + 1], pz = pos[3 * i + 2];
        REAL f[3], m[3];
        for (int k = 0; k < 3; k++)
            f[k] = FLOOR(FN(dot3_gemm)(px, g.inv[k], py, g.inv[3 + k], pz, g.inv[6 + k]));
        for (int k = 0; k < 3; k++)
            m[k] = FN(dot3_gemm)(f[0], g.cell[k], f[1], g.cell[3 + k], f[2], g.cell[6 + k]);
        pw[3 * i] = px - m[0];
        pw[3 * i + 1] = py - m[1];
        pw[3 * i + 2] = pz - m[2];
        ff[3 * i] = (int32_t)f[0];
        ff[3 * i + 1] = (int32_t)f[1];
        ff[3 * i + 2] = (int32_t)f[2];
        /* image count (:34-66), s from the wrapped position with nvcc's contraction */
        REAL wx = pw[3 * i], wy = pw[3 * i + 1], wz = pw[3 * i + 2];
        REAL s[3];
        for (int k = 0; k < 3; k++)
            s[k] = FN(dot3_nvcc)(wx, g.inv[k], wy, g.inv[3 + k], wz, g.inv[6 + k]);
        int c = 0;
        for (int dx = -g.rep[0]; dx <= g.rep[0]; dx++)
            for (int dy = -g.rep[1]; dy <= g.rep[1]; dy++)
                for (int dz = -g.rep[2]; dz <= g.rep[2]; dz++) {
                    int dd[3] = { dx, dy, dz };
                    c += FN(image_needed)(&g, s, dd);
                }
        nimg[i] = c;
    }
    int64_t *ioff = (int64_t *)malloc(sizeof(int64_t) * ((size_t)N + 1));
    ioff[0] = 0;
    for (int64_t i = 0; i < N; i++)
        ioff[i + 1] = ioff[i] + nimg[i];
    const int64_t M = ioff[N];
    out->M = M;

    /* images (:90-134) */
    FN(src_t) *src = (FN(src_t) *)malloc(sizeof(FN(src_t)) * (size_t)(M > 0 ? M : 1));
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < N; i++) {
        REAL wx = pw[3 * i], wy = pw[3 * i + 1], wz = pw[3 * i + 2];
        REAL s[3];
        for (int k = 0; k < 3; k++)
            s[k] = FN(dot3_nvcc)(wx, g.inv[k], wy, g.inv[3 + k], wz, g.inv[6 + k]);
        int64_t o = ioff[i];
        for (int dx = -g.rep[0]; dx <= g.rep[0]; dx++)
            for (int dy = -g.rep[1]; dy <= g.rep[1]; dy++)
                for (int dz = -g.rep[2]; dz <= g.rep[2]; dz++) {
                    int dd[3] = { dx, dy, dz };
                    if (!FN(image_needed)(&g, s, dd))
                        continue;
                    REAL fx = (REAL)dx, fy = (REAL)dy, fz = (REAL)dz;
                    REAL shx = FN(dot3_nvcc)(fx, g.cell[0], fy, g.cell[3], fz, g.cell[6]);
                    REAL shy = FN(dot3_nvcc)(fx, g.cell[1], fy, g.cell[4], fz, g.cell[7]);
                    REAL shz = FN(dot3_nvcc)(fx, g.cell[2], fy, g.cell[5], fz, g.cell[8]);
                    FN(src_t) *r = &src[o++];
                    r->x = wx + shx;
                    r->y = wy + shy;
                    r->z = wz + shz;
                    r->atom = (int32_t)i;
                    r->sh[0] = dx - ff[3 * i];
                    r->sh[1] = dy - ff[3 * i + 1];
                    r->sh[2] = dz - ff[3 * i + 2];
                }
    }

    /* the oracle's own grid: cells of edge `radius`, 3x3x3 scan window */
    REAL lo[3] = { src[0].x, src[0].y, src[0].z }, hi[3] = { src[0].x, src[0].y, src[0].z };
    for (int64_t j = 0; j < M; j++) {
        REAL p[3] = { src[j].x, src[j].y, src[j].z };
        for (int k = 0; k < 3; k++) {
            if (p[k] < lo[k]) lo[k] = p[k];
            if (p[k] > hi[k]) hi[k] = p[k];
        }
    }
    double res = (double)radius * 1.0001;
    int64_t n[3];
    for (int k = 0; k < 3; k++) {
        n[k] = (int64_t)floor(((double)hi[k] - (double)lo[k]) / res) + 1;
        if (n[k] < 1) n[k] = 1;
    }
    /* keep the grid bounded for sparse clusters in large boxes */
    while ((double)n[0] * (double)n[1] * (double)n[2] > 4.0 * (double)M + 1024.0) {
        res *= 1.5;
        for (int k = 0; k < 3; k++) {
            n[k] = (int64_t)floor(((double)hi[k] - (double)lo[k]) / res) + 1;
            if (n[k] < 1) n[k] = 1;
        }
    }
    const int64_t ncell = n[0] * n[1] * n[2];
#define ORC_CELL_OF(px, py, pz, cx, cy, cz)                              \
    do {                                                                 \
        cx = (int64_t)floor(((double)(px) - (double)lo[0]) / res);       \
        cy = (int64_t)floor(((double)(py) - (double)lo[1]) / res);       \
        cz = (int64_t)floor(((double)(pz) - (double)lo[2]) / res);       \
        if (cx < 0) cx = 0; if (cx >= n[0]) cx = n[0] - 1;               \
        if (cy < 0) cy = 0; if (cy >= n[1]) cy = n[1] - 1;               \
        if (cz < 0) cz = 0; if (cz >= n[2]) cz = n[2] - 1;               \
    } while (0)
    int64_t *cstart = (int64_t *)calloc((size_t)ncell + 1, sizeof(int64_t));
    int64_t *scell = (int64_t *)malloc(sizeof(int64_t) * (size_t)M);
    for (int64_t j = 0; j < M; j++) {
        int64_t cx, cy, cz;
        ORC_CELL_OF(src[j].x, src[j].y, src[j].z, cx, cy, cz);
        scell[j] = cx + n[0] * (cy + n[1] * cz);
        cstart[scell[j] + 1]++;
    }
    for (int64_t c = 0; c < ncell; c++)
        cstart[c + 1] += cstart[c];
    int64_t *cfill = (int64_t *)malloc(sizeof(int64_t) * (size_t)ncell);
    memcpy(cfill, cstart, sizeof(int64_t) * (size_t)ncell);
    int64_t *order = (int64_t *)malloc(sizeof(int64_t) * (size_t)M);
    for (int64_t j = 0; j < M; j++)
        order[cfill[scell[j]]++] = j;

    const REAL r2 = radius * radius;
    const REAL eps = (REAL)1e-8f; /* the literal is a float in both instantiations */

    int64_t *eoff = (int64_t *)malloc(sizeof(int64_t) * ((size_t)Nt + 1));
    for (int pass = 0; pass < 2; pass++) {
        if (pass == 1) {
            eoff[0] = 0;
            for (int64_t t = 0; t < Nt; t++)
                eoff[t + 1] = eoff[t] + out->counts[t];
            out->E = eoff[Nt];
            size_t e = (size_t)(out->E > 0 ? out->E : 1);
            out->src = (int64_t *)malloc(sizeof(int64_t) * e);
            out->dst = (int64_t *)malloc(sizeof(int64_t) * e);
            out->shift = (int32_t *)malloc(sizeof(int32_t) * 3 * e);
            out->d2 = (double *)malloc(sizeof(double) * e);
        }
#pragma omp parallel for schedule(dynamic, 256)
        for (int64_t t = 0; t < Nt; t++) {
            const int64_t a = targets ? targets[t] : t;
            const REAL tx = pw[3 * a], ty = pw[3 * a + 1], tz = pw[3 * a + 2];
            int64_t cx, cy, cz;
            ORC_CELL_OF(tx, ty, tz, cx, cy, cz);
            int64_t w = pass ? eoff[t] : 0;
            int32_t cnt = 0;
            for (int64_t z = (cz > 0 ? cz - 1 : 0); z <= (cz + 1 < n[2] ? cz + 1 : n[2] - 1); z++)
                for (int64_t y = (cy > 0 ? cy - 1 : 0); y <= (cy + 1 < n[1] ? cy + 1 : n[1] - 1); y++) {
                    int64_t x0 = cx > 0 ? cx - 1 : 0, x1 = cx + 1 < n[0] ? cx + 1 : n[0] - 1;
                    int64_t b = cstart[x0 + n[0] * (y + n[1] * z)];
                    int64_t e = cstart[x1 + n[0] * (y + n[1] * z) + 1];
                    for (int64_t q = b; q < e; q++) {
                        const FN(src_t) *s = &src[order[q]];
                        REAL ddx = tx - s->x, ddy = ty - s->y, ddz = tz - s->z;
                        /* (tx-sx)*(tx-sx) + (ty-sy)*(ty-sy) + (tz-sz)*(tz-sz), :399 */
                        REAL d2 = FN(dot3_nvcc)(ddx, ddx, ddy, ddy, ddz, ddz);
                        if (d2 <= r2 && d2 > eps) {
                            if (pass) {
                                out->src[w] = s->atom;
                                out->dst[w] = a;
                                out->shift[3 * w] = s->sh[0] + ff[3 * a];
                                out->shift[3 * w + 1] = s->sh[1] + ff[3 * a + 1];
                                out->shift[3 * w + 2] = s->sh[2] + ff[3 * a + 2];
                                out->d2[w] = (double)d2;
                                w++;
                            }
                            cnt++;
                        }
                    }
                }
            if (!pass)
                out->counts[t] = cnt;
        }
    }
#undef ORC_CELL_OF
    free(eoff); free(order); free(cfill); free(scell); free(cstart);
    free(src); free(ioff); free(nimg); free(ff); free(pw);
    return out;
}
