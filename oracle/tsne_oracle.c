/*
 * CPU restatement (OpenMP C) of the FIt-SNE pipeline that the reference runs on the GPU.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker for the CUDA engine and the timed CPU
 * baseline; no product code path may call it.
 *
 * Parity status: pinned against the reference's own CUDA kernels (compiled for sm_100 from the
 * reference tree, see oracle/ref_build/) through the fixtures under tests/golden/, which were
 * produced by running those kernels on a B200.  The reference ships no golden vectors of its own.
 *
 * Every function cites the reference file:line it restates (paths relative to the reference
 * project root).  Arithmetic is kept in fp32 where the reference's order of operations is
 * deterministic, and accumulated in fp64 where the reference's order is unspecified (atomics,
 * library reductions).
 *
 * Build: see oracle/build.py  (gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_N_BOXES 130          /* src/fit_tsne.cu:246-262: 125 rounded up through the allowed list */
#define ORC_N_INTERP 3           /* src/fit_tsne.cu:247 */
#define ORC_G (ORC_N_BOXES * ORC_N_INTERP) /* 390 interpolation nodes per dimension */
#define ORC_N_TERMS 4            /* src/fit_tsne.cu:252 */
#define ORC_M 1024               /* transform length; any M >= 2*G-1 gives the same linear convolution */

int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------------------ */
/* Exact kNN.  Replaces the FAISS IVF search of src/util/distance_utils.cu:79-121 (FAISS is an
 * external, un-vendored dependency) by the canonical exact search: squared L2 accumulated
 * sequentially over d in fp32, every subtract / multiply / add rounded separately (no FMA),
 * self included, ordered by (distance, index) ascending.                                      */
static inline float canon_dist(const float *a, const float *b, int D)
{
    float acc = 0.0f;
    for (int d = 0; d < D; d++) {
        float t = a[d] - b[d];
        float s = t * t;
        acc = acc + s;
    }
    return acc;
}

/* queries [q_lo, q_hi) against database rows [db_lo, db_hi); ids/d2 are [(q_hi-q_lo)][K].
 * Unfilled slots (database smaller than K) hold id -1 and distance +inf. */
void orc_knn(const float *X, int N, int D, int K, int q_lo, int q_hi, int db_lo, int db_hi,
             int32_t *ids, float *d2)
{
    (void)N;
#pragma omp parallel for schedule(dynamic, 16)
    for (int q = q_lo; q < q_hi; q++) {
        int32_t *oi = ids + (size_t)(q - q_lo) * K;
        float *od = d2 + (size_t)(q - q_lo) * K;
        int cnt = 0;
        const float *xq = X + (size_t)q * D;
        for (int j = db_lo; j < db_hi; j++) {
            float dist = canon_dist(xq, X + (size_t)j * D, D);
            if (cnt == K) {
                /* reject unless (dist, j) < (od[K-1], oi[K-1]) */
                if (dist > od[K - 1] || (dist == od[K - 1] && j > oi[K - 1]))
                    continue;
            }
            int pos = (cnt < K) ? cnt : K - 1;
            while (pos > 0 && (od[pos - 1] > dist || (od[pos - 1] == dist && oi[pos - 1] > j))) {
                od[pos] = od[pos - 1];
                oi[pos] = oi[pos - 1];
                pos--;
            }
            od[pos] = dist;
            oi[pos] = j;
            if (cnt < K) cnt++;
        }
        for (int s = cnt; s < K; s++) { od[s] = INFINITY; oi[s] = -1; }
    }
}

/* Merge `parts` sorted candidate lists per query (each [n][K]) into the best K by (d, id).
 * Host-side model of the multi-GPU merge that follows a database-sharded search. */
void orc_knn_merge(const int32_t *ids_parts, const float *d2_parts, int parts, int n, int K,
                   int32_t *ids, float *d2)
{
#pragma omp parallel for
    for (int q = 0; q < n; q++) {
        int head[64];
        for (int p = 0; p < parts; p++) head[p] = 0;
        for (int s = 0; s < K; s++) {
            int best = -1; float bd = 0; int32_t bi = 0;
            for (int p = 0; p < parts; p++) {
                if (head[p] >= K) continue;
                size_t o = ((size_t)p * n + q) * K + head[p];
                int32_t ci = ids_parts[o]; float cd = d2_parts[o];
                if (ci < 0) continue;
                if (best < 0 || cd < bd || (cd == bd && ci < bi)) { best = p; bd = cd; bi = ci; }
            }
            if (best < 0) { ids[(size_t)q * K + s] = -1; d2[(size_t)q * K + s] = INFINITY; }
            else { ids[(size_t)q * K + s] = bi; d2[(size_t)q * K + s] = bd; head[best]++; }
        }
    }
}

/* src/util/math_utils.cu:66-74 — divide every distance by the global max |d|. Returns the max. */
float orc_max_normalize(float *d2, size_t n)
{
    float m = 0.0f;
    for (size_t i = 0; i < n; i++) { float a = fabsf(d2[i]); if (a > m) m = a; }
    for (size_t i = 0; i < n; i++) d2[i] = d2[i] / m;
    return m;
}

/* src/kernels/perplexity_search.cu:10-141 — per-row bisection on beta.  A row that is found
 * keeps its beta in the reference's lock-step loop, so the per-row early exit is equivalent.
 * The reference evaluates exp/log with the fast device intrinsics; here they are libm's.
 * betas_out may be NULL. */
void orc_perplexity(const float *dhat, int N, int K, float perplexity, float eps, float *p,
                    float *betas_out)
{
    const float log_perp = logf(perplexity);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; i++) {
        const float *d = dhat + (size_t)i * K;
        float *pr = p + (size_t)i * K;
        float beta = 1.0f, lo = -FLT_MAX, hi = FLT_MAX, S = 0.0f;
        for (int it = 0; it < 200; it++) {
            S = 0.0f;
            float ent = 0.0f; /* sum p*log p */
            for (int s = 0; s < K; s++) {
                float v = (s == 0 && d[s] == 0.0f) ? 0.0f : expf(-beta * d[s]);
                pr[s] = v;
                S += v;
                float e = v * logf(v);
                if (e != e || isinf(e)) e = 0.0f; /* thrust_transform_functions.h:32-37 */
                ent += e;
            }
            float neg_ent = -ent;
            float H = (neg_ent / S) + logf(S);
            float diff = H - log_perp;
            int found = (diff < eps && -diff < eps);
            if (found) break;
            if (diff > 0) {
                lo = beta;
                beta = (hi == FLT_MAX || hi == -FLT_MAX) ? beta * 2.0f : (beta + hi) / 2.0f;
            } else {
                hi = beta;
                beta = (lo == -FLT_MAX || lo == FLT_MAX) ? beta / 2.0f : (beta + lo) / 2.0f;
            }
        }
        /* note: after 200 unsuccessful rounds p holds the values of the beta *before* the last
         * update, exactly as in the reference, whose final division uses the last row sums. */
        for (int s = 0; s < K; s++) pr[s] = pr[s] / S;
        if (betas_out) betas_out[i] = beta;
    }
}

/* src/util/math_utils.cu:269-291 — fixed-width "symmetrisation": row i keeps its own K slots and
 * adds p_{j->i} only when i is in the list of j.  Division by 2N is done in double. */
void orc_symmetrize(const float *p, const int32_t *ids, int N, int K, float *P)
{
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; i++) {
        for (int s = 0; s < K; s++) {
            size_t t = (size_t)i * K + s;
            int j = ids[t];
            float acc = p[t];
            const int32_t *rj = ids + (size_t)j * K;
            const float *pj = p + (size_t)j * K;
            for (int u = 0; u < K; u++) acc += (rj[u] == i) ? pj[u] : 0.0f;
            P[t] = (float)(acc / (2.0 * N));
        }
    }
}

/* src/kernels/attr_forces.cu:129-184 — Y is SoA [x(0..N) | y(0..N)], F likewise. Rows [lo,hi). */
void orc_attractive(const float *P, const int32_t *ids, const float *Y, int N, int K, int lo, int hi,
                    float *F)
{
#pragma omp parallel for schedule(static)
    for (int i = lo; i < hi; i++) {
        float ix = Y[i], iy = Y[N + i], ax = 0.0f, ay = 0.0f;
        for (int s = 0; s < K; s++) {
            size_t t = (size_t)i * K + s;
            int j = ids[t];
            float dx = ix - Y[j], dy = iy - Y[N + j];
            float pq = P[t] / (1 + dx * dx + dy * dy);
            ax += pq * dx;
            ay += pq * dy;
        }
        F[i] = ax;
        F[N + i] = ay;
    }
}

/* ------------------------------ FFT (double, radix-2, length ORC_M) ------------------------ */
typedef struct { double re, im; } cplx;

static void fft1d(cplx *a, int n, int inverse, const cplx *tw /* n/2 forward twiddles */)
{
    for (int i = 1, j = 0; i < n; i++) {
        int bit = n >> 1;
        for (; j & bit; bit >>= 1) j ^= bit;
        j ^= bit;
        if (i < j) { cplx t = a[i]; a[i] = a[j]; a[j] = t; }
    }
    for (int len = 2; len <= n; len <<= 1) {
        int step = n / len;
        for (int i = 0; i < n; i += len) {
            for (int k = 0; k < len / 2; k++) {
                cplx w = tw[k * step];
                if (inverse) w.im = -w.im;
                cplx u = a[i + k], v = a[i + k + len / 2];
                cplx vw = { v.re * w.re - v.im * w.im, v.re * w.im + v.im * w.re };
                a[i + k].re = u.re + vw.re; a[i + k].im = u.im + vw.im;
                a[i + k + len / 2].re = u.re - vw.re; a[i + k + len / 2].im = u.im - vw.im;
            }
        }
    }
}

/* 2-D transform of an M x M array with row pruning: only rows [r0, r1) are transformed along the
 * row direction (the others are known to be zero on input, or not needed on output). */
static void fft2d(cplx *a, int inverse, int r0, int r1, const cplx *tw)
{
    const int M = ORC_M;
    if (!inverse) {
#pragma omp parallel for schedule(static)
        for (int r = r0; r < r1; r++) fft1d(a + (size_t)r * M, M, 0, tw);
    }
#pragma omp parallel
    {
        cplx *col = (cplx *)malloc(sizeof(cplx) * M);
#pragma omp for schedule(static)
        for (int c = 0; c < M; c++) {
            for (int r = 0; r < M; r++) col[r] = a[(size_t)r * M + c];
            fft1d(col, M, inverse, tw);
            for (int r = 0; r < M; r++) a[(size_t)r * M + c] = col[r];
        }
        free(col);
    }
    if (inverse) {
#pragma omp parallel for schedule(static)
        for (int r = r0; r < r1; r++) fft1d(a + (size_t)r * M, M, 1, tw);
    }
}

/* Joint min / max over all 2N coordinates (src/fit_tsne.cu:430-432). */
void orc_minmax(const float *Y, int N, float *mn, float *mx)
{
    float a = Y[0], b = Y[0];
    for (int i = 1; i < 2 * N; i++) { if (Y[i] < a) a = Y[i]; if (Y[i] > b) b = Y[i]; }
    *mn = a; *mx = b;
}

/* Per-point box and Lagrange weights: src/kernels/nbodyfft.cu:43-105 with the node positions and
 * denominators of src/fit_tsne.cu:303-323. */
static inline void point_weights(float x, float coord_min, float box_width, const float *sp,
                                 const float *den, int *box, float *L)
{
    int idx = (int)((x - coord_min) / box_width);
    if (idx < 0) idx = 0;
    if (idx > ORC_N_BOXES - 1) idx = ORC_N_BOXES - 1;
    float lb = idx * box_width + coord_min;      /* nbodyfft.cu:222 */
    float xin = (x - lb) / box_width;
    for (int j = 0; j < ORC_N_INTERP; j++) {
        float v = 1;
        for (int k = 0; k < ORC_N_INTERP; k++) if (j != k) v *= xin - sp[k];
        L[j] = v / den[j];
    }
    *box = idx;
}

static void interp_constants(float *sp, float *den)
{
    float h = 1 / (float)ORC_N_INTERP;
    sp[0] = h / 2;
    for (int i = 1; i < ORC_N_INTERP; i++) sp[i] = sp[i - 1] + h;
    for (int i = 0; i < ORC_N_INTERP; i++) {
        den[i] = 1;
        for (int j = 0; j < ORC_N_INTERP; j++) if (i != j) den[i] *= sp[i] - sp[j];
    }
}

/* Spread (nbodyfft.cu:107-139 with the charges of rep_forces.cu:57-76): w is [G][G][4] with the
 * x node index slowest, accumulated in double (the reference's atomic order is unspecified) and
 * rounded to float.  Points [lo,hi) only, so a sharded spread can be modelled. */
void orc_spread(const float *Y, int N, int lo, int hi, float coord_min, float coord_max, float *w)
{
    const int G = ORC_G;
    float sp[ORC_N_INTERP], den[ORC_N_INTERP];
    interp_constants(sp, den);
    float box_width = (coord_max - coord_min) / (float)ORC_N_BOXES;
    double *acc = (double *)calloc((size_t)G * G * 4, sizeof(double));
    for (int i = lo; i < hi; i++) {
        float x = Y[i], y = Y[N + i];
        int bx, by; float Lx[3], Ly[3];
        point_weights(x, coord_min, box_width, sp, den, &bx, Lx);
        point_weights(y, coord_min, box_width, sp, den, &by, Ly);
        float c[4] = { 1, x, y, x * x + y * y };
        for (int a = 0; a < 3; a++)
            for (int b = 0; b < 3; b++) {
                size_t node = (size_t)(bx * 3 + a) * G + (by * 3 + b);
                for (int t = 0; t < 4; t++) acc[node * 4 + t] += (double)(Lx[a] * Ly[b] * c[t]);
            }
    }
    for (size_t k = 0; k < (size_t)G * G * 4; k++) w[k] = (float)acc[k];
    free(acc);
}

/* Convolution of the node charges with the squared-Cauchy kernel:
 * nbodyfft.cu:175-203 (kernel values, evaluated in double from float node coordinates and mirrored
 * around index G of the zero-padded array), :3-41 and :395-424 (zero-padded transform, product,
 * inverse, read-back of the [G,2G)^2 quadrant).  The reference uses a 780-point cuFFT in fp32;
 * this uses a 1024-point transform in fp64: the linear convolution is the same for any length
 * >= 779.  ytilde is [G][G][4]. */
void orc_convolve(const float *w, float coord_min, float coord_max, float *ytilde)
{
    const int G = ORC_G, M = ORC_M;
    float box_width = (coord_max - coord_min) / (float)ORC_N_BOXES;
    float h = box_width / (float)ORC_N_INTERP;
    float x_min = coord_min, y_min = coord_min;
    cplx *tw = (cplx *)malloc(sizeof(cplx) * M / 2);
    for (int k = 0; k < M / 2; k++) { tw[k].re = cos(-2.0 * M_PI * k / M); tw[k].im = sin(-2.0 * M_PI * k / M); }
    cplx *kt = (cplx *)calloc((size_t)M * M, sizeof(cplx));
    cplx *s0 = (cplx *)calloc((size_t)M * M, sizeof(cplx));
    cplx *s1 = (cplx *)calloc((size_t)M * M, sizeof(cplx));
#pragma omp parallel for schedule(static)
    for (int i = 0; i < G; i++)
        for (int j = 0; j < G; j++) {
            float x1 = y_min + h / 2, x2 = x_min + h / 2;
            float y1 = y_min + h / 2 + i * h, y2 = x_min + h / 2 + j * h;
            float d1 = x1 - y1, d2 = x2 - y2;
            double v = pow(1.0 + (double)(d1 * d1) + (double)(d2 * d2), -2);
            float tmp = (float)v;
            kt[(size_t)(G + i) * M + (G + j)].re = tmp;
            kt[(size_t)(G - i) * M + (G + j)].re = tmp;
            kt[(size_t)(G + i) * M + (G - j)].re = tmp;
            kt[(size_t)(G - i) * M + (G - j)].re = tmp;
        }
    for (int i = 0; i < G; i++)
        for (int j = 0; j < G; j++) {
            const float *c = w + ((size_t)i * G + j) * 4;
            s0[(size_t)i * M + j].re = c[0]; s0[(size_t)i * M + j].im = c[1];
            s1[(size_t)i * M + j].re = c[2]; s1[(size_t)i * M + j].im = c[3];
        }
    fft2d(kt, 0, 0, M, tw);
    fft2d(s0, 0, 0, G, tw);
    fft2d(s1, 0, 0, G, tw);
#pragma omp parallel for schedule(static)
    for (size_t k = 0; k < (size_t)M * M; k++) {
        cplx a = s0[k], b = s1[k], c = kt[k];
        s0[k].re = a.re * c.re - a.im * c.im; s0[k].im = a.re * c.im + a.im * c.re;
        s1[k].re = b.re * c.re - b.im * c.im; s1[k].im = b.re * c.im + b.im * c.re;
    }
    fft2d(s0, 1, G, 2 * G, tw);
    fft2d(s1, 1, G, 2 * G, tw);
    const double scale = 1.0 / ((double)M * M);
    for (int i = 0; i < G; i++)
        for (int j = 0; j < G; j++) {
            float *o = ytilde + ((size_t)i * G + j) * 4;
            size_t k = (size_t)(G + i) * M + (G + j);
            o[0] = (float)(s0[k].re * scale); o[1] = (float)(s0[k].im * scale);
            o[2] = (float)(s1[k].re * scale); o[3] = (float)(s1[k].im * scale);
        }
    free(tw); free(kt); free(s0); free(s1);
}

/* Gather (nbodyfft.cu:141-173), normalisation terms and repulsive force (rep_forces.cu:3-31).
 * Returns sum_i Z_i over points [lo,hi) in double (rep_forces.cu:51-54 subtracts N afterwards).
 * Frep is SoA [2][N]; phi (may be NULL) is [N][4]. */
double orc_gather(const float *Y, int N, int lo, int hi, float coord_min, float coord_max,
                  const float *ytilde, float *Frep, float *phi_out)
{
    const int G = ORC_G;
    float sp[ORC_N_INTERP], den[ORC_N_INTERP];
    interp_constants(sp, den);
    float box_width = (coord_max - coord_min) / (float)ORC_N_BOXES;
    double zsum = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : zsum)
    for (int i = lo; i < hi; i++) {
        float x = Y[i], y = Y[N + i];
        int bx, by; float Lx[3], Ly[3];
        point_weights(x, coord_min, box_width, sp, den, &bx, Lx);
        point_weights(y, coord_min, box_width, sp, den, &by, Ly);
        double phi[4] = { 0, 0, 0, 0 };
        for (int a = 0; a < 3; a++)
            for (int b = 0; b < 3; b++) {
                size_t node = (size_t)(bx * 3 + a) * G + (by * 3 + b);
                for (int t = 0; t < 4; t++) phi[t] += (double)(Lx[a] * Ly[b] * ytilde[node * 4 + t]);
            }
        float p1 = (float)phi[0], p2 = (float)phi[1], p3 = (float)phi[2], p4 = (float)phi[3];
        if (phi_out) { phi_out[4 * (size_t)i] = p1; phi_out[4 * (size_t)i + 1] = p2; phi_out[4 * (size_t)i + 2] = p3; phi_out[4 * (size_t)i + 3] = p4; }
        float zi = (1 + x * x + y * y) * p1 - 2 * (x * p2 + y * p3) + p4;
        zsum += (double)zi;
        Frep[i] = x * p1 - p2;
        Frep[N + i] = y * p1 - p3;
    }
    return zsum;
}

/* One complete repulsive evaluation as in one iteration of src/fit_tsne.cu:425-469.
 * Z_out = sum Z_i - N.  w_out / ytilde_out / phi_out may be NULL. */
void orc_repulsive(const float *Y, int N, float *Frep, float *Z_out, float *w_out, float *ytilde_out,
                   float *phi_out)
{
    const size_t gs = (size_t)ORC_G * ORC_G * 4;
    float mn, mx;
    orc_minmax(Y, N, &mn, &mx);
    float *w = w_out ? w_out : (float *)malloc(gs * sizeof(float));
    float *yt = ytilde_out ? ytilde_out : (float *)malloc(gs * sizeof(float));
    orc_spread(Y, N, 0, N, mn, mx, w);
    orc_convolve(w, mn, mx, yt);
    double zs = orc_gather(Y, N, 0, N, mn, mx, yt, Frep, phi_out);
    *Z_out = (float)zs - (float)N;
    if (!w_out) free(w);
    if (!ytilde_out) free(yt);
}

/* Exact O(N^2) evaluation of the same quantities in double (independent of the grid): checks the
 * interpolation scheme itself.  F_i = sum_j (y_i-y_j)/(1+d^2)^2 ; Z = sum_{i != j} 1/(1+d^2). */
void orc_repulsive_exact(const float *Y, int N, double *Frep, double *Z_out)
{
    double z = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : z)
    for (int i = 0; i < N; i++) {
        double fx = 0, fy = 0, xi = Y[i], yi = Y[N + i];
        for (int j = 0; j < N; j++) {
            if (j == i) continue;
            double dx = xi - Y[j], dy = yi - Y[N + j];
            double q = 1.0 / (1.0 + dx * dx + dy * dy);
            z += q;
            fx += q * q * dx;
            fy += q * q * dy;
        }
        Frep[i] = fx; Frep[N + i] = fy;
    }
    *Z_out = z;
}

/* src/kernels/apply_forces.cu:11-57 — gradient (no factor 4), gains (+0.2 / *0.8 evaluated in
 * double, floor 0.01), momentum, position update; the force arrays are zeroed afterwards. */
void orc_apply_forces(float *Y, float *attr, float *rep, float *gains, float *old_forces, float eta,
                      float normalization, float momentum, float exaggeration, int N)
{
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; i++) {
        float ux = old_forces[i], uy = old_forces[N + i];
        float gx = gains[i], gy = gains[N + i];
        float dx = exaggeration * attr[i] - (rep[i] / normalization);
        float dy = exaggeration * attr[i + N] - (rep[i + N] / normalization);
        gx = (float)((signbit(dx) != signbit(ux)) ? gx + 0.2 : gx * 0.8);
        gy = (float)((signbit(dy) != signbit(uy)) ? gy + 0.2 : gy * 0.8);
        gx = (gx < 0.01) ? (float)0.01 : gx;
        gy = (gy < 0.01) ? (float)0.01 : gy;
        ux = momentum * ux - eta * gx * dx;
        uy = momentum * uy - eta * gy * dy;
        Y[i] += ux; Y[i + N] += uy;
        attr[i] = 0.0f; attr[N + i] = 0.0f; rep[i] = 0.0f; rep[N + i] = 0.0f;
        old_forces[i] = ux; old_forces[N + i] = uy;
        gains[i] = gx; gains[N + i] = gy;
    }
}

/* The iteration loop of src/fit_tsne.cu:402-580 on a given P / ids / Y (in place).
 * gains / old_forces are [2][N] state (gains start at 1, old_forces at 0: fit_tsne.cu:163-164).
 * `first_step` lets a caller continue a run; Z of the last iteration is returned. */
float orc_iterate(const float *P, const int32_t *ids, float *Y, float *gains, float *old_forces, int N,
                  int K, int first_step, int n_steps, float eta, float early_exaggeration,
                  int force_magnify_iters, float pre_momentum, float post_momentum)
{
    float *attr = (float *)calloc((size_t)2 * N, sizeof(float));
    float *rep = (float *)calloc((size_t)2 * N, sizeof(float));
    float Z = 0.0f;
    for (int step = first_step; step < first_step + n_steps; step++) {
        float momentum = (step >= force_magnify_iters) ? post_momentum : pre_momentum;
        float exag = (step >= force_magnify_iters) ? 1.0f : early_exaggeration;
        orc_repulsive(Y, N, rep, &Z, NULL, NULL, NULL);
        orc_attractive(P, ids, Y, N, K, 0, N, attr);
        orc_apply_forces(Y, attr, rep, gains, old_forces, eta, Z, momentum, exag, N);
    }
    free(attr); free(rep);
    return Z;
}

/* Set-up of src/fit_tsne.cu:84-153 from X to the fixed-width P: exact kNN, global max
 * normalisation, perplexity search, symmetrisation.  ids/P are [N][K]. */
void orc_affinities(const float *X, int N, int D, int K, float perplexity, float eps, int32_t *ids,
                    float *P)
{
    float *d2 = (float *)malloc(sizeof(float) * (size_t)N * K);
    float *p = (float *)malloc(sizeof(float) * (size_t)N * K);
    orc_knn(X, N, D, K, 0, N, 0, N, ids, d2);
    orc_max_normalize(d2, (size_t)N * K);
    orc_perplexity(d2, N, K, perplexity, eps, p, NULL);
    orc_symmetrize(p, ids, N, K, P);
    free(d2); free(p);
}

/* ------------------------------- quality evaluators (not in the reference) ----------------- */
/* KL(P || Q) over the stored entries of the fixed-width P, Q_ij = (1+d^2)^-1 / Z with the exact
 * Z = sum_{k != l} (1+d_kl^2)^-1.  P is renormalised to sum 1 over its stored entries. */
double orc_kl_divergence(const float *P, const int32_t *ids, const float *Y, int N, int K)
{
    double Z = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : Z)
    for (int i = 0; i < N; i++) {
        double xi = Y[i], yi = Y[N + i];
        for (int j = 0; j < N; j++) {
            if (j == i) continue;
            double dx = xi - Y[j], dy = yi - Y[N + j];
            Z += 1.0 / (1.0 + dx * dx + dy * dy);
        }
    }
    double ps = 0.0;
    for (size_t t = 0; t < (size_t)N * K; t++) ps += P[t];
    double kl = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : kl)
    for (int i = 0; i < N; i++)
        for (int s = 0; s < K; s++) {
            size_t t = (size_t)i * K + s;
            double pv = P[t] / ps;
            int j = ids[t];
            if (pv <= 0.0 || j == i) continue;
            double dx = (double)Y[i] - Y[j], dy = (double)Y[N + i] - Y[N + j];
            double q = (1.0 / (1.0 + dx * dx + dy * dy)) / Z;
            kl += pv * log(pv / q);
        }
    return kl;
}

/* Mean fraction of each point's k nearest high-dimensional neighbours (ids_hi, [N][K_hi], slot 0
 * is the point itself) that are among its k nearest neighbours in the embedding. */
double orc_nn_preservation(const int32_t *ids_hi, int K_hi, const float *Y, int N, int k)
{
    double total = 0.0;
#pragma omp parallel for schedule(dynamic, 16) reduction(+ : total)
    for (int i = 0; i < N; i++) {
        int32_t best_i[64]; double best_d[64]; int cnt = 0;
        double xi = Y[i], yi = Y[N + i];
        for (int j = 0; j < N; j++) {
            if (j == i) continue;
            double dx = xi - Y[j], dy = yi - Y[N + j];
            double d = dx * dx + dy * dy;
            if (cnt == k && d >= best_d[k - 1]) continue;
            int pos = (cnt < k) ? cnt : k - 1;
            while (pos > 0 && best_d[pos - 1] > d) { best_d[pos] = best_d[pos - 1]; best_i[pos] = best_i[pos - 1]; pos--; }
            best_d[pos] = d; best_i[pos] = j;
            if (cnt < k) cnt++;
        }
        int hit = 0, seen = 0;
        for (int s = 0; s < K_hi && seen < k; s++) {
            int j = ids_hi[(size_t)i * K_hi + s];
            if (j == i) continue;
            seen++;
            for (int u = 0; u < cnt; u++) if (best_i[u] == j) { hit++; break; }
        }
        total += (double)hit / (double)k;
    }
    return total / N;
}
