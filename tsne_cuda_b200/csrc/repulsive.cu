// FIt-SNE repulsive force: spread of the point charges onto the 390x390 Lagrange grid, convolution
// of the grid with the squared-Cauchy kernel, interpolation back, normalisation terms.
//
// Reference: src/kernels/nbodyfft.cu (binning :43-73, Lagrange weights :75-105, spread :107-139,
// kernel evaluation :175-203, FFT convolution :3-41 + :395-424, gather :141-173) and
// src/kernels/rep_forces.cu (charges :57-76, forces and Z_i :3-31), sequenced as in
// src/fit_tsne.cu:411-469.
//
// Design (nothing here is a translation of the reference's kernels):
//  * One kernel per point pass.  Box index, in-box coordinate, Lagrange weights and charges are
//    recomputed in registers by spread and gather; the reference's nine N-sized intermediate
//    arrays do not exist.  The grid is AoS float4 per node, stored as (x-charge, y-charge, count,
//    r^2-charge) = two packed complex numbers, so a point issues 9 vector reductions instead of 36
//    scalar atomics.  The pairing is deliberate: a complex FFT leaks rounding error of the larger
//    component into the smaller one, so the x and y charges (same magnitude) share one plane and the
//    r^2 charge is multiplied by a power of two that brings it to the magnitude of the counts before
//    it shares the other (scaling by a power of two is exact and is undone on the way out).
//  * The convolution is a hand-written zero-padded 1024x1024 FFT (any length >= 779 gives the same
//    linear convolution as the reference's 780) in three kernels: forward row pass, fused column
//    pass (forward FFT, product with the kernel spectrum, inverse FFT, never leaving the SM), inverse
//    row pass.  The four real charge grids travel as two complex planes; convolving with a real
//    kernel acts on real and imaginary parts independently, so nothing is ever unpacked.
//    The kernel is placed around index 0 instead of index G: its spectrum is then real (a cosine
//    transform of one quadrant), is produced by the same two passes as a third plane and the
//    result appears in the [0,G)^2 corner.  Only the G non-zero input rows and the G needed output
//    rows are transformed.
//  * A 1024-point FFT is done by one warp: 32 points per lane in registers (radix-32 as five
//    unrolled radix-2 stages), one transposition through shared memory, 32 points per lane again.
#include "common.cuh"

#include <algorithm>

namespace b200 {

InterpConsts make_interp_consts()
{
    InterpConsts c;
    float h = 1 / (float)kInterp;
    c.sp[0] = h / 2;
    for (int i = 1; i < kInterp; i++) c.sp[i] = c.sp[i - 1] + h;
    for (int i = 0; i < kInterp; i++) {
        c.den[i] = 1;
        for (int j = 0; j < kInterp; j++)
            if (i != j) c.den[i] *= c.sp[i] - c.sp[j];
    }
    return c;
}

namespace {

// ------------------------------------------------------------------------------------------
// per-point geometry shared by spread and gather
// ------------------------------------------------------------------------------------------
struct GridGeom {
    float cmin, box_width;
    float r2_scale, r2_unscale;   // powers of two: r2_scale * max possible (x^2+y^2) lies in [4, 8)
};

__device__ __forceinline__ GridGeom load_geom(const IterState *state, int slot)
{
    GridGeom g;
    const float cmin = dec_float(state->min_enc[slot]);
    const float cmax = dec_float(state->max_enc[slot]);
    g.cmin = cmin;
    g.box_width = (cmax - cmin) / (float)kBoxes;
    // All points identical: the reference divides by zero here.  Use a tiny positive width so that
    // every point falls in box 0 with in-box coordinate 0 and all results stay finite.
    if (!(g.box_width > 0.0f)) g.box_width = 1e-30f;
    const float r = fmaxf(fabsf(cmin), fabsf(cmax));
    const float r2max = 2.0f * r * r;
    int e = 0;
    if (r2max > 0.0f && r2max < INFINITY) e = min(100, max(-100, 2 - ilogbf(r2max)));
    g.r2_scale = scalbnf(1.0f, e);
    g.r2_unscale = scalbnf(1.0f, -e);
    return g;
}

__device__ __forceinline__ void axis_weights(float c, const GridGeom &g, const InterpConsts &ic, int &box, float (&L)[kInterp])
{
    int idx = (int)((c - g.cmin) / g.box_width);
    idx = max(0, idx);
    idx = min(kBoxes - 1, idx);
    const float lower = idx * g.box_width + g.cmin;
    const float in_box = (c - lower) / g.box_width;
#pragma unroll
    for (int j = 0; j < kInterp; j++) {
        float v = 1;
#pragma unroll
        for (int k = 0; k < kInterp; k++)
            if (j != k) v *= in_box - ic.sp[k];
        L[j] = v / ic.den[j];
    }
    box = idx;
}

// ------------------------------------------------------------------------------------------
// min / max of the embedding into a state slot (start-up and after an exchange of Y)
// ------------------------------------------------------------------------------------------
__global__ void state_reset_kernel(IterState *state, int slot, int all)
{
    state->min_enc[slot] = 0xffffffffu;
    state->max_enc[slot] = 0u;
    if (all) {
        state->min_enc[slot ^ 1] = 0xffffffffu;
        state->max_enc[slot ^ 1] = 0u;
        state->zsum[0] = 0.0;
        state->zsum[1] = 0.0;
        state->unorm2 = 0.0;
        state->bad = 0;
    }
}

__global__ void __launch_bounds__(256) minmax_kernel(const float2 *__restrict__ Y2, long long N, IterState *state, int slot)
{
    float mn = INFINITY, mx = -INFINITY;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (long long)gridDim.x * blockDim.x) {
        const float2 y = Y2[i];
        mn = fminf(mn, fminf(y.x, y.y));
        mx = fmaxf(mx, fmaxf(y.x, y.y));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0 && mn <= mx) {
        atomicMin(&state->min_enc[slot], enc_float(mn));
        atomicMax(&state->max_enc[slot], enc_float(mx));
    }
}

// ------------------------------------------------------------------------------------------
// spread
// ------------------------------------------------------------------------------------------
// Same-address floating-point reductions serialise in L2, and an embedding is anything but uniform
// over its bounding square (during early exaggeration half the points sit in a few hundred boxes).
// So the spread walks the points in an order that is sorted by box (refreshed every few iterations
// by a counting sort; a stale order only costs efficiency, never correctness, because the box of
// every point is recomputed here): lanes that fall into the same box are neighbours in the warp,
// their 36 contributions are combined with a segmented shuffle reduction, and only the first lane of
// each run issues the nine vector reductions.
__device__ __forceinline__ int axis_box(float c, const GridGeom &g)
{
    int idx = (int)((c - g.cmin) / g.box_width);
    idx = max(0, idx);
    return min(kBoxes - 1, idx);
}

// A lane takes kSpreadPerLane consecutive points of the order.  While they stay in one box it sums their 36
// contributions in registers; a box change inside the lane sends the finished sum to the grid directly.  The
// lane's last (open) run is then combined with those of its neighbours as described above, so the 180
// shuffles of the segmented reduction are paid once per 32 * kSpreadPerLane points.
constexpr int kSpreadPerLane = 4;

__device__ __forceinline__ void spread_flush(float4 *__restrict__ w, int bx, int by, const float (&v)[kInterp][kInterp][4])
{
#pragma unroll
    for (int a = 0; a < kInterp; a++)
#pragma unroll
        for (int b = 0; b < kInterp; b++) {
            float4 *dst = w + (size_t)(bx * kInterp + a) * kG + (by * kInterp + b);
            atomicAdd(dst, make_float4(v[a][b][0], v[a][b][1], v[a][b][2], v[a][b][3]));
        }
}

__global__ void __launch_bounds__(256)
spread_kernel(const float2 *__restrict__ Y2, long long row_lo, long long n_rows, const int32_t *__restrict__ order,
              const IterState *state, int slot, InterpConsts ic, float4 *__restrict__ w)
{
    const long long t0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * kSpreadPerLane;
    const int lane = threadIdx.x & 31;
    const GridGeom g = load_geom(state, slot);
    int key = -1, bx = 0, by = 0;
    float v[kInterp][kInterp][4];
#pragma unroll
    for (int a = 0; a < kInterp; a++)
#pragma unroll
        for (int b = 0; b < kInterp; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) v[a][b][c] = 0.0f;
    // all loads of the lane first: they are independent of each other
    float2 ys[kSpreadPerLane];
#pragma unroll
    for (int p = 0; p < kSpreadPerLane; p++) {
        const long long t = t0 + p;
        if (t < n_rows) {
            const long long r = order ? (long long)order[t] : t;
            ys[p] = Y2[row_lo + r];
        }
    }
#pragma unroll
    for (int p = 0; p < kSpreadPerLane; p++) {
        if (t0 + p >= n_rows) break;
        const float2 y = ys[p];
        int kx, ky;
        float Lx[kInterp], Ly[kInterp];
        axis_weights(y.x, g, ic, kx, Lx);
        axis_weights(y.y, g, ic, ky, Ly);
        const int k = ky * kBoxes + kx;
        if (k != key && key >= 0) {
            spread_flush(w, bx, by, v);
#pragma unroll
            for (int a = 0; a < kInterp; a++)
#pragma unroll
                for (int b = 0; b < kInterp; b++)
#pragma unroll
                    for (int c = 0; c < 4; c++) v[a][b][c] = 0.0f;
        }
        key = k; bx = kx; by = ky;
        const float c3 = y.x * y.x + y.y * y.y;
#pragma unroll
        for (int a = 0; a < kInterp; a++)
#pragma unroll
            for (int b = 0; b < kInterp; b++) {
                const float l = Lx[a] * Ly[b];
                v[a][b][0] += l * y.x; v[a][b][1] += l * y.y; v[a][b][2] += l; v[a][b][3] += l * c3;  // (x, y, count, r^2)
            }
    }
    // runs of equal keys among neighbouring lanes (their open runs)
    const int prev = __shfl_up_sync(0xffffffffu, key, 1);
    const bool head = (lane == 0) || (key != prev);
    const unsigned heads = __ballot_sync(0xffffffffu, head);
    const unsigned above = (lane == 31) ? 0u : (heads & (0xffffffffu << (lane + 1)));
    const int run_end = above ? (__ffs(above) - 2) : 31;   // last lane of this lane's run
    if (heads != 0xffffffffu) {                             // at least one run longer than one lane
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const bool take = lane + d <= run_end;
#pragma unroll
            for (int a = 0; a < kInterp; a++)
#pragma unroll
                for (int b = 0; b < kInterp; b++)
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const float o = __shfl_down_sync(0xffffffffu, v[a][b][c], d);
                        if (take) v[a][b][c] += o;
                    }
        }
    }
    if (head && key >= 0) spread_flush(w, bx, by, v);
}

// ---- counting sort of the owned points by box (order[t] = local row index) ----
__global__ void order_identity_kernel(int32_t *order, long long n)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) order[t] = (int32_t)t;
}

// Both passes of the counting sort give a thread kOrderPerThread consecutive entries of the previous order,
// so that it has that many independent loads and atomics in flight (a pass is a chain of dependent L2
// round trips).  Atomics are combined across the warp: for each of its entries in turn, the lanes that
// hold the same key elect a leader that adds their number.  The points of a box are (nearly) contiguous in
// the previous order, so a warp sees few distinct keys.
constexpr int kOrderPerThread = 4;

__device__ __forceinline__ int point_key(const float2 *__restrict__ Y2, long long row, const GridGeom &g)
{
    const float2 y = Y2[row];
    return axis_box(y.y, g) * kBoxes + axis_box(y.x, g);
}

// keys[t] = box of point order[t]; hist[box] += 1
__global__ void __launch_bounds__(256)
order_histogram_kernel(const float2 *__restrict__ Y2, long long row_lo, long long n_rows, const int32_t *__restrict__ order,
                       const IterState *state, int slot, int32_t *__restrict__ keys, int32_t *__restrict__ hist)
{
    const long long t0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * kOrderPerThread;
    const int lane = threadIdx.x & 31;
    const GridGeom g = load_geom(state, slot);
    int k[kOrderPerThread] = {-1, -1, -1, -1};
    if (t0 + kOrderPerThread <= n_rows) {
        const int4 o = *reinterpret_cast<const int4 *>(order + t0);
        k[0] = point_key(Y2, row_lo + o.x, g);
        k[1] = point_key(Y2, row_lo + o.y, g);
        k[2] = point_key(Y2, row_lo + o.z, g);
        k[3] = point_key(Y2, row_lo + o.w, g);
        *reinterpret_cast<int4 *>(keys + t0) = make_int4(k[0], k[1], k[2], k[3]);
    } else {
#pragma unroll
        for (int p = 0; p < kOrderPerThread; p++)
            if (t0 + p < n_rows) {
                k[p] = point_key(Y2, row_lo + order[t0 + p], g);
                keys[t0 + p] = k[p];
            }
    }
#pragma unroll
    for (int p = 0; p < kOrderPerThread; p++) {
        const unsigned same = __match_any_sync(0xffffffffu, k[p]);
        if (k[p] >= 0 && lane == __ffs(same) - 1) atomicAdd(hist + k[p], __popc(same));
    }
}

// exclusive scan of the kBoxes^2 counters in place: one block, warp w owns the contiguous bins
// [w * kPerWarp, (w + 1) * kPerWarp) and walks them 32 at a time (coalesced), carrying its running total;
// one pass over the 32 warp totals gives every warp its offset
__global__ void __launch_bounds__(1024) order_scan_kernel(int32_t *hist)
{
    constexpr int kBins = kBoxes * kBoxes;
    constexpr int kPerWarp = (kBins + 31) / 32;
    constexpr int kRounds = (kPerWarp + 31) / 32;
    __shared__ int warp_tot[32];
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    int v[kRounds], excl[kRounds];
#pragma unroll
    for (int j = 0; j < kRounds; j++) {
        const int off = j * 32 + lane, idx = wi * kPerWarp + off;
        v[j] = (off < kPerWarp && idx < kBins) ? hist[idx] : 0;
    }
    int carry = 0;
#pragma unroll
    for (int j = 0; j < kRounds; j++) {
        int incl = v[j];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        excl[j] = carry + incl - v[j];
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) warp_tot[wi] = carry;
    __syncthreads();
    if (wi == 0) {
        int t = warp_tot[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, t, d);
            if (lane >= d) t += o;
        }
        warp_tot[lane] = t;   // inclusive totals of the warps
    }
    __syncthreads();
    const int offset = wi > 0 ? warp_tot[wi - 1] : 0;
#pragma unroll
    for (int j = 0; j < kRounds; j++) {
        const int off = j * 32 + lane, idx = wi * kPerWarp + off;
        if (off < kPerWarp && idx < kBins) hist[idx] = excl[j] + offset;
    }
}

__global__ void __launch_bounds__(256)
order_scatter_kernel(const int32_t *__restrict__ order_in, const int32_t *__restrict__ keys, long long n_rows,
                     int32_t *__restrict__ cursor, int32_t *__restrict__ order_out)
{
    const long long t0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * kOrderPerThread;
    const int lane = threadIdx.x & 31;
    int k[kOrderPerThread] = {-1, -1, -1, -1}, o[kOrderPerThread] = {0, 0, 0, 0};
    if (t0 + kOrderPerThread <= n_rows) {
        const int4 kk = *reinterpret_cast<const int4 *>(keys + t0);
        const int4 oo = *reinterpret_cast<const int4 *>(order_in + t0);
        k[0] = kk.x; k[1] = kk.y; k[2] = kk.z; k[3] = kk.w;
        o[0] = oo.x; o[1] = oo.y; o[2] = oo.z; o[3] = oo.w;
    } else {
#pragma unroll
        for (int p = 0; p < kOrderPerThread; p++)
            if (t0 + p < n_rows) { k[p] = keys[t0 + p]; o[p] = order_in[t0 + p]; }
    }
    unsigned same[kOrderPerThread];
    int base[kOrderPerThread];
#pragma unroll
    for (int p = 0; p < kOrderPerThread; p++) {   // all the atomics first: their round trips overlap
        same[p] = __match_any_sync(0xffffffffu, k[p]);
        base[p] = 0;
        if (k[p] >= 0 && lane == __ffs(same[p]) - 1) base[p] = atomicAdd(cursor + k[p], __popc(same[p]));
    }
#pragma unroll
    for (int p = 0; p < kOrderPerThread; p++) {
        const int b = __shfl_sync(0xffffffffu, base[p], __ffs(same[p]) - 1);
        if (k[p] >= 0) order_out[b + __popc(same[p] & ((1u << lane) - 1u))] = o[p];
    }
}

// ------------------------------------------------------------------------------------------
// gather + normalisation terms + repulsive force
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_kernel(const float2 *__restrict__ Y2, long long row_lo, long long n_rows, IterState *state, int slot,
              InterpConsts ic, const float4 *__restrict__ ytilde, float2 *__restrict__ Frep2, int sum_z)
{
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    float zi = 0.0f;
    if (r < n_rows) {
        const GridGeom g = load_geom(state, slot);
        const float2 y = Y2[row_lo + r];
        int bx, by;
        float Lx[kInterp], Ly[kInterp];
        axis_weights(y.x, g, ic, bx, Lx);
        axis_weights(y.y, g, ic, by, Ly);
        float p1 = 0.0f, p2 = 0.0f, p3 = 0.0f, p4 = 0.0f;
#pragma unroll
        for (int a = 0; a < kInterp; a++) {
#pragma unroll
            for (int b = 0; b < kInterp; b++) {
                const float l = Lx[a] * Ly[b];
                const float4 v = __ldg(ytilde + (size_t)(bx * kInterp + a) * kG + (by * kInterp + b));
                p1 += l * v.z; p2 += l * v.x; p3 += l * v.y; p4 += l * v.w;  // node = (x, y, count, r^2) potentials
            }
        }
        zi = (1 + y.x * y.x + y.y * y.y) * p1 - 2 * (y.x * p2 + y.y * p3) + p4;
        Frep2[row_lo + r] = make_float2(y.x * p1 - p2, y.y * p1 - p3);
    }
    // block sum of Z_i in double, one atomic per block
    double z = (double)zi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    __shared__ double sz[8];
    if ((threadIdx.x & 31) == 0) sz[threadIdx.x >> 5] = z;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int k = 0; k < 8; k++) t += sz[k];
        if (sum_z) atomicAdd(&state->zsum[slot], t);
        if (blockIdx.x == 0) {  // recycle the other slot's min/max for this iteration's update
            state->min_enc[slot ^ 1] = 0xffffffffu;
            state->max_enc[slot ^ 1] = 0u;
        }
    }
}

// ------------------------------------------------------------------------------------------
// FFT building blocks
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 cmul(const float2 a, const float2 b)
{
    return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}

// e^{+2 pi i k / 32}, k = 0..15 (conjugated by the caller for the forward transform)
__device__ __forceinline__ float2 w32(int k)
{
    switch (k) {
        case 0: return make_float2(1.0f, 0.0f);
        case 1: return make_float2(0.98078528f, 0.195090322f);
        case 2: return make_float2(0.923879533f, 0.382683432f);
        case 3: return make_float2(0.831469612f, 0.555570233f);
        case 4: return make_float2(0.707106781f, 0.707106781f);
        case 5: return make_float2(0.555570233f, 0.831469612f);
        case 6: return make_float2(0.382683432f, 0.923879533f);
        case 7: return make_float2(0.195090322f, 0.98078528f);
        case 8: return make_float2(0.0f, 1.0f);
        case 9: return make_float2(-0.195090322f, 0.98078528f);
        case 10: return make_float2(-0.382683432f, 0.923879533f);
        case 11: return make_float2(-0.555570233f, 0.831469612f);
        case 12: return make_float2(-0.707106781f, 0.707106781f);
        case 13: return make_float2(-0.831469612f, 0.555570233f);
        case 14: return make_float2(-0.923879533f, 0.382683432f);
        default: return make_float2(-0.98078528f, 0.195090322f);
    }
}

__device__ __forceinline__ constexpr int rev5(int i)
{
    return ((i & 1) << 4) | ((i & 2) << 2) | (i & 4) | ((i & 8) >> 2) | ((i & 16) >> 4);
}

// 32-point transform held entirely in registers: natural order in, natural order out.
// INV = false: e^{-2 pi i nk/32};  INV = true: e^{+2 pi i nk/32} (unnormalised).
template <bool INV>
__device__ __forceinline__ void fft32(float2 (&v)[32])
{
#pragma unroll
    for (int s = 0; s < 5; s++) {
        const int half = 16 >> s;
#pragma unroll
        for (int b = 0; b < 32; b += 2 * half) {
#pragma unroll
            for (int j = 0; j < half; j++) {
                const float2 a = v[b + j], c = v[b + j + half];
                v[b + j] = make_float2(a.x + c.x, a.y + c.y);
                const float2 d = make_float2(a.x - c.x, a.y - c.y);
                const int t = j * (16 / half);
                if (t == 0) {
                    v[b + j + half] = d;
                } else if (t == 8) {
                    v[b + j + half] = INV ? make_float2(-d.y, d.x) : make_float2(d.y, -d.x);
                } else {
                    float2 w = w32(t);
                    if (!INV) w.y = -w.y;
                    v[b + j + half] = cmul(d, w);
                }
            }
        }
    }
    float2 t[32];
#pragma unroll
    for (int i = 0; i < 32; i++) t[rev5(i)] = v[i];
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = t[i];
}

constexpr int kExchStride = 33;                       // float2 per row of the per-warp exchange buffer
constexpr int kExchFloat2 = 32 * kExchStride;         // 1056 float2 = 8448 bytes per warp

// 1024-point transform by one warp.  In: lane l holds x[32*r + l] in v[r].  Out: lane l holds
// X[l + 32*r] in v[r] (the same register/lane pattern, so transforms chain without reshuffling).
// tws[k*32 + l] = e^{-2 pi i (k*l) / 1024}.
template <bool INV>
__device__ __forceinline__ void fft1024_warp(float2 (&v)[32], float2 *exch, const float2 *tws, int lane)
{
    fft32<INV>(v);
#pragma unroll
    for (int k = 0; k < 32; k++) {
        float2 w = tws[k * 32 + lane];
        if (INV) w.y = -w.y;
        exch[k * kExchStride + lane] = cmul(v[k], w);
    }
    __syncwarp();
#pragma unroll
    for (int n = 0; n < 32; n++) v[n] = exch[lane * kExchStride + n];
    __syncwarp();
    fft32<INV>(v);
}

__device__ __forceinline__ void fill_twiddles(float2 *tws, const float2 *__restrict__ tw)
{
    for (int idx = threadIdx.x; idx < 1024; idx += blockDim.x) tws[idx] = tw[((idx >> 5) * (idx & 31)) & (kM - 1)];
}

__global__ void twiddle_init_kernel(float2 *tw)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < kM) {
        double s, c;
        sincospi(-2.0 * (double)k / (double)kM, &s, &c);
        tw[k] = make_float2((float)c, (float)s);
    }
}

// ---- pass A: forward transform along the y-node index of the G non-zero rows ----
// 6 warps per block = 2 rows x {plane 0, plane 1, kernel plane}.
constexpr int kRowsPerBlockA = 2;
__global__ void __launch_bounds__(kRowsPerBlockA * 3 * 32)
fft_rows_forward_kernel(float4 *__restrict__ w, float2 *__restrict__ A, float *__restrict__ Rk, const IterState *state,
                        int slot, const float2 *__restrict__ tw, int zero_w)
{
    extern __shared__ float2 smem[];
    float2 *tws = smem;
    float2 *exch = smem + 1024 + (threadIdx.x >> 5) * kExchFloat2;
    fill_twiddles(tws, tw);
    __syncthreads();
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int row = blockIdx.x * kRowsPerBlockA + wi / 3, plane = wi % 3;
    if (row >= kG) return;
    float2 v[32];
    const GridGeom g = load_geom(state, slot);
    if (plane < 2) {
        float2 *wrow = reinterpret_cast<float2 *>(w + (size_t)row * kG) + plane;  // .xy or .zw of each node
        const float imag_scale = (plane == 1) ? g.r2_scale : 1.0f;
#pragma unroll
        for (int r = 0; r < 32; r++) {
            const int j = 32 * r + lane;
            if (j < kG) {
                v[r] = wrow[2 * j];
                v[r].y *= imag_scale;
                if (zero_w) wrow[2 * j] = make_float2(0.0f, 0.0f);
            } else {
                v[r] = make_float2(0.0f, 0.0f);
            }
        }
    } else {
        // Kernel values at node offsets (row, j), from float node coordinates exactly as the
        // reference forms them, summed and inverted in double (nbodyfft.cu:175-195); the weights
        // c_row * c_j (1 on the axes, 2 elsewhere) fold the three mirrored quadrants in.
        const float h = g.box_width / (float)kInterp;
        const float x_min = g.cmin, y_min = g.cmin;
        const float x1 = y_min + h / 2;
        const float y1 = y_min + h / 2 + row * h;
        const float d1 = x1 - y1;
        const float d1sq = d1 * d1;
#pragma unroll
        for (int r = 0; r < 32; r++) {
            const int j = 32 * r + lane;
            float val = 0.0f;
            if (j < kG) {
                const float x2 = x_min + h / 2;
                const float y2 = x_min + h / 2 + j * h;
                const float d2 = x2 - y2;
                const double s = 1.0 + (double)d1sq + (double)(d2 * d2);
                val = (float)(1.0 / (s * s));
                val *= ((row == 0) ? 1.0f : 2.0f) * ((j == 0) ? 1.0f : 2.0f);
            }
            v[r] = make_float2(val, 0.0f);
        }
    }
    fft1024_warp<false>(v, exch, tws, lane);
    if (plane < 2) {
        float2 *out = A + ((size_t)plane * kG + row) * kM;
#pragma unroll
        for (int r = 0; r < 32; r++) out[lane + 32 * r] = v[r];
    } else {
        float *out = Rk + (size_t)row * kM;
#pragma unroll
        for (int r = 0; r < 32; r++) out[lane + 32 * r] = v[r].x;
    }
}

// ---- pass B: per column: forward FFT, product with the (real) kernel spectrum, inverse FFT ----
// 12 warps per block = 4 adjacent columns x {plane 0, plane 1, kernel plane}.
constexpr int kColsPerBlockB = 4;
__global__ void __launch_bounds__(kColsPerBlockB * 3 * 32)
fft_columns_kernel(const float2 *__restrict__ A, const float *__restrict__ Rk, float2 *__restrict__ B,
                   const float2 *__restrict__ tw)
{
    extern __shared__ float2 smem[];
    float2 *tws = smem;
    float *kspec = reinterpret_cast<float *>(smem + 1024);                 // [4][1024]
    float2 *exch = smem + 1024 + (kColsPerBlockB * 1024) / 2 + (threadIdx.x >> 5) * kExchFloat2;
    fill_twiddles(tws, tw);
    __syncthreads();
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int c = wi % kColsPerBlockB, plane = wi / kColsPerBlockB;
    const int ky = blockIdx.x * kColsPerBlockB + c;
    float2 v[32];
    if (plane < 2) {
        const float2 *in = A + (size_t)plane * kG * kM + ky;
#pragma unroll
        for (int r = 0; r < 32; r++) {
            const int a = 32 * r + lane;
            v[r] = (a < kG) ? __ldg(in + (size_t)a * kM) : make_float2(0.0f, 0.0f);
        }
    } else {
        const float *in = Rk + ky;
#pragma unroll
        for (int r = 0; r < 32; r++) {
            const int a = 32 * r + lane;
            v[r] = make_float2((a < kG) ? __ldg(in + (size_t)a * kM) : 0.0f, 0.0f);
        }
    }
    fft1024_warp<false>(v, exch, tws, lane);
    if (plane == 2) {
#pragma unroll
        for (int r = 0; r < 32; r++) kspec[c * 1024 + r * 32 + lane] = v[r].x;
    }
    __syncthreads();
    if (plane == 2) return;
#pragma unroll
    for (int r = 0; r < 32; r++) {
        const float k = kspec[c * 1024 + r * 32 + lane];
        v[r].x *= k;
        v[r].y *= k;
    }
    fft1024_warp<true>(v, exch, tws, lane);
    float2 *out = B + (size_t)plane * kG * kM + ky;
#pragma unroll
    for (int r = 0; r < 32; r++) {
        const int a = lane + 32 * r;
        if (a < kG) out[(size_t)a * kM] = v[r];
    }
}

// ---- pass C: inverse transform along the y-node index of the G needed rows ----
constexpr int kRowsPerBlockC = 2;
__global__ void __launch_bounds__(kRowsPerBlockC * 2 * 32)
fft_rows_inverse_kernel(const float2 *__restrict__ B, float4 *__restrict__ ytilde, const IterState *state, int slot,
                        const float2 *__restrict__ tw)
{
    extern __shared__ float2 smem[];
    float2 *tws = smem;
    float2 *exch = smem + 1024 + (threadIdx.x >> 5) * kExchFloat2;
    fill_twiddles(tws, tw);
    __syncthreads();
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int row = blockIdx.x * kRowsPerBlockC + wi / 2, plane = wi % 2;
    if (row >= kG) return;
    float2 v[32];
    const float2 *in = B + ((size_t)plane * kG + row) * kM;
#pragma unroll
    for (int r = 0; r < 32; r++) v[r] = __ldg(in + 32 * r + lane);
    fft1024_warp<true>(v, exch, tws, lane);
    const float scale = 1.0f / ((float)kM * (float)kM);
    const float imag_scale = (plane == 1) ? scale * load_geom(state, slot).r2_unscale : scale;
    float2 *out = reinterpret_cast<float2 *>(ytilde + (size_t)row * kG) + plane;
#pragma unroll
    for (int r = 0; r < 32; r++) {
        const int j = lane + 32 * r;
        if (j < kG) out[2 * j] = make_float2(v[r].x * scale, v[r].y * imag_scale);
    }
}

inline unsigned nblk(long long n, int t) { return (unsigned)((n + t - 1) / t); }

constexpr size_t kSmemA = (1024 + (size_t)kRowsPerBlockA * 3 * kExchFloat2) * sizeof(float2);
constexpr size_t kSmemB = (1024 + (kColsPerBlockB * 1024) / 2 + (size_t)kColsPerBlockB * 3 * kExchFloat2) * sizeof(float2);
constexpr size_t kSmemC = (1024 + (size_t)kRowsPerBlockC * 2 * kExchFloat2) * sizeof(float2);

int configure_fft_kernels()
{
    static int done_for_device[64] = {0};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && done_for_device[dev]) return 0;
    B200_CUDA(cudaFuncSetAttribute(fft_rows_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemA));
    B200_CUDA(cudaFuncSetAttribute(fft_columns_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemB));
    B200_CUDA(cudaFuncSetAttribute(fft_rows_inverse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemC));
    if (dev >= 0 && dev < 64) done_for_device[dev] = 1;
    return 0;
}

}  // namespace

size_t fft_workspace_bytes()
{
    return sizeof(float2) * (size_t)2 * kG * kM * 2 + sizeof(float) * (size_t)kG * kM + sizeof(float2) * kM;
}

int fft_workspace_init(FftWorkspace *ws, void *mem, cudaStream_t st)
{
    char *p = static_cast<char *>(mem);
    ws->A = reinterpret_cast<float2 *>(p); p += sizeof(float2) * (size_t)2 * kG * kM;
    ws->B = reinterpret_cast<float2 *>(p); p += sizeof(float2) * (size_t)2 * kG * kM;
    ws->Rk = reinterpret_cast<float *>(p); p += sizeof(float) * (size_t)kG * kM;
    ws->tw = reinterpret_cast<float2 *>(p);
    B200_TRY(configure_fft_kernels());
    twiddle_init_kernel<<<kM / 256, 256, 0, st>>>(ws->tw);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_minmax_init(const float2 *Y2, int64_t N, IterState *state, int slot, cudaStream_t st)
{
    state_reset_kernel<<<1, 1, 0, st>>>(state, slot, 0);
    B200_CUDA(cudaGetLastError());
    if (N > 0) {
        const unsigned blocks = (unsigned)std::min<long long>(nblk(N, 256), 148 * 8);
        minmax_kernel<<<blocks, 256, 0, st>>>(Y2, N, state, slot);
        B200_CUDA(cudaGetLastError());
    }
    return 0;
}

int launch_state_reset(IterState *state, cudaStream_t st)
{
    state_reset_kernel<<<1, 1, 0, st>>>(state, 0, 1);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_spread(const float2 *Y2, int64_t row_lo, int64_t row_hi, const int32_t *order, const IterState *state,
                  int slot, InterpConsts ic, float4 *w, cudaStream_t st)
{
    const long long n = row_hi - row_lo;
    if (n <= 0) return 0;
    spread_kernel<<<nblk((n + kSpreadPerLane - 1) / kSpreadPerLane, 256), 256, 0, st>>>(Y2, row_lo, n, order, state, slot, ic, w);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_order_identity(int32_t *order, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    order_identity_kernel<<<nblk(n, 256), 256, 0, st>>>(order, n);
    B200_CUDA(cudaGetLastError());
    return 0;
}

// order_in -> order_out sorted by the box of the points' current position; keys: n ints of scratch,
// hist: kBoxes^2 ints of scratch.
int launch_order_refresh(const float2 *Y2, int64_t row_lo, int64_t row_hi, const int32_t *order_in, int32_t *order_out,
                         int32_t *keys, int32_t *hist, const IterState *state, int slot, cudaStream_t st)
{
    const long long n = row_hi - row_lo;
    if (n <= 0) return 0;
    B200_CUDA(cudaMemsetAsync(hist, 0, sizeof(int32_t) * kBoxes * kBoxes, st));
    const long long n_thr = (n + kOrderPerThread - 1) / kOrderPerThread;
    order_histogram_kernel<<<nblk(n_thr, 256), 256, 0, st>>>(Y2, row_lo, n, order_in, state, slot, keys, hist);
    B200_CUDA(cudaGetLastError());
    order_scan_kernel<<<1, 1024, 0, st>>>(hist);
    B200_CUDA(cudaGetLastError());
    order_scatter_kernel<<<nblk(n_thr, 256), 256, 0, st>>>(order_in, keys, n, hist, order_out);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_convolve(float4 *w, float4 *ytilde, const IterState *state, int slot, const FftWorkspace &ws, bool zero_w,
                    cudaStream_t st)
{
    B200_TRY(configure_fft_kernels());
    fft_rows_forward_kernel<<<kG / kRowsPerBlockA, kRowsPerBlockA * 3 * 32, kSmemA, st>>>(w, ws.A, ws.Rk, state, slot,
                                                                                         ws.tw, zero_w ? 1 : 0);
    B200_CUDA(cudaGetLastError());
    fft_columns_kernel<<<kM / kColsPerBlockB, kColsPerBlockB * 3 * 32, kSmemB, st>>>(ws.A, ws.Rk, ws.B, ws.tw);
    B200_CUDA(cudaGetLastError());
    fft_rows_inverse_kernel<<<kG / kRowsPerBlockC, kRowsPerBlockC * 2 * 32, kSmemC, st>>>(ws.B, ytilde, state, slot, ws.tw);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_gather(const float2 *Y2, int64_t row_lo, int64_t row_hi, IterState *state, int slot, InterpConsts ic,
                  const float4 *ytilde, float2 *Frep2, bool sum_z, cudaStream_t st)
{
    const long long n = row_hi - row_lo;
    // an empty shard still runs one block: it recycles the other slot's min/max
    gather_kernel<<<n > 0 ? nblk(n, 256) : 1, 256, 0, st>>>(Y2, row_lo, n, state, slot, ic, ytilde, Frep2, sum_z ? 1 : 0);
    B200_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace b200
