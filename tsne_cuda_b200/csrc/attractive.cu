// Attractive force: F_i = sum_s P[i][s] / (1 + |y_i - y_j|^2) * (y_i - y_j),  j = ids[i][s].
// Arithmetic of the reference's ComputePijxQijKernelV3 + reduce_sum_kernel
// (src/kernels/attr_forces.cu:129-184) without its [2][N*K] workspace round trip.
//
// One warp per row.  The row's ids and P values (8*K bytes, the only large stream: read once with
// evict-first loads) are all requested before the first neighbour coordinate is, and all neighbour
// coordinates (AoS float2, L2-resident) before the first is used, so every lane keeps ceil(K/32)
// independent gathers in flight.  Measured on B200: with the loads issued one slot at a time the
// kernel is latency-bound (627 us for N = 10^6, K = 90 on a random graph); batched it runs at the
// rate the L1 serves fully divergent 8-byte reads, about one 128-byte line per clock and SM
// (369 us, against 324 us for the bare gathers and 112 us for the HBM stream alone).  A
// shared-memory ring filled by bulk asynchronous copies and texture fetches were measured too and
// change nothing: the stream is not the limit, the divergent gather is.
#include "common.cuh"

namespace b200 {

namespace {
constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ void accumulate(float2 yi, float2 yj, float p, float &ax, float &ay)
{
    const float dx = yi.x - yj.x, dy = yi.y - yj.y;
    const float pq = p / (1 + dx * dx + dy * dy);
    ax += pq * dx;
    ay += pq * dy;
}

// KPL = slots per lane (K <= 32*KPL)
template <int KPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attractive_kernel(const float *__restrict__ P, const int32_t *__restrict__ ids, const float2 *__restrict__ Y2,
                  long long N, int K, long long row_lo, long long n_rows, float2 *__restrict__ F2)
{
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const long long i = row_lo + r;
    int j[KPL];
    float p[KPL];
#pragma unroll
    for (int k = 0; k < KPL; k++) {
        const int s = lane + 32 * k;
        const bool in_row = s < K;
        j[k] = in_row ? __ldcs(ids + r * K + s) : -1;
        p[k] = in_row ? __ldcs(P + r * K + s) : 0.0f;
    }
    const float2 yi = __ldg(Y2 + i);
    float2 yj[KPL];
#pragma unroll
    for (int k = 0; k < KPL; k++) {
        const bool valid = (unsigned long long)j[k] < (unsigned long long)N;   // -1 marks an unfilled slot
        yj[k] = __ldg(Y2 + (valid ? (long long)j[k] : i));
        if (!valid) p[k] = 0.0f;
    }
    float ax = 0.0f, ay = 0.0f;
#pragma unroll
    for (int k = 0; k < KPL; k++) accumulate(yi, yj[k], p[k], ax, ay);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ax += __shfl_xor_sync(0xffffffffu, ax, o);
        ay += __shfl_xor_sync(0xffffffffu, ay, o);
    }
    if (lane == 0) F2[i] = make_float2(ax, ay);
}

// any K: four slots per lane and round
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attractive_long_rows_kernel(const float *__restrict__ P, const int32_t *__restrict__ ids, const float2 *__restrict__ Y2,
                            long long N, int K, long long row_lo, long long n_rows, float2 *__restrict__ F2)
{
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const long long i = row_lo + r;
    const float2 yi = __ldg(Y2 + i);
    float ax = 0.0f, ay = 0.0f;
    for (int s0 = 0; s0 < K; s0 += 128) {
        int j[4];
        float p[4];
        float2 yj[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int s = s0 + lane + 32 * k;
            j[k] = (s < K) ? __ldcs(ids + r * K + s) : -1;
            p[k] = (s < K) ? __ldcs(P + r * K + s) : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const bool valid = (unsigned long long)j[k] < (unsigned long long)N;
            yj[k] = __ldg(Y2 + (valid ? (long long)j[k] : i));
            if (!valid) p[k] = 0.0f;
        }
#pragma unroll
        for (int k = 0; k < 4; k++) accumulate(yi, yj[k], p[k], ax, ay);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ax += __shfl_xor_sync(0xffffffffu, ax, o);
        ay += __shfl_xor_sync(0xffffffffu, ay, o);
    }
    if (lane == 0) F2[i] = make_float2(ax, ay);
}
// the rows' extra entries (variable width): one warp per row, added to what the fixed-width kernel wrote
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attractive_extra_kernel(const int *__restrict__ ptr, const int32_t *__restrict__ ext_ids, const float *__restrict__ ext_val,
                        const float2 *__restrict__ Y2, long long N, long long row_lo, long long n_rows, float2 *__restrict__ F2)
{
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const long long i = row_lo + r;
    const int lo = ptr[r], hi = ptr[r + 1];
    if (lo == hi) return;
    const float2 yi = __ldg(Y2 + i);
    float ax = 0.0f, ay = 0.0f;
    for (int e = lo + lane; e < hi; e += 32) {
        const int j = __ldcs(ext_ids + e);
        if ((unsigned long long)j < (unsigned long long)N) accumulate(yi, __ldg(Y2 + j), __ldcs(ext_val + e), ax, ay);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ax += __shfl_xor_sync(0xffffffffu, ax, o);
        ay += __shfl_xor_sync(0xffffffffu, ay, o);
    }
    if (lane == 0) {
        float2 f = F2[i];
        f.x += ax;
        f.y += ay;
        F2[i] = f;
    }
}
}  // namespace

int launch_attractive_extra(const int *ptr, const int32_t *ext_ids, const float *ext_val, const float2 *Y2, int64_t N, int64_t row_lo,
                            int64_t row_hi, float2 *F2, cudaStream_t st)
{
    const long long n_rows = row_hi - row_lo;
    if (n_rows <= 0) return 0;
    const unsigned blocks = (unsigned)((n_rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    attractive_extra_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>(ptr, ext_ids, ext_val, Y2, N, row_lo, n_rows, F2);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_attractive(const float *P_rows, const int32_t *ids_rows, const float2 *Y2, int64_t N, int K, int64_t row_lo,
                      int64_t row_hi, float2 *F2, cudaStream_t st)
{
    const long long n_rows = row_hi - row_lo;
    if (n_rows <= 0) return 0;
    const unsigned blocks = (unsigned)((n_rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const int threads = kWarpsPerBlock * 32;
#define B200_ATTR(KPL) attractive_kernel<KPL><<<blocks, threads, 0, st>>>(P_rows, ids_rows, Y2, N, K, row_lo, n_rows, F2)
    if (K <= 32) B200_ATTR(1);
    else if (K <= 64) B200_ATTR(2);
    else if (K <= 96) B200_ATTR(3);
    else if (K <= 128) B200_ATTR(4);
    else if (K <= 160) B200_ATTR(5);
    else if (K <= 192) B200_ATTR(6);
    else attractive_long_rows_kernel<<<blocks, threads, 0, st>>>(P_rows, ids_rows, Y2, N, K, row_lo, n_rows, F2);
#undef B200_ATTR
    B200_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace b200
