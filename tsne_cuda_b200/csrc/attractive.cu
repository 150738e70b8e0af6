// Attractive force: F_i = sum_s P[i][s] / (1 + |y_i - y_j|^2) * (y_i - y_j),  j = ids[i][s].
// Arithmetic of the reference's ComputePijxQijKernelV3 + reduce_sum_kernel
// (src/kernels/attr_forces.cu:129-184) without its [2][N*K] workspace round trip.
//
// HBM roofline kernel: the fixed-width P and ids rows (8*K bytes per point) are streamed once
// with evict-first loads, one warp per row; the embedding (8 bytes per point, AoS float2) stays
// L2-resident and is gathered through the read-only path.
#include "common.cuh"

namespace b200 {

namespace {
constexpr int kWarpsPerBlock = 8;

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attractive_kernel(const float *__restrict__ P, const int32_t *__restrict__ ids, const float2 *__restrict__ Y2,
                  long long N, int K, long long row_lo, long long n_rows, float2 *__restrict__ F2)
{
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const long long i = row_lo + r;
    const float2 yi = __ldg(Y2 + i);
    const float *pr = P + r * K;
    const int32_t *ir = ids + r * K;
    float ax = 0.0f, ay = 0.0f;
#pragma unroll 3
    for (int s = lane; s < K; s += 32) {
        const int j = __ldcs(ir + s);
        const float p = __ldcs(pr + s);
        if ((unsigned long long)j < (unsigned long long)N) {
            const float2 yj = __ldg(Y2 + j);
            const float dx = yi.x - yj.x, dy = yi.y - yj.y;
            const float pq = p / (1 + dx * dx + dy * dy);
            ax += pq * dx;
            ay += pq * dy;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ax += __shfl_xor_sync(0xffffffffu, ax, o);
        ay += __shfl_xor_sync(0xffffffffu, ay, o);
    }
    if (lane == 0) F2[i] = make_float2(ax, ay);
}
}  // namespace

int launch_attractive(const float *P_rows, const int32_t *ids_rows, const float2 *Y2, int64_t N, int K, int64_t row_lo,
                      int64_t row_hi, float2 *F2, cudaStream_t st)
{
    const long long n_rows = row_hi - row_lo;
    if (n_rows <= 0) return 0;
    const unsigned blocks = (unsigned)((n_rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    attractive_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>(P_rows, ids_rows, Y2, N, K, row_lo, n_rows, F2);
    B200_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace b200
