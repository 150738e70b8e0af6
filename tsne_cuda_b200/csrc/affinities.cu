// From neighbour distances to the fixed-width affinity matrix P:
//   global max-normalisation   (reference: util::MaxNormalizeDeviceVector, src/util/math_utils.cu:66-74)
//   per-row perplexity search  (reference: src/kernels/perplexity_search.cu:10-141: two elementwise
//                               kernels, two cuBLAS gemv row reductions and three device syncs per round)
//   symmetrisation             (reference: syv2k, src/util/math_utils.cu:269-291)
//
// Here one warp owns one row for the whole bisection: the row's normalised distances sit in shared
// memory, the row sums are warp shuffles, and p is written once (4*K bytes read + 4*K written per
// point).  The update rule, the fast exp/log intrinsics and the 200-round cap follow the reference.
#include <float.h>

#include "common.cuh"

namespace b200 {
namespace {

__global__ void __launch_bounds__(256) absmax_kernel(const float *__restrict__ v, long long n, unsigned int *max_enc)
{
    float m = 0.0f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float a = fabsf(v[i]);
        if (a > m && a < INFINITY) m = a;  // +inf marks an unfilled slot, never a distance
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(max_enc, enc_float(m));
}

__device__ __forceinline__ float cond_p(int s, float dist, float beta)
{
    // slot 0 is the point itself (distance exactly 0): p_ii = 0   (perplexity_search.cu:32)
    return (s == 0 & dist == 0.0f) ? 0.0f : __expf(-beta * dist);
}

constexpr int kPerpWarps = 8;

__global__ void __launch_bounds__(kPerpWarps * 32)
perplexity_kernel(const float *__restrict__ d2, long long n_rows, int K, float perplexity, float eps,
                  const unsigned int *__restrict__ max_enc, float *__restrict__ p, float *__restrict__ betas)
{
    extern __shared__ float srow[];
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * kPerpWarps + wi;
    if (row >= n_rows) return;
    float *d = srow + (size_t)wi * K;
    const float maxv = dec_float(*max_enc);
    for (int s = lane; s < K; s += 32) d[s] = d2[row * K + s] / maxv;
    __syncwarp();
    const float log_perp = __logf(perplexity);
    float beta = 1.0f, lo = -FLT_MAX, hi = FLT_MAX;
    float beta_eval = beta, S = 0.0f;
    for (int it = 0; it < 200; it++) {
        float sum = 0.0f, ent = 0.0f;
        for (int s = lane; s < K; s += 32) {
            const float v = cond_p(s, d[s], beta);
            float e = v * logf(v);
            e = (e != e || isinf(e)) ? 0.0f : e;  // FunctionalEntropy, thrust_transform_functions.h:32-37
            sum += v;
            ent += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            ent += __shfl_xor_sync(0xffffffffu, ent, o);
        }
        S = sum;
        beta_eval = beta;
        const float neg_ent = -ent;
        const float H = (neg_ent / S) + __logf(S);
        const float diff = H - log_perp;
        if (diff < eps && -diff < eps) break;
        if (diff > 0) {
            lo = beta;
            beta = (hi == FLT_MAX || hi == -FLT_MAX) ? beta * 2.0f : (beta + hi) / 2.0f;
        } else {
            hi = beta;
            beta = (lo == -FLT_MAX || lo == FLT_MAX) ? beta / 2.0f : (beta + lo) / 2.0f;
        }
    }
    // p of the last evaluated beta divided by its row sum.  A row that exhausts the 200 rounds keeps,
    // like the reference, the values of the beta evaluated last, not of the beta it would try next.
    for (int s = lane; s < K; s += 32) p[row * K + s] = cond_p(s, d[s], beta_eval) / S;
    if (lane == 0 && betas) betas[row] = beta;
}

// One warp per row i.  For each slot s: j = ids[i][s]; scan the K ids of row j for i and add the
// matching p[j][.]; divide by 2N in double like the reference.
// visit (optional, n_rows entries, all inside [row_lo, row_lo + n_rows)): the order in which the warps take the rows.
// The kernel is bound by the K random row reads per row (32 GB at N = 10^6, K = 90); rows visited cluster by cluster
// find the rows of their neighbours, which lie in the same cluster, in L2.
constexpr int kSymWarps = 8;
constexpr int kSymAhead = 4;   // neighbour rows whose loads are in flight together (8: 15.9 ms against 7.0 at N = 10^6, K = 90; 1: 8.5)
__global__ void __launch_bounds__(kSymWarps * 32)
symmetrize_kernel(const float *__restrict__ p, const int32_t *__restrict__ ids, long long N, int K, long long row_lo,
                  long long n_rows, const int32_t *__restrict__ visit, float *__restrict__ P_rows)
{
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * kSymWarps + (threadIdx.x >> 5);
    if (w >= n_rows) return;
    const long long i = visit ? (long long)visit[w] : row_lo + w;
    const long long r = i - row_lo;
    if (r < 0 || r >= n_rows) return;
    const double inv = 2.0 * (double)N;
    for (int s0 = 0; s0 < K; s0 += 32) {
        const int s_mine = s0 + lane;
        int j_mine = -1;
        float p_mine = 0.0f;
        if (s_mine < K) {
            j_mine = ids[i * K + s_mine];
            p_mine = p[i * K + s_mine];
        }
        float acc_mine = p_mine;
        const int cnt = min(32, K - s0);
        // kSymAhead neighbours' rows at a time: their loads are independent and in flight together (a warp that takes
        // one row after the other waits for each round trip to L2 in turn)
        for (int t = 0; t < cnt; t += kSymAhead) {
            int j[kSymAhead];
            const int32_t *rj[kSymAhead];
#pragma unroll
            for (int q = 0; q < kSymAhead; q++) {
                j[q] = __shfl_sync(0xffffffffu, j_mine, min(t + q, 31));
                if (t + q >= cnt || (unsigned long long)j[q] >= (unsigned long long)N) j[q] = -1;
                rj[q] = ids + (long long)max(j[q], 0) * K;
            }
            float add[kSymAhead];
#pragma unroll
            for (int q = 0; q < kSymAhead; q++) add[q] = 0.0f;
            for (int u0 = 0; u0 < K; u0 += 32) {
                const int u = u0 + lane;
                int32_t v[kSymAhead];
#pragma unroll
                for (int q = 0; q < kSymAhead; q++) v[q] = (u < K && j[q] >= 0) ? rj[q][u] : -1;
#pragma unroll
                for (int q = 0; q < kSymAhead; q++)
                    if (v[q] == (int32_t)i && j[q] >= 0) add[q] += p[(long long)j[q] * K + u];
            }
            // matches are rare (at most one for a valid neighbour list): reduce only when some lane has one
#pragma unroll
            for (int q = 0; q < kSymAhead; q++) {
                if (__any_sync(0xffffffffu, add[q] != 0.0f)) {
                    float a = add[q];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                    if (lane == t + q) acc_mine += a;
                }
            }
        }
        if (s_mine < K) P_rows[r * K + s_mine] = (float)((double)acc_mine / inv);
    }
}

// The entries the fixed-width P leaves out.  The fixed-width symmetrisation stores P_ij only where j is a neighbour
// of i; where j has i as a neighbour but not the other way round, the reference drops P_ji's mirror image
// (src/util/math_utils.cu:269-291).  A truly symmetric P = (p + p^T) / 2N has it: for every edge i -> j whose
// reverse is missing, row j gets the extra entry (column i, p_j|i / 2N).
// One warp per source row i (all N rows); PASS 0 counts the extra entries of the owned target rows, PASS 1 writes them
// (order inside a row: as the atomics fall, which only reorders a row's sum).
template <int PASS>
__global__ void __launch_bounds__(kSymWarps * 32)
reverse_only_kernel(const float *__restrict__ p, const int32_t *__restrict__ ids, long long N, int K, long long row_lo, long long row_hi,
                    int *__restrict__ count, const int *__restrict__ ptr, int *__restrict__ cursor, int32_t *__restrict__ ext_ids,
                    float *__restrict__ ext_val)
{
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * kSymWarps + (threadIdx.x >> 5);
    if (i >= N) return;
    const double inv = 2.0 * (double)N;
    for (int s0 = 0; s0 < K; s0 += 32) {
        const int s_mine = s0 + lane;
        int j_mine = -1;
        float p_mine = 0.0f;
        if (s_mine < K) {
            j_mine = ids[i * K + s_mine];
            p_mine = p[i * K + s_mine];
        }
        const int cnt = min(32, K - s0);
        for (int t = 0; t < cnt; t++) {
            const int j = __shfl_sync(0xffffffffu, j_mine, t);
            if (j < row_lo || j >= row_hi || j == i) continue;          // not an owned target, or the point itself
            const int32_t *rj = ids + (long long)j * K;
            bool found = false;
            for (int u = lane; u < K; u += 32) found |= rj[u] == (int32_t)i;
            if (__any_sync(0xffffffffu, found)) continue;               // mutual: the fixed-width entry has both halves
            if (lane == t) {
                const long long r = j - row_lo;
                if (PASS == 0) {
                    atomicAdd(&count[r], 1);
                } else {
                    const int at = ptr[r] + atomicAdd(&cursor[r], 1);
                    ext_ids[at] = (int32_t)i;
                    ext_val[at] = (float)((double)p_mine / inv);
                }
            }
        }
    }
}

inline unsigned nblk(long long n, int t) { return (unsigned)((n + t - 1) / t); }
}  // namespace

// ptr: [rows + 1] ints (device), filled here; returns the number of extra entries in *count_host (synchronises st).
int launch_reverse_only_count(const float *p_all, const int32_t *ids_all, int64_t N, int K, int64_t row_lo, int64_t row_hi, int *ptr,
                              int64_t *count_host, cudaStream_t st)
{
    const long long rows = row_hi - row_lo;
    *count_host = 0;
    if (rows <= 0) return 0;
    B200_CUDA(cudaMemsetAsync(ptr, 0, sizeof(int) * (rows + 1), st));
    reverse_only_kernel<0><<<nblk(N, kSymWarps), kSymWarps * 32, 0, st>>>(p_all, ids_all, N, K, row_lo, row_hi, ptr, nullptr, nullptr, nullptr,
                                                                          nullptr);
    B200_CUDA(cudaGetLastError());
    B200_TRY(launch_exclusive_scan_i32(ptr, rows + 1, st));
    int total = 0;
    B200_CUDA(cudaMemcpyAsync(&total, ptr + rows, sizeof(int), cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    if (total < 0) { set_error("symmetric P: more than 2^31 reverse-only entries"); return -4; }
    *count_host = total;
    return 0;
}

// cursor: [rows] ints of scratch (device)
int launch_reverse_only_fill(const float *p_all, const int32_t *ids_all, int64_t N, int K, int64_t row_lo, int64_t row_hi, const int *ptr,
                             int *cursor, int32_t *ext_ids, float *ext_val, cudaStream_t st)
{
    const long long rows = row_hi - row_lo;
    if (rows <= 0) return 0;
    B200_CUDA(cudaMemsetAsync(cursor, 0, sizeof(int) * rows, st));
    reverse_only_kernel<1><<<nblk(N, kSymWarps), kSymWarps * 32, 0, st>>>(p_all, ids_all, N, K, row_lo, row_hi, nullptr, ptr, cursor, ext_ids,
                                                                          ext_val);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_absmax(const float *v, int64_t n, unsigned int *max_enc, cudaStream_t st)
{
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    absmax_kernel<<<blocks, 256, 0, st>>>(v, n, max_enc);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_perplexity(const float *d2, int64_t n_rows, int K, float perplexity, float eps, const unsigned int *max_enc,
                      float *p, float *betas, cudaStream_t st)
{
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)kPerpWarps * K * sizeof(float);
    if (smem > 200 * 1024) { set_error("perplexity: num_neighbors too large for the shared-memory row buffer"); return -4; }
    if (smem > 48 * 1024)
        B200_CUDA(cudaFuncSetAttribute(perplexity_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    perplexity_kernel<<<nblk(n_rows, kPerpWarps), kPerpWarps * 32, smem, st>>>(d2, n_rows, K, perplexity, eps, max_enc, p,
                                                                              betas);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_symmetrize(const float *p_all, const int32_t *ids_all, int64_t N, int K, int64_t row_lo, int64_t row_hi,
                      float *P_rows, cudaStream_t st, const int32_t *visit)
{
    const long long n_rows = row_hi - row_lo;
    if (n_rows <= 0) return 0;
    symmetrize_kernel<<<nblk(n_rows, kSymWarps), kSymWarps * 32, 0, st>>>(p_all, ids_all, N, K, row_lo, n_rows, visit, P_rows);
    B200_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace b200
