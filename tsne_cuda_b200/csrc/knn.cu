// Exact k-nearest-neighbour search, SIMT path.
//
// Replaces the reference's FAISS IVF-Flat call (src/util/distance_utils.cu:79-121, approximate, with
// results returned to the host as int64 and re-uploaded) by an exact search that stays on the device
// and writes int32 ids directly (so src/util/distance_utils.cu:125-154 has no counterpart).
//
// Canonical distance: squared L2 accumulated sequentially over d = 0..D-1 in fp32 with every
// subtract, multiply and add rounded separately (no FMA); results ordered by (distance, id); the
// query itself is included.  This is reproducible bit for bit on the CPU, which is what makes
// "identical neighbour ids" a testable statement.
//
// Structure: a block owns 64 queries and walks the database in tiles of 128 points.  Distances of a
// 64x128 tile are accumulated in registers (4x8 per thread) from dimension-major shared-memory
// tiles, parked in shared memory, and then each warp filters its queries' rows against the current
// k-th best; the rare survivors are inserted into the sorted result rows by the whole warp.
// No N x N matrix is ever written.
#include <limits.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>

#include "common.cuh"

#include <atomic>
#include "session.h"

namespace b200 {
namespace {

constexpr int BQ = 64;     // queries per block
constexpr int BP = 128;    // database points per tile
constexpr int DCH = 32;    // dimensions per shared-memory chunk
constexpr int kThreads = 256;
constexpr int DSTR = BP + 4;  // row stride of the parked distance tile (keeps float4 alignment)

__global__ void transpose_kernel(const float *__restrict__ X, long long N, int D, float *__restrict__ XT)
{
    __shared__ float tile[32][33];
    const long long r0 = (long long)blockIdx.x * 32;
    const int d0 = blockIdx.y * 32;
    for (int k = threadIdx.y; k < 32; k += blockDim.y) {
        const long long r = r0 + k;
        const int d = d0 + threadIdx.x;
        tile[k][threadIdx.x] = (r < N && d < D) ? X[r * D + d] : 0.0f;
    }
    __syncthreads();
    for (int k = threadIdx.y; k < 32; k += blockDim.y) {
        const int d = d0 + k;
        const long long r = r0 + threadIdx.x;
        if (d < D && r < N) XT[(long long)d * N + r] = tile[threadIdx.x][k];
    }
}

__global__ void knn_init_kernel(int32_t *ids, float *d2, long long n)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { ids[i] = INT_MAX; d2[i] = INFINITY; }
}

__global__ void knn_finalize_kernel(int32_t *ids, float *d2, long long n)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && ids[i] == INT_MAX) { ids[i] = -1; d2[i] = INFINITY; }
}

// Insert (d, id) into the ascending list (ld, li) of length K held in global memory; whole warp.
__device__ __forceinline__ void warp_insert(volatile float *ld, volatile int32_t *li, int K, float d, int id, int lane)
{
    int pos = 0;
    for (int e = lane; e < K; e += 32) {
        const float de = ld[e];
        const int ie = li[e];
        pos += (de < d || (de == d && ie < id)) ? 1 : 0;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) pos += __shfl_xor_sync(0xffffffffu, pos, o);
    for (int base = ((K - 1) / 32) * 32; base >= 0; base -= 32) {
        const int e = base + lane;
        const bool mv = (e > pos && e < K);
        float de = 0.0f;
        int ie = 0;
        if (mv) { de = ld[e - 1]; ie = li[e - 1]; }
        __syncwarp();
        if (mv) { ld[e] = de; li[e] = ie; }
        __syncwarp();
    }
    if (lane == 0) { ld[pos] = d; li[pos] = id; }
    __syncwarp();
}

// XT: dimension-major copy of X ([D][N]).  The nq queries are rows q_lo, q_lo+1, ... or, when q_index is
// given, the rows it lists; database rows [db_lo,db_hi).  The list of query row g is written to row
// (g - out_base) of ids/d2 ([.][K], pre-set to (INT_MAX, +inf)).
__global__ void __launch_bounds__(kThreads, 2)
knn_exact_kernel(const float *__restrict__ XT, long long N, int D, int K, long long q_lo, long long nq,
                 const int *__restrict__ q_index, long long out_base, long long db_lo, long long db_hi, int32_t *ids,
                 float *d2, long long slice_step, long long slice_out_stride)
{
    // slice_step > 0: block row y searches the database slice [db_lo + y * slice_step, ... + slice_step) and
    // writes its lists slice_out_stride elements after those of row y - 1
    if (slice_step > 0) {
        db_lo += (long long)blockIdx.y * slice_step;
        db_hi = min(db_hi, db_lo + slice_step);
        ids += (long long)blockIdx.y * slice_out_stride;
        d2 += (long long)blockIdx.y * slice_out_stride;
    }
    extern __shared__ __align__(16) float sm[];
    float *Qs = sm;                          // [DCH][BQ]
    float *Ps = Qs + DCH * BQ;               // [DCH][BP]
    float *Dist = Ps + DCH * BP;             // [BQ][DSTR]
    float *thr_d = Dist + BQ * DSTR;         // [BQ]
    int *thr_i = reinterpret_cast<int *>(thr_d + BQ);  // [BQ]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tx = tid & 15, ty = tid >> 4;
    const long long q0 = (long long)blockIdx.x * BQ;   // position in the query list
    int *q_row = thr_i + BQ;                            // [BQ] global row of each query, -1 beyond the list
    if (tid < BQ) {
        thr_d[tid] = INFINITY;
        thr_i[tid] = INT_MAX;
        const long long pos = q0 + tid;
        q_row[tid] = (pos < nq) ? (q_index ? q_index[pos] : (int)(q_lo + pos)) : -1;
    }
    __syncthreads();

    for (long long p0 = db_lo; p0 < db_hi; p0 += BP) {
        float acc[4][8];
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int b = 0; b < 8; b++) acc[a][b] = 0.0f;

        for (int d0 = 0; d0 < D; d0 += DCH) {
            const int dlen = min(DCH, D - d0);
            __syncthreads();  // previous chunk / previous tile's selection done with the buffers
            for (int idx = tid; idx < dlen * BQ; idx += kThreads) {
                const int dd = idx / BQ, q = idx % BQ;
                const int gq = q_row[q];
                Qs[dd * BQ + q] = (gq >= 0) ? XT[(long long)(d0 + dd) * N + gq] : 0.0f;
            }
            for (int idx = tid; idx < dlen * BP; idx += kThreads) {
                const int dd = idx / BP, pp = idx % BP;
                const long long gp = p0 + pp;
                Ps[dd * BP + pp] = (gp < db_hi) ? XT[(long long)(d0 + dd) * N + gp] : 0.0f;
            }
            __syncthreads();
#pragma unroll 4
            for (int dd = 0; dd < dlen; dd++) {
                const float4 q4 = *reinterpret_cast<const float4 *>(Qs + dd * BQ + ty * 4);
                const float4 pa = *reinterpret_cast<const float4 *>(Ps + dd * BP + tx * 4);
                const float4 pb = *reinterpret_cast<const float4 *>(Ps + dd * BP + 64 + tx * 4);
                const float qv[4] = {q4.x, q4.y, q4.z, q4.w};
                const float pv[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int b = 0; b < 8; b++) {
                        const float t = __fsub_rn(qv[a], pv[b]);
                        acc[a][b] = __fadd_rn(acc[a][b], __fmul_rn(t, t));
                    }
            }
        }
        // park the tile
#pragma unroll
        for (int a = 0; a < 4; a++) {
            float *row = Dist + (ty * 4 + a) * DSTR;
            *reinterpret_cast<float4 *>(row + tx * 4) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
            *reinterpret_cast<float4 *>(row + 64 + tx * 4) = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
        }
        __syncthreads();
        // selection: warp `warp` owns queries warp, warp+8, ...
        for (int q = warp; q < BQ; q += kThreads / 32) {
            const long long gq = q_row[q];
            if (gq < 0) break;
            const float4 dv = *reinterpret_cast<const float4 *>(Dist + q * DSTR + lane * 4);
            const float dl[4] = {dv.x, dv.y, dv.z, dv.w};
            float td = thr_d[q];
            int ti = thr_i[q];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const long long gp = p0 + lane * 4 + c;
                const bool in_db = gp < db_hi;
                unsigned m = __ballot_sync(0xffffffffu, in_db && (dl[c] < td || (dl[c] == td && (int)gp < ti)));
                while (m) {
                    const int src = __ffs(m) - 1;
                    m &= m - 1;
                    const float cd = __shfl_sync(0xffffffffu, dl[c], src);
                    const int ci = (int)(p0 + src * 4 + c);
                    if (cd < td || (cd == td && ci < ti)) {   // the threshold may have moved since the ballot
                        const long long orow = (out_base < 0) ? (q0 + q) : (gq - out_base);   // out_base < 0: by list position
                        volatile float *ld = d2 + orow * K;
                        volatile int32_t *li = ids + orow * K;
                        warp_insert(ld, li, K, cd, ci, lane);
                        td = ld[K - 1];
                        ti = li[K - 1];
                    }
                }
            }
            if (lane == 0) { thr_d[q] = td; thr_i[q] = ti; }
        }
    }
}

// Merge `parts` ascending lists per row (list p of row r at parts_base + p*part_stride + r*K) into the
// K best by (distance, id).  One thread per row; used after a database-sharded search.
__global__ void knn_merge_kernel(const int32_t *__restrict__ ids_parts, const float *__restrict__ d2_parts, int parts,
                                 long long part_stride, long long n_rows, int K, const int *__restrict__ row_index,
                                 long long out_base, int32_t *__restrict__ ids, float *__restrict__ d2)
{
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const long long orow = row_index ? (row_index[r] - out_base) : r;   // where the merged list goes
    int head[16];
    for (int p = 0; p < 16; p++) head[p] = 0;
    for (int s = 0; s < K; s++) {
        int best = -1, bi = INT_MAX;
        float bd = INFINITY;
        for (int p = 0; p < parts; p++) {
            if (head[p] >= K) continue;
            const long long o = (long long)p * part_stride + r * K + head[p];
            const int ci = ids_parts[o];
            const float cd = d2_parts[o];
            if (best < 0 || cd < bd || (cd == bd && ci < bi)) { best = p; bd = cd; bi = ci; }
        }
        ids[orow * K + s] = bi;
        d2[orow * K + s] = bd;
        if (best >= 0) head[best]++;
    }
}

// The same merge for many short lists (up to 1024 parts): one warp per row, lane l owns the parts
// l, l + 32, ...; every round each lane offers the best head among its parts and the warp takes the
// smallest offer by (distance, id).
__global__ void __launch_bounds__(128)
knn_merge_many_kernel(const int32_t *__restrict__ ids_parts, const float *__restrict__ d2_parts, int parts,
                      long long part_stride, long long n_rows, int K, const int *__restrict__ row_index, long long out_base,
                      int32_t *__restrict__ ids, float *__restrict__ d2)
{
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const long long orow = row_index ? (row_index[r] - out_base) : r;
    int head[32];
#pragma unroll
    for (int j = 0; j < 32; j++) head[j] = 0;
    for (int s = 0; s < K; s++) {
        float bd = INFINITY;
        int bi = INT_MAX, bj = -1;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int p = lane + 32 * j;
            if (p < parts && head[j] < K) {
                const long long o = (long long)p * part_stride + r * K + head[j];
                const float cd = d2_parts[o];
                const int ci = ids_parts[o];
                if (cd < bd || (cd == bd && ci < bi)) { bd = cd; bi = ci; bj = j; }
            }
        }
        float wd = bd;
        int wi = bi;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float od = __shfl_xor_sync(0xffffffffu, wd, o);
            const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
            if (od < wd || (od == wd && oi < wi)) { wd = od; wi = oi; }
        }
        // ids are unique across the parts (disjoint database slices), so exactly one lane holds the winner
        if (bj >= 0 && bd == wd && bi == wi) {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (j == bj) head[j]++;
        }
        if (lane == 0) { ids[orow * K + s] = wi; d2[orow * K + s] = wd; }
    }
}

constexpr size_t kKnnSmem = sizeof(float) * (DCH * BQ + DCH * BP + BQ * DSTR + BQ) + sizeof(int) * 2 * BQ;

__global__ void knn_init_rows_kernel(int32_t *ids, float *d2, const int *__restrict__ q_index, long long nq, long long out_base, int K)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nq * K) return;
    const long long row = (out_base < 0) ? (t / K) : (q_index[t / K] - out_base);
    ids[row * K + t % K] = INT_MAX;
    d2[row * K + t % K] = INFINITY;
}
}  // namespace

int launch_knn_finalize(int32_t *ids, float *d2, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    knn_finalize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ids, d2, n);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_knn_merge(const int32_t *ids_parts, const float *d2_parts, int parts, int64_t part_stride, int64_t n_rows,
                     int K, int32_t *ids, float *d2, cudaStream_t st)
{
    if (n_rows <= 0) return 0;
    if (parts > 16) { set_error("knn merge: more than 16 partial lists"); return -4; }
    knn_merge_kernel<<<(unsigned)((n_rows + 127) / 128), 128, 0, st>>>(ids_parts, d2_parts, parts, part_stride, n_rows, K,
                                                                      nullptr, 0, ids, d2);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_transpose(const float *X, int64_t N, int D, float *XT, cudaStream_t st)
{
    if (N <= 0 || D <= 0) return 0;
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)((D + 31) / 32));
    transpose_kernel<<<grid, dim3(32, 8), 0, st>>>(X, N, D, XT);
    B200_CUDA(cudaGetLastError());
    return 0;
}

// XT is the dimension-major copy of X produced by launch_transpose.
int launch_knn_exact(const float *XT, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo,
                     int64_t db_hi, int32_t *ids, float *d2, cudaStream_t st)
{
    const long long nq = q_hi - q_lo;
    if (nq <= 0) return 0;
    const long long n = nq * K;
    knn_init_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ids, d2, n);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaFuncSetAttribute(knn_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKnnSmem));
    knn_exact_kernel<<<(unsigned)((nq + BQ - 1) / BQ), kThreads, kKnnSmem, st>>>(XT, N, D, K, q_lo, nq, nullptr, q_lo, db_lo, db_hi,
                                                                                 ids, d2, 0, 0);
    B200_CUDA(cudaGetLastError());
    return 0;
}

// Same search for an explicit list of query rows (device array q_index of nq global row ids); the list
// of row g replaces row (g - out_base) of ids/d2.
int launch_knn_exact_rows(const float *XT, int64_t N, int D, int K, const int *q_index, int64_t nq, int64_t out_base,
                          int64_t db_lo, int64_t db_hi, int32_t *ids, float *d2, cudaStream_t st)
{
    if (nq <= 0) return 0;
    const long long n = nq * K;
    knn_init_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ids, d2, q_index, nq, out_base, K);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaFuncSetAttribute(knn_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKnnSmem));
    knn_exact_kernel<<<(unsigned)((nq + BQ - 1) / BQ), kThreads, kKnnSmem, st>>>(XT, N, D, K, 0, nq, q_index, out_base, db_lo, db_hi,
                                                                                 ids, d2, 0, 0);
    B200_CUDA(cudaGetLastError());
    return 0;
}


// SIMT search for a short list of rows.  A block serves 64 queries against the whole database, so a handful
// of rows would occupy a handful of SMs for the whole scan: the database is cut into slices searched by
// the block rows of one launch (enough of them to fill the GPU four times over), and the partial lists
// are merged.
static int knn_exact_few_rows(const float *XT, int64_t N, int D, int K, const int *rows, int64_t n_rows, int64_t out_base,
                              int64_t db_lo, int64_t db_hi, int32_t *ids, float *d2, DeviceArena &tmp, cudaStream_t st)
{
    const int64_t span = db_hi - db_lo;
    const int64_t q_blocks = (n_rows + BQ - 1) / BQ;
    const int slices = (int)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(span / 2048, 1024), 592 / q_blocks));
    if (slices == 1)
        return launch_knn_exact_rows(XT, N, D, K, rows, n_rows, out_base, db_lo, db_hi, ids, d2, st);
    int32_t *pi = nullptr;
    float *pd = nullptr;
    const long long per_slice = (long long)n_rows * K;
    B200_TRY(tmp.alloc((void **)&pi, sizeof(int32_t) * (size_t)slices * per_slice));
    B200_TRY(tmp.alloc((void **)&pd, sizeof(float) * (size_t)slices * per_slice));
    const int64_t step = (span + slices - 1) / slices;
    knn_init_kernel<<<(unsigned)((slices * per_slice + 255) / 256), 256, 0, st>>>(pi, pd, slices * per_slice);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaFuncSetAttribute(knn_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKnnSmem));
    knn_exact_kernel<<<dim3((unsigned)q_blocks, (unsigned)slices), kThreads, kKnnSmem, st>>>(XT, N, D, K, 0, n_rows, rows, -1, db_lo, db_hi,
                                                                                            pi, pd, step, per_slice);
    B200_CUDA(cudaGetLastError());
    knn_merge_many_kernel<<<(unsigned)((n_rows + 3) / 4), 128, 0, st>>>(pi, pd, slices, per_slice, n_rows, K, rows, out_base, ids, d2);
    B200_CUDA(cudaGetLastError());
    return 0;
}

// Exact search of queries [q_lo,q_hi) against database rows [db_lo,db_hi) of X ([N][D], device),
// choosing the tensor-core path where it applies and falling back to the SIMT search for the rows it
// cannot certify.  Unfilled slots keep (INT_MAX, +inf); see launch_knn_finalize.
int knn_search(const float *X, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo, int64_t db_hi,
               int32_t *ids, float *d2, KnnStats *stats, cudaStream_t st)
{
    KnnStats local;
    if (!stats) stats = &local;
    *stats = KnnStats();
    const int64_t nq = q_hi - q_lo;
    if (nq <= 0) return 0;
    const char *force = getenv("B200TSNE_KNN");
    const bool want_tc = knn_tc_supported(db_hi - db_lo, D, K) && !(force && strcmp(force, "simt") == 0);
    DeviceArena tmp;
    tmp.serve(st);
    float *XT = nullptr;
    auto ensure_xt = [&]() -> int {
        if (XT) return 0;
        B200_TRY(tmp.alloc((void **)&XT, sizeof(float) * (size_t)N * D));
        return launch_transpose(X, N, D, XT, st);
    };
    if (!want_tc) {
        B200_TRY(ensure_xt());
        B200_TRY(launch_knn_exact(XT, N, D, K, q_lo, q_hi, db_lo, db_hi, ids, d2, st));
        B200_CUDA(cudaStreamSynchronize(st));   // XT is released on return
        return 0;
    }
    // Queries go through in batches of 2^20 so that the candidate buffers (about 10 KB per query) stay
    // bounded however large N is; the operand images are rebuilt per batch (a millisecond per million points).
    const int64_t batch = (int64_t)1 << 20;
    void *ws = nullptr;
    B200_TRY(tmp.alloc(&ws, knn_tc_workspace_bytes(D, K, std::min(nq, batch), db_hi - db_lo)));
    stats->tensor_core = 1;
    for (int64_t b_lo = q_lo; b_lo < q_hi; b_lo += batch) {
        const int64_t b_hi = std::min(q_hi, b_lo + batch);
        int *failed_list = nullptr;
        int n_failed = 0;
        float ratio = 0.0f;
        int32_t *ids_b = ids + (b_lo - q_lo) * K;
        float *d2_b = d2 + (b_lo - q_lo) * K;
        B200_TRY(launch_knn_tc(X, N, D, K, b_lo, b_hi, db_lo, db_hi, ids_b, d2_b, ws, &failed_list, &n_failed, &ratio, st));
        stats->rows_recomputed += n_failed;
        stats->filter_error_ratio = std::max(stats->filter_error_ratio, ratio);
        if (n_failed > 0) {
            B200_TRY(ensure_xt());
            B200_TRY(knn_exact_few_rows(XT, N, D, K, failed_list, n_failed, b_lo, db_lo, db_hi, ids_b, d2_b, tmp, st));
            B200_CUDA(cudaStreamSynchronize(st));   // the failed list lives in the workspace the next batch reuses
        }
    }
    B200_CUDA(cudaStreamSynchronize(st));
    return 0;
}


// ---------------------------------------------------------------------------------------------------
// Exact search for callers that must not allocate.
//
// Some hosts own every byte of device memory themselves (a framework with its own pool, a service that
// pre-sizes its footprint at start-up, a real-time loop in which cudaMalloc's implicit device
// synchronisation is not acceptable).  For them the dimension-major copy of the points that the SIMT
// search reads lives in a fixed array that is part of the library image: every GPU that loads the
// library carries kNoAllocMaxElems floats (16 MiB) for it until the process exits.
// ---------------------------------------------------------------------------------------------------
constexpr long long kNoAllocMaxElems = 4ll << 20;   // N * D may not exceed this
static __device__ __align__(256) float g_noalloc_xt[kNoAllocMaxElems];

// In host code `g_noalloc_xt` is only a handle; the address a kernel can use comes from the runtime and
// differs per device.  Looked up once per device, with that device current.
static int noalloc_scratch(float **out)
{
    static std::atomic<float *> cached[64];   // zero-initialised; two threads racing here store the same address
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { set_error("knn_noalloc: device ordinal out of range"); return -4; }
    float *p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        B200_CUDA(cudaGetSymbolAddress((void **)&p, g_noalloc_xt));
        cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return 0;
}

long long knn_noalloc_max_elems() { return kNoAllocMaxElems; }

// X, ids, d2: device memory of the current device.  Queues the search on `st` and returns.
int knn_noalloc(const float *X, int64_t N, int D, int K, int32_t *ids, float *d2, cudaStream_t st)
{
    if (N <= 0 || D <= 0 || K <= 0) { set_error("knn_noalloc: invalid sizes"); return -1; }
    if (D > 65535 * 32) { set_error("knn_noalloc: more than 2,097,120 dimensions are not supported"); return -4; }
    if ((long long)N * D > kNoAllocMaxElems) {
        set_error("knn_noalloc: N * D = " + std::to_string((long long)N * D) + " exceeds the built-in scratch of " +
                  std::to_string(kNoAllocMaxElems) + " floats; use b200tsne_knn");
        return -4;
    }
    float *XT = nullptr;
    B200_TRY(noalloc_scratch(&XT));
    B200_TRY(launch_transpose(X, N, D, XT, st));      // overwrites every element the search will read
    B200_TRY(launch_knn_exact(XT, N, D, K, 0, N, 0, N, ids, d2, st));
    B200_TRY(launch_knn_finalize(ids, d2, N * K, st));
    return 0;
}

}  // namespace b200
