// Gradient, gains and momentum update (reference: IntegrationKernel, src/kernels/apply_forces.cu:11-57)
// fused with the min/max reduction the next iteration's grid needs (reference: thrust::minmax_element
// + two host reads, src/fit_tsne.cu:430-432) and the optional update-norm reduction
// (src/fit_tsne.cu:522-527).  Pure streaming kernel: 40 bytes read and 24 written per point.
#include "common.cuh"

namespace b200 {

namespace {

__device__ __forceinline__ float gain_rule(float g, float grad, float u)
{
    // the reference evaluates g + 0.2 and g * 0.8 in double and rounds once
    g = (signbit(grad) != signbit(u)) ? (float)((double)g + 0.2) : (float)((double)g * 0.8);
    return (g < 0.01) ? (float)0.01 : g;
}

__device__ __forceinline__ void step_point(float2 &y, const float2 fa, const float2 fr, float2 &g, float2 &u, float eta,
                                           float Z, float momentum, float exaggeration)
{
    const float dx = exaggeration * fa.x - (fr.x / Z);
    const float dy = exaggeration * fa.y - (fr.y / Z);
    g.x = gain_rule(g.x, dx, u.x);
    g.y = gain_rule(g.y, dy, u.y);
    u.x = momentum * u.x - eta * g.x * dx;
    u.y = momentum * u.y - eta * g.y * dy;
    y.x += u.x;
    y.y += u.y;
}

// Rows [row_lo, row_lo+n_rows) of the embedding are updated: read from Y2, written to every array of
// `dst` (in place: Y2 itself; sharded over peer memory: the next embedding buffer of every rank, which
// replaces an all-gather).  Reads the normalisation
// from state->zsum[slot] (sum of Z_i; Z = sum - n_total as in src/kernels/rep_forces.cu:51-54),
// accumulates min/max of the new coordinates into slot^1 and clears zsum[slot^1] for the next
// iteration's gather.
__global__ void __launch_bounds__(256)
update_kernel(const float2 *Y2, UpdateTargets dst, const float2 *__restrict__ Fa, const float2 *__restrict__ Fr,
              float2 *__restrict__ gains, float2 *__restrict__ u2, long long row_lo, long long n_rows,
              long long n_total, IterState *state, int slot, float eta, float momentum, float exaggeration,
              int want_norm)
{
    const float Z = (float)state->zsum[slot] - (float)n_total;
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    float mn = INFINITY, mx = -INFINITY, nrm = 0.0f;
    int bad = 0;
    if (r < n_rows) {
        const long long i = row_lo + r;
        float2 y = Y2[i], g = gains[r], u = u2[r];
        const float2 fa = __ldcs(Fa + i), fr = __ldcs(Fr + i);
        step_point(y, fa, fr, g, u, eta, Z, momentum, exaggeration);
#pragma unroll
        for (int t = 0; t < kMaxUpdateTargets; t++)
            if (t < dst.n) dst.p[t][i] = y;
        gains[r] = g;
        u2[r] = u;
        mn = fminf(y.x, y.y);
        mx = fmaxf(y.x, y.y);
        nrm = u.x * u.x + u.y * u.y;
        bad = !(isfinite(y.x) && isfinite(y.y));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (want_norm) nrm += __shfl_xor_sync(0xffffffffu, nrm, o);
    }
    bad = __any_sync(0xffffffffu, bad);
    __shared__ float s_mn[8], s_mx[8], s_n[8];
    __shared__ int s_bad[8];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_mn[w] = mn; s_mx[w] = mx; s_n[w] = nrm; s_bad[w] = bad; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int k = 0; k < 8; k++) {
            mn = fminf(mn, s_mn[k]); mx = fmaxf(mx, s_mx[k]); tot += (double)s_n[k]; bad |= s_bad[k];
        }
        if (mn <= mx) {
            atomicMin(&state->min_enc[slot ^ 1], enc_float(mn));
            atomicMax(&state->max_enc[slot ^ 1], enc_float(mx));
        }
        if (want_norm) atomicAdd(&state->unorm2, tot);
        if (bad) state->bad = 1;
        if (blockIdx.x == 0) state->zsum[slot ^ 1] = 0.0;
    }
}

// Stand-alone form with the reference's SoA buffers and an explicit Z, for the stage entry point.
__global__ void apply_forces_soa_kernel(float *Y, float *attr, float *rep, float *gains, float *old_forces, float eta,
                                        float Z, float momentum, float exaggeration, long long N)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    float2 y = make_float2(Y[i], Y[N + i]), g = make_float2(gains[i], gains[N + i]);
    float2 u = make_float2(old_forces[i], old_forces[N + i]);
    const float2 fa = make_float2(attr[i], attr[N + i]), fr = make_float2(rep[i], rep[N + i]);
    step_point(y, fa, fr, g, u, eta, Z, momentum, exaggeration);
    Y[i] = y.x; Y[N + i] = y.y;
    gains[i] = g.x; gains[N + i] = g.y;
    old_forces[i] = u.x; old_forces[N + i] = u.y;
    attr[i] = 0.0f; attr[N + i] = 0.0f; rep[i] = 0.0f; rep[N + i] = 0.0f;
}

// perm (optional): position q of the pair array holds point perm[q] of the block-wise array
__global__ void soa_to_aos_kernel(const float *soa, float2 *aos, long long N, const int32_t *perm)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) { const long long j = perm ? perm[i] : i; aos[i] = make_float2(soa[j], soa[N + j]); }
}
__global__ void aos_to_soa_kernel(const float2 *aos, float *soa, long long N, const int32_t *perm)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) { const long long j = perm ? perm[i] : i; const float2 v = aos[i]; soa[j] = v.x; soa[N + j] = v.y; }
}
// dst[q] = src[perm[q]] (gather) or dst[perm[q]] = src[q] (scatter)
__global__ void reorder_pairs_kernel(const float2 *src, float2 *dst, long long N, const int32_t *perm, int scatter)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    if (scatter) dst[perm[i]] = src[i];
    else dst[i] = src[perm[i]];
}
__global__ void fill_kernel(float *p, float v, long long n)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

inline unsigned nblk(long long n, int t) { return (unsigned)((n + t - 1) / t); }
}  // namespace

int launch_update(const float2 *Y2, const UpdateTargets &dst, const float2 *Fattr2, const float2 *Frep2, float2 *gains2, float2 *u2,
                  int64_t N, int64_t row_lo, int64_t row_hi, IterState *state, int slot, float eta, float momentum,
                  float exaggeration, int want_norm, cudaStream_t st)
{
    const long long n_rows = row_hi - row_lo;
    // even an empty shard must run one block so that the state slots are recycled
    const unsigned blocks = n_rows > 0 ? nblk(n_rows, 256) : 1;
    update_kernel<<<blocks, 256, 0, st>>>(Y2, dst, Fattr2, Frep2, gains2, u2, row_lo, n_rows, N, state, slot, eta, momentum,
                                          exaggeration, want_norm);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_apply_forces_soa(float *Y, float *attr, float *rep, float *gains, float *old_forces, float eta, float Z,
                            float momentum, float exaggeration, int64_t N, cudaStream_t st)
{
    if (N <= 0) return 0;
    apply_forces_soa_kernel<<<nblk(N, 256), 256, 0, st>>>(Y, attr, rep, gains, old_forces, eta, Z, momentum,
                                                         exaggeration, N);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_soa_to_aos(const float *soa, float2 *aos, int64_t N, cudaStream_t st, const int32_t *perm)
{
    if (N <= 0) return 0;
    soa_to_aos_kernel<<<nblk(N, 256), 256, 0, st>>>(soa, aos, N, perm);
    B200_CUDA(cudaGetLastError());
    return 0;
}
int launch_aos_to_soa(const float2 *aos, float *soa, int64_t N, cudaStream_t st, const int32_t *perm)
{
    if (N <= 0) return 0;
    aos_to_soa_kernel<<<nblk(N, 256), 256, 0, st>>>(aos, soa, N, perm);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_reorder_pairs(const float2 *src, float2 *dst, int64_t N, const int32_t *perm, bool scatter, cudaStream_t st)
{
    if (N <= 0) return 0;
    reorder_pairs_kernel<<<nblk(N, 256), 256, 0, st>>>(src, dst, N, perm, scatter ? 1 : 0);
    B200_CUDA(cudaGetLastError());
    return 0;
}
int launch_fill(float *p, float v, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    fill_kernel<<<nblk(n, 256), 256, 0, st>>>(p, v, n);
    B200_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace b200
