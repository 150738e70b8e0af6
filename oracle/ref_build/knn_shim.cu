// Stand-in for the two functions of the reference's src/util/distance_utils.cu, which cannot be
// compiled here because FAISS (an external dependency of the reference) is not installed.
// Test infrastructure: linked only into oracle/_ref/libtsnecuda_ref.so together with the
// reference's own, unmodified sources.
//
//  * tsnecuda::util::KNearestNeighbors  (reference: src/util/distance_utils.cu:79-121, FAISS IVF-Flat)
//    is replaced by an exact search.  When a neighbour list has been injected with
//    ref_set_knn(), that list is returned (so that both engines can be given identical graphs and
//    large inputs need no second search); otherwise a plain one-thread-per-query exact search
//    with the canonical fp32 distance runs on the GPU.
//  * tsnecuda::util::PostprocessNeighborIndices (reference: src/util/distance_utils.cu:139-154).
#include "include/util/distance_utils.h"

namespace {
const int64_t *g_inj_ids = nullptr;
const float *g_inj_d2 = nullptr;
long long g_inj_n = 0;
int g_inj_k = 0;

__global__ void exact_knn_kernel(const float *__restrict__ X, int N, int D, int K, int64_t *ids, float *d2)
{
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= N) return;
    int64_t *oi = ids + (size_t)q * K;
    float *od = d2 + (size_t)q * K;
    int cnt = 0;
    const float *xq = X + (size_t)q * D;
    for (int j = 0; j < N; j++) {
        const float *xj = X + (size_t)j * D;
        float acc = 0.0f;
        for (int d = 0; d < D; d++) {
            float t = __fsub_rn(xq[d], xj[d]);
            acc = __fadd_rn(acc, __fmul_rn(t, t));
        }
        if (cnt == K && (acc > od[K - 1] || (acc == od[K - 1] && j > oi[K - 1]))) continue;
        int pos = (cnt < K) ? cnt : K - 1;
        while (pos > 0 && (od[pos - 1] > acc || (od[pos - 1] == acc && oi[pos - 1] > j))) {
            od[pos] = od[pos - 1];
            oi[pos] = oi[pos - 1];
            pos--;
        }
        od[pos] = acc;
        oi[pos] = j;
        if (cnt < K) cnt++;
    }
}

__global__ void narrow_ids_kernel(int *out, const long *in, size_t n)
{
    size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (t < n) out[t] = (int)in[t];
}
} // namespace

extern "C" void ref_set_knn(const int64_t *ids, const float *d2, long long n, int k)
{
    g_inj_ids = ids; g_inj_d2 = d2; g_inj_n = n; g_inj_k = k;
}

void tsnecuda::util::KNearestNeighbors(tsnecuda::GpuOptions &gpu_opt, tsnecuda::Options &base_opt,
                                       int64_t *indices, float *distances, const float *const points,
                                       const int num_dims, const int num_points, const int num_near_neighbors)
{
    (void)gpu_opt; (void)base_opt;
    const size_t nk = (size_t)num_points * num_near_neighbors;
    if (g_inj_ids != nullptr && g_inj_n == num_points && g_inj_k == num_near_neighbors) {
        memcpy(indices, g_inj_ids, nk * sizeof(int64_t));
        memcpy(distances, g_inj_d2, nk * sizeof(float));
        return;
    }
    thrust::device_vector<float> X(points, points + (size_t)num_points * num_dims);
    thrust::device_vector<int64_t> ids(nk);
    thrust::device_vector<float> d2(nk);
    exact_knn_kernel<<<(num_points + 127) / 128, 128>>>(thrust::raw_pointer_cast(X.data()), num_points, num_dims,
                                                       num_near_neighbors, thrust::raw_pointer_cast(ids.data()),
                                                       thrust::raw_pointer_cast(d2.data()));
    GpuErrorCheck(cudaDeviceSynchronize());
    thrust::copy(ids.begin(), ids.end(), indices);
    thrust::copy(d2.begin(), d2.end(), distances);
}

void tsnecuda::util::PostprocessNeighborIndices(tsnecuda::GpuOptions &gpu_opt, thrust::device_vector<int> &indices,
                                                thrust::device_vector<int64_t> &long_indices, const int num_points,
                                                const int num_neighbors)
{
    (void)gpu_opt;
    const size_t n = (size_t)num_points * num_neighbors;
    narrow_ids_kernel<<<(unsigned)((n + 255) / 256), 256>>>(thrust::raw_pointer_cast(indices.data()),
                                                            (const long *)thrust::raw_pointer_cast(long_indices.data()), n);
    GpuErrorCheck(cudaDeviceSynchronize());
}
