// Stage-level entry points into the reference's own host wrappers, for parity tests and golden
// fixtures.  Test infrastructure: linked only into oracle/_ref/libtsnecuda_ref.so.  Every function
// takes host pointers, fills thrust device vectors, calls the reference's wrapper(s) with the
// argument lists the reference's orchestrator uses (src/fit_tsne.cu, cited per function) and
// copies the results back.
#include "include/fit_tsne.h"
#include "include/kernels/apply_forces.h"
#include "include/kernels/attr_forces.h"
#include "include/kernels/nbodyfft.h"
#include "include/kernels/perplexity_search.h"
#include "include/kernels/rep_forces.h"
#include "include/util/math_utils.h"

namespace {
template <class T> T *raw(thrust::device_vector<T> &v) { return thrust::raw_pointer_cast(v.data()); }
}

// src/fit_tsne.cu:125-127 (MaxNormalizeDeviceVector), in place on a host array.
extern "C" void ref_max_normalize(float *d2, long long n)
{
    thrust::device_vector<float> d(d2, d2 + n);
    tsnecuda::util::MaxNormalizeDeviceVector(d);
    thrust::copy(d.begin(), d.end(), d2);
}

// src/fit_tsne.cu:138-140 (SearchPerplexity) on already max-normalised distances.
extern "C" void ref_perplexity(const float *dhat, int N, int K, float perplexity, float eps, float *p_out)
{
    tsnecuda::GpuOptions gpu_opt(0);
    cublasHandle_t handle;
    CublasSafeCall(cublasCreate(&handle));
    thrust::device_vector<float> d(dhat, dhat + (size_t)N * K);
    thrust::device_vector<float> p((size_t)N * K);
    tsnecuda::SearchPerplexity(gpu_opt, handle, p, d, perplexity, eps, N, K);
    cudaDeviceSynchronize();
    thrust::copy(p.begin(), p.end(), p_out);
    cublasDestroy(handle);
}

// src/fit_tsne.cu:152-153 (SymmetrizeMatrixV2).
extern "C" void ref_symmetrize(const float *p, const int *ids, int N, int K, float *P_out)
{
    thrust::device_vector<float> pd(p, p + (size_t)N * K), out((size_t)N * K);
    thrust::device_vector<int> id(ids, ids + (size_t)N * K);
    tsnecuda::util::SymmetrizeMatrixV2(out, pd, id, N, K);
    thrust::copy(out.begin(), out.end(), P_out);
}

// src/fit_tsne.cu:487-496 (ComputeAttractiveForcesV3). Y and F are SoA [2][N].
extern "C" void ref_attractive(const float *P, const int *ids, const float *Y, int N, int K, float *F_out)
{
    tsnecuda::GpuOptions gpu_opt(0);
    cublasHandle_t handle;
    CublasSafeCall(cublasCreate(&handle));
    thrust::device_vector<float> pd(P, P + (size_t)N * K), ws((size_t)N * K * 2), y(Y, Y + 2 * (size_t)N);
    thrust::device_vector<float> f(2 * (size_t)N, 0.0f), ones(2 * (size_t)N, 1.0f);
    thrust::device_vector<int> id(ids, ids + (size_t)N * K);
    tsnecuda::ComputeAttractiveForcesV3(handle, gpu_opt, f, pd, id, ws, y, ones, N, K);
    cudaDeviceSynchronize();
    thrust::copy(f.begin(), f.end(), F_out);
    cublasDestroy(handle);
}

// One repulsive evaluation with the call sequence of src/fit_tsne.cu:246-342 (constants, buffers,
// plans) and :411-469 (charges, min/max, PrecomputeFFT2D, NbodyFFT2D, ComputeRepulsiveForces).
// Outputs: Frep SoA [2][N], Z (= sum Z_i - N), and optionally w [G][G][4], ytilde [G][G][4], phi [N][4].
extern "C" void ref_repulsive(const float *Y, int N, float *Frep, float *Z_out, float *w_out, float *ytilde_out,
                              float *phi_out)
{
    tsnecuda::GpuOptions gpu_opt(0);
    const int n_interpolation_points = 3, n_terms = 4, n_boxes_per_dim = 130;
    const int n_total_boxes = n_boxes_per_dim * n_boxes_per_dim;
    const int total_interpolation_points = n_total_boxes * n_interpolation_points * n_interpolation_points;
    const int n_fft_coeffs_half = n_interpolation_points * n_boxes_per_dim;
    const int n_fft_coeffs = 2 * n_fft_coeffs_half;
    const int n_interpolation_points_1d = n_fft_coeffs_half;
    const size_t big = (size_t)n_terms * n_interpolation_points * n_interpolation_points * N;

    thrust::device_vector<float> points(Y, Y + 2 * (size_t)N);
    thrust::device_vector<int> point_box_idx(N);
    thrust::device_vector<float> x_in_box(N), y_in_box(N);
    thrust::device_vector<float> y_tilde_values((size_t)total_interpolation_points * n_terms);
    thrust::device_vector<float> x_interp((size_t)N * n_interpolation_points), y_interp((size_t)N * n_interpolation_points);
    thrust::device_vector<float> potentials((size_t)N * n_terms, 0.0f);
    thrust::device_vector<float> w_coefficients((size_t)total_interpolation_points * n_terms, 0.0f);
    thrust::device_vector<float> all_interp_values(1), output_values(1);     // unused by the wrapper
    thrust::device_vector<int> all_interp_indices(1), output_indices(1);     // unused by the wrapper
    (void)big;
    thrust::device_vector<float> charges((size_t)N * n_terms);
    thrust::device_vector<float> box_lower(2 * n_total_boxes), box_upper(2 * n_total_boxes);
    thrust::device_vector<float> kernel_tilde((size_t)n_fft_coeffs * n_fft_coeffs);
    thrust::device_vector<thrust::complex<float>> fft_kernel_tilde((size_t)n_fft_coeffs * n_fft_coeffs);
    thrust::device_vector<float> fft_input((size_t)n_terms * n_fft_coeffs * n_fft_coeffs);
    thrust::device_vector<thrust::complex<float>> fft_w((size_t)n_terms * n_fft_coeffs * (n_fft_coeffs / 2 + 1));
    thrust::device_vector<float> fft_output((size_t)n_terms * n_fft_coeffs * n_fft_coeffs);
    thrust::device_vector<float> rep(2 * (size_t)N, 0.0f), norm_vec(N);

    float h = 1 / (float)n_interpolation_points;
    float spacings[3], denominator[3];
    spacings[0] = h / 2;
    for (int i = 1; i < 3; i++) spacings[i] = spacings[i - 1] + h;
    for (int i = 0; i < 3; i++) {
        denominator[i] = 1;
        for (int j = 0; j < 3; j++)
            if (i != j) denominator[i] *= spacings[i] - spacings[j];
    }
    thrust::device_vector<float> spacings_d(spacings, spacings + 3), denominator_d(denominator, denominator + 3);

    cufftHandle plan_kernel_tilde, plan_dft, plan_idft;
    CufftSafeCall(cufftCreate(&plan_kernel_tilde));
    CufftSafeCall(cufftCreate(&plan_dft));
    CufftSafeCall(cufftCreate(&plan_idft));
    size_t ws0, ws1, ws2;
    int dims[2] = {n_fft_coeffs, n_fft_coeffs};
    CufftSafeCall(cufftMakePlan2d(plan_kernel_tilde, dims[0], dims[1], CUFFT_R2C, &ws0));
    CufftSafeCall(cufftMakePlanMany(plan_dft, 2, dims, NULL, 1, n_fft_coeffs * n_fft_coeffs, NULL, 1,
                                    n_fft_coeffs * (n_fft_coeffs / 2 + 1), CUFFT_R2C, n_terms, &ws1));
    CufftSafeCall(cufftMakePlanMany(plan_idft, 2, dims, NULL, 1, n_fft_coeffs * (n_fft_coeffs / 2 + 1), NULL, 1,
                                    n_fft_coeffs * n_fft_coeffs, CUFFT_C2R, n_terms, &ws2));

    tsnecuda::ComputeChargesQij(gpu_opt, charges, points, N, n_terms);
    auto mm = thrust::minmax_element(points.begin(), points.end());
    float min_coord = mm.first[0];
    float max_coord = mm.second[0];
    tsnecuda::PrecomputeFFT2D(plan_kernel_tilde, max_coord, min_coord, max_coord, min_coord, n_boxes_per_dim,
                              n_interpolation_points, box_lower, box_upper, kernel_tilde, fft_kernel_tilde);
    float box_width = ((max_coord - min_coord) / (float)n_boxes_per_dim);
    tsnecuda::NbodyFFT2D(gpu_opt, plan_dft, plan_idft, N, n_terms, n_boxes_per_dim, n_interpolation_points,
                         fft_kernel_tilde, n_total_boxes, total_interpolation_points, min_coord, box_width,
                         n_fft_coeffs_half, n_fft_coeffs, fft_input, fft_w, fft_output, point_box_idx, x_in_box,
                         y_in_box, points, box_lower, spacings_d, denominator_d, y_tilde_values, all_interp_values,
                         output_values, all_interp_indices, output_indices, w_coefficients, charges, x_interp,
                         y_interp, potentials);
    float Z = tsnecuda::ComputeRepulsiveForces(gpu_opt, rep, norm_vec, points, potentials, N, n_terms);
    cudaDeviceSynchronize();
    thrust::copy(rep.begin(), rep.end(), Frep);
    *Z_out = Z;
    if (w_out) thrust::copy(w_coefficients.begin(), w_coefficients.end(), w_out);
    if (ytilde_out) thrust::copy(y_tilde_values.begin(), y_tilde_values.end(), ytilde_out);
    if (phi_out) thrust::copy(potentials.begin(), potentials.end(), phi_out);
    CufftSafeCall(cufftDestroy(plan_kernel_tilde));
    CufftSafeCall(cufftDestroy(plan_dft));
    CufftSafeCall(cufftDestroy(plan_idft));
    (void)n_interpolation_points_1d;
}

// src/fit_tsne.cu:504-515 (ApplyForces); all arrays SoA [2][N], updated in place.
extern "C" void ref_apply_forces(float *Y, float *attr, float *rep, float *gains, float *old_forces, float eta,
                                 float normalization, float momentum, float exaggeration, int N)
{
    tsnecuda::GpuOptions gpu_opt(0);
    const size_t n2 = 2 * (size_t)N;
    thrust::device_vector<float> y(Y, Y + n2), a(attr, attr + n2), r(rep, rep + n2), g(gains, gains + n2),
        o(old_forces, old_forces + n2);
    tsnecuda::ApplyForces(gpu_opt, y, a, r, g, o, eta, normalization, momentum, exaggeration, N, gpu_opt.sm_count);
    cudaDeviceSynchronize();
    thrust::copy(y.begin(), y.end(), Y);
    thrust::copy(a.begin(), a.end(), attr);
    thrust::copy(r.begin(), r.end(), rep);
    thrust::copy(g.begin(), g.end(), gains);
    thrust::copy(o.begin(), o.end(), old_forces);
}

// The reference's whole entry point with a caller-chosen seed (Options::random_seed is a public field that
// its C symbol never sets: src/include/options.h:104, src/ext/pymodule_ext.cu).  With iterations = 0 the
// returned embedding is the initial one (src/fit_tsne.cu:181-235 draw order, :610-613 copy-out).
extern "C" void ref_run_seeded(float *points, int N, int D, int init_type, int seed, int iterations, int num_neighbors,
                               float perplexity, float *Y_out)
{
    tsnecuda::GpuOptions gpu_opt(0);
    tsnecuda::Options opt(Y_out, points, N, D);
    opt.random_seed = seed;
    opt.iterations = iterations;
    opt.num_neighbors = num_neighbors;
    opt.perplexity = perplexity;
    opt.verbosity = 0;
    opt.initialization = static_cast<tsnecuda::TSNE_INIT>(init_type);
    opt.return_style = tsnecuda::RETURN_STYLE::ONCE;
    tsnecuda::RunTsne(opt, gpu_opt);
}
