// A C++ caller of the drop-in entry point, written against the reference's public interface
// (src/include/fit_tsne.h:33-35, src/include/options.h; the reference's own caller is src/exe/main.cu:174-217):
// two Gaussian blobs, RunTsne, then the fields the reference fills in.  Compiled by tests/test_cpp_caller.py
// against include/tsnecuda/ and linked with -ltsnecuda.
#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

#include "tsnecuda/fit_tsne.h"

int main(int argc, char **argv)
{
    const int n = 3000, d = 24, iterations = argc > 1 ? std::atoi(argv[1]) : 300;
    std::vector<float> x((size_t)n * d), y((size_t)n * 2, 0.0f);
    std::default_random_engine gen(1);
    std::normal_distribution<float> blob_a(-10.0f, 1.0f), blob_b(10.0f, 1.0f);
    for (int i = 0; i < n; i++)
        for (int k = 0; k < d; k++) x[(size_t)i * d + k] = (i < n / 2) ? blob_a(gen) : blob_b(gen);

    tsnecuda::GpuOptions gpu_opt(0);
    tsnecuda::Options opt(y.data(), x.data(), n, d);
    opt.perplexity = 30.0f;
    opt.num_neighbors = 90;
    opt.iterations = iterations;
    opt.verbosity = 0;
    opt.random_seed = 7;
    opt.initialization = tsnecuda::TSNE_INIT::GAUSSIAN;
    opt.return_style = tsnecuda::RETURN_STYLE::ONCE;
    if (!opt.validate()) { std::printf("invalid options\n"); return 2; }
    tsnecuda::RunTsne(opt, gpu_opt);
    if (!opt.trained) { std::printf("not trained\n"); return 3; }

    // the two blobs must end up apart: compare the blob centres with the spread inside a blob
    double ca[2] = {0, 0}, cb[2] = {0, 0};
    for (int i = 0; i < n; i++) {
        double *c = (i < n / 2) ? ca : cb;
        c[0] += y[i];
        c[1] += y[n + i];
    }
    for (int k = 0; k < 2; k++) { ca[k] /= n / 2; cb[k] /= n - n / 2; }
    double spread = 0;
    bool finite = true;
    for (int i = 0; i < n; i++) {
        const double *c = (i < n / 2) ? ca : cb;
        spread += std::hypot(y[i] - c[0], y[n + i] - c[1]);
        finite = finite && std::isfinite(y[i]) && std::isfinite(y[n + i]);
    }
    spread /= n;
    const double apart = std::hypot(ca[0] - cb[0], ca[1] - cb[1]);
    std::printf("trained=%d trained_norm=%g finite=%d apart=%g spread=%g\n", (int)opt.trained, opt.trained_norm, (int)finite, apart,
                spread);
    return (finite && opt.trained_norm > 0.0f && apart > 2.0 * spread) ? 0 : 4;
}
