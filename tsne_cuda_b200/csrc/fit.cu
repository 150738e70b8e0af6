// tsnecuda::RunTsne, pymodule_tsne and b200tsne_fit: the drop-in entry points.
//
// Replaces the reference's orchestrator (src/fit_tsne.cu:16-627) and its ctypes shim
// (src/ext/pymodule_ext.cu:6-123).  The phases, their order, the progress messages and the
// "_time_*" lines printed at verbosity > 0 (which the reference's tuning harness parses) are kept;
// everything between host X and host Y stays on the device.
#include <chrono>
#include <thread>
#include <fstream>
#include <iostream>
#include <random>
#include <vector>

#include "../../include/tsnecuda/fit_tsne.h"
#include "../../include/tsnecuda_b200.h"
#include "session.h"

namespace tsnecuda {

bool Options::validate()
{
    if (points == nullptr || num_points == 0 || num_dims == 0) return false;
    if (num_snapshots < 2 && return_style == RETURN_STYLE::SNAPSHOT) {
        std::cout << "E: Need to record more than 1 snapshot when using snapshot capture. Use 'once' capture if you "
                     "only want one return."
                  << std::endl;
        return false;
    }
    return true;
}

GpuOptions::GpuOptions(int device_) : device(device_)
{
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_) == cudaSuccess) {
        warp_size = prop.warpSize;
        sm_count = prop.multiProcessorCount;
    }
    cudaSetDevice(device_);
}

namespace {
// Where the embedding goes while the loop runs (the reference's live visualisation feed, src/fit_tsne.cu:354-389 and
// :546-561, without the socket): set for the calling thread by b200tsne_fit_with_frames around one run.
struct FrameSink {
    int (*send)(void *user, const void *data, size_t bytes) = nullptr;
    void *user = nullptr;
    int every = 1;
};
thread_local FrameSink g_frames;

struct PhaseTimer {
    std::chrono::high_resolution_clock::time_point t0 = std::chrono::high_resolution_clock::now();
    double lap()
    {
        auto t1 = std::chrono::high_resolution_clock::now();
        double s = std::chrono::duration<double>(t1 - t0).count();
        t0 = t1;
        return s;
    }
};

// Initial embedding exactly as the reference draws it (src/fit_tsne.cu:181-235): the engine is
// seeded with random_seed, 2N normal draws are consumed for a vector the reference never uses,
// then GAUSSIAN takes the next 2N draws times 1e-4, UNIFORM takes 2N uniform draws in [-5, 5).
int initial_embedding(const Options &opt, std::vector<float> &y)
{
    const size_t n2 = (size_t)opt.num_points * 2;
    y.resize(n2);
    std::default_random_engine generator(opt.random_seed);
    std::normal_distribution<float> normal(0.0, 1.0);
    for (size_t i = 0; i < n2; i++) (void)normal(generator);
    switch (opt.initialization) {
        case TSNE_INIT::UNIFORM: {
            std::uniform_real_distribution<float> uni(-5, 5);
            for (size_t i = 0; i < n2; i++) y[i] = uni(generator);
            return 0;
        }
        case TSNE_INIT::GAUSSIAN:
            for (size_t i = 0; i < n2; i++) y[i] = 0.0001 * normal(generator);
            return 0;
        case TSNE_INIT::RESUME:
        case TSNE_INIT::VECTOR:
            if (opt.preinit_data == nullptr) {
                b200::set_error("Invalid initialization. Initialization points are null.");
                return -1;
            }
            for (size_t i = 0; i < n2; i++) y[i] = opt.preinit_data[i];
            return 0;
        default:
            b200::set_error("Invalid initialization type specified.");
            return -1;
    }
}

int run(Options &opt, GpuOptions &gpu_opt)
{
    double t_init = 0, t_knn = 0, t_sym = 0, t_lowdim = 0, t_fft = 0, t_loop = 0;
    PhaseTimer timer;
    const bool verbose = opt.verbosity > 0;
    if (verbose) std::cout << "Initializing cuda handles... " << std::flush;

    const int N = opt.num_points;
    const int K = (opt.num_neighbors < N) ? opt.num_neighbors : N;
    if (K <= 0) { b200::set_error("num_neighbors must be positive"); return -1; }
    b200::Session s;
    struct Guard { b200::Session &s; ~Guard() { s.destroy(); } } guard{s};
    B200_TRY(s.init(N, K, 0, N, gpu_opt.device));
    s.eta = opt.learning_rate;
    s.exaggeration = opt.early_exaggeration;
    s.pre_momentum = opt.pre_exaggeration_momentum;
    s.post_momentum = opt.post_exaggeration_momentum;
    s.force_magnify_iters = opt.force_magnify_iters;
    if (getenv("B200TSNE_STAGE_TIMERS") && atoi(getenv("B200TSNE_STAGE_TIMERS")) != 0) s.stage_timers = true;
    t_init = timer.lap();

    if (verbose) std::cout << "done.\nKNN Computation... " << std::flush;
    // The initial embedding is drawn on the host (the reference's generator and draw order, 4N normal
    // draws): a host thread does that while the device searches the neighbours.
    std::vector<float> y0;
    std::string y0_error;
    int y0_rc = 0;
    std::thread y0_thread([&]() {
        y0_rc = initial_embedding(opt, y0);
        if (y0_rc != 0) y0_error = b200::last_error();
    });
    // kNN, max-normalisation, perplexity search and symmetrisation run back to back on the device;
    // the split between the two printed phases is only meaningful with stage timers on.
    const int aff_rc = s.affinities_from_points(opt.points, opt.num_dims, opt.perplexity, opt.perplexity_search_epsilon);
    y0_thread.join();
    if (aff_rc != 0) return aff_rc;
    if (verbose) std::cout << "done.\nComputing Pij matrix... " << std::endl;
    const double t_aff = timer.lap();
    if (s.stage_timers) {
        t_knn = s.stage_ms[b200::kStKnn] * 1e-3;
        t_sym = t_aff - t_knn;
    } else {
        t_knn = t_aff;
    }

    if (verbose) std::cout << "done.\nInitializing low dim points... " << std::flush;
    if (y0_rc != 0) { b200::set_error(y0_error); return y0_rc; }
    B200_TRY(s.set_embedding_soa(y0.data(), true));
    t_lowdim = timer.lap();
    if (verbose) std::cout << "done.\nInitializing CUDA memory... " << std::flush;

    std::ofstream dump_file;
    std::vector<float> host_ys;
    if (opt.get_dump_points()) {
        dump_file.open(opt.get_dump_file());
        host_ys.resize((size_t)N * 2);
        dump_file << N << " " << 2 << std::endl;
    }
    // The reference's feed: first the number of points as decimal text, then after every iteration the raw
    // embedding (2N floats, x block then y block); a send that fails ends the feed, not the run.
    FrameSink frames = g_frames;
    std::vector<float> frame_buf;
    if (frames.send) {
        const std::string hello = std::to_string(N);
        if (frames.send(frames.user, hello.data(), hello.size()) != 0) {
            std::cout << "No Visualization Terminal, continuing..." << std::endl;
            frames.send = nullptr;
        } else {
            frame_buf.resize((size_t)N * 2);
        }
    } else if (opt.get_use_interactive()) {
        std::cout << "This version is not built with ZMQ for interative viz. Rebuild with WITH_ZMQ=TRUE for viz."
                  << std::endl;
    }
    if (verbose) std::cout << "done." << std::endl;
    t_fft = timer.lap();

    int snap_num = 0, snap_interval = 1;
    if (opt.return_style == RETURN_STYLE::SNAPSHOT) snap_interval = std::max(1, opt.iterations / (opt.num_snapshots - 1));

    // The loop runs in chunks that end where the host has something to do.  The reference does its
    // host work (print, dump, snapshot) right after every iteration whose index is a multiple of the
    // respective interval (src/fit_tsne.cu:539-579); such an iteration runs as a chunk of one, all
    // others run asynchronously up to the next such index.
    const int print_iv = std::max(1, opt.print_interval), dump_iv = std::max(1, opt.get_dump_interval());
    const bool want_print = opt.verbosity >= 1;
    const bool want_dump = opt.get_dump_points();
    const bool want_snap = opt.return_style == RETURN_STYLE::SNAPSHOT && opt.return_data != nullptr;
    const int frame_iv = std::max(1, frames.every);
    auto host_work_after = [&](long long st) {
        return (want_print && st % print_iv == 0) || (want_dump && st % dump_iv == 0) ||
               (want_snap && st % snap_interval == 0) || (frames.send && st % frame_iv == 0);
    };
    auto next_multiple = [](long long st, long long iv) { return (st / iv + 1) * iv; };
    float loop_ms = 0.0f;
    long long step = 0;
    const long long total = opt.iterations;  // negative: run until the gradient-norm stop ends the loop
    while (total < 0 || step < total) {
        long long stop = total < 0 ? step + 1000 : total;
        const bool alone = host_work_after(step);
        if (alone) {
            stop = step + 1;
        } else {
            if (want_print) stop = std::min(stop, next_multiple(step, print_iv));
            if (want_dump) stop = std::min(stop, next_multiple(step, dump_iv));
            if (want_snap) stop = std::min(stop, next_multiple(step, snap_interval));
            if (frames.send) stop = std::min(stop, next_multiple(step, frame_iv));
        }
        int done = 0;
        float ms = 0.0f;
        s.force_norm = alone && want_print && step % print_iv == 0;
        B200_TRY(s.iterate((int)(stop - step), opt.min_gradient_norm, &ms, &done));
        loop_ms += ms;
        const long long first = step;
        step += done;
        if (opt.min_gradient_norm > 0.0f && done > 0 && s.last_unorm < opt.min_gradient_norm) {
            if (opt.verbosity >= 1) std::cout << "Reached minimum gradient norm: " << s.last_unorm << std::endl;
            break;
        }
        if (!alone) continue;
        // the reference prints the 2-norm of the update vector under this label (fit_tsne.cu:539-542)
        if (want_print && first % print_iv == 0)
            std::cout << "[Step " << first << "] Avg. Gradient Norm: " << s.last_unorm << std::endl;
        if (frames.send && first % frame_iv == 0) {
            B200_TRY(s.get_embedding_soa(frame_buf.data()));
            if (frames.send(frames.user, frame_buf.data(), sizeof(float) * frame_buf.size()) != 0) {
                std::cout << "Server Disconnected, Not sending anymore for this session." << std::endl;
                frames.send = nullptr;
            }
        }
        if (want_dump && first % dump_iv == 0) {
            B200_TRY(s.get_embedding_soa(host_ys.data()));
            for (int i = 0; i < N; i++) dump_file << host_ys[i] << " " << host_ys[i + N] << std::endl;
        }
        if (want_snap && first % snap_interval == 0 && snap_num < opt.num_snapshots - 1) {
            B200_TRY(s.get_embedding_soa(opt.return_data + (size_t)snap_num * N * 2));
            snap_num++;
        }
    }
    t_loop = loop_ms * 1e-3;
    (void)timer.lap();

    if (verbose) {
        auto pr = [](const char *name, double v) { std::cout << name << ": " << (float)v << "s" << std::endl; };
        pr("_time_initialization", t_init);
        pr("_time_knn", t_knn);
        pr("_time_symmetry", t_sym);
        pr("_time_init_low_dim", t_lowdim);
        pr("_time_init_fft", t_fft);
        pr("_time_compute_charges", 0.0);
        pr("_time_precompute_2d", 0.0);
        pr("_time_nbodyfft", (s.stage_ms[b200::kStSpread] + s.stage_ms[b200::kStConvolve]) * 1e-3);
        pr("_time_norm", s.stage_ms[b200::kStGather] * 1e-3);
        pr("_time_attr", s.stage_ms[b200::kStAttractive] * 1e-3);
        pr("_time_apply_forces", s.stage_ms[b200::kStUpdate] * 1e-3);
        pr("_time_other", 0.0);
        pr("total_time", t_init + t_knn + t_sym + t_lowdim + t_fft + t_loop);
    }
    if (opt.get_dump_points()) dump_file.close();

    if (opt.return_data != nullptr) {
        if (opt.return_style == RETURN_STYLE::ONCE) B200_TRY(s.get_embedding_soa(opt.return_data));
        else B200_TRY(s.get_embedding_soa(opt.return_data + (size_t)snap_num * N * 2));
    }
    opt.trained = true;
    opt.trained_norm = s.last_Z;
    return 0;
}
}  // namespace

void RunTsne(Options &opt, GpuOptions &gpu_opt)
{
    if (!opt.validate()) {
        std::cout << "E: Invalid options file. Terminating." << std::endl;
        return;
    }
    if (run(opt, gpu_opt) != 0) std::cerr << "E: " << b200::last_error() << std::endl;
}

}  // namespace tsnecuda

// ------------------------------------------------------------------------------------------------
extern "C" {

void b200tsne_default_options(b200tsne_options *o)
{
    if (!o) return;
    tsnecuda::Options d;
    o->perplexity = d.perplexity;
    o->learning_rate = d.learning_rate;
    o->early_exaggeration = d.early_exaggeration;
    o->num_neighbors = d.num_neighbors;
    o->iterations = d.iterations;
    o->force_magnify_iters = d.force_magnify_iters;
    o->perplexity_search_epsilon = d.perplexity_search_epsilon;
    o->pre_exaggeration_momentum = d.pre_exaggeration_momentum;
    o->post_exaggeration_momentum = d.post_exaggeration_momentum;
    o->min_gradient_norm = d.min_gradient_norm;
    o->initialization_type = 1;
    o->preinit_data = nullptr;
    o->random_seed = 0;
    o->verbosity = 0;
    o->print_interval = d.print_interval;
    o->gpu_device = 0;
    o->return_style = 0;
    o->num_snapshots = 0;
    o->dump_file = nullptr;
    o->dump_interval = 1;
}

int b200tsne_fit(const float *points, int64_t num_points, int num_dims, const b200tsne_options *o, float *result,
                 float *trained_norm)
{
    if (!points || !o || !result || num_points <= 0 || num_dims <= 0 || num_points > 2147483647LL) {
        b200::set_error("b200tsne_fit: invalid arguments");
        return B200TSNE_ERR_INVALID;
    }
    if (o->initialization_type < 0 || o->initialization_type > 3) {
        b200::set_error("Invalid initialization supplied");
        return B200TSNE_ERR_INVALID;
    }
    if (o->return_style != 0 && o->return_style != 1) {
        b200::set_error("Invalid return style supplied");
        return B200TSNE_ERR_INVALID;
    }
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || o->gpu_device < 0 || o->gpu_device >= n_dev) {
        b200::set_error("no such CUDA device");
        return B200TSNE_ERR_CUDA;
    }
    tsnecuda::GpuOptions gpu_opt(o->gpu_device);
    tsnecuda::Options opt(result, const_cast<float *>(points), (int)num_points, num_dims);
    opt.perplexity = o->perplexity;
    opt.learning_rate = o->learning_rate;
    opt.early_exaggeration = o->early_exaggeration;
    opt.num_neighbors = o->num_neighbors;
    opt.iterations = o->iterations;
    opt.force_magnify_iters = o->force_magnify_iters;
    opt.perplexity_search_epsilon = o->perplexity_search_epsilon;
    opt.pre_exaggeration_momentum = o->pre_exaggeration_momentum;
    opt.post_exaggeration_momentum = o->post_exaggeration_momentum;
    opt.min_gradient_norm = o->min_gradient_norm;
    opt.initialization = (tsnecuda::TSNE_INIT)o->initialization_type;
    opt.preinit_data = const_cast<float *>(o->preinit_data);
    if (o->random_seed != 0) opt.random_seed = o->random_seed;
    opt.verbosity = o->verbosity;
    opt.print_interval = o->print_interval;
    opt.return_style = (tsnecuda::RETURN_STYLE)o->return_style;
    opt.num_snapshots = o->num_snapshots;
    if (o->dump_file) opt.enable_dump(std::string(o->dump_file), o->dump_interval);
    if (!opt.validate()) {
        b200::set_error("Invalid options file.");
        return B200TSNE_ERR_INVALID;
    }
    const int rc = tsnecuda::run(opt, gpu_opt);
    if (trained_norm) *trained_norm = opt.trained_norm;
    return rc;
}

int b200tsne_fit_with_frames(const float *points, int64_t num_points, int num_dims, const b200tsne_options *o, float *result,
                             float *trained_norm, b200tsne_frame_fn send, void *user, int every)
{
    if (!send || every <= 0) { b200::set_error("b200tsne_fit_with_frames: invalid arguments"); return B200TSNE_ERR_INVALID; }
    tsnecuda::g_frames.send = send;
    tsnecuda::g_frames.user = user;
    tsnecuda::g_frames.every = every;
    const int rc = b200tsne_fit(points, num_points, num_dims, o, result, trained_norm);
    tsnecuda::g_frames = tsnecuda::FrameSink();
    return rc;
}

void pymodule_tsne(float *result, float *points, ssize_t *dims, float perplexity, float learning_rate,
                   float early_exaggeration, float magnitude_factor, int num_neighbors, int iterations,
                   int iterations_no_progress, int force_magnify_iters, float perplexity_search_epsilon,
                   float pre_exaggeration_momentum, float post_exaggeration_momentum, float theta, float epssq,
                   float min_gradient_norm, int initialization_type, float *preinit_data, bool dump_points,
                   char *dump_file, int dump_interval, bool use_interactive, char *viz_server, int viz_timeout,
                   int verbosity, int print_interval, int gpu_device, int return_style, int num_snapshots,
                   int distance_metric)
{
    (void)magnitude_factor; (void)iterations_no_progress; (void)theta; (void)epssq; (void)viz_server;
    (void)viz_timeout; (void)distance_metric;
    b200tsne_options o;
    b200tsne_default_options(&o);
    o.perplexity = perplexity;
    o.learning_rate = learning_rate;
    o.early_exaggeration = early_exaggeration;
    o.num_neighbors = num_neighbors;
    o.iterations = iterations;
    o.force_magnify_iters = force_magnify_iters;
    o.perplexity_search_epsilon = perplexity_search_epsilon;
    o.pre_exaggeration_momentum = pre_exaggeration_momentum;
    o.post_exaggeration_momentum = post_exaggeration_momentum;
    o.min_gradient_norm = min_gradient_norm;
    o.verbosity = verbosity;
    o.print_interval = print_interval;
    o.gpu_device = gpu_device;
    o.return_style = return_style;
    o.num_snapshots = num_snapshots;
    if (initialization_type == 2) {
        std::cerr << "E: RESUME initialization not yet supported fully..." << std::endl;  // pymodule_ext.cu:78-81
        return;
    }
    o.initialization_type = initialization_type;
    o.preinit_data = (initialization_type == 3) ? preinit_data : nullptr;
    if (dump_points) { o.dump_file = dump_file; o.dump_interval = dump_interval; }
    if (use_interactive)
        std::cout << "This version is not built with ZMQ for interative viz. Rebuild with WITH_ZMQ=TRUE for viz."
                  << std::endl;
    if (!dims) { std::cerr << "E: Invalid options file. Terminating." << std::endl; return; }
    if (b200tsne_fit(points, (int64_t)dims[0], (int)dims[1], &o, result, nullptr) != 0)
        std::cerr << "E: " << b200::last_error() << std::endl;
    cudaDeviceSynchronize();
}

}  // extern "C"
