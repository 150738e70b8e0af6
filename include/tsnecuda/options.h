// Source-compatible stand-ins for the reference's option carriers, so that C++ callers of
// tsnecuda::RunTsne(Options&, GpuOptions&) compile against this library unchanged.
//
// Replaces: src/include/options.h:18-376 of the reference (same namespace, type names, public
// field names, defaults, constructors and helper methods).  Fields that the reference carries but
// never reads (theta, epssq, magnitude_factor, iterations_no_progress, distance_metric, the
// Barnes-Hut launch factors of GpuOptions) are kept and ignored here as well.
#ifndef TSNECUDA_B200_OPTIONS_H_
#define TSNECUDA_B200_OPTIONS_H_

#include <ctime>
#include <string>

#if defined(__has_include)
#if __has_include(<faiss/MetricType.h>)
#include <faiss/MetricType.h>
#define TSNECUDA_B200_HAVE_FAISS_METRIC 1
#endif
#endif
#ifndef TSNECUDA_B200_HAVE_FAISS_METRIC
// The reference stores a faiss::MetricType in Options; FAISS is not needed by this library, so a
// value-compatible enum stands in when its header is absent.
namespace faiss {
enum MetricType { METRIC_INNER_PRODUCT = 0, METRIC_L2 = 1, METRIC_L1 = 2, METRIC_Linf = 3, METRIC_Lp = 4,
                  METRIC_Canberra = 20, METRIC_BrayCurtis = 21, METRIC_JensenShannon = 22 };
}
#endif

namespace tsnecuda {

enum TSNE_INIT { UNIFORM, GAUSSIAN, RESUME, VECTOR };
enum RETURN_STYLE { ONCE, SNAPSHOT };
enum DISTANCE_METRIC { INNER_PRODUCT, L2, L1, LINF, CANBERRA, BRAYCURTIS, JENSENSHANNON };

class Options {
  private:
    bool dump_points = false;
    int dump_interval = 100;
    std::string dump_file = "";
    bool use_interactive = false;
    std::string viz_server = "tcp://localhost:5556";
    int viz_timeout = 10000;

  public:
    // required
    float *points = nullptr;   // host, [num_points][num_dims] row-major
    int num_points = 0;
    int num_dims = 0;

    // optimisation
    float perplexity = 50.0f;
    float learning_rate = 200.0f;
    float early_exaggeration = 12.0f;
    float magnitude_factor = 5.0f;
    int num_neighbors = 1023;
    int iterations = 1000;
    int iterations_no_progress = 1000;
    int force_magnify_iters = 250;
    float perplexity_search_epsilon = 1e-4f;
    float pre_exaggeration_momentum = 0.5f;
    float post_exaggeration_momentum = 0.8f;
    float theta = 0.5f;
    float epssq = 0.05f * 0.05f;
    float min_gradient_norm = 0.0f;
    faiss::MetricType distance_metric = faiss::METRIC_INNER_PRODUCT;

    // initialisation
    TSNE_INIT initialization = TSNE_INIT::GAUSSIAN;
    float *preinit_data = nullptr;   // host, 2*num_points floats, x block then y block

    // reporting
    int verbosity = 20;
    int print_interval = 10;

    // output
    RETURN_STYLE return_style = RETURN_STYLE::ONCE;
    float *return_data = nullptr;    // host, 2*num_points floats (num_snapshots blocks for SNAPSHOT)
    int num_snapshots = 0;

    // results
    float trained_norm = -1.0f;
    bool trained = false;
    int random_seed = 0;

    Options() {}
    Options(float *return_data, float *points, int num_points, int num_dims)
        : points(points), num_points(num_points), num_dims(num_dims), return_data(return_data)
    {
        random_seed = (int)time(NULL);
    }
    Options(float *points, int num_points, int num_dims, float perplexity, float learning_rate, float magnitude_factor,
            int num_neighbors, int iterations, int iterations_no_progress, int force_magnify_iters,
            float perplexity_search_epsilon, float pre_exaggeration_momentum, float post_exaggeration_momentum,
            float theta, float epssq, float min_gradient_norm, TSNE_INIT initialization, float *preinit_data,
            bool dump_points, int dump_interval, RETURN_STYLE return_style, float *return_data, int num_snapshots,
            bool use_interactive, std::string viz_server, int verbosity, int print_interval,
            faiss::MetricType distance_metric)
        : dump_points(dump_points), dump_interval(dump_interval), use_interactive(use_interactive),
          viz_server(viz_server), points(points), num_points(num_points), num_dims(num_dims), perplexity(perplexity),
          learning_rate(learning_rate), magnitude_factor(magnitude_factor), num_neighbors(num_neighbors),
          iterations(iterations), iterations_no_progress(iterations_no_progress),
          force_magnify_iters(force_magnify_iters), perplexity_search_epsilon(perplexity_search_epsilon),
          pre_exaggeration_momentum(pre_exaggeration_momentum), post_exaggeration_momentum(post_exaggeration_momentum),
          theta(theta), epssq(epssq), min_gradient_norm(min_gradient_norm), distance_metric(distance_metric),
          initialization(initialization), preinit_data(preinit_data), verbosity(verbosity),
          print_interval(print_interval), return_style(return_style), return_data(return_data),
          num_snapshots(num_snapshots)
    {
        random_seed = (int)time(NULL);
    }

    bool enable_dump(std::string filename, int interval = 1)
    {
        dump_points = true;
        dump_file = filename;
        dump_interval = interval;
        return true;
    }
    bool enable_viz(std::string server_address = "tcp://localhost:5556", int timeout = 10000)
    {
        use_interactive = true;
        viz_server = server_address;
        viz_timeout = timeout;
        return true;
    }
    // Same acceptance rule as the reference (options.h:163-180).
    bool validate();

    bool get_dump_points() { return dump_points; }
    std::string get_dump_file() { return dump_file; }
    int get_dump_interval() { return dump_interval; }
    bool get_use_interactive() { return use_interactive; }
    int get_viz_timeout() { return viz_timeout; }
    std::string get_viz_server() { return viz_server; }
};

// Device selection and launch hints.  The launch-shape fields exist for source compatibility; the
// kernels of this library choose their own shapes.  Constructing a GpuOptions makes `device` the
// current CUDA device, as in the reference (options.h:222-229).
class GpuOptions {
  public:
    int device = 0;
    int integration_kernel_threads = 1024;
    int integration_kernel_factor = 1;
    int fft_kernel_threads = 128;
    int attr_kernel_threads = 1024;
    int rep_kernel_threads = 1024;
    int repulsive_kernel_threads = 256;
    int repulsive_kernel_factor = 5;
    int bounding_kernel_threads = 512;
    int bounding_kernel_factor = 3;
    int tree_kernel_threads = 1024;
    int tree_kernel_factor = 2;
    int sort_kernel_threads = 64;
    int sort_kernel_factor = 6;
    int summary_kernel_threads = 128;
    int summary_kernel_factor = 6;
    int warp_size = 32;
    int sm_count = 0;

    explicit GpuOptions(int device);
};

}  // namespace tsnecuda
#endif
