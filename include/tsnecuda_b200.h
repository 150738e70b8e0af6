/*
 * C ABI of the B200-native FIt-SNE engine (libtsnecuda.so).
 *
 * Plain pointers and sizes only.  Unless a function says "device", every pointer is HOST memory,
 * borrowed for the duration of the call.  Functions returning int return 0 on success and a
 * negative b200tsne_status otherwise; b200tsne_last_error() then describes the failure for the
 * calling thread.  Nothing in this library calls exit() or throws across the boundary.
 *
 * Layout conventions (same as the reference):
 *   X        [N][D] float32 row-major
 *   ids, d2  [N][K] (int32 neighbour ids, float32 squared distances), slot 0 is the point itself
 *   p, P     [N][K] float32, fixed-width rows aligned with ids
 *   Y, F, gains, old_forces   "SoA": 2N floats, x[0..N) followed by y[0..N)  (== numpy (N,2) F-order)
 *   w, ytilde  [390][390][4] float32, x-node index slowest, 4 charge terms innermost
 *
 * Each declaration cites the reference interface it replaces (paths relative to the reference
 * project root).
 */
#ifndef TSNECUDA_B200_H_
#define TSNECUDA_B200_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <sys/types.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200tsne_status {
    B200TSNE_OK = 0,
    B200TSNE_ERR_INVALID = -1,   /* bad argument / invalid options            */
    B200TSNE_ERR_CUDA = -2,      /* a CUDA runtime call failed                */
    B200TSNE_ERR_NUMERIC = -3,   /* NaN/Inf detected in the embedding         */
    B200TSNE_ERR_UNSUPPORTED = -4,
    B200TSNE_ERR_COMM = -5       /* multi-GPU communicator failure            */
} b200tsne_status;

/* Message for the last failure on the calling thread ("" if none). */
const char *b200tsne_last_error(void);
/* Library version, (major<<16)|(minor<<8)|patch. */
int b200tsne_version(void);

/* ------------------------------------------------------------------------------------------- *
 * The drop-in symbol.  Replaces: extern "C" void pymodule_tsne(...) of
 * src/include/ext/pymodule_ext.h:10-43 (implementation src/ext/pymodule_ext.cu:6-123), the one
 * symbol src/python/tsnecuda/TSNE.py:138-183 binds with ctypes.  Same 31 positional arguments,
 * same meaning.  Differences: errors print "E: ..." and return (result untouched) instead of
 * exit(1); k-nearest neighbours are exact.
 * ------------------------------------------------------------------------------------------- */
void pymodule_tsne(float *result, float *points, ssize_t *dims, float perplexity, float learning_rate,
                   float early_exaggeration, float magnitude_factor, int num_neighbors, int iterations,
                   int iterations_no_progress, int force_magnify_iters, float perplexity_search_epsilon,
                   float pre_exaggeration_momentum, float post_exaggeration_momentum, float theta, float epssq,
                   float min_gradient_norm, int initialization_type, float *preinit_data, bool dump_points,
                   char *dump_file, int dump_interval, bool use_interactive, char *viz_server, int viz_timeout,
                   int verbosity, int print_interval, int gpu_device, int return_style, int num_snapshots,
                   int distance_metric);

/* Status-returning form of the same call with a plain-C options block.
 * Replaces: tsnecuda::RunTsne(Options&, GpuOptions&) (src/include/fit_tsne.h:33-35,
 * src/fit_tsne.cu:16-627) for callers that cannot use the C++ header. */
typedef struct b200tsne_options {
    float perplexity;                  /* Options::perplexity              (options.h:66) */
    float learning_rate;
    float early_exaggeration;
    int num_neighbors;
    int iterations;
    int force_magnify_iters;
    float perplexity_search_epsilon;
    float pre_exaggeration_momentum;
    float post_exaggeration_momentum;
    float min_gradient_norm;
    int initialization_type;           /* 0 UNIFORM, 1 GAUSSIAN, 2 RESUME, 3 VECTOR (options.h:20-26) */
    const float *preinit_data;         /* SoA 2N floats when initialization_type is 2 or 3           */
    int random_seed;                   /* Options::random_seed (options.h:104); 0 = seed from the clock, as the reference's constructors do */
    int verbosity;
    int print_interval;
    int gpu_device;
    int return_style;                  /* 0 ONCE, 1 SNAPSHOT (options.h:28-32)                       */
    int num_snapshots;
    const char *dump_file;             /* NULL = no dump (Options::enable_dump, options.h:149-155)   */
    int dump_interval;
} b200tsne_options;

void b200tsne_default_options(b200tsne_options *opt);
/* result: 2N floats SoA (num_snapshots blocks of 2N for SNAPSHOT).  trained_norm (may be NULL)
 * receives the last normalisation Z (Options::trained_norm, src/fit_tsne.cu:624). */
int b200tsne_fit(const float *points, int64_t num_points, int num_dims, const b200tsne_options *opt,
                 float *result, float *trained_norm);

/* The reference's live feed of the embedding without its socket.  The reference (built WITH_ZMQ) connects a
 * REQ socket to its plotting server, sends the number of points as decimal text, and after every iteration
 * sends the embedding as raw float32 (2N values, x block then y block), each time waiting for the server's
 * reply; a send or reply that fails ends the feed, not the run (src/fit_tsne.cu:354-389, :546-561; server:
 * visualization/vis_rt.py:8-38).  Here the same frames go to a callback: first the text frame, then one
 * embedding frame after every `every`-th iteration (the reference: every = 1).  The callback returns 0 for
 * "received" and anything else for "gone"; it is called on the calling thread and must not call back into the
 * library.  A socket, a file or a plotting front end is the caller's side. */
typedef int (*b200tsne_frame_fn)(void *user, const void *data, size_t bytes);
int b200tsne_fit_with_frames(const float *points, int64_t num_points, int num_dims, const b200tsne_options *opt,
                             float *result, float *trained_norm, b200tsne_frame_fn send, void *user, int every);

/* ------------------------------------------------------------------------------------------- *
 * Stage entry points with host buffers (one call = upload, kernels, download).  These are what
 * the parity tests drive; `device` is the CUDA ordinal.
 * ------------------------------------------------------------------------------------------- */

/* Exact k nearest neighbours of rows [q_lo,q_hi) of X among rows [db_lo,db_hi), ordered by
 * (squared distance, id), self included.  ids/d2 are [(q_hi-q_lo)][K]; slots that cannot be
 * filled (database smaller than K) hold id -1 and +inf.
 * Replaces: tsnecuda::util::KNearestNeighbors + PostprocessNeighborIndices
 * (src/util/distance_utils.cu:79-154; approximate FAISS IVF-Flat in the reference). */
int b200tsne_knn(const float *X, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo,
                 int64_t db_hi, int32_t *ids, float *d2, int device);

/* How the last b200tsne_knn call of this thread ran: whether the tensor-core path was used, how many rows
 * its proof could not certify (recomputed by the SIMT search) and the largest observed filter error as a
 * fraction of the assumed bound.  No counterpart in the reference. */
int b200tsne_knn_last_stats(int *tensor_core, int *rows_recomputed, float *filter_error_ratio);

/* Exact k nearest neighbours without any allocation.  This entry point has no counterpart in the
 * reference.  It is for hosts that must not allocate device memory when they call in: a framework that
 * hands out all device memory from its own pool, a service whose footprint is fixed at start-up, a
 * latency-bound loop where cudaMalloc's implicit synchronisation is unacceptable.  X_device ([N][D]),
 * ids_device and d2_device ([N][K]) are DEVICE pointers on the current device, owned by the caller; the
 * one piece of scratch the search needs (a dimension-major copy of X) lives in a fixed array inside the
 * library, so N * D must not exceed b200tsne_knn_noalloc_max_elements() (4 Mi floats = 16 MiB, resident
 * on every GPU that loads the library); larger inputs are rejected with B200TSNE_ERR_UNSUPPORTED.
 * The work is queued on cuda_stream (a cudaStream_t, NULL = default stream) and the call returns without
 * waiting, on the device that is current (cuda_stream must belong to it).  The first call on a device looks up
 * the array's device address and sets kernel attributes, which may load the library's device code: make that
 * call once at start-up, before any stream capture.  All calls share the one array, which keeps the previous
 * call's contents (every element the search reads is rewritten first): two calls whose GPU work overlaps, on different streams or from
 * different threads, race on it.  Results equal b200tsne_knn's (SIMT search; whole database, all queries). */
int b200tsne_knn_noalloc(const float *X_device, int64_t N, int D, int K, int32_t *ids_device, float *d2_device,
                         void *cuda_stream);
int64_t b200tsne_knn_noalloc_max_elements(void);

/* Global max-normalisation of the squared distances followed by the per-row perplexity search;
 * p receives the row-normalised conditional probabilities, betas (may be NULL) the found betas,
 * max_out (may be NULL) the normalising maximum.  If max_override > 0 it is used instead of the
 * maximum of d2 (a rank that holds a shard of the rows passes the global maximum).
 * Replaces: util::MaxNormalizeDeviceVector (src/util/math_utils.cu:66-74) and
 * tsnecuda::SearchPerplexity (src/kernels/perplexity_search.cu:81-141). */
int b200tsne_perplexity(const float *d2, int64_t N, int K, float perplexity, float epsilon,
                        float max_override, float *p, float *betas, float *max_out, int device);

/* Fixed-width symmetrisation P_ij = (p_j|i + [i in kNN(j)] p_i|j) / 2N.
 * Replaces: util::SymmetrizeMatrixV2 (src/util/math_utils.cu:269-308). */
int b200tsne_symmetrize(const float *p, const int32_t *ids, int64_t N, int K, float *P, int device);

/* Attractive force of rows [row_lo,row_hi) on a fixed Y; F is 2N floats SoA (other rows zero).
 * Replaces: tsnecuda::ComputeAttractiveForcesV3 (src/kernels/attr_forces.cu:186-240). */
int b200tsne_attractive(const float *P, const int32_t *ids, const float *Y, int64_t N, int K,
                        int64_t row_lo, int64_t row_hi, float *F, int device);

/* The same force from the column-blocked copy of P that the gradient loop uses when the graph suits it: the
 * points are ordered by Voronoi cell (from X [N][D] when given, else the natural order), every stored entry
 * moves into the stream of the tile (<= 28,672 points) that holds its column, and the kernel gathers the
 * neighbour coordinates from shared memory.  entries_per_group (may be NULL) receives the sampled average
 * number of entries a row has per tile; the copy is not built (B200TSNE_ERR_UNSUPPORTED) when that is below 2.5
 * unless the environment says B200TSNE_ATTRACTIVE=blocked.  Same arithmetic per entry as b200tsne_attractive,
 * other summation order.  Replaces: tsnecuda::ComputeAttractiveForcesV3 (src/kernels/attr_forces.cu:186-240). */
int b200tsne_attractive_blocked(const float *P, const int32_t *ids, const float *Y, int64_t N, int K, int64_t row_lo,
                                int64_t row_hi, const float *X, int D, float *F, float *entries_per_group, int device);

/* Attractive force under a TRULY symmetric P = (p + p^T) / 2N (opt-in; not what the reference computes).  The
 * reference's fixed-width symmetrisation stores P_ij only where j is one of i's neighbours, so where j has i as a
 * neighbour but not the other way round, row i never sees that edge (src/util/math_utils.cu:269-291).  Here every such
 * edge also gets its mirror image, kept beside the fixed-width P as a variable-width list per row, and the force
 * sums both.  p: conditional probabilities [N][K] as b200tsne_perplexity returns them; X ([N][D], may be NULL) orders
 * the points for the blocked kernel.  Outputs besides F (2N floats SoA; all may be NULL): the fixed-width part
 * P_fixed [N][K], the number of extra entries, their sum (fixed-width sum + extra sum = 1), and whether the blocked
 * kernel ran.  No counterpart in the reference (a "next" row of the scope table: true symmetric P as an opt-in). */
int b200tsne_attractive_symmetric(const float *p, const int32_t *ids, const float *Y, int64_t N, int K, const float *X, int D, float *F,
                                  float *P_fixed, int64_t *extra_entries, float *extra_sum, int *blocked, int device);

/* One FIt-SNE repulsive evaluation on a fixed Y: min/max, charges, spread, FFT convolution with
 * the squared-Cauchy kernel, gather, Z.  Frep: 2N floats SoA; Z = sum_i Z_i - N.
 * w_out / ytilde_out ([390][390][4]) may be NULL.
 * Replaces: ComputeChargesQij, PrecomputeFFT2D, NbodyFFT2D, ComputeRepulsiveForces as sequenced
 * in src/fit_tsne.cu:425-469 (src/kernels/nbodyfft.cu, src/kernels/rep_forces.cu). */
int b200tsne_repulsive(const float *Y, int64_t N, float *Frep, float *Z, float *w_out, float *ytilde_out,
                       int device);

/* Gradient, gains and momentum update, in place.  attr and rep are zeroed like the reference does.
 * Replaces: tsnecuda::ApplyForces (src/kernels/apply_forces.cu:59-82). */
int b200tsne_apply_forces(float *Y, float *attr, float *rep, float *gains, float *old_forces, float eta,
                          float normalization, float momentum, float exaggeration, int64_t N, int device);

/* ------------------------------------------------------------------------------------------- *
 * Device-resident session: the gradient loop with everything kept in HBM, as RunTsne runs it.
 * This is what bench.py times (inputs already resident) and what a multi-GPU driver steps.
 * No counterpart in the reference's public API (RunTsne is monolithic); the loop body it runs is
 * src/fit_tsne.cu:402-580.
 * ------------------------------------------------------------------------------------------- */
typedef struct b200tsne_session b200tsne_session;

/* N = total number of points; this session owns rows [row_lo,row_hi) (whole range on one GPU). */
int b200tsne_session_create(b200tsne_session **out, int64_t N, int K, int64_t row_lo, int64_t row_hi, int device);
void b200tsne_session_destroy(b200tsne_session *s);
/* Upload the owned rows of the fixed-width P and ids: [(row_hi-row_lo)][K]. */
int b200tsne_session_set_affinities(b200tsne_session *s, const float *P_rows, const int32_t *ids_rows);
/* Compute the owned rows' affinities on the device from X (all N rows, host): exact kNN of the
 * owned rows against the whole database, perplexity, symmetrisation.  Multi-GPU sessions exchange
 * what they need through the communicator. */
int b200tsne_session_affinities_from_points(b200tsne_session *s, const float *X, int D, float perplexity,
                                            float epsilon);
/* Set the full embedding (2N floats SoA); resets gains to 1 and momentum to 0 when reset != 0. */
int b200tsne_session_set_embedding(b200tsne_session *s, const float *Y, int reset);
int b200tsne_session_get_embedding(b200tsne_session *s, float *Y);
/* Checkpoint and resume of the loop: the embedding (2N floats SoA, all points), the owned rows' momentum (the
 * reference's old_forces) and gains (2 * rows floats SoA each; NULL = skip) and the iteration number, which
 * selects momentum, exaggeration and the spread-order refresh.  A session restored with set_state continues
 * as the saved one would have.  Replaces: TSNE_INIT::RESUME (src/include/options.h:24), which the reference
 * declares for this purpose but implements as a copy of the points alone (src/fit_tsne.cu:205-217). */
int b200tsne_session_get_state(b200tsne_session *s, float *Y, float *momentum, float *gains, int *step);
int b200tsne_session_set_state(b200tsne_session *s, const float *Y, const float *momentum, const float *gains, int step);
/* Download the owned rows of P / ids. */
int b200tsne_session_get_affinities(b200tsne_session *s, float *P_rows, int32_t *ids_rows);
/* Opt-in before b200tsne_session_affinities_from_points: build P truly symmetric (see b200tsne_attractive_symmetric).
 * The environment variable B200TSNE_SYMMETRIC_P=1 does the same for every run, pymodule_tsne included.
 * b200tsne_session_get_affinities still returns the fixed-width part. */
int b200tsne_session_set_symmetric(b200tsne_session *s, int on);
/* Which attractive kernel the session's loop runs: 1 = column-blocked copy of P (built with the affinities),
 * 0 = row-major P / ids.  entries_per_group (may be NULL): see b200tsne_attractive_blocked. */
int b200tsne_session_attractive_mode(b200tsne_session *s, float *entries_per_group);
/* Hyper-parameters of the loop (Options::learning_rate, early_exaggeration, force_magnify_iters,
 * pre/post momentum; src/include/options.h:67-77). */
int b200tsne_session_set_schedule(b200tsne_session *s, float learning_rate, float early_exaggeration,
                                  int force_magnify_iters, float pre_momentum, float post_momentum);
/* Run n_iters gradient iterations starting at the session's current step.  elapsed_ms (may be
 * NULL) receives the device time of the loop measured with CUDA events on the session's stream.
 * Returns the iteration count actually run in *iters_done when min_gradient_norm > 0 stops early. */
int b200tsne_session_run(b200tsne_session *s, int n_iters, float min_gradient_norm, float *elapsed_ms,
                         int *iters_done);
/* Last normalisation Z and last update norm ||u||_2. */
int b200tsne_session_stats(b200tsne_session *s, float *Z, float *update_norm, int *step);
/* Per-stage device time accumulated since creation, in ms, into out[B200TSNE_N_STAGES]
 * (only collected after b200tsne_session_enable_stage_timers(s, 1), which serialises stages). */
#define B200TSNE_N_STAGES 9
int b200tsne_session_enable_stage_timers(b200tsne_session *s, int enable);
int b200tsne_session_stage_times(b200tsne_session *s, float *out_ms, int64_t *out_launches);
const char *b200tsne_stage_name(int stage);
/* Number of kernel launches issued by the session so far. */
int64_t b200tsne_session_launch_count(b200tsne_session *s);

/* Multi-GPU: attach an NCCL communicator created from a unique id that rank 0 obtained from
 * b200tsne_comm_unique_id (128 bytes) and distributed to all ranks by any means.  Creating a
 * communicator takes seconds, so the library keeps it for the life of the process: a later session
 * attached with the same (id, rank, world_size) shares it.  b200tsne_comm_release_all destroys
 * the cached communicators; every session that used one must have been destroyed before. */
int b200tsne_comm_unique_id(void *id128);
int b200tsne_session_attach_comm(b200tsne_session *s, const void *id128, int rank, int world_size);
void b200tsne_comm_release_all(void);
/* How the session exchanges data per iteration: 0 = single GPU, nothing to exchange; 1 = NCCL collectives
 * (grid all-reduce, normalisation all-reduce, embedding all-gather); 2 = peer memory: the ranks map each
 * other's buffers (CUDA IPC), sum the partial grids with peer loads, evaluate the normalisation on the
 * summed grid and store updated rows into every rank's embedding.  attach_comm selects 2 when every rank
 * could map all others and the environment does not say B200TSNE_EXCHANGE=nccl (set alike on all
 * ranks).  With mode 2, destroying the session is collective: all ranks must call it. */
int b200tsne_session_exchange_mode(b200tsne_session *s);
/* Limit of one meeting of the ranks in exchange mode 2 (default 2000 ms, or B200TSNE_PEER_TIMEOUT_MS when the
 * exchange was created).  A rank that waits longer gives up: it tells every rank (an abort word in each
 * rank's exchange block), all later meetings of that exchange return at once, and b200tsne_session_run
 * returns B200TSNE_ERR_COMM on every rank that met it.  After that status the embedding is not meaningful;
 * destroy the sessions and call b200tsne_comm_release_all on all ranks before starting over.  No counterpart
 * in the reference (single GPU). */
int b200tsne_session_set_peer_timeout_ms(b200tsne_session *s, int timeout_ms);

/* Self-test of the two bounded device-side waits of this library, without a peer and without faulting or
 * hanging anything: (1) a meeting of two ranks whose second rank is local memory that nothing writes, (2) a
 * shared-memory barrier of the kNN pipeline that expects an arrival that never comes.  Each must give up after
 * timeout_ms (1..2000) and leave the device usable.  *_status receive the status the wait produced
 * (B200TSNE_ERR_COMM = gave up as designed, 0 = wrongly got through), *_ms the device time spent waiting.
 * Returns 0 when both ran.  No counterpart in the reference. */
int b200tsne_selftest_bounded_waits(int device, int timeout_ms, int *peer_status, float *peer_ms, int *barrier_status,
                                    float *barrier_ms);

/* Device memory the library has freed stays in the device's default memory pool so that the next call
 * gets it back without going to the driver (no reference counterpart: the reference allocates with
 * thrust per call).  This returns the pool of `device` to the driver. */
int b200tsne_release_cached_memory(int device);

#ifdef __cplusplus
}
#endif
#endif /* TSNECUDA_B200_H_ */
