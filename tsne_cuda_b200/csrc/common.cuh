// Internal declarations shared by the kernels and the host orchestration of libtsnecuda.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace b200 {

// ---- FIt-SNE grid constants (reference: src/fit_tsne.cu:246-272) ----
constexpr int kBoxes = 130;            // boxes per dimension (125 rounded up through the allowed list)
constexpr int kInterp = 3;             // Lagrange nodes per box and dimension
constexpr int kG = kBoxes * kInterp;   // 390 nodes per dimension
constexpr int kTerms = 4;              // charges (1, x, y, x^2+y^2)
constexpr int kM = 1024;               // transform length of the zero-padded convolution (>= 2*kG-1)
constexpr int kStages = 9;             // instrumented stages (== B200TSNE_N_STAGES)

// ---- error plumbing ----
void set_error(const std::string &msg);
const std::string &last_error();
int release_cached_memory();   // session.cu: hand the device memory pool of the current device back to the driver
int cuda_fail(cudaError_t e, const char *what, const char *file, int line);

#define B200_CUDA(expr)                                                        \
    do {                                                                       \
        cudaError_t _e = (expr);                                               \
        if (_e != cudaSuccess) return ::b200::cuda_fail(_e, #expr, __FILE__, __LINE__); \
    } while (0)

#define B200_TRY(expr)            \
    do {                          \
        int _s = (expr);          \
        if (_s != 0) return _s;   \
    } while (0)

// Per-iteration scalars that live in device memory so that an iteration needs no host round trip.
// Slots are double-buffered by iteration parity: iteration `it` reads slot it&1 and prepares slot
// (it+1)&1 for its successor.
struct IterState {
    unsigned int min_enc[2];   // order-preserving encodings of min / max over all coordinates
    unsigned int max_enc[2];
    double zsum[2];            // sum_i Z_i accumulated by the gather kernel
    double unorm2;             // sum of squared updates (only maintained on request)
    int bad;                   // set when a non-finite coordinate is produced
    int pad;
};

// Lagrange constants evaluated on the host exactly as the reference does (src/fit_tsne.cu:303-320).
struct InterpConsts {
    float sp[kInterp];
    float den[kInterp];
};
InterpConsts make_interp_consts();

__host__ __device__ inline unsigned int enc_float(float f)
{
#ifdef __CUDA_ARCH__
    unsigned int b = __float_as_uint(f);
#else
    union { float f; unsigned int u; } c; c.f = f; unsigned int b = c.u;
#endif
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ inline float dec_float(unsigned int e)
{
    unsigned int b = (e & 0x80000000u) ? (e & 0x7fffffffu) : ~e;
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    union { float f; unsigned int u; } c; c.u = b; return c.f;
#endif
}

// ---- kernel launchers (all asynchronous on `st`; pointers are device memory) ----

// knn.cu
int launch_transpose(const float *X, int64_t N, int D, float *XT, cudaStream_t st);   // [N][D] -> [D][N]
int launch_knn_exact(const float *XT, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo,
                     int64_t db_hi, int32_t *ids, float *d2, cudaStream_t st);   // ids/d2 keep (INT_MAX,+inf) in unfilled slots
int launch_knn_exact_rows(const float *XT, int64_t N, int D, int K, const int *q_index, int64_t nq, int64_t out_base,
                          int64_t db_lo, int64_t db_hi, int32_t *ids, float *d2, cudaStream_t st);
// knn_tc.cu: tensor-core filter + exact re-rank + proof (nd = database rows to scan)
bool knn_tc_supported(int64_t nd, int D, int K);
size_t knn_tc_workspace_bytes(int D, int K, int64_t nq, int64_t nd);
int launch_knn_tc(const float *X, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo, int64_t db_hi,
                  int32_t *ids, float *d2, void *workspace, int **failed_list, int *n_failed_host, float *err_ratio_host,
                  cudaStream_t st);
int mbar_wait_selftest(int timeout_ms, float *waited_ms, cudaStream_t st);   // see b200tsne_selftest_bounded_waits
struct KnnStats {
    int tensor_core = 0;            // 1 when the tensor-core path ran
    int rows_recomputed = 0;        // rows the proof could not certify, recomputed by the SIMT search
    float filter_error_ratio = 0;   // largest observed filter error on the candidates / assumed bound
};
// X: [N][D] row-major on the device; picks the path, handles the fallback rows, synchronises `st`.
int knn_search(const float *X, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo, int64_t db_hi,
               int32_t *ids, float *d2, KnnStats *stats, cudaStream_t st);
// knn.cu: search with the scratch in a fixed device array of the library (no allocation)
long long knn_noalloc_max_elems();
int knn_noalloc(const float *X, int64_t N, int D, int K, int32_t *ids, float *d2, cudaStream_t st);
int launch_knn_merge(const int32_t *ids_parts, const float *d2_parts, int parts, int64_t part_stride, int64_t n_rows,
                     int K, int32_t *ids, float *d2, cudaStream_t st);
int launch_knn_finalize(int32_t *ids, float *d2, int64_t n, cudaStream_t st);

// affinities.cu
int launch_absmax(const float *v, int64_t n, unsigned int *max_enc, cudaStream_t st);  // max_enc: enc_float accumulator, pre-set to enc(0)
int launch_perplexity(const float *d2, int64_t n_rows, int K, float perplexity, float eps, const unsigned int *max_enc,
                      float *p, float *betas, cudaStream_t st);
int launch_reverse_only_count(const float *p_all, const int32_t *ids_all, int64_t N, int K, int64_t row_lo, int64_t row_hi, int *ptr,
                              int64_t *count_host, cudaStream_t st);
int launch_reverse_only_fill(const float *p_all, const int32_t *ids_all, int64_t N, int K, int64_t row_lo, int64_t row_hi, const int *ptr,
                             int *cursor, int32_t *ext_ids, float *ext_val, cudaStream_t st);
// visit (optional): row_hi - row_lo row numbers inside [row_lo, row_hi), the order in which the rows are taken
int launch_symmetrize(const float *p_all, const int32_t *ids_all, int64_t N, int K, int64_t row_lo, int64_t row_hi,
                      float *P_rows, cudaStream_t st, const int32_t *visit = nullptr);

// attractive.cu   (Y2: AoS float2 [N]; F2: AoS float2, rows [row_lo,row_hi) written at their global index)
int launch_attractive(const float *P_rows, const int32_t *ids_rows, const float2 *Y2, int64_t N, int K, int64_t row_lo,
                      int64_t row_hi, float2 *F2, cudaStream_t st);
// F2[row] += force of the rows' extra entries (variable-width list, see ExtraEntries below)
int launch_attractive_extra(const int *ptr, const int32_t *ext_ids, const float *ext_val, const float2 *Y2, int64_t N, int64_t row_lo,
                            int64_t row_hi, float2 *F2, cudaStream_t st);

// attractive_blocked.cu: column-blocked copy of P whose gathers come from shared memory (see that file)
struct DeviceArena;
// Further stored entries of the owned rows in variable-width form: row r (0-based among the owned rows) has the
// entries ptr[r] .. ptr[r + 1].  Used for the reverse-only edges that make P truly symmetric (affinities.cu).
struct ExtraEntries {
    const int *ptr = nullptr;        // [rows + 1]
    const int32_t *ids = nullptr;    // columns (point numbers)
    const float *val = nullptr;
    int64_t count = 0;
};
struct BlockedAttractive {
    const float *ev = nullptr;
    const uint16_t *ec = nullptr;
    const int *chunk_row0 = nullptr, *tile_chunk0 = nullptr;
    const float *extra_ev = nullptr;       // second stream: the extra entries (none: extra_C = 0)
    const uint16_t *extra_ec = nullptr;
    const int *extra_chunk_row0 = nullptr, *extra_tile_chunk0 = nullptr;
    int extra_C = 0;
    int64_t extra_E = 0;
    const int32_t *perm = nullptr, *own_perm = nullptr, *own_pos = nullptr;
    float2 *Yp = nullptr, *Yown = nullptr, *Fp = nullptr;
    int ntiles = 0, T = 0, C = 0;
    int64_t E = 0, groups = 0, N = 0, row_lo = 0, rows = 0;
    float entries_per_group = 0.0f;   // of the sampled rows, under the chosen order
    bool ready = false;
    void clear();
};
int order_points_by_cell(const float *X, int64_t N, int D, int32_t *perm, cudaStream_t st);
int blocked_attractive_build(BlockedAttractive *b, DeviceArena &arena, const float *P_rows, const int32_t *ids_rows, int64_t N, int K,
                             int64_t row_lo, int64_t row_hi, const int32_t *perm, const ExtraEntries *extra, cudaStream_t st);
int launch_exclusive_scan_i32(int *data, int64_t n, cudaStream_t st);   // in place; small arrays (one block)
// in_cell_order: Y2 and F2 are in the copy's own point order (one GPU): no conversion before or after the kernel
int launch_attractive_blocked(const BlockedAttractive &b, const float2 *Y2, float2 *F2, cudaStream_t st, bool in_cell_order = false);

// repulsive.cu
struct FftWorkspace {
    float2 *A;      // [2][kG][kM] row-transformed signal planes
    float *Rk;      // [kG][kM] row-transformed kernel plane (real part)
    float2 *B;      // [2][kG][kM] after the fused column pass
    float2 *tw;     // [kM] forward twiddles e^{-2 pi i k / kM}
};
size_t fft_workspace_bytes();
int fft_workspace_init(FftWorkspace *ws, void *mem, cudaStream_t st);
int launch_state_reset(IterState *state, cudaStream_t st);   // both slots, sums and flags
int launch_minmax_init(const float2 *Y2, int64_t N, IterState *state, int slot, cudaStream_t st);
// order: local row indices sorted by box (null = natural order); see launch_order_refresh
int launch_spread(const float2 *Y2, int64_t row_lo, int64_t row_hi, const int32_t *order, const IterState *state,
                  int slot, InterpConsts ic, float4 *w, cudaStream_t st);
int launch_order_identity(int32_t *order, int64_t n, cudaStream_t st);
int launch_order_refresh(const float2 *Y2, int64_t row_lo, int64_t row_hi, const int32_t *order_in, int32_t *order_out,
                         int32_t *keys, int32_t *hist, const IterState *state, int slot, cudaStream_t st);
int launch_convolve(float4 *w, float4 *ytilde, const IterState *state, int slot, const FftWorkspace &ws, bool zero_w,
                    cudaStream_t st);
// sum_z: add the rows' Z_i to state->zsum[slot] (off when the caller evaluates the sum on the grid)
int launch_gather(const float2 *Y2, int64_t row_lo, int64_t row_hi, IterState *state, int slot, InterpConsts ic,
                  const float4 *ytilde, float2 *Frep2, bool sum_z, cudaStream_t st);

// update.cu
// where the updated rows go: one array (in place) or the embedding copy of every rank (peer memory)
constexpr int kMaxUpdateTargets = 16;
struct UpdateTargets {
    float2 *p[kMaxUpdateTargets];
    int n;
};
int launch_update(const float2 *Y2, const UpdateTargets &dst, const float2 *Fattr2, const float2 *Frep2, float2 *gains2, float2 *u2,
                  int64_t N, int64_t row_lo, int64_t row_hi, IterState *state, int slot, float eta, float momentum,
                  float exaggeration, int want_norm, cudaStream_t st);
int launch_apply_forces_soa(float *Y, float *attr, float *rep, float *gains, float *old_forces, float eta, float Z,
                            float momentum, float exaggeration, int64_t N, cudaStream_t st);
// perm (optional): position q of the pair array holds point perm[q] of the block-wise (x block, y block) array
int launch_soa_to_aos(const float *soa, float2 *aos, int64_t N, cudaStream_t st, const int32_t *perm = nullptr);
int launch_aos_to_soa(const float2 *aos, float *soa, int64_t N, cudaStream_t st, const int32_t *perm = nullptr);
// dst[q] = src[perm[q]], or with scatter dst[perm[q]] = src[q]
int launch_reorder_pairs(const float2 *src, float2 *dst, int64_t N, const int32_t *perm, bool scatter, cudaStream_t st);
int launch_fill(float *p, float v, int64_t n, cudaStream_t st);

}  // namespace b200
