#include "comm.h"
#include "peer.h"

#include <dlfcn.h>
#include <string.h>

#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace b200 {
namespace {

// Minimal NCCL surface, declared here so that no NCCL header is needed at build time.
typedef struct { char internal[128]; } nccl_unique_id;
typedef int (*fn_get_unique_id)(nccl_unique_id *);
typedef int (*fn_comm_init_rank)(void **, int, nccl_unique_id, int);
typedef int (*fn_comm_destroy)(void *);
typedef const char *(*fn_get_error_string)(int);
typedef int (*fn_all_reduce)(const void *, void *, size_t, int, int, void *, cudaStream_t);
typedef int (*fn_all_gather)(const void *, void *, size_t, int, void *, cudaStream_t);
typedef int (*fn_send)(const void *, size_t, int, int, void *, cudaStream_t);
typedef int (*fn_recv)(void *, size_t, int, int, void *, cudaStream_t);
typedef int (*fn_group)(void);

// ncclDataType_t / ncclRedOp_t values (stable across NCCL 2.x)
enum { kNcclInt8 = 0, kNcclUint32 = 3, kNcclFloat32 = 7, kNcclFloat64 = 8 };
enum { kNcclSum = 0, kNcclMax = 2 };

struct Api {
    void *h = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_get_error_string get_error_string = nullptr;
    fn_all_reduce all_reduce = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_send send = nullptr;
    fn_recv recv = nullptr;
    fn_group group_start = nullptr, group_end = nullptr;
};

Api *api()
{
    static Api a;
    static bool tried = false;
    if (!tried) {
        tried = true;
        a.h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!a.h) a.h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (a.h) {
            a.get_unique_id = (fn_get_unique_id)dlsym(a.h, "ncclGetUniqueId");
            a.comm_init_rank = (fn_comm_init_rank)dlsym(a.h, "ncclCommInitRank");
            a.comm_destroy = (fn_comm_destroy)dlsym(a.h, "ncclCommDestroy");
            a.get_error_string = (fn_get_error_string)dlsym(a.h, "ncclGetErrorString");
            a.all_reduce = (fn_all_reduce)dlsym(a.h, "ncclAllReduce");
            a.all_gather = (fn_all_gather)dlsym(a.h, "ncclAllGather");
            a.send = (fn_send)dlsym(a.h, "ncclSend");
            a.recv = (fn_recv)dlsym(a.h, "ncclRecv");
            a.group_start = (fn_group)dlsym(a.h, "ncclGroupStart");
            a.group_end = (fn_group)dlsym(a.h, "ncclGroupEnd");
        }
    }
    const bool ok = a.h && a.get_unique_id && a.comm_init_rank && a.comm_destroy && a.all_reduce && a.all_gather &&
                    a.send && a.recv && a.group_start && a.group_end;
    if (!ok) {
        set_error("NCCL (libnccl.so.2) could not be loaded: multi-GPU runs are unavailable");
        return nullptr;
    }
    return &a;
}

int nccl_fail(int rc, const char *what)
{
    Api *a = api();
    std::string msg = std::string("NCCL error in ") + what + ": " +
                      ((a && a->get_error_string) ? a->get_error_string(rc) : "unknown");
    set_error(msg);
    return -5;
}
#define B200_NCCL(call, what)                  \
    do {                                       \
        int _rc = (call);                      \
        if (_rc != 0) return nccl_fail(_rc, what); \
    } while (0)

}  // namespace

int comm_unique_id(void *id128)
{
    Api *a = api();
    if (!a) return -5;
    B200_NCCL(a->get_unique_id(reinterpret_cast<nccl_unique_id *>(id128)), "ncclGetUniqueId");
    return 0;
}

// Creating a communicator costs seconds (bootstrap, topology search, channel set-up), a session a few
// milliseconds, so communicators are kept for the life of the process: a second session attached
// with the same (unique id, rank, world size) gets the communicator of the first.
namespace {
struct Cached { nccl_unique_id id; Comm *comm; };
std::mutex g_cache_mutex;
std::vector<Cached> g_cache;
}  // namespace

int comm_acquire(Comm **out, const void *id128, int rank, int world)
{
    Api *a = api();
    if (!a) return -5;
    if (world < 1 || rank < 0 || rank >= world) { set_error("comm_acquire: bad rank/world_size"); return -1; }
    nccl_unique_id id = *reinterpret_cast<const nccl_unique_id *>(id128);
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    for (const Cached &c : g_cache)
        if (memcmp(&c.id, &id, sizeof(id)) == 0 && c.comm->rank == rank && c.comm->world == world) { *out = c.comm; return 0; }
    Comm *c = new Comm();
    c->rank = rank;
    c->world = world;
    int rc = a->comm_init_rank(&c->nccl, world, id, rank);
    if (rc != 0) { delete c; return nccl_fail(rc, "ncclCommInitRank"); }
    g_cache.push_back({id, c});
    *out = c;
    return 0;
}

void comm_release_all()
{
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    for (Cached &c : g_cache) {
        if (c.comm->px_idle) { peer_exchange_destroy(c.comm->px_idle, c.comm, nullptr); c.comm->px_idle = nullptr; }
        c.comm->destroy();
        delete c.comm;
    }
    g_cache.clear();
}

void Comm::destroy()
{
    Api *a = api();
    if (a && nccl) a->comm_destroy(nccl);
    nccl = nullptr;
}

int Comm::all_reduce_sum_f32(float *buf, size_t n, cudaStream_t st)
{
    B200_NCCL(api()->all_reduce(buf, buf, n, kNcclFloat32, kNcclSum, nccl, st), "ncclAllReduce(f32)");
    return 0;
}
int Comm::all_reduce_sum_f64(double *buf, size_t n, cudaStream_t st)
{
    B200_NCCL(api()->all_reduce(buf, buf, n, kNcclFloat64, kNcclSum, nccl, st), "ncclAllReduce(f64)");
    return 0;
}
int Comm::all_reduce_max_u32(unsigned int *buf, size_t n, cudaStream_t st)
{
    B200_NCCL(api()->all_reduce(buf, buf, n, kNcclUint32, kNcclMax, nccl, st), "ncclAllReduce(u32 max)");
    return 0;
}
int Comm::all_gather_inplace(void *buf, size_t bytes_per_rank, cudaStream_t st)
{
    const char *mine = static_cast<const char *>(buf) + (size_t)rank * bytes_per_rank;
    B200_NCCL(api()->all_gather(mine, buf, bytes_per_rank, kNcclInt8, nccl, st), "ncclAllGather");
    return 0;
}
int Comm::all_to_all(const void *send, void *recv, size_t bytes, cudaStream_t st)
{
    Api *a = api();
    B200_NCCL(a->group_start(), "ncclGroupStart");
    for (int o = 0; o < world; o++) {
        B200_NCCL(a->send(static_cast<const char *>(send) + (size_t)o * bytes, bytes, kNcclInt8, o, nccl, st), "ncclSend");
        B200_NCCL(a->recv(static_cast<char *>(recv) + (size_t)o * bytes, bytes, kNcclInt8, o, nccl, st), "ncclRecv");
    }
    B200_NCCL(a->group_end(), "ncclGroupEnd");
    return 0;
}

}  // namespace b200
