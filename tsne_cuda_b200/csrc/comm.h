// Thin wrapper over NCCL for the few collectives a sharded run needs.  NCCL is bound at run time
// (dlopen) so that a single-GPU user of libtsnecuda.so needs no NCCL at all; inside a PyTorch process
// the already-loaded libnccl.so.2 is picked up.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200 {

struct PeerExchange;   // peer.h

struct Comm {
    void *nccl = nullptr;   // ncclComm_t
    int rank = 0, world = 1;
    // Mapping the peers' memory costs hundreds of milliseconds (the first mapping enables peer access), so
    // the exchange block of the last sharded session stays with the communicator and the next session of
    // the same size takes it over.
    PeerExchange *px_idle = nullptr;
    int all_reduce_sum_f32(float *buf, size_t n, cudaStream_t st);
    int all_reduce_sum_f64(double *buf, size_t n, cudaStream_t st);
    int all_reduce_max_u32(unsigned int *buf, size_t n, cudaStream_t st);
    // in place: rank r's contribution sits at buf + r*bytes_per_rank
    int all_gather_inplace(void *buf, size_t bytes_per_rank, cudaStream_t st);
    // rank r sends send + o*bytes to rank o and receives into recv + o*bytes from rank o
    int all_to_all(const void *send, void *recv, size_t bytes, cudaStream_t st);
    void destroy();
};

int comm_unique_id(void *id128);
// The communicator for (id, rank, world): created on first use, owned by a process-wide cache and
// shared by later sessions; comm_release_all destroys them (no session may still be using one).
int comm_acquire(Comm **out, const void *id128, int rank, int world);
void comm_release_all();

}  // namespace b200
