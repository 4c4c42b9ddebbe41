// Tensor-parallel plumbing: NCCL (resolved at run time from the copy already loaded in the
// process, or from the system library) and the peer-memory exchange buffers.
#pragma once
#include "internal.h"

struct NcclApi;  // dlopen'ed entry points

struct TpNccl {
    void* comm = nullptr;
    int rank = 0, size = 1;
};

int nccl_unique_id(void* id128);
int nccl_init(TpNccl* t, const void* id128, int rank, int size);
int nccl_destroy(TpNccl* t);
int nccl_allreduce_f32(TpNccl* t, float* buf, size_t count, cudaStream_t stream);
int nccl_allgather_f32(TpNccl* t, const float* send, float* recv, size_t count_per_rank, cudaStream_t stream);
