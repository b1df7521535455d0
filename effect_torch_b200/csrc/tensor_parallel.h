// Tensor-parallel plumbing of the decoder: a communicator per decoder, bound at run time to the NCCL library that
// is already loaded in the process (the one torch.distributed brought in) or else to the system's libnccl.so.2.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <string>

namespace etc {

struct TpComm;  // opaque: an ncclComm_t plus the rank geometry

// 128 bytes that rank 0 creates and every rank passes to tp_comm_create (exchange them with the host's own transport).
bool tp_unique_id(unsigned char out[128], std::string* error);
// Collective over all ranks: blocks until every rank has joined.
TpComm* tp_comm_create(int rank, int world, const unsigned char id[128], std::string* error);
void tp_comm_destroy(TpComm* comm);
// In-place f32 sum over all ranks, enqueued on `stream` (may be captured into a CUDA graph).
bool tp_allreduce_sum(TpComm* comm, float* data, size_t count, cudaStream_t stream, std::string* error);

}  // namespace etc
