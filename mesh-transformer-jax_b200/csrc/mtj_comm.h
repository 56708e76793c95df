// Internal interface of the "shard"-axis collectives.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <string>

namespace mtj {

int32_t comm_unique_id(uint8_t* out128, std::string* err);
int32_t comm_init(const uint8_t* id128, int rank, int world, void** comm_out, std::string* err);
void comm_destroy(void* comm);
int32_t comm_all_reduce(void* comm, float* buf, size_t count, bool max_op, cudaStream_t s, std::string* err);
int32_t comm_all_gather(void* comm, const float* send, float* recv, size_t count, cudaStream_t s,
                        std::string* err);

cudaError_t launch_residual_stats(float* x, const float* reduced, float* stats, int rows, int d,
                                  bool accumulate, cudaStream_t s, bool pdl);
cudaError_t launch_gather_rows(const float* src, float* dst, int mp, int rows, int vl, cudaStream_t s);

}  // namespace mtj
