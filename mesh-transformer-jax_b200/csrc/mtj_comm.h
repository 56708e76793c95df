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

// Peer-memory all-reduce of [rows, d] fp32 partial sums fused with the residual add and the
// LayerNorm statistics (mtj_p2p.cu).
constexpr int kP2pMaxWorld = 8;
struct P2pArgs {
  int rank, world, d;
  size_t slot_elems;                       // floats per data slot
  const float* peer_data[kP2pMaxWorld];    // every rank's buffer (own one included)
  uint32_t* peer_flags[kP2pMaxWorld];      // every rank's flag row [world]
  const uint32_t* local_flags;             // this rank's flag row
  uint32_t* seq;                           // all-reduces completed (this rank's device counter)
  uint32_t* ticket;                        // block arrival counter, self-resetting
  float* x;                                // [rows, d] residual stream, updated in place
  float* stats;                            // [rows, 2]
  int accumulate;                          // 1: x += sum, 0: x = sum
  uint32_t* dev_err;
};
cudaError_t launch_p2p_allreduce(const P2pArgs& a, int rows, cudaStream_t s, bool pdl);

cudaError_t launch_residual_stats(float* x, const float* reduced, float* stats, int rows, int d,
                                  bool accumulate, cudaStream_t s, bool pdl);
cudaError_t launch_gather_rows(const float* src, float* dst, int mp, int rows, int vl, cudaStream_t s);

}  // namespace mtj
