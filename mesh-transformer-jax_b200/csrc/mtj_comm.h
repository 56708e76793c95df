// Internal interface of the "shard"-axis collectives.
#pragma once
#include <cuda_bf16.h>
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
  int wait_limit;                          // spins before a wait on a peer flag gives up (sets kDevErrTimeout)
};
cudaError_t launch_p2p_allreduce(const P2pArgs& a, int rows, cudaStream_t s, bool pdl);

// Push-style exchanges of the tensor-parallel decode step (mtj_tp_push.cu).
struct TpReduceArgs {
  int rank, world, d, rows_cap;
  const float* partial;                    // this rank's partial sums [ksplit, rows, d]
  int ksplit;
  const float* bias;                       // [d] or null
  float* peer_recv[kP2pMaxWorld];          // every rank's receive area [2 slots][world][rows_cap][d]
  uint32_t* peer_flags[kP2pMaxWorld];      // every rank's row flags [world][rows_cap]
  uint32_t* seq;                           // exchanges completed (this rank's device counter)
  uint32_t* ticket;                        // block arrival counter, self-resetting
  float* x;                                // [rows, d] residual stream, updated in place
  float* stats;                            // [rows, 2] or null
  int accumulate;                          // 1: x += sum, 0: x = sum
  const float* ln_scale;                   // LayerNorm of the finished rows to the next GEMM's operand (xn != null)
  const float* ln_offset;
  __nv_bfloat16* xn;                       // [rows, d] or null
  __nv_bfloat16* xn_lo;                    // optional bf16 rounding error of xn
  uint32_t* dev_err;
  int wait_limit;
};
cudaError_t launch_tp_push_reduce(const TpReduceArgs& a, int rows, cudaStream_t s, bool pdl);

struct TpArgmaxArgs {
  const float* logits;                     // [B, Vl] this rank's vocabulary slice
  int Vl, vocab_start, rank, world, rows_cap;
  uint2* peer_amax[kP2pMaxWorld];          // every rank's packets [2 slots][world][rows_cap][2]
  uint32_t* seq;
  uint32_t* ticket;
  uint32_t* tokens;                        // [B]
  int32_t* cur_dev;                        // incremented by one after the step (may be null)
  uint32_t* dev_err;
  int wait_limit;
};
cudaError_t launch_tp_argmax(const TpArgmaxArgs& a, int B, cudaStream_t s, bool pdl);

cudaError_t launch_residual_stats(float* x, const float* reduced, float* stats, int rows, int d,
                                  bool accumulate, cudaStream_t s, bool pdl);
cudaError_t launch_gather_rows(const float* src, float* dst, int mp, int rows, int vl, cudaStream_t s);

}  // namespace mtj
