// Backward pass of the Yemong trunk's sequence forward (grad_kernels.cu).
#pragma once
#include <cuda_runtime.h>

#include "bnb_trunk.h"

namespace bnb {
namespace grad {

struct TrunkBwdArgs {
  const BnbSpatialWeights* spatial;
  const BnbTemporalWeights* temporal;
  const BnbSpatialGrads* d_spatial;
  const BnbTemporalGrads* d_temporal;
  int n_blocks, n_spatial, n_temporal, D, H;
  const float* x;
  const uint8_t* alive;
  const BnbBullets* bullets;
  const float* hidden_in;
  const uint8_t* done;
  const BnbBatch* batch;
  int T;
  bool bf16_products;   // products round their operands to bfloat16 (forward ran under autocast)
  const float* dy;
  const float* d_hidden_out;
  float* dx;
  float* d_hidden_in;
  float* d_bullets;
  void* scratch;
  size_t scratch_bytes;
  void* kept;           // activations kept by trunk_sequence_fwd_train, or null: recompute
  size_t kept_bytes;
  cudaStream_t stream;
};

struct TrunkFwdTrainArgs {
  const BnbSpatialWeights* spatial;
  const BnbTemporalWeights* temporal;
  int n_blocks, n_spatial, n_temporal, D, H;
  const float* x;
  const uint8_t* alive;
  const BnbBullets* bullets;
  const float* hidden_in;
  const uint8_t* done;
  const BnbBatch* batch;
  int T;
  bool bf16_products;
  float* y;
  float* hidden_out;
  void* scratch;
  size_t scratch_bytes;
  void* kept;
  size_t kept_bytes;
  cudaStream_t stream;
};

// Bytes of scratch trunk_sequence_bwd needs for this structure and batch.
size_t scratch_bytes(int n_blocks, int n_spatial, int n_temporal, int D, const BnbBatch& b, int T, int bullets_per_env,
                     bool bf16);

// Bytes of the activations trunk_sequence_fwd_train keeps for the backward (0: unsupported geometry).
size_t kept_bytes(int n_blocks, int n_spatial, int n_temporal, int D, int H, const BnbBatch& b, int T, int bullets_per_env,
                  bool bf16);

// y (M, N) = x (M, K) . W (N, K)^T, row-major, on the tiled product kernels: with bf16_operands the
// operands are rounded to bfloat16 and accumulated in float32 (y is not rounded), else 3 x tf32.
void linear_nt(const float* x, const float* W, float* y, int M, int N, int K, bool bf16_operands, cudaStream_t st);

int trunk_sequence_fwd_train(const TrunkFwdTrainArgs& a);
int trunk_sequence_bwd(const TrunkBwdArgs& a);

}  // namespace grad
}  // namespace bnb
