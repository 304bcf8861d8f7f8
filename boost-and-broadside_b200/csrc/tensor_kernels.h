// Host interface of the tensor-core (tcgen05) trunk kernels (tensor_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "bnb_trunk.h"

namespace bnb {
namespace tensor {

// True when the tensor-core kernels are built for this width, head count and environment size.
bool supported(int D, int H, int max_tokens_per_env);
// The same, for one concrete batch (uniform geometry only).
bool supported_batch(int D, int H, const BnbBatch& b);

// Host-only: pack the environments of a ragged batch into tiles of whole environments.
int plan_tiles(const int32_t* tok_off_host, int n_envs, int32_t* tile_env_begin_host, int32_t* tile_env_ids_host,
               int capacity, int* n_tiles);

// True when the attention kernel can stage this many bullet keys beside an environment's tokens.
bool supported_bullets(const BnbBatch& b, int bullets_per_env);

size_t scratch_bytes(int D, const BnbBatch& b, int T, int bullets_per_env);
size_t packed_spatial_bytes(int D);
size_t packed_temporal_bytes(int D);
int pack_spatial(const BnbSpatialWeights& w, int D, int H, void* packed, cudaStream_t st);
int pack_temporal(const BnbTemporalWeights& w, int D, void* packed, cudaStream_t st);
// Every weight image of a trunk (each struct's `packed` names its destination) in one launch.
int pack_trunk(const BnbSpatialWeights* spatial, int n_spatial, const BnbTemporalWeights* temporal, int n_temporal,
               int D, int H, cudaStream_t st);

// Status word of the bounded waits, as last copied to the host for the current device (sticky
// until cleared); and the test hooks that make a wait run out.
int last_status();
void clear_status();
void debug_wait_test(int skip_op, int poll_limit);

int spatial_block(const BnbSpatialWeights& w, int D, int H, const float* x, const uint8_t* alive,
                  const BnbBullets* bullets, float* y, const BnbBatch& b, int n_groups, void* scratch,
                  size_t scratch_bytes, cudaStream_t st);

int temporal_block(const BnbTemporalWeights& w, int D, const float* x, float* y, const float* hidden_in,
                   float* hidden_out, const uint8_t* done, const uint8_t* reset_env, const BnbBatch& b, int T,
                   void* scratch, size_t scratch_bytes, cudaStream_t st);

int trunk(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal, int n_blocks, int n_spatial,
          int n_temporal, int D, int H, const float* x, const uint8_t* alive, const BnbBullets* bullets, float* y,
          const float* hidden_in, float* hidden_out, const uint8_t* done, const uint8_t* reset_env, const BnbBatch& b, int T,
          void* scratch, size_t scratch_bytes, cudaStream_t st, bool io_bf16 = false);

}  // namespace tensor
}  // namespace bnb
