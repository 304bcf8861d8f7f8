// Host launchers of the SIMT trunk kernels (exact_kernels.cu).
#pragma once
#include <cuda_runtime.h>

#include "bnb_trunk.h"

namespace bnb {
namespace exact {

// Spatial sublayer.  qkv_scratch holds n_rows*3D floats, o_scratch n_rows*D floats.  When the
// sublayer reads bullets (bullets != null and w.kv_bullet_w set), kvb_scratch holds the bullet
// keys and values of kvb_envs environments at a time: kvb_envs * per_env * 2D floats.
int spatial_block(const BnbSpatialWeights& w, int D, int H, const float* x, const uint8_t* alive,
                  const BnbBullets* bullets, float* y, const BnbBatch& b, int n_groups, bool emulate_bf16,
                  float* qkv_scratch, float* o_scratch, float* kvb_scratch, int kvb_envs, cudaStream_t st);

// Temporal sublayer over T steps (ships with state, fields without).
int temporal_block(const BnbTemporalWeights& w, int D, const float* x, float* y, const float* hidden_in,
                   float* hidden_out, const uint8_t* done, const uint8_t* reset_env, const BnbBatch& b,
                   int T, bool emulate_bf16, cudaStream_t st);

int reset_hidden(const float* in, float* out, const uint8_t* done, int n_slots, int D,
                 const BnbBatch& b, cudaStream_t st);

}  // namespace exact
}  // namespace bnb
