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

// GatedMLP on its own: y (n_rows, D) = down(gelu(gate x) * up x).
int gated_mlp(const float* gate_w, const float* up_w, const float* down_w, int D, const float* x, float* y,
              int n_rows, bool emulate_bf16, cudaStream_t st);

// RG-LRU on its own over T steps: x, y (T, n_rows, D) time-major, h0 / h_out (n_rows, D),
// done (T, n_rows) bytes or null.
int rglru(const float* a_w, const float* a_b, const float* x_w, const float* x_b, const float* log_lambda, int D,
          const float* x, float* y, const float* h0, float* h_out, const uint8_t* done, int n_rows, int T,
          bool emulate_bf16, cudaStream_t st);

// Encoder chain Linear + b -> RMSNorm -> GELU -> Linear + b -> RMSNorm on rows of raw features.
// w1 is (hidden, in_pad) with zero columns beyond in_dim; g2 null leaves the last norm out (the
// policy's heads); y is (n_rows, out_store), float32, or bfloat16 when emulate_bf16.
int encoder_mlp(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2, const float* g2,
                int in_dim, int in_pad, int hidden, int out_dim, int out_store, const float* x, void* y, int n_rows,
                bool emulate_bf16, cudaStream_t st);

// TeamPMA: pooling by attention over each team's alive ships, broadcast back to the ships.
// kv holds n_envs * N * 2D floats of scratch, q 2D floats; y is (n_envs, N, D) float32 or bfloat16.
int team_pma(const float* seeds, const float* in_proj_w, const float* out_w, const float* norm_w, int D, int H, const float* x,
             const int32_t* team_id, const uint8_t* alive, void* y, bool y_bf16, int n_envs, int N, float* kv, float* q,
             bool emulate_bf16, cudaStream_t st);

// Factored categorical over the 12 action logits: draws from `uniforms` (n_rows, 3) into `action`,
// or scores the `given` actions; logprob (n_rows) and, when asked, entropy (n_rows).
int sample_action(const float* logits, const float* uniforms, const int64_t* given, int64_t* action, float* logprob,
                  float* entropy, int n_rows, bool emulate_bf16, cudaStream_t st);

}  // namespace exact
}  // namespace bnb
