// Shared device helpers for the Yemong trunk kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bnb_trunk.h"

namespace bnb {

constexpr float kRmsEps = 1.1920928955078125e-07f;  // finfo(float32).eps: nn.RMSNorm(eps=None)
constexpr float kMaskedScore = -1.0e30f;            // score of a dead key; exp(kMaskedScore - m) == 0
constexpr float kRglruC = 8.0f;                     // models/yemong/griffin.py:160
constexpr float kGateFloor = 1e-6f;                 // models/yemong/griffin.py:184

// Round-to-nearest-even to bf16, returned in a float container.
__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

template <bool EMU>
__device__ __forceinline__ float rnd(float v) {
  if constexpr (EMU) return round_bf16(v);
  return v;
}

// erf GeLU, the F.gelu default (models/yemong/attention.py:37).
__device__ __forceinline__ float gelu_erf(float v) {
  return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
}

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

// Geometry of a batch on the device: maps environments, ships and fields to rows.
struct EnvMap {
  int n_envs;
  int tokens_per_env;
  int ships_per_env;
  int total_tokens;
  int total_ships;
  const int* tok_off;   // null for uniform batches
  const int* ship_off;

  __device__ __forceinline__ int env_tok_begin(int e) const {
    return tok_off ? tok_off[e] : e * tokens_per_env;
  }
  __device__ __forceinline__ int env_tok_count(int e) const {
    return tok_off ? tok_off[e + 1] - tok_off[e] : tokens_per_env;
  }
  __device__ __forceinline__ int env_ship_begin(int e) const {
    return ship_off ? ship_off[e] : e * ships_per_env;
  }
  __device__ __forceinline__ int env_ship_count(int e) const {
    return ship_off ? ship_off[e + 1] - ship_off[e] : ships_per_env;
  }
  __device__ __forceinline__ int total_fields() const { return total_tokens - total_ships; }

  // largest e with key(e) <= v, key non-decreasing, key(0) = 0
  template <class F>
  __device__ __forceinline__ int search(int v, F key) const {
    int lo = 0, hi = n_envs - 1;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (key(mid) <= v) lo = mid; else hi = mid - 1;
    }
    return lo;
  }
  __device__ __forceinline__ int env_of_ship(int s) const {
    if (!ship_off) return s / ships_per_env;
    // skip environments without ships: the last e whose ship range starts at or before s
    return search(s, [&](int e) { return ship_off[e]; });
  }
  __device__ __forceinline__ int env_of_token(int r) const {
    if (!tok_off) return r / tokens_per_env;
    return search(r, [&](int e) { return tok_off[e]; });
  }
  // token row (within one timestep) of ship s
  __device__ __forceinline__ int ship_token_row(int s, int* env_out) const {
    int e = env_of_ship(s);
    *env_out = e;
    return env_tok_begin(e) + (s - env_ship_begin(e));
  }
  // token row of the f-th field token of the batch
  __device__ __forceinline__ int field_token_row(int f) const {
    if (!tok_off) {
      int m = tokens_per_env - ships_per_env;
      int e = f / m;
      return e * tokens_per_env + ships_per_env + (f - e * m);
    }
    int e = search(f, [&](int i) { return tok_off[i] - ship_off[i]; });
    int fb = tok_off[e] - ship_off[e];
    return tok_off[e] + (ship_off[e + 1] - ship_off[e]) + (f - fb);
  }
};

inline EnvMap make_env_map(const BnbBatch& b) {
  EnvMap m;
  m.n_envs = b.n_envs;
  m.tokens_per_env = b.tokens_per_env;
  m.ships_per_env = b.ships_per_env;
  m.total_tokens = b.total_tokens;
  m.total_ships = b.total_ships;
  m.tok_off = b.tok_off;
  m.ship_off = b.ship_off;
  return m;
}

}  // namespace bnb
