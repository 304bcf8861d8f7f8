// Argument validation shared by the C-ABI entry points (capi.cu, static_scratch.cu): every check
// runs on the host before anything is launched.
#pragma once
#include <stdint.h>

#include "bnb_trunk.h"

namespace bnb {
namespace validate {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int check_dims(int D, int H) {
  if (D <= 0 || H <= 0 || D % H != 0) return BNB_ERR_BAD_ARGUMENT;
  if (D % 32 != 0 || D > 128) return BNB_ERR_UNSUPPORTED_DIMS;
  int dh = D / H;
  if (dh != 8 && dh != 16 && dh != 32 && dh != 64) return BNB_ERR_UNSUPPORTED_DIMS;
  return BNB_OK;
}

inline int check_batch(const BnbBatch* b) {
  if (!b) return BNB_ERR_NULL_POINTER;
  if (b->n_envs < 0 || b->total_tokens < 0 || b->total_ships < 0 || b->total_ships > b->total_tokens)
    return BNB_ERR_BAD_ARGUMENT;
  if ((b->tok_off == nullptr) != (b->ship_off == nullptr)) return BNB_ERR_BAD_ARGUMENT;
  if (!b->tok_off) {
    if (b->tokens_per_env < 0 || b->ships_per_env < 0 || b->ships_per_env > b->tokens_per_env)
      return BNB_ERR_BAD_ARGUMENT;
    if ((long long)b->n_envs * b->tokens_per_env != b->total_tokens) return BNB_ERR_BAD_ARGUMENT;
    if ((long long)b->n_envs * b->ships_per_env != b->total_ships) return BNB_ERR_BAD_ARGUMENT;
    if (b->max_tokens_per_env < b->tokens_per_env) return BNB_ERR_BAD_ARGUMENT;
  } else if (b->max_tokens_per_env <= 0) {
    return BNB_ERR_BAD_ARGUMENT;
  }
  return BNB_OK;
}

inline int check_spatial(const BnbSpatialWeights* w) {
  if (!w) return BNB_ERR_NULL_POINTER;
  const void* ps[] = {w->norm1_w, w->qkv_w, w->out_w, w->norm2_w, w->gate_w, w->up_w, w->down_w};
  for (const void* p : ps) {
    if (!p) return BNB_ERR_NULL_POINTER;
    if (!aligned16(p)) return BNB_ERR_MISALIGNED;
  }
  if ((w->norm_bullet_w == nullptr) != (w->kv_bullet_w == nullptr)) return BNB_ERR_NULL_POINTER;
  if (!aligned16(w->norm_bullet_w) || !aligned16(w->kv_bullet_w)) return BNB_ERR_MISALIGNED;
  return BNB_OK;
}

}  // namespace validate
}  // namespace bnb
