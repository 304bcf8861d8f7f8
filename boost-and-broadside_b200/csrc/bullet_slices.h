// Slicing of the bullet key/value projection: both engines project the bullet tokens of a
// bounded number of environments at a time into scratch, attend, and move on, so the scratch
// share of the bullets does not grow with the batch.
#pragma once
#include <stddef.h>

namespace bnb {

constexpr size_t kBulletScratchCap = (size_t)512 << 20;

// Environments per slice: as many as keep nb rows of [k | v] (2D elements of `elt` bytes) per
// environment under the cap, at least one, at most all.
inline int bullet_slice_envs(long long total_envs, int nb, int D, size_t elt) {
  size_t per_env = (size_t)nb * 2 * (size_t)D * elt;
  long long n = per_env ? (long long)(kBulletScratchCap / per_env) : total_envs;
  if (n < 1) n = 1;
  if (n > total_envs) n = total_envs;
  return (int)n;
}

inline size_t bullet_slice_bytes(long long total_envs, int nb, int D, size_t elt) {
  if (nb <= 0 || total_envs <= 0) return 0;
  return (size_t)bullet_slice_envs(total_envs, nb, D, elt) * (size_t)nb * 2 * (size_t)D * elt;
}

}  // namespace bnb
