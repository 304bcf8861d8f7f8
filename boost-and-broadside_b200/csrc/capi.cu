// C ABI of the trunk kernels: argument validation and engine dispatch.
// Every entry point is declared, with the reference interface it replaces, in
// include/bnb_trunk.h.
#include <cuda_runtime.h>

#include "bnb_trunk.h"
#include "bullet_slices.h"
#include "exact_kernels.h"
#include "mlp_kernels.h"
#include "grad_kernels.h"
#include "launch_count.h"
#include "validate.h"
#include "tensor_kernels.h"

namespace bnb {
std::atomic<unsigned long long> g_launches{0};
}

namespace {

using namespace bnb::validate;

// bullets may be null (no cross-attention in this call); otherwise it must be complete.
int check_bullets(const BnbBullets* b) {
  if (!b) return BNB_OK;
  if (!b->tokens) return BNB_ERR_NULL_POINTER;
  if (!aligned16(b->tokens)) return BNB_ERR_MISALIGNED;
  if (b->per_env < 1) return BNB_ERR_BAD_ARGUMENT;
  return BNB_OK;
}

bool any_reads_bullets(const BnbSpatialWeights* s, int ns, const BnbBullets* b) {
  if (!b) return false;
  for (int i = 0; i < ns; ++i) if (s[i].kv_bullet_w) return true;
  return false;
}

int check_temporal(const BnbTemporalWeights* w, bool need_field) {
  if (!w) return BNB_ERR_NULL_POINTER;
  const void* ps[] = {w->norm1_w, w->linear1_w, w->conv_w, w->conv_b, w->log_lambda, w->a_w, w->a_b, w->x_w,
                      w->x_b, w->linear2_w, w->out_w, w->norm2_w, w->gate_w, w->up_w, w->down_w};
  for (const void* p : ps) {
    if (!p) return BNB_ERR_NULL_POINTER;
    if (!aligned16(p)) return BNB_ERR_MISALIGNED;
  }
  if (need_field) {
    if (!w->field_sub_w) return BNB_ERR_NULL_POINTER;
    if (!aligned16(w->field_sub_w)) return BNB_ERR_MISALIGNED;
  }
  return BNB_OK;
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Scratch {
  float* qkv;
  float* o;
  float* kvb;     // bullet keys and values of one slice of environments, or null
  int kvb_envs;   // environments per slice
};

size_t simt_scratch_bytes(size_t n_rows, int D, long long total_envs, int nb) {
  return round_up(n_rows * 3 * D * sizeof(float), 256) + round_up(n_rows * D * sizeof(float), 256) +
         round_up(bnb::bullet_slice_bytes(total_envs, nb, D, sizeof(float)), 256);
}

// SIMT spatial scratch: qkv (rows, 3D), o (rows, D), then the bullet slice, float32.
int carve(void* scratch, size_t bytes, size_t n_rows, int D, long long total_envs, int nb, Scratch* out) {
  size_t need = simt_scratch_bytes(n_rows, D, total_envs, nb);
  *out = Scratch{nullptr, nullptr, nullptr, 0};
  if (need == 0) return BNB_OK;
  if (!scratch) return BNB_ERR_NULL_POINTER;
  if (!aligned16(scratch)) return BNB_ERR_MISALIGNED;
  if (bytes < need) return BNB_ERR_SCRATCH_TOO_SMALL;
  char* p = static_cast<char*>(scratch);
  out->qkv = reinterpret_cast<float*>(p);
  p += round_up(n_rows * 3 * D * sizeof(float), 256);
  out->o = reinterpret_cast<float*>(p);
  p += round_up(n_rows * D * sizeof(float), 256);
  if (nb > 0 && total_envs > 0) {
    out->kvb = reinterpret_cast<float*>(p);
    out->kvb_envs = bnb::bullet_slice_envs(total_envs, nb, D, sizeof(float));
  }
  return BNB_OK;
}

// BNB_BF16 calls that asked for BNB_ENGINE_AUTO and were served by the exact kernels because the
// tensor-core kernels are not built for their shape (read by bnb_auto_fallback_count).
std::atomic<unsigned long long> g_auto_fallbacks{0};

bool use_tensor(int precision, int engine, int D, int H, const BnbBatch* b, const BnbBullets* bullets) {
  if (precision != BNB_BF16 || engine == BNB_ENGINE_SIMT) return false;
  bool ok = bnb::tensor::supported_batch(D, H, *b);
  if (ok && bullets && !bnb::tensor::supported_bullets(*b, bullets->per_env)) ok = false;
  if (!ok && engine == BNB_ENGINE_AUTO) g_auto_fallbacks.fetch_add(1, std::memory_order_relaxed);
  return ok;
}

// The tensor engine needs the packed weight image of every sublayer it runs.
bool all_packed(const BnbSpatialWeights* s, int ns, const BnbTemporalWeights* t, int nt) {
  for (int i = 0; i < ns; ++i) if (!s[i].packed) return false;
  for (int i = 0; i < nt; ++i) if (!t[i].packed) return false;
  return true;
}

}  // namespace

extern "C" {

int bnb_abi_version(void) { return BNB_ABI_VERSION; }

unsigned long long bnb_launch_count(void) { return bnb::g_launches.load(std::memory_order_relaxed); }
unsigned long long bnb_auto_fallback_count(void) { return g_auto_fallbacks.load(std::memory_order_relaxed); }

const char* bnb_status_string(int status) {
  switch (status) {
    case BNB_OK: return "ok";
    case BNB_ERR_NULL_POINTER: return "a required pointer is null";
    case BNB_ERR_MISALIGNED: return "a pointer is not 16-byte aligned";
    case BNB_ERR_UNSUPPORTED_DIMS: return "d_model / n_heads / engine combination is not built";
    case BNB_ERR_TOO_MANY_TOKENS: return "an environment holds more tokens than the kernels take";
    case BNB_ERR_BAD_ARGUMENT: return "inconsistent argument";
    case BNB_ERR_SCRATCH_TOO_SMALL: return "scratch buffer smaller than bnb_scratch_bytes";
    case BNB_ERR_LAUNCH: return "CUDA launch failed";
    case BNB_ERR_NO_DEVICE: return "no CUDA device";
    case BNB_STATUS_WAIT_WEIGHTS: return "a bounded wait for a weight copy ran out inside a tensor-core kernel";
    case BNB_STATUS_WAIT_SLOT: return "a bounded wait for a free weight slot ran out inside a tensor-core kernel";
    case BNB_STATUS_WAIT_MMA: return "a bounded wait for tensor-core results ran out inside a tensor-core kernel";
    case BNB_STATUS_WAIT_OPERAND: return "a bounded wait for an operand ran out inside a tensor-core kernel";
    case BNB_ERR_EXCEEDS_STATIC_LIMIT: return "batch has more rows than the fixed scratch of the no-allocation entry point holds";
    default: return "unknown status";
  }
}

int bnb_supported(int d_model, int n_heads, int max_tokens_per_env, int precision, int engine) {
  if (check_dims(d_model, n_heads) != BNB_OK) return 0;
  if (max_tokens_per_env <= 0) return 0;
  if (precision != BNB_FP32 && precision != BNB_BF16) return 0;
  if (engine == BNB_ENGINE_TENSOR)
    return precision == BNB_BF16 && bnb::tensor::supported(d_model, n_heads, max_tokens_per_env) ? 1 : 0;
  return 1;
}

int bnb_plan_tiles(const int32_t* tok_off_host, int n_envs, int32_t* tile_env_begin_host,
                   int32_t* tile_env_ids_host, int capacity, int* n_tiles) {
  if (!tok_off_host || !tile_env_begin_host || !tile_env_ids_host || !n_tiles) return BNB_ERR_NULL_POINTER;
  if (n_envs < 0 || capacity < 1) return BNB_ERR_BAD_ARGUMENT;
  return bnb::tensor::plan_tiles(tok_off_host, n_envs, tile_env_begin_host, tile_env_ids_host, capacity, n_tiles);
}

size_t bnb_scratch_bytes(int d_model, const BnbBatch* batch, int timesteps, int bullets_per_env) {
  if (!batch || d_model <= 0 || timesteps <= 0) return 0;
  if (bullets_per_env < 0) bullets_per_env = 0;
  size_t n_rows = (size_t)timesteps * (size_t)batch->total_tokens;
  size_t simt = simt_scratch_bytes(n_rows, d_model, (long long)timesteps * batch->n_envs, bullets_per_env);
  size_t tc = bnb::tensor::scratch_bytes(d_model, *batch, timesteps, bullets_per_env);
  return (simt > tc ? simt : tc) + 256;
}

int bnb_spatial_block_fwd(const BnbSpatialWeights* w, int d_model, int n_heads, const float* x,
                          const uint8_t* alive, const BnbBullets* bullets, float* y, const BnbBatch* batch,
                          int n_groups, int precision, int engine, void* scratch, size_t scratch_bytes,
                          void* stream) {
  int st = check_dims(d_model, n_heads);
  if (st) return st;
  if ((st = check_batch(batch))) return st;
  if ((st = check_spatial(w))) return st;
  if ((st = check_bullets(bullets))) return st;
  if (!any_reads_bullets(w, 1, bullets)) bullets = nullptr;
  if (n_groups < 0) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  size_t n_rows = (size_t)n_groups * batch->total_tokens;
  if (n_rows == 0) return BNB_OK;
  if (!x || !y) return BNB_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(y)) return BNB_ERR_MISALIGNED;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (use_tensor(precision, engine, d_model, n_heads, batch, bullets) && (w->packed || engine == BNB_ENGINE_TENSOR))
    return bnb::tensor::spatial_block(*w, d_model, n_heads, x, alive, bullets, y, *batch, n_groups, scratch,
                                      scratch_bytes, cs);
  if (engine == BNB_ENGINE_TENSOR) return BNB_ERR_UNSUPPORTED_DIMS;
  Scratch s;
  if ((st = carve(scratch, scratch_bytes, n_rows, d_model, (long long)n_groups * batch->n_envs,
                  bullets ? bullets->per_env : 0, &s)))
    return st;
  return bnb::exact::spatial_block(*w, d_model, n_heads, x, alive, bullets, y, *batch, n_groups,
                                   precision == BNB_BF16, s.qkv, s.o, s.kvb, s.kvb_envs, cs);
}

int bnb_temporal_block_fwd(const BnbTemporalWeights* w, int d_model, const float* x, float* y,
                           const float* hidden_in, float* hidden_out, const uint8_t* done,
                           const BnbBatch* batch, int timesteps, int precision, int engine,
                           void* scratch, size_t scratch_bytes, void* stream) {
  int st = check_dims(d_model, d_model / 32);
  if (st) return st;
  if ((st = check_batch(batch))) return st;
  if ((st = check_temporal(w, batch->total_tokens > batch->total_ships))) return st;
  if (timesteps < 1) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (batch->total_tokens == 0) return BNB_OK;
  if (!x || !y) return BNB_ERR_NULL_POINTER;
  if (batch->total_ships > 0 && (!hidden_in || !hidden_out)) return BNB_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(y) || !aligned16(hidden_in) || !aligned16(hidden_out)) return BNB_ERR_MISALIGNED;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (use_tensor(precision, engine, d_model, 4, batch, nullptr) && (w->packed || engine == BNB_ENGINE_TENSOR))
    return bnb::tensor::temporal_block(*w, d_model, x, y, hidden_in, hidden_out, done, nullptr, *batch, timesteps,
                                       scratch, scratch_bytes, cs);
  if (engine == BNB_ENGINE_TENSOR) return BNB_ERR_UNSUPPORTED_DIMS;
  return bnb::exact::temporal_block(*w, d_model, x, y, hidden_in, hidden_out, done, nullptr, *batch, timesteps,
                                    precision == BNB_BF16, cs);
}

static int trunk_common(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal, int n_blocks,
                        int n_spatial, int n_temporal, int D, int H, const float* x, const uint8_t* alive,
                        const BnbBullets* bullets, float* y, const float* hidden_in, float* hidden_out, const uint8_t* done,
                        const uint8_t* reset_env, const BnbBatch* batch, int T, int precision, int engine,
                        void* scratch, size_t scratch_bytes, void* stream, bool is_sequence) {
  int st = check_dims(D, H);
  if (st) return st;
  if ((st = check_batch(batch))) return st;
  if (n_blocks < 0 || n_spatial < 0 || n_temporal < 0 || T < 1) return BNB_ERR_BAD_ARGUMENT;
  const bool io_bf16 = precision == BNB_BF16_IO;
  if (io_bf16) precision = BNB_BF16;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_blocks * n_spatial > 0 && !spatial) return BNB_ERR_NULL_POINTER;
  if (n_blocks * n_temporal > 0 && !temporal) return BNB_ERR_NULL_POINTER;
  for (int i = 0; i < n_blocks * n_spatial; ++i)
    if ((st = check_spatial(&spatial[i]))) return st;
  for (int i = 0; i < n_blocks * n_temporal; ++i)
    if ((st = check_temporal(&temporal[i], batch->total_tokens > batch->total_ships))) return st;
  if ((st = check_bullets(bullets))) return st;
  if (!any_reads_bullets(spatial, n_blocks * n_spatial, bullets)) bullets = nullptr;
  size_t n_rows = (size_t)T * batch->total_tokens;
  if (n_rows == 0) return BNB_OK;
  if (!x || !y) return BNB_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(y) || !aligned16(hidden_in) || !aligned16(hidden_out)) return BNB_ERR_MISALIGNED;
  const bool has_state = n_blocks * n_temporal > 0 && batch->total_ships > 0;
  if (has_state && !hidden_in) return BNB_ERR_NULL_POINTER;
  if (has_state && !is_sequence && !hidden_out) return BNB_ERR_NULL_POINTER;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  if (use_tensor(precision, engine, D, H, batch, bullets) &&
      (engine == BNB_ENGINE_TENSOR || all_packed(spatial, n_blocks * n_spatial, temporal, n_blocks * n_temporal)))
    return bnb::tensor::trunk(spatial, temporal, n_blocks, n_spatial, n_temporal, D, H, x, alive, bullets, y, hidden_in,
                              hidden_out, done, reset_env, *batch, T, scratch, scratch_bytes, cs, io_bf16);
  if (engine == BNB_ENGINE_TENSOR || io_bf16 || (bullets && bullets->tokens_bf16)) return BNB_ERR_UNSUPPORTED_DIMS;

  Scratch s{nullptr, nullptr, nullptr, 0};
  if (n_blocks * n_spatial > 0 &&
      (st = carve(scratch, scratch_bytes, n_rows, D, (long long)T * batch->n_envs, bullets ? bullets->per_env : 0, &s)))
    return st;
  const bool emu = precision == BNB_BF16;
  const float* cur = x;
  const size_t slot_stride = (size_t)batch->total_ships * 4 * D;
  if (n_blocks * (n_spatial + n_temporal) == 0) {
    if (y != x && cudaMemcpyAsync(y, x, n_rows * D * sizeof(float), cudaMemcpyDeviceToDevice, cs) != cudaSuccess)
      return BNB_ERR_LAUNCH;
    return BNB_OK;
  }
  for (int i = 0; i < n_blocks; ++i) {
    for (int j = 0; j < n_spatial; ++j) {
      st = bnb::exact::spatial_block(spatial[i * n_spatial + j], D, H, cur, alive, bullets, y, *batch, T, emu, s.qkv,
                                     s.o, s.kvb, s.kvb_envs, cs);
      if (st) return st;
      cur = y;
    }
    for (int j = 0; j < n_temporal; ++j) {
      int slot = i * n_temporal + j;
      st = bnb::exact::temporal_block(temporal[slot], D, cur, y, hidden_in ? hidden_in + slot * slot_stride : nullptr,
                                      hidden_out ? hidden_out + slot * slot_stride : nullptr, done, reset_env,
                                      *batch, T, emu, cs);
      if (st) return st;
      cur = y;
    }
  }
  return BNB_OK;
}

int bnb_trunk_step(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal, int n_blocks,
                   int n_spatial, int n_temporal, int d_model, int n_heads, const float* x,
                   const uint8_t* alive, const BnbBullets* bullets, float* y, const float* hidden_in,
                   float* hidden_out, const uint8_t* reset_env, const BnbBatch* batch, int precision, int engine,
                   void* scratch, size_t scratch_bytes, void* stream) {
  return trunk_common(spatial, temporal, n_blocks, n_spatial, n_temporal, d_model, n_heads, x, alive, bullets, y,
                      hidden_in, hidden_out, nullptr, reset_env, batch, 1, precision, engine, scratch, scratch_bytes, stream,
                      false);
}

int bnb_trunk_sequence(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal, int n_blocks,
                       int n_spatial, int n_temporal, int d_model, int n_heads, const float* x,
                       const uint8_t* alive, const BnbBullets* bullets, float* y, const float* hidden_in,
                       float* hidden_out, const uint8_t* done, const BnbBatch* batch, int timesteps, int precision, int engine,
                       void* scratch, size_t scratch_bytes, void* stream) {
  return trunk_common(spatial, temporal, n_blocks, n_spatial, n_temporal, d_model, n_heads, x, alive, bullets, y,
                      hidden_in, hidden_out, done, nullptr, batch, timesteps, precision, engine, scratch, scratch_bytes, stream,
                      true);
}

size_t bnb_trunk_bwd_scratch_bytes(int n_blocks, int n_spatial, int n_temporal, int d_model, const BnbBatch* batch,
                                   int timesteps, int bullets_per_env, int precision) {
  if (!batch || n_blocks < 0 || n_spatial < 0 || n_temporal < 0 || d_model <= 0 || timesteps < 1) return 0;
  return bnb::grad::scratch_bytes(n_blocks, n_spatial, n_temporal, d_model, *batch, timesteps, bullets_per_env,
                                  precision == BNB_BF16);
}

size_t bnb_trunk_kept_bytes(int n_blocks, int n_spatial, int n_temporal, int d_model, int n_heads, const BnbBatch* batch,
                            int timesteps, int bullets_per_env, int precision) {
  if (!batch || n_blocks < 0 || n_spatial < 0 || n_temporal < 0 || d_model <= 0 || timesteps < 1) return 0;
  if (check_dims(d_model, n_heads) || check_batch(batch)) return 0;
  return bnb::grad::kept_bytes(n_blocks, n_spatial, n_temporal, d_model, n_heads, *batch, timesteps, bullets_per_env,
                               precision == BNB_BF16);
}

int bnb_trunk_sequence_fwd_train(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal, int n_blocks,
                                 int n_spatial, int n_temporal, int d_model, int n_heads, const float* x,
                                 const uint8_t* alive, const BnbBullets* bullets, float* y, const float* hidden_in,
                                 float* hidden_out, const uint8_t* done, const BnbBatch* batch, int timesteps, int precision,
                                 void* kept, size_t kept_bytes, void* scratch, size_t scratch_bytes, void* stream) {
  int st = check_dims(d_model, n_heads);
  if (st) return st;
  if ((st = check_batch(batch))) return st;
  if (batch->tok_off) return BNB_ERR_UNSUPPORTED_DIMS;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_blocks < 0 || n_spatial < 0 || n_temporal < 0 || timesteps < 1) return BNB_ERR_BAD_ARGUMENT;
  if ((size_t)timesteps * batch->total_tokens == 0) return BNB_OK;
  const int ns = n_blocks * n_spatial, nt = n_blocks * n_temporal;
  if ((ns && !spatial) || (nt && !temporal)) return BNB_ERR_NULL_POINTER;
  if (!x || !y || !scratch || !kept) return BNB_ERR_NULL_POINTER;
  if (nt && batch->total_ships > 0 && !hidden_in) return BNB_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(y) || !aligned16(hidden_in) || !aligned16(hidden_out)) return BNB_ERR_MISALIGNED;
  for (int i = 0; i < ns; ++i)
    if ((st = check_spatial(&spatial[i]))) return st;
  for (int i = 0; i < nt; ++i)
    if ((st = check_temporal(&temporal[i], batch->total_tokens > batch->total_ships))) return st;
  if ((st = check_bullets(bullets))) return st;
  if (!any_reads_bullets(spatial, ns, bullets)) bullets = nullptr;
  bnb::grad::TrunkFwdTrainArgs a{spatial, temporal, n_blocks, n_spatial, n_temporal, d_model, n_heads, x, alive, bullets,
                                 hidden_in, done, batch, timesteps, precision == BNB_BF16, y, hidden_out, scratch,
                                 scratch_bytes, kept, kept_bytes, static_cast<cudaStream_t>(stream)};
  return bnb::grad::trunk_sequence_fwd_train(a);
}

int bnb_trunk_sequence_bwd(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal,
                           const BnbSpatialGrads* d_spatial, const BnbTemporalGrads* d_temporal, int n_blocks,
                           int n_spatial, int n_temporal, int d_model, int n_heads, const float* x, const uint8_t* alive,
                           const BnbBullets* bullets, const float* hidden_in, const uint8_t* done, const BnbBatch* batch,
                           int timesteps, int precision, const float* dy, const float* d_hidden_out, float* dx,
                           float* d_hidden_in, float* d_bullets, void* kept, size_t kept_bytes, void* scratch,
                           size_t scratch_bytes, void* stream) {
  int st = check_dims(d_model, n_heads);
  if (st) return st;
  if ((st = check_batch(batch))) return st;
  if (batch->tok_off) return BNB_ERR_UNSUPPORTED_DIMS;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_blocks < 0 || n_spatial < 0 || n_temporal < 0 || timesteps < 1) return BNB_ERR_BAD_ARGUMENT;
  if ((size_t)timesteps * batch->total_tokens == 0) return BNB_OK;
  const int ns = n_blocks * n_spatial, nt = n_blocks * n_temporal;
  if ((ns && (!spatial || !d_spatial)) || (nt && (!temporal || !d_temporal))) return BNB_ERR_NULL_POINTER;
  if (!x || !dy || !dx || !scratch) return BNB_ERR_NULL_POINTER;
  if (nt && batch->total_ships > 0 && !hidden_in) return BNB_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(hidden_in) || !aligned16(d_hidden_out) ||
      !aligned16(d_hidden_in) || !aligned16(d_bullets))
    return BNB_ERR_MISALIGNED;
  for (int i = 0; i < ns; ++i) {
    if ((st = check_spatial(&spatial[i]))) return st;
    const BnbSpatialGrads& g = d_spatial[i];
    const void* ps[] = {g.norm1_w, g.qkv_w, g.out_w, g.norm2_w, g.gate_w, g.up_w, g.down_w};
    for (const void* p : ps) {
      if (!p) return BNB_ERR_NULL_POINTER;
      if (!aligned16(p)) return BNB_ERR_MISALIGNED;
    }
    if (bullets && spatial[i].kv_bullet_w && (!g.norm_bullet_w || !g.kv_bullet_w)) return BNB_ERR_NULL_POINTER;
    if (!aligned16(g.kv_bullet_w)) return BNB_ERR_MISALIGNED;
  }
  const bool fields = batch->total_tokens > batch->total_ships;
  for (int i = 0; i < nt; ++i) {
    const BnbTemporalWeights& w = temporal[i];
    const BnbTemporalGrads& g = d_temporal[i];
    const void* ws[] = {w.norm1_w, w.linear1_w, w.conv_w, w.conv_b, w.log_lambda, w.a_w, w.a_b, w.x_w, w.x_b,
                        w.linear2_w, w.out_w, w.norm2_w, w.gate_w, w.up_w, w.down_w,
                        g.norm1_w, g.linear1_w, g.conv_w, g.conv_b, g.log_lambda, g.a_w, g.a_b, g.x_w, g.x_b,
                        g.linear2_w, g.out_w, g.norm2_w, g.gate_w, g.up_w, g.down_w};
    for (const void* p : ws) {
      if (!p) return BNB_ERR_NULL_POINTER;
      if (!aligned16(p)) return BNB_ERR_MISALIGNED;
    }
    if (fields && (!w.field_sub_w || !g.field_sub_w)) return BNB_ERR_NULL_POINTER;
    if (!aligned16(w.field_sub_w) || !aligned16(g.field_sub_w)) return BNB_ERR_MISALIGNED;
  }
  if (bullets) {
    if (bullets->per_env < 1 || !bullets->tokens) return BNB_ERR_BAD_ARGUMENT;
    if (!aligned16(bullets->tokens)) return BNB_ERR_MISALIGNED;
    if (bullets->tokens_bf16) return BNB_ERR_UNSUPPORTED_DIMS;
  }
  bnb::grad::TrunkBwdArgs a{spatial, temporal, d_spatial, d_temporal, n_blocks, n_spatial, n_temporal, d_model, n_heads,
                            x, alive, bullets, hidden_in, done, batch, timesteps, precision == BNB_BF16, dy, d_hidden_out, dx, d_hidden_in,
                            d_bullets, scratch, scratch_bytes, kept, kept_bytes, static_cast<cudaStream_t>(stream)};
  if (bullets && !any_reads_bullets(spatial, ns, bullets)) a.bullets = nullptr;
  return bnb::grad::trunk_sequence_bwd(a);
}

int bnb_reset_hidden(const float* hidden_in, float* hidden_out, const uint8_t* done, int n_slots, int d_model,
                     const BnbBatch* batch, void* stream) {
  int st = check_batch(batch);
  if (st) return st;
  if (d_model <= 0 || d_model % 4 != 0 || n_slots < 0) return BNB_ERR_BAD_ARGUMENT;
  if ((size_t)n_slots * batch->total_ships == 0) return BNB_OK;
  if (!hidden_in || !hidden_out || !done) return BNB_ERR_NULL_POINTER;
  if (!aligned16(hidden_in) || !aligned16(hidden_out)) return BNB_ERR_MISALIGNED;
  return bnb::exact::reset_hidden(hidden_in, hidden_out, done, n_slots, d_model, *batch,
                                  static_cast<cudaStream_t>(stream));
}

int bnb_gated_mlp_fwd(const float* gate_w, const float* up_w, const float* down_w, int d_model, const float* x,
                      float* y, int n_rows, int precision, void* stream) {
  if (d_model <= 0 || d_model % 32 != 0 || d_model > 128) return BNB_ERR_UNSUPPORTED_DIMS;
  if (n_rows < 0) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_rows == 0) return BNB_OK;
  const void* ps[] = {gate_w, up_w, down_w, x, y};
  for (const void* p : ps) {
    if (!p) return BNB_ERR_NULL_POINTER;
    if (!aligned16(p)) return BNB_ERR_MISALIGNED;
  }
  return bnb::exact::gated_mlp(gate_w, up_w, down_w, d_model, x, y, n_rows, precision == BNB_BF16,
                               static_cast<cudaStream_t>(stream));
}

int bnb_rglru_fwd(const float* a_w, const float* a_b, const float* x_w, const float* x_b, const float* log_lambda,
                  int d_model, const float* x, float* y, const float* h0, float* h_out, const uint8_t* done,
                  int n_rows, int timesteps, int precision, void* stream) {
  if (d_model <= 0 || d_model % 32 != 0 || d_model > 128) return BNB_ERR_UNSUPPORTED_DIMS;
  if (n_rows < 0 || timesteps < 1) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_rows == 0) return BNB_OK;
  const void* ps[] = {a_w, a_b, x_w, x_b, log_lambda, x, y, h0, h_out};
  for (const void* p : ps) {
    if (!p) return BNB_ERR_NULL_POINTER;
    if (!aligned16(p)) return BNB_ERR_MISALIGNED;
  }
  return bnb::exact::rglru(a_w, a_b, x_w, x_b, log_lambda, d_model, x, y, h0, h_out, done, n_rows, timesteps,
                           precision == BNB_BF16, static_cast<cudaStream_t>(stream));
}

int bnb_encoder_mlp_fwd(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2,
                        const float* g2, int in_dim, int in_pad, int hidden, int out_dim, const float* x, void* y,
                        int n_rows, int precision, void* stream) {
  if (in_dim <= 0 || in_pad < in_dim || in_pad % 32 != 0 || in_pad > 128) return BNB_ERR_UNSUPPORTED_DIMS;
  if (hidden <= 0 || hidden % 32 != 0 || hidden > 256) return BNB_ERR_UNSUPPORTED_DIMS;
  if (out_dim <= 0 || out_dim % 32 != 0 || out_dim > 128) return BNB_ERR_UNSUPPORTED_DIMS;
  if (n_rows < 0) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_rows == 0) return BNB_OK;
  const void* ps[] = {w1, b1, g1, w2, b2, g2, x, y};
  for (const void* p : ps) if (!p) return BNB_ERR_NULL_POINTER;
  if (!aligned16(w1) || !aligned16(w2)) return BNB_ERR_MISALIGNED;
  if (precision == BNB_BF16 && bnb::mlp::supported(in_pad, hidden, out_dim))
    return bnb::mlp::encoder_mlp_bf16(w1, b1, g1, w2, b2, g2, in_dim, in_pad, hidden, out_dim, out_dim, x, false, y, n_rows,
                                      static_cast<cudaStream_t>(stream));
  return bnb::exact::encoder_mlp(w1, b1, g1, w2, b2, g2, in_dim, in_pad, hidden, out_dim, out_dim, x, y, n_rows,
                                 precision == BNB_BF16, static_cast<cudaStream_t>(stream));
}

int bnb_head_mlp_fwd(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2, int in_dim,
                     int hidden, int out_dim, int out_pad, const float* x, void* y, int n_rows, int precision,
                     void* stream) {
  if (in_dim <= 0 || in_dim % 32 != 0 || in_dim > 128) return BNB_ERR_UNSUPPORTED_DIMS;
  if (hidden <= 0 || hidden % 32 != 0 || hidden > 256) return BNB_ERR_UNSUPPORTED_DIMS;
  if (out_dim <= 0 || out_pad < out_dim || out_pad % 32 != 0 || out_pad > 128) return BNB_ERR_UNSUPPORTED_DIMS;
  if (n_rows < 0) return BNB_ERR_BAD_ARGUMENT;
  const bool x_bf16 = precision == BNB_BF16_IO;   // x holds bfloat16 tokens (the trunk's output under autocast)
  if (x_bf16) precision = BNB_BF16;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_rows == 0) return BNB_OK;
  const void* ps[] = {w1, b1, g1, w2, b2, x, y};
  for (const void* p : ps) if (!p) return BNB_ERR_NULL_POINTER;
  if (!aligned16(w1) || !aligned16(w2)) return BNB_ERR_MISALIGNED;
  if (precision == BNB_BF16 && bnb::mlp::supported(in_dim, hidden, out_pad))
    return bnb::mlp::encoder_mlp_bf16(w1, b1, g1, w2, b2, nullptr, in_dim, in_dim, hidden, out_pad, out_dim, x, x_bf16, y, n_rows,
                                      static_cast<cudaStream_t>(stream));
  if (x_bf16) return BNB_ERR_UNSUPPORTED_DIMS;   // only the tiled kernel reads bfloat16 rows
  return bnb::exact::encoder_mlp(w1, b1, g1, w2, b2, nullptr, in_dim, in_dim, hidden, out_pad, out_dim, x, y, n_rows,
                                 precision == BNB_BF16, static_cast<cudaStream_t>(stream));
}

size_t bnb_team_pma_scratch_bytes(int d_model, int n_envs, int n_ships) {
  if (d_model <= 0 || n_envs < 0 || n_ships < 0) return 0;
  return ((size_t)n_envs * n_ships * 2 * d_model + 2 * (size_t)d_model) * sizeof(float) + 256;
}

int bnb_team_pma_fwd(const float* seeds, const float* in_proj_w, const float* out_w, const float* norm_w, int d_model,
                     int n_heads, const float* x, const int32_t* team_id, const uint8_t* alive, void* y, int y_is_bf16,
                     int n_envs, int n_ships, int precision, void* scratch, size_t scratch_bytes, void* stream) {
  int st = check_dims(d_model, n_heads);
  if (st) return st;
  if (n_envs < 0 || n_ships < 0) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if ((size_t)n_envs * n_ships == 0) return BNB_OK;
  const void* ps[] = {seeds, in_proj_w, out_w, norm_w, x, team_id, alive, y, scratch};
  for (const void* p : ps)
    if (!p) return BNB_ERR_NULL_POINTER;
  if (!aligned16(in_proj_w) || !aligned16(out_w) || !aligned16(x) || !aligned16(y)) return BNB_ERR_MISALIGNED;
  if (scratch_bytes < bnb_team_pma_scratch_bytes(d_model, n_envs, n_ships)) return BNB_ERR_SCRATCH_TOO_SMALL;
  uintptr_t base = (reinterpret_cast<uintptr_t>(scratch) + 255) & ~(uintptr_t)255;
  float* kv = reinterpret_cast<float*>(base);
  float* q = kv + (size_t)n_envs * n_ships * 2 * d_model;
  return bnb::exact::team_pma(seeds, in_proj_w, out_w, norm_w, d_model, n_heads, x, team_id, alive, y, y_is_bf16 != 0, n_envs,
                              n_ships, kv, q, precision == BNB_BF16, static_cast<cudaStream_t>(stream));
}

int bnb_action_dist_fwd(const float* logits, const float* uniforms, const int64_t* given_action, int64_t* action,
                        float* logprob, float* entropy, int n_rows, int precision, void* stream) {
  if (n_rows < 0) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  if (n_rows == 0) return BNB_OK;
  if (!logits || !logprob) return BNB_ERR_NULL_POINTER;
  if (!given_action && (!uniforms || !action)) return BNB_ERR_NULL_POINTER;
  return bnb::exact::sample_action(logits, uniforms, given_action, action, logprob, entropy, n_rows, precision == BNB_BF16,
                                   static_cast<cudaStream_t>(stream));
}

size_t bnb_packed_spatial_bytes(int d_model) { return bnb::tensor::packed_spatial_bytes(d_model); }
size_t bnb_packed_temporal_bytes(int d_model) { return bnb::tensor::packed_temporal_bytes(d_model); }

int bnb_pack_spatial(const BnbSpatialWeights* w, int d_model, int n_heads, void* packed, void* stream) {
  int st = check_dims(d_model, n_heads);
  if (st) return st;
  if ((st = check_spatial(w))) return st;
  if (!packed) return BNB_ERR_NULL_POINTER;
  if (!aligned16(packed)) return BNB_ERR_MISALIGNED;
  return bnb::tensor::pack_spatial(*w, d_model, n_heads, packed, static_cast<cudaStream_t>(stream));
}

int bnb_pack_trunk(const BnbSpatialWeights* spatial, int n_spatial_total, const BnbTemporalWeights* temporal,
                   int n_temporal_total, int d_model, int n_heads, void* stream) {
  int st = check_dims(d_model, n_heads);
  if (st) return st;
  if (n_spatial_total < 0 || n_temporal_total < 0) return BNB_ERR_BAD_ARGUMENT;
  if ((n_spatial_total > 0 && !spatial) || (n_temporal_total > 0 && !temporal)) return BNB_ERR_NULL_POINTER;
  for (int i = 0; i < n_spatial_total; ++i) {
    if ((st = check_spatial(&spatial[i]))) return st;
    if (!spatial[i].packed) return BNB_ERR_NULL_POINTER;
    if (!aligned16(spatial[i].packed)) return BNB_ERR_MISALIGNED;
  }
  for (int i = 0; i < n_temporal_total; ++i) {
    if ((st = check_temporal(&temporal[i], false))) return st;
    if (!temporal[i].packed) return BNB_ERR_NULL_POINTER;
    if (!aligned16(temporal[i].packed)) return BNB_ERR_MISALIGNED;
  }
  return bnb::tensor::pack_trunk(spatial, n_spatial_total, temporal, n_temporal_total, d_model, n_heads,
                                 static_cast<cudaStream_t>(stream));
}

int bnb_last_status(void) { return bnb::tensor::last_status(); }
void bnb_clear_status(void) { bnb::tensor::clear_status(); }
void bnb_debug_wait_test(int skip_op, int poll_limit) { bnb::tensor::debug_wait_test(skip_op, poll_limit); }

int bnb_pack_temporal(const BnbTemporalWeights* w, int d_model, void* packed, void* stream) {
  int st = check_dims(d_model, d_model / 32);
  if (st) return st;
  if ((st = check_temporal(w, false))) return st;
  if (!packed) return BNB_ERR_NULL_POINTER;
  if (!aligned16(packed)) return BNB_ERR_MISALIGNED;
  return bnb::tensor::pack_temporal(*w, d_model, packed, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
