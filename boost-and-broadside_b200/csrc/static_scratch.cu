// bnb_spatial_block_fwd_static: the spatial sublayer for callers that cannot allocate.
//
// bnb_spatial_block_fwd needs (rows x 4 x d_model) floats of scratch for the projected
// q/k/v and the attention output, and expects the caller to bring that memory.  Some callers
// have no way to get it: a thin ctypes / cgo / JNI stub owns no device allocator, and a host
// process that has already handed the whole device to another framework's memory pool must
// not call cudaMalloc behind that pool's back.  For them this entry point keeps the scratch
// in a fixed array that is part of the library image.  The price: every GPU that loads the
// library holds BNB_STATIC_SCRATCH_BYTES of device memory until the process exits, and the
// batch is limited to BNB_STATIC_MAX_ROWS token rows.
#include <cuda_runtime.h>

#include <mutex>

#include "bnb_trunk.h"
#include "exact_kernels.h"
#include "validate.h"

namespace {

constexpr int kMaxRows = BNB_STATIC_MAX_ROWS;
constexpr int kMaxWidth = 128;                            // largest d_model the kernels take
constexpr size_t kFloats = (size_t)kMaxRows * 4 * kMaxWidth;  // q, k, v and attention output
static_assert(kFloats * sizeof(float) == BNB_STATIC_SCRATCH_BYTES, "header and array disagree");

// The scratch itself.  In host code this name is only a handle for the runtime, not a
// device address: the address is looked up per device below and handed to the kernels.
static __device__ __align__(256) float g_static_scratch[kFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float* g_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch on each GPU

// Device address of the array on the current device; looked up once per device (again with
// `refresh`, after a launch failed on the cached address).
int scratch_address(float** out, bool refresh) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return BNB_ERR_NO_DEVICE;
  if (dev >= kMaxDevices) return BNB_ERR_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_ptr[dev] || refresh) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) return BNB_ERR_LAUNCH;
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return BNB_OK;
}

}  // namespace

extern "C" int bnb_spatial_block_fwd_static(const BnbSpatialWeights* w, int d_model, int n_heads, const float* x,
                                            const uint8_t* alive, float* y, const BnbBatch* batch, int n_groups,
                                            int precision, void* stream) {
  // the same checks, in the same order, as bnb_spatial_block_fwd
  int st = bnb::validate::check_dims(d_model, n_heads);
  if (st) return st;
  if ((st = bnb::validate::check_batch(batch))) return st;
  if ((st = bnb::validate::check_spatial(w))) return st;
  if (n_groups < 0) return BNB_ERR_BAD_ARGUMENT;
  if (precision != BNB_FP32 && precision != BNB_BF16) return BNB_ERR_BAD_ARGUMENT;
  const long long n_rows = (long long)n_groups * batch->total_tokens;
  if (n_rows > kMaxRows) return BNB_ERR_EXCEEDS_STATIC_LIMIT;
  if (n_rows == 0) return BNB_OK;
  if (!x || !y) return BNB_ERR_NULL_POINTER;
  if (!bnb::validate::aligned16(x) || !bnb::validate::aligned16(y)) return BNB_ERR_MISALIGNED;
  // Nothing in the array has to start at zero: the q/k/v rows and the attention rows this
  // call reads are all written by this call first.  What an earlier call left is ignored.
  for (int attempt = 0; attempt < 2; ++attempt) {
    float* scratch = nullptr;
    if ((st = scratch_address(&scratch, attempt == 1))) return st;
    float* qkv = scratch;
    float* o = scratch + (size_t)kMaxRows * 3 * kMaxWidth;
    st = bnb::exact::spatial_block(*w, d_model, n_heads, x, alive, nullptr, y, *batch, n_groups,
                                   precision == BNB_BF16, qkv, o, nullptr, 0, static_cast<cudaStream_t>(stream));
    // A launch that fails may mean the cached address belongs to a context that is gone (the
    // caller reset the device): look the array up again, once.
    if (st != BNB_ERR_LAUNCH) break;
    (void)cudaGetLastError();
  }
  return st;
}
