// The encoder / head MLP of the policy under the autocast contract, on bf16 tensor-core tiles.
//
//   Linear(in, hidden) + b -> RMSNorm(hidden) -> GELU -> Linear(hidden, out) + b [-> RMSNorm(out)]
//
// is the chain of the reference's ShipEncoder and BulletEncoder (models/yemong/encoder.py:45-51,
// 84-102) and, without the last norm and with only the first out_store columns stored, of the four
// heads of the policy (models/yemong/policy.py:185-214).  Every stage hands on bfloat16 as under
// torch.autocast: operands of both products are bfloat16, accumulation is float32, a Linear output
// is rounded once after its bias, an RMSNorm of a bfloat16 input is computed in float32 and rounded
// once, and so is the GELU.  The float32 contract stays on the CUDA-core engine (exact_kernels.cu).
//
// One persistent CTA per SM slot: both weight matrices are converted to bfloat16 once per CTA and stay
// in shared memory; the CTA then walks tiles of 128 rows.  Warp w owns rows [16 w, 16 w + 16) of the
// tile through every stage, so only the loading of a tile needs a CTA-wide barrier.
#include "mlp_kernels.h"

#include "common.cuh"
#include "launch_count.h"
#include "tensor_common.cuh"

namespace bnb {
namespace mlp {

using tensor::ldsm_x4;
using tensor::mma_bf16;
using tensor::pack_bf16;
using tensor::smem_u32;

namespace {

constexpr int TILE = 128;      // rows per tile
constexpr int THREADS = 256;   // 8 warps x 16 rows
constexpr int PAD = 8;         // bf16 elements of padding per staged row: ldmatrix stays conflict-free
constexpr size_t SMEM_MAX = 227 * 1024;

struct Layout {
  int ldx, ldh;   // row strides (bf16 elements) of the in_pad-wide and the hidden-wide arrays
  size_t w1, w2, x, h, vec, total;
};
__host__ __device__ inline Layout layout(int in_pad, int hidden, int out_dim) {
  Layout l;
  l.ldx = in_pad + PAD;
  l.ldh = hidden + PAD;
  size_t off = 0;
  l.w1 = off; off += (size_t)hidden * l.ldx * 2;
  l.w2 = off; off += (size_t)out_dim * l.ldh * 2;
  l.x = off; off += (size_t)TILE * l.ldx * 2;
  l.h = off; off += (size_t)TILE * l.ldh * 2;
  l.vec = off; off += (size_t)(2 * hidden + 2 * out_dim + TILE) * 4;   // b1, g1, b2, g2, 1/rms per row
  l.total = off;
  return l;
}

}  // namespace

namespace {

__device__ __forceinline__ float2 unpack2(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}

__global__ void __launch_bounds__(THREADS, 2)
k_mlp_bf16(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, int n_rows, int in_dim, int in_pad, int hidden,
           int out_dim, int out_store, int vec_store, const float* __restrict__ w1, const float* __restrict__ b1,
           const float* __restrict__ g1, const float* __restrict__ w2, const float* __restrict__ b2,
           const float* __restrict__ g2) {
  extern __shared__ __align__(16) uint8_t sm[];
  const Layout L = layout(in_pad, hidden, out_dim);
  __nv_bfloat16* W1 = reinterpret_cast<__nv_bfloat16*>(sm + L.w1);
  __nv_bfloat16* W2 = reinterpret_cast<__nv_bfloat16*>(sm + L.w2);
  __nv_bfloat16* X = reinterpret_cast<__nv_bfloat16*>(sm + L.x);
  __nv_bfloat16* H = reinterpret_cast<__nv_bfloat16*>(sm + L.h);
  float* b1s = reinterpret_cast<float*>(sm + L.vec);
  float* g1s = b1s + hidden;
  float* b2s = g1s + hidden;
  float* g2s = b2s + out_dim;
  float* rinv = g2s + out_dim;
  const int ldx = L.ldx, ldh = L.ldh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  // the weights, once per CTA: float32 in global memory, bfloat16 operands here
  for (int idx = tid; idx < hidden * in_pad; idx += THREADS) {
    const int r = idx / in_pad, c = idx - r * in_pad;
    W1[r * ldx + c] = __float2bfloat16_rn(w1[idx]);
  }
  for (int idx = tid; idx < out_dim * hidden; idx += THREADS) {
    const int r = idx / hidden, c = idx - r * hidden;
    W2[r * ldh + c] = __float2bfloat16_rn(w2[idx]);
  }
  for (int i = tid; i < hidden; i += THREADS) {
    b1s[i] = round_bf16(b1[i]);
    g1s[i] = g1[i];
  }
  for (int i = tid; i < out_dim; i += THREADS) {
    b2s[i] = round_bf16(b2[i]);
    g2s[i] = g2 ? g2[i] : 1.0f;
  }

  const int n_tiles = (n_rows + TILE - 1) / TILE;
  const int wr = warp * 16;
  const uint32_t sX = smem_u32(X), sH = smem_u32(H), sW1 = smem_u32(W1), sW2 = smem_u32(W2);
  // ldmatrix lane addressing: A rows by lane % 16, k half by lane / 16; B rows (output columns) by
  // lane % 8 + 8 (lane / 16), k half by (lane / 8) % 2
  const int a_row = wr + (lane & 15), a_k = (lane >> 4) * 8;
  const int b_row = (lane & 7) + (lane >> 4) * 8, b_k = ((lane >> 3) & 1) * 8;

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int row0 = tile * TILE;
    const int n_valid = min(TILE, n_rows - row0);
    __syncthreads();   // the weights are staged; every warp is done with the previous tile's X
    if ((in_dim & 3) == 0 && in_dim == in_pad) {
      const int q_per_row = in_pad >> 2;
      for (int idx = tid; idx < TILE * q_per_row; idx += THREADS) {
        const int r = idx / q_per_row, q = idx - r * q_per_row;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < n_valid) v = *reinterpret_cast<const float4*>(x + (size_t)(row0 + r) * in_dim + q * 4);
        *reinterpret_cast<uint2*>(X + r * ldx + q * 4) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
      }
    } else {
      for (int idx = tid; idx < TILE * in_pad; idx += THREADS) {
        const int r = idx / in_pad, c = idx - r * in_pad;
        float v = 0.f;
        if (r < n_valid && c < in_dim) v = x[(size_t)(row0 + r) * in_dim + c];
        X[r * ldx + c] = __float2bfloat16_rn(v);
      }
    }
    __syncthreads();

    // ---- Linear 1 + bias, 64 output columns at a time; the rounded result goes to H, its squares are summed
    float ss0 = 0.f, ss1 = 0.f;
    for (int c0 = 0; c0 < hidden; c0 += 64) {
      const int npairs = min(4, (hidden - c0) >> 4);
      float acc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
      for (int k0 = 0; k0 < in_pad; k0 += 16) {
        uint32_t a0, a1, a2, a3;
        ldsm_x4(sX + (a_row * ldx + k0 + a_k) * 2, a0, a1, a2, a3);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          if (np < npairs) {
            uint32_t q0, q1, q2, q3;
            ldsm_x4(sW1 + ((c0 + np * 16 + b_row) * ldx + k0 + b_k) * 2, q0, q1, q2, q3);
            mma_bf16(acc[2 * np], a0, a1, a2, a3, q0, q1);
            mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, q2, q3);
          }
        }
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt < 2 * npairs) {
          const int c = c0 + nt * 8 + 2 * t;
          const float bb0 = b1s[c], bb1 = b1s[c + 1];
          const float h00 = round_bf16(acc[nt][0] + bb0), h01 = round_bf16(acc[nt][1] + bb1);
          const float h10 = round_bf16(acc[nt][2] + bb0), h11 = round_bf16(acc[nt][3] + bb1);
          ss0 = fmaf(h00, h00, fmaf(h01, h01, ss0));
          ss1 = fmaf(h10, h10, fmaf(h11, h11, ss1));
          *reinterpret_cast<uint32_t*>(H + (wr + g) * ldh + c) = pack_bf16(h00, h01);
          *reinterpret_cast<uint32_t*>(H + (wr + g + 8) * ldh + c) = pack_bf16(h10, h11);
        }
      }
    }
    ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
    ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
    ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
    ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
    if (t == 0) {
      rinv[wr + g] = rsqrtf(ss0 / (float)hidden + kRmsEps);
      rinv[wr + g + 8] = rsqrtf(ss1 / (float)hidden + kRmsEps);
    }
    __syncwarp();
    // ---- RMSNorm (float32, rounded once) and GELU (rounded once) over this warp's 16 rows of H
    {
      const int half = hidden >> 1;
      for (int idx = lane; idx < 16 * half; idx += 32) {
        const int r = idx / half, c = (idx - r * half) * 2;
        uint32_t* p = reinterpret_cast<uint32_t*>(H + (wr + r) * ldh + c);
        const float2 h = unpack2(*p);
        const float inv = rinv[wr + r];
        const float v0 = round_bf16(h.x * inv * g1s[c]), v1 = round_bf16(h.y * inv * g1s[c + 1]);
        *p = pack_bf16(gelu_erf(v0), gelu_erf(v1));
      }
    }
    __syncwarp();

    // ---- Linear 2 + bias [+ RMSNorm], all out_dim columns in registers
    const int npairs2 = out_dim >> 4;
    float acc[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
    for (int k0 = 0; k0 < hidden; k0 += 16) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(sH + (a_row * ldh + k0 + a_k) * 2, a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        if (np < npairs2) {
          uint32_t q0, q1, q2, q3;
          ldsm_x4(sW2 + ((np * 16 + b_row) * ldh + k0 + b_k) * 2, q0, q1, q2, q3);
          mma_bf16(acc[2 * np], a0, a1, a2, a3, q0, q1);
          mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, q2, q3);
        }
      }
    }
    __syncwarp();   // every lane has read its part of this warp's rows of H: they now stage the output
    ss0 = 0.f;
    ss1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      if (nt < 2 * npairs2) {
        const int c = nt * 8 + 2 * t;
        const float bb0 = b2s[c], bb1 = b2s[c + 1];
        acc[nt][0] = round_bf16(acc[nt][0] + bb0);
        acc[nt][1] = round_bf16(acc[nt][1] + bb1);
        acc[nt][2] = round_bf16(acc[nt][2] + bb0);
        acc[nt][3] = round_bf16(acc[nt][3] + bb1);
        ss0 = fmaf(acc[nt][0], acc[nt][0], fmaf(acc[nt][1], acc[nt][1], ss0));
        ss1 = fmaf(acc[nt][2], acc[nt][2], fmaf(acc[nt][3], acc[nt][3], ss1));
      }
    }
    float inv0 = 1.0f, inv1 = 1.0f;
    if (g2) {   // the encoders end in a norm, the heads do not
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
      inv0 = rsqrtf(ss0 / (float)out_dim + kRmsEps);
      inv1 = rsqrtf(ss1 / (float)out_dim + kRmsEps);
    }
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      if (nt < 2 * npairs2) {
        const int c = nt * 8 + 2 * t;
        const float s0 = g2s[c], s1 = g2s[c + 1];
        *reinterpret_cast<uint32_t*>(H + (wr + g) * ldh + c) = pack_bf16(acc[nt][0] * inv0 * s0, acc[nt][1] * inv0 * s1);
        *reinterpret_cast<uint32_t*>(H + (wr + g + 8) * ldh + c) = pack_bf16(acc[nt][2] * inv1 * s0, acc[nt][3] * inv1 * s1);
      }
    }
    __syncwarp();
    if (vec_store) {   // whole 16-byte pieces of a row
      const int pieces = out_store >> 3;
      for (int idx = lane; idx < 16 * pieces; idx += 32) {
        const int r = idx / pieces, q = idx - r * pieces;
        if (wr + r < n_valid)
          *reinterpret_cast<uint4*>(y + (size_t)(row0 + wr + r) * out_store + q * 8) =
              *reinterpret_cast<const uint4*>(H + (wr + r) * ldh + q * 8);
      }
    } else {
      for (int idx = lane; idx < 16 * out_store; idx += 32) {
        const int r = idx / out_store, c = idx - r * out_store;
        if (wr + r < n_valid) y[(size_t)(row0 + wr + r) * out_store + c] = H[(wr + r) * ldh + c];
      }
    }
    __syncwarp();   // the staged output is read before the next tile's Linear 1 writes these rows
  }
}

}  // namespace

bool supported(int in_pad, int hidden, int out_dim) {
  if (in_pad <= 0 || in_pad % 16 != 0 || hidden <= 0 || hidden % 32 != 0 || out_dim <= 0 || out_dim % 32 != 0) return false;
  if (in_pad > 128 || hidden > 256 || out_dim > 128 || out_dim > hidden) return false;
  return layout(in_pad, hidden, out_dim).total <= SMEM_MAX;
}

int encoder_mlp_bf16(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2, const float* g2,
                     int in_dim, int in_pad, int hidden, int out_dim, int out_store, const float* x, void* y, int n_rows,
                     cudaStream_t st) {
  if (!supported(in_pad, hidden, out_dim)) return BNB_ERR_UNSUPPORTED_DIMS;
  if (n_rows <= 0) return BNB_OK;
  const size_t smem = layout(in_pad, hidden, out_dim).total;
  if (cudaFuncSetAttribute(k_mlp_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return BNB_ERR_LAUNCH;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return BNB_ERR_NO_DEVICE;
  const int per_sm = smem * 2 + 2048 <= SMEM_MAX ? 2 : 1;
  const int n_tiles = (n_rows + TILE - 1) / TILE;
  const int grid = n_tiles < sms * per_sm ? n_tiles : sms * per_sm;
  // a 16-byte row store needs y and every row of it on a 16-byte boundary
  const int vec_store = (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (out_store & 7) == 0;
  count_launch();
  k_mlp_bf16<<<grid, THREADS, smem, st>>>(x, static_cast<__nv_bfloat16*>(y), n_rows, in_dim, in_pad, hidden, out_dim, out_store, vec_store,
                                          w1, b1, g1, w2, b2, g2);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

}  // namespace mlp
}  // namespace bnb
