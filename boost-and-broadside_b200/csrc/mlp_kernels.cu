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
// One persistent CTA per SM: both weight matrices are converted to bfloat16 once per CTA and stay in
// shared memory.  After that the warps (up to 16, 28 for the heads) are independent: each walks slices of 16 rows of
// its own, stages the slice's input rows in its own shared-memory rows and keeps everything else in
// registers.  The hidden activations never leave the register file: the accumulator fragment of
// Linear 1 (row g, columns 2t, 2t+1 of two adjacent 8-column blocks) is exactly the A fragment of
// mma.sync for a 16-wide k step of Linear 2, so each 64-column chunk of the hidden layer is normed,
// passed through the GELU and multiplied into the output accumulators straight away.  The RMSNorm
// needs the whole row's sum of squares first: for a hidden layer wider than one chunk Linear 1 is
// computed twice, once for the sum alone (cheaper than a trip through shared memory: the kernel is
// bound by instruction issue, not by the tensor pipe).  No CTA-wide barrier after the weights.
#include "mlp_kernels.h"

#include "common.cuh"
#include "launch_count.h"
#include "tensor_common.cuh"

namespace bnb {
namespace mlp {

using tensor::gelu_fast;   // the fused trunk kernel's fit of the erf GELU (max relative error 1.2e-3, below bfloat16 rounding)
using tensor::ldsm_x4;
using tensor::mma_bf16;
using tensor::pack_bf16;
using tensor::smem_u32;

namespace {

constexpr int SLICE = 16;      // rows per warp slice (one mma.sync row block)
// Warps per CTA: 16 where the output accumulators take 64 registers (out_dim 128), 28 where they
// take 16 (out_dim 32: the heads, whose 65 536 rows are then one 16-row slice per warp of the grid).
__host__ __device__ constexpr int max_warps(int out_dim) { return out_dim <= 32 ? 28 : 16; }
constexpr int PAD = 8;         // bf16 elements of padding per staged row: ldmatrix stays conflict-free
constexpr size_t SMEM_MAX = 227 * 1024;

struct Layout {
  int ldx, ldw;   // row strides (bf16 elements): in_pad-wide arrays, the second weight
  int warps;      // warps per CTA
  size_t w1, w2, vec, slices, per_warp, total;
};
__host__ __device__ inline Layout layout(int in_pad, int hidden, int out_dim) {
  Layout l;
  l.ldx = in_pad + PAD;
  l.ldw = hidden + PAD;
  size_t off = 0;
  l.w1 = off; off += (size_t)hidden * l.ldx * 2;
  l.w2 = off; off += (size_t)out_dim * l.ldw * 2;
  l.vec = off; off += (size_t)(2 * hidden + 2 * out_dim) * 4;   // b1, g1, b2, g2
  l.slices = off;
  l.per_warp = (size_t)SLICE * l.ldx * 2;                        // a warp's staged input rows
  const size_t room = SMEM_MAX > off ? SMEM_MAX - off : 0;
  int w = (int)(room / l.per_warp);
  w = w > max_warps(out_dim) ? max_warps(out_dim) : w & ~1;
  l.warps = w;
  l.total = off + (size_t)w * l.per_warp;
  return l;
}

// One 64-column chunk of Linear 1 for the warp's 16 rows: acc[nt] = X W1[c0 + 8 nt ..]^T.
template <int IN16>
__device__ __forceinline__ void linear1_chunk(float (&acc)[8][4], uint32_t sX, uint32_t sW1, int ldx, int c0,
                                              int a_off, int b_row, int b_k) {
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
#pragma unroll
  for (int ks = 0; ks < IN16; ++ks) {
    const int k0 = ks * 16;
    uint32_t a0, a1, a2, a3;
    ldsm_x4(sX + (a_off + k0) * 2, a0, a1, a2, a3);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t q0, q1, q2, q3;
      ldsm_x4(sW1 + ((c0 + np * 16 + b_row) * ldx + k0 + b_k) * 2, q0, q1, q2, q3);
      mma_bf16(acc[2 * np], a0, a1, a2, a3, q0, q1);
      mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, q2, q3);
    }
  }
}

// NP2: pairs of 8-column output blocks (out_dim = 16 NP2: 32 for the heads, 128 for the encoders);
// NCH: 64-column chunks of the hidden layer (hidden = 64 NCH).  Both are compile-time so that every
// loop over fragments unrolls without guards; so is IN16, the 16-wide k steps of the first product
// (in_pad = 16 IN16).
template <int NP2, int NCH, int IN16>
__global__ void __launch_bounds__(32 * max_warps(16 * NP2), 1)
k_mlp_bf16(const float* __restrict__ x, int x_bf16, __nv_bfloat16* __restrict__ y, int n_rows, int in_dim, int in_pad, int hidden,
           int out_dim, int out_store, const float* __restrict__ w1, const float* __restrict__ b1,
           const float* __restrict__ g1, const float* __restrict__ w2, const float* __restrict__ b2,
           const float* __restrict__ g2) {
  extern __shared__ __align__(16) uint8_t sm[];
  const Layout L = layout(in_pad, hidden, out_dim);
  __nv_bfloat16* W1 = reinterpret_cast<__nv_bfloat16*>(sm + L.w1);
  __nv_bfloat16* W2 = reinterpret_cast<__nv_bfloat16*>(sm + L.w2);
  float* b1s = reinterpret_cast<float*>(sm + L.vec);
  float* g1s = b1s + hidden;
  float* b2s = g1s + hidden;
  float* g2s = b2s + out_dim;
  const int ldx = L.ldx, ldw = L.ldw;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_threads = blockDim.x;
  const int g = lane >> 2, t = lane & 3;

  // the weights, once per CTA: float32 in global memory (rows of whole 16-byte pieces on 16-byte
  // boundaries), bfloat16 operands here; four loads in flight per thread
  {
    constexpr int Q1 = 4 * IN16, Q2 = 16 * NCH;   // 16-byte pieces per row of w1 (in_pad wide) and w2 (hidden wide)
    const float4* s1 = reinterpret_cast<const float4*>(w1);
    for (int i0 = tid; i0 < hidden * Q1; i0 += 4 * n_threads) {
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int idx = i0 + j * n_threads;
        if (idx < hidden * Q1) v[j] = s1[idx];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int idx = i0 + j * n_threads;
        if (idx < hidden * Q1) {
          const int r = idx / Q1, q = idx - r * Q1;
          *reinterpret_cast<uint2*>(W1 + r * ldx + q * 4) = make_uint2(pack_bf16(v[j].x, v[j].y), pack_bf16(v[j].z, v[j].w));
        }
      }
    }
    const float4* s2 = reinterpret_cast<const float4*>(w2);
    for (int i0 = tid; i0 < out_dim * Q2; i0 += 4 * n_threads) {
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int idx = i0 + j * n_threads;
        if (idx < out_dim * Q2) v[j] = s2[idx];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int idx = i0 + j * n_threads;
        if (idx < out_dim * Q2) {
          const int r = idx / Q2, q = idx - r * Q2;
          *reinterpret_cast<uint2*>(W2 + r * ldw + q * 4) = make_uint2(pack_bf16(v[j].x, v[j].y), pack_bf16(v[j].z, v[j].w));
        }
      }
    }
  }
  for (int i = tid; i < hidden; i += n_threads) {
    b1s[i] = round_bf16(b1[i]);
    g1s[i] = g1[i];
  }
  for (int i = tid; i < out_dim; i += n_threads) {
    b2s[i] = round_bf16(b2[i]);
    g2s[i] = g2 ? g2[i] : 1.0f;
  }
  __syncthreads();   // the only CTA-wide barrier: from here on every warp works alone

  __nv_bfloat16* X = reinterpret_cast<__nv_bfloat16*>(sm + L.slices + (size_t)warp * L.per_warp);
  const uint32_t sX = smem_u32(X), sW1 = smem_u32(W1), sW2 = smem_u32(W2);
  // ldmatrix lane addressing: A rows by lane % 16, k half by lane / 16; B rows (output columns) by
  // lane % 8 + 8 (lane / 16), k half by (lane / 8) % 2
  const int a_off = (lane & 15) * ldx + (lane >> 4) * 8;
  const int b_row = (lane & 7) + (lane >> 4) * 8, b_k = ((lane >> 3) & 1) * 8;
  const int n_slices = (n_rows + SLICE - 1) / SLICE;
  const int warps = n_threads >> 5;
  constexpr bool two_pass = NCH > 1;
  // input rows as 16-byte pieces when rows are whole pieces on 16-byte boundaries, else element by
  // element; idx / d for idx < 2048 and d <= 128 as a multiplication (exact: the error stays below 1 / 512)
  const bool vec_in = in_dim == in_pad && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int q_per_row = in_pad >> 2;
  const int recip = ((1 << 20) + (vec_in ? q_per_row : in_pad) - 1) / (vec_in ? q_per_row : in_pad);

  for (int slice = blockIdx.x * warps + warp; slice < n_slices; slice += gridDim.x * warps) {
    const int row0 = slice * SLICE;
    const int n_valid = min(SLICE, n_rows - row0);
    // ---- this slice's input rows: one contiguous span of global memory.  Eight loads (four 16-byte
    // ones) are issued before the first is used: a warp keeps that many requests in flight.
    if (x_bf16) {   // rows already hold bfloat16 (in_dim == in_pad, a multiple of 16): 16-byte pieces, copied as they are
      const int p_per_row = in_pad >> 3, pieces = n_valid * p_per_row;
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)row0 * in_dim);
      for (int i0 = 0; i0 < (in_pad >> 4); i0 += 4) {   // SLICE * p_per_row / 32 iterations in all
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int idx = lane + 32 * (i0 + j);
          v[j] = make_uint4(0u, 0u, 0u, 0u);
          if (idx < pieces) v[j] = src[idx];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int idx = lane + 32 * (i0 + j);
          if (idx < SLICE * p_per_row) {
            const int r = idx / p_per_row, q = idx - r * p_per_row;
            *reinterpret_cast<uint4*>(X + r * ldx + q * 8) = v[j];
          }
        }
      }
    } else if (vec_in) {
      const int quads = n_valid * q_per_row;
      const float4* src = reinterpret_cast<const float4*>(x + (size_t)row0 * in_dim);
      for (int i0 = 0; i0 < (in_pad >> 3); i0 += 4) {   // SLICE * q_per_row / 32 iterations in all, a multiple of 4 or just 2
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int idx = lane + 32 * (i0 + j);
          v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (idx < quads) v[j] = src[idx];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int idx = lane + 32 * (i0 + j);
          if (idx < SLICE * q_per_row) {
            const int r = (idx * recip) >> 20, q = idx - r * q_per_row;
            *reinterpret_cast<uint2*>(X + r * ldx + q * 4) = make_uint2(pack_bf16(v[j].x, v[j].y), pack_bf16(v[j].z, v[j].w));
          }
        }
      }
    } else {
      const float* src = x + (size_t)row0 * in_dim;
      for (int i0 = 0; i0 < (in_pad >> 1); i0 += 8) {   // SLICE * in_pad / 32 iterations in all, a multiple of 8
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int idx = lane + 32 * (i0 + j);
          const int r = (idx * recip) >> 20, c = idx - r * in_pad;
          v[j] = 0.f;
          if (r < n_valid && c < in_dim) v[j] = src[r * in_dim + c];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int idx = lane + 32 * (i0 + j);
          const int r = (idx * recip) >> 20, c = idx - r * in_pad;
          X[r * ldx + c] = __float2bfloat16_rn(v[j]);
        }
      }
    }
    __syncwarp();

    float acc[8][4];
    float ss0 = 0.f, ss1 = 0.f;
    if (two_pass) {   // the sum of squares of the rounded Linear 1 output, every chunk
#pragma unroll 1
      for (int ch = 0; ch < NCH; ++ch) {
        const int c0 = ch * 64;
        linear1_chunk<IN16>(acc, sX, sW1, ldx, c0, a_off, b_row, b_k);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const float2 bb = *reinterpret_cast<const float2*>(b1s + c0 + nt * 8 + 2 * t);
          const float h00 = round_bf16(acc[nt][0] + bb.x), h01 = round_bf16(acc[nt][1] + bb.y);
          const float h10 = round_bf16(acc[nt][2] + bb.x), h11 = round_bf16(acc[nt][3] + bb.y);
          ss0 = fmaf(h00, h00, fmaf(h01, h01, ss0));
          ss1 = fmaf(h10, h10, fmaf(h11, h11, ss1));
        }
      }
    }
    float inv0 = 0.f, inv1 = 0.f;
    float acc2[2 * NP2][4];
#pragma unroll
    for (int nt = 0; nt < 2 * NP2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc2[nt][i] = 0.f;
#pragma unroll 1
    for (int ch = 0; ch < NCH; ++ch) {
      const int c0 = ch * 64;
      linear1_chunk<IN16>(acc, sX, sW1, ldx, c0, a_off, b_row, b_k);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float2 bb = *reinterpret_cast<const float2*>(b1s + c0 + nt * 8 + 2 * t);
        acc[nt][0] = round_bf16(acc[nt][0] + bb.x);
        acc[nt][1] = round_bf16(acc[nt][1] + bb.y);
        acc[nt][2] = round_bf16(acc[nt][2] + bb.x);
        acc[nt][3] = round_bf16(acc[nt][3] + bb.y);
        if (!two_pass) {
          ss0 = fmaf(acc[nt][0], acc[nt][0], fmaf(acc[nt][1], acc[nt][1], ss0));
          ss1 = fmaf(acc[nt][2], acc[nt][2], fmaf(acc[nt][3], acc[nt][3], ss1));
        }
      }
      if (c0 == 0) {   // the row sums are complete: after the first pass, or with this only chunk
        ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
        ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
        ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
        ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
        inv0 = rsqrtf(ss0 / (float)hidden + kRmsEps);
        inv1 = rsqrtf(ss1 / (float)hidden + kRmsEps);
      }
      // RMSNorm (float32, rounded once), GELU (rounded once by the pack), then straight into Linear 2
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        {
          uint32_t a[4];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int nt = 2 * kk + hf;
            const float2 gg = *reinterpret_cast<const float2*>(g1s + c0 + nt * 8 + 2 * t);
            a[2 * hf] = pack_bf16(gelu_fast(round_bf16(acc[nt][0] * inv0 * gg.x)), gelu_fast(round_bf16(acc[nt][1] * inv0 * gg.y)));
            a[2 * hf + 1] = pack_bf16(gelu_fast(round_bf16(acc[nt][2] * inv1 * gg.x)), gelu_fast(round_bf16(acc[nt][3] * inv1 * gg.y)));
          }
#pragma unroll
          for (int np = 0; np < NP2; ++np) {
            {
              uint32_t q0, q1, q2, q3;
              ldsm_x4(sW2 + ((np * 16 + b_row) * ldw + c0 + kk * 16 + b_k) * 2, q0, q1, q2, q3);
              mma_bf16(acc2[2 * np], a[0], a[1], a[2], a[3], q0, q1);
              mma_bf16(acc2[2 * np + 1], a[0], a[1], a[2], a[3], q2, q3);
            }
          }
        }
      }
    }

    // ---- bias [+ RMSNorm] of Linear 2, then the first out_store columns of the 16 rows
    ss0 = 0.f;
    ss1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2 * NP2; ++nt) {
      {
        const float2 bb = *reinterpret_cast<const float2*>(b2s + nt * 8 + 2 * t);
        acc2[nt][0] = round_bf16(acc2[nt][0] + bb.x);
        acc2[nt][1] = round_bf16(acc2[nt][1] + bb.y);
        acc2[nt][2] = round_bf16(acc2[nt][2] + bb.x);
        acc2[nt][3] = round_bf16(acc2[nt][3] + bb.y);
        ss0 = fmaf(acc2[nt][0], acc2[nt][0], fmaf(acc2[nt][1], acc2[nt][1], ss0));
        ss1 = fmaf(acc2[nt][2], acc2[nt][2], fmaf(acc2[nt][3], acc2[nt][3], ss1));
      }
    }
    float o0 = 1.0f, o1 = 1.0f;
    if (g2) {   // the encoders end in a norm, the heads do not
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
      o0 = rsqrtf(ss0 / (float)out_dim + kRmsEps);
      o1 = rsqrtf(ss1 / (float)out_dim + kRmsEps);
    }
    __nv_bfloat16* y0 = y + (size_t)(row0 + g) * out_store;
    __nv_bfloat16* y1 = y + (size_t)(row0 + g + 8) * out_store;
    const bool pair_store = (out_store & 1) == 0;   // columns 2t, 2t+1 of a row share an aligned 4-byte word
#pragma unroll
    for (int nt = 0; nt < 2 * NP2; ++nt) {
      {
        const int c = nt * 8 + 2 * t;
        if (c < out_store) {
          const float2 s = *reinterpret_cast<const float2*>(g2s + c);
          const uint32_t v0 = pack_bf16(acc2[nt][0] * o0 * s.x, acc2[nt][1] * o0 * s.y);
          const uint32_t v1 = pack_bf16(acc2[nt][2] * o1 * s.x, acc2[nt][3] * o1 * s.y);
          if (pair_store) {
            if (g < n_valid) *reinterpret_cast<uint32_t*>(y0 + c) = v0;
            if (g + 8 < n_valid) *reinterpret_cast<uint32_t*>(y1 + c) = v1;
          } else {
            const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&v0), p1 = *reinterpret_cast<const __nv_bfloat162*>(&v1);
            if (g < n_valid) {
              y0[c] = p0.x;
              if (c + 1 < out_store) y0[c + 1] = p0.y;
            }
            if (g + 8 < n_valid) {
              y1[c] = p1.x;
              if (c + 1 < out_store) y1[c + 1] = p1.y;
            }
          }
        }
      }
    }
    __syncwarp();   // every lane is done with the staged input rows before the next slice overwrites them
  }
}

}  // namespace

bool supported(int in_pad, int hidden, int out_dim) {
  if (in_pad != 32 && in_pad != 64 && in_pad != 96 && in_pad != 128) return false;   // the instantiated k-step counts
  if (hidden != 64 && hidden != 128 && hidden != 256) return false;   // the instantiated chunk counts
  if (out_dim != 32 && out_dim != 128) return false;                  // and output widths
  return layout(in_pad, hidden, out_dim).warps >= 4;
}

int encoder_mlp_bf16(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2, const float* g2,
                     int in_dim, int in_pad, int hidden, int out_dim, int out_store, const void* x, bool x_bf16, void* y,
                     int n_rows, cudaStream_t st) {
  if (!supported(in_pad, hidden, out_dim)) return BNB_ERR_UNSUPPORTED_DIMS;
  if (x_bf16 && (in_dim != in_pad || (reinterpret_cast<uintptr_t>(x) & 15))) return BNB_ERR_UNSUPPORTED_DIMS;
  if (n_rows <= 0) return BNB_OK;
  if (reinterpret_cast<uintptr_t>(y) & 3) return BNB_ERR_MISALIGNED;
  const Layout L = layout(in_pad, hidden, out_dim);
  using Kernel = void (*)(const float*, int, __nv_bfloat16*, int, int, int, int, int, int, const float*, const float*, const float*,
                          const float*, const float*, const float*);
#define BNB_MLP_ROW(NP2, NCH) {k_mlp_bf16<NP2, NCH, 2>, k_mlp_bf16<NP2, NCH, 4>, k_mlp_bf16<NP2, NCH, 6>, k_mlp_bf16<NP2, NCH, 8>}
  static const Kernel table[2][3][4] = {{BNB_MLP_ROW(2, 1), BNB_MLP_ROW(2, 2), BNB_MLP_ROW(2, 4)},
                                        {BNB_MLP_ROW(8, 1), BNB_MLP_ROW(8, 2), BNB_MLP_ROW(8, 4)}};
#undef BNB_MLP_ROW
  const Kernel kernel = table[out_dim == 32 ? 0 : 1][hidden == 64 ? 0 : hidden == 128 ? 1 : 2][in_pad / 32 - 1];
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total) != cudaSuccess) return BNB_ERR_LAUNCH;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return BNB_ERR_NO_DEVICE;
  const int n_slices = (n_rows + SLICE - 1) / SLICE;
  const int want = (n_slices + L.warps - 1) / L.warps;
  const int grid = want < sms ? want : sms;
  count_launch();
  kernel<<<grid, 32 * L.warps, L.total, st>>>(static_cast<const float*>(x), x_bf16 ? 1 : 0, static_cast<__nv_bfloat16*>(y), n_rows, in_dim, in_pad, hidden, out_dim, out_store,
                                              w1, b1, g1, w2, b2, g2);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

}  // namespace mlp
}  // namespace bnb
