// Exact-arithmetic kernels of the Yemong trunk: float32 results throughout (elementwise math on
// the CUDA cores, Linear products as 3 x tf32 tensor-core MMAs with float32 accumulation), with
// the bf16 roundings of the autocast contract applied in software when EMU is set.
//
// These kernels serve BNB_FP32 calls (1e-4 parity needs float32 products, which the
// bf16 tensor-core path cannot give) and BNB_BF16 calls whose shapes the tensor-core
// kernels are not built for.  They follow
//   TransformerBlock.forward        models/yemong/attention.py:76-169
//   GatedMLP.forward                models/yemong/attention.py:21-37
//   GriffinTemporalBlock.*          models/yemong/griffin.py:249-317
//   RGLRU gates / update            models/yemong/griffin.py:169-219
//   causal conv + tap validity      models/yemong/griffin.py:67-140
// of the reference.
#include "common.cuh"
#include "exact_kernels.h"
#include "grad_kernels.h"
#include "launch_count.h"

namespace bnb {
namespace exact {

constexpr int ROWS = 32;        // token rows per CTA
constexpr int NTHREADS = 256;   // 8 warps; warp w owns rows 4w..4w+3
constexpr int KC = 32;          // K chunk staged per pass
constexpr int WS_STRIDE = KC + 4;
constexpr int NCHUNK = 128;     // output columns per tile_linear call

// Split of a float into two tf32 numbers, hi + lo = v to about 2^-21: the products
// lo*hi + hi*lo + hi*hi of two such pairs, accumulated in float32 by the tensor cores, keep
// float32-level accuracy (the dropped lo*lo term is below 2^-22 relative).
__device__ __forceinline__ uint32_t to_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ void split_tf32(float v, uint32_t& hi, uint32_t& lo) {
  hi = to_tf32(v);
  lo = to_tf32(v - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc[i][j] += sum_k A[4*warp+i][k] * W[(lane + 32 j)][k]   for lane + 32 j < N
// A: shared, row stride lda (floats, lda = 4 mod 32), already rounded for EMU.  W: global, row
// stride ldw.  Ws: shared staging of NCHUNK x WS_STRIDE floats.  All threads of the CTA must call.
//
// The products run on the tensor cores as m16n8k8 tf32 MMAs with float32 accumulation: warp w
// owns rows 16 (w & 1) .. +15 and the 8-column blocks (w >> 1) + 4 q.  With EMU the operands are
// bf16 values, exact in tf32, so one MMA per block; otherwise each operand is split in two tf32
// numbers and three MMAs give the float32 product.  The result goes through shared memory into
// the (4 rows x 4 strided columns) per-thread layout the callers' epilogues use.
template <bool EMU>
__device__ __forceinline__ void tile_linear(const float* __restrict__ A, int lda,
                                            const float* __restrict__ W, int ldw, int N, int K,
                                            float* __restrict__ Ws, float (&acc)[4][4]) {
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int mrow = 16 * (warp & 1) + g;
  float c[4][4];
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[q][i] = 0.f;
  for (int k0 = 0; k0 < K; k0 += KC) {
    __syncthreads();  // previous users of Ws are done
    for (int idx = tid; idx < N * (KC / 4); idx += NTHREADS) {
      int cc = idx >> 3, q = idx & 7;
      float4 v = *reinterpret_cast<const float4*>(W + (size_t)cc * ldw + k0 + q * 4);
      if constexpr (EMU) {
        v.x = round_bf16(v.x); v.y = round_bf16(v.y); v.z = round_bf16(v.z); v.w = round_bf16(v.w);
      }
      *reinterpret_cast<float4*>(Ws + cc * WS_STRIDE + q * 4) = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KC; kk += 8) {
      const float* ap = A + mrow * lda + k0 + kk + t;
      const float af[4] = {ap[0], ap[8 * lda], ap[4], ap[8 * lda + 4]};
      uint32_t ah[4], al[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if constexpr (EMU) ah[i] = __float_as_uint(af[i]);
        else split_tf32(af[i], ah[i], al[i]);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int n0 = 8 * ((warp >> 1) + 4 * q);
        if (n0 < N) {
          const float* bp = Ws + (n0 + g) * WS_STRIDE + kk + t;
          if constexpr (EMU) {
            mma_tf32(c[q], ah, __float_as_uint(bp[0]), __float_as_uint(bp[4]));
          } else {
            uint32_t bh0, bl0, bh1, bl1;
            split_tf32(bp[0], bh0, bl0);
            split_tf32(bp[4], bh1, bl1);
            mma_tf32(c[q], al, bh0, bh1);
            mma_tf32(c[q], ah, bl0, bl1);
            mma_tf32(c[q], ah, bh0, bh1);
          }
        }
      }
    }
  }
  // fragments -> shared (the staging area is free now) -> the callers' per-thread layout
  constexpr int LDC = NCHUNK + 4;
  static_assert(ROWS * LDC <= NCHUNK * WS_STRIDE, "the staging area must hold one output tile");
  __syncthreads();
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int n0 = 8 * ((warp >> 1) + 4 * q);
    if (n0 < N) {
      *reinterpret_cast<float2*>(Ws + mrow * LDC + n0 + 2 * t) = make_float2(c[q][0], c[q][1]);
      *reinterpret_cast<float2*>(Ws + (mrow + 8) * LDC + n0 + 2 * t) = make_float2(c[q][2], c[q][3]);
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = lane + 32 * j;
      if (col < N) acc[i][j] += Ws[(4 * warp + i) * LDC + col];
    }
}

__device__ __forceinline__ void zero_acc(float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
}

// RMS norm of the rows of X (ROWS x D, stride ld) into Nrm (rounded for EMU).
// Warp w handles rows 4w..4w+3.  Rows >= n_valid produce zeros.
template <bool EMU>
__device__ __forceinline__ void tile_rmsnorm(const float* X, float* Nrm, int ld, int D,
                                             const float* __restrict__ g, int n_valid) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = 0; i < 4; ++i) {
    int r = 4 * warp + i;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) { float v = X[r * ld + c]; ss = fmaf(v, v, ss); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float inv = rsqrtf(ss / (float)D + kRmsEps);
    for (int c = lane; c < D; c += 32) {
      float v = (r < n_valid) ? X[r * ld + c] * inv * g[c] : 0.f;
      Nrm[r * ld + c] = rnd<EMU>(v);
    }
  }
}

// x2 = x1 + down(gelu(gate(m)) * up(m)) for the tile; m = rmsnorm(x1).  X holds x1 on entry
// and is left untouched; the result is returned in out[i][j] for columns of chunk `oc`.
// Shared buffers: Nrm (normed input), P (gated product chunk).  D <= 128.
template <bool EMU>
__device__ __forceinline__ void tile_gated_mlp(const float* Nrm, float* P, int ld, int D,
                                               const float* __restrict__ Wg, const float* __restrict__ Wu,
                                               const float* __restrict__ Wd, float* Ws,
                                               float (&down)[4][4]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = 4 * D;
  zero_acc(down);
  for (int h0 = 0; h0 < H; h0 += NCHUNK) {
    int hn = min(NCHUNK, H - h0);
    float g[4][4], u[4][4];
    zero_acc(g);
    zero_acc(u);
    tile_linear<EMU>(Nrm, ld, Wg + (size_t)h0 * D, D, hn, D, Ws, g);
    tile_linear<EMU>(Nrm, ld, Wu + (size_t)h0 * D, D, hn, D, Ws, u);
    __syncthreads();  // previous readers of P are done
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        if (c < hn) {
          float ge = rnd<EMU>(gelu_erf(rnd<EMU>(g[i][j])));
          P[(4 * warp + i) * ld + c] = rnd<EMU>(ge * rnd<EMU>(u[i][j]));
        }
      }
    __syncthreads();
    tile_linear<EMU>(P, ld, Wd + h0, H, D, hn, Ws, down);
  }
}

// ------------------------------------------------------------------ spatial, stage 1
// qkv = Linear(rmsnorm(x))  -> (rows, n_out) float32 scratch (values bf16-rounded for EMU).
// n_out = 3D for the entity tokens (qkv), 2D for the bullet tokens (kv_bullet of norm_bullet).
template <bool EMU>
__global__ void __launch_bounds__(NTHREADS)
k_spatial_qkv(const float* __restrict__ x, float* __restrict__ qkv, int n_rows, int D, int n_out,
              const float* __restrict__ g1, const float* __restrict__ Wqkv) {
  extern __shared__ __align__(16) float smem[];
  const int ld = D + 4;
  float* X = smem;
  float* Nrm = X + ROWS * ld;
  float* Ws = Nrm + ROWS * ld;
  const int row0 = blockIdx.x * ROWS;
  const int n_valid = min(ROWS, n_rows - row0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int idx = tid; idx < ROWS * (D / 4); idx += NTHREADS) {
    int r = idx / (D / 4), q = idx % (D / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < n_valid) v = *reinterpret_cast<const float4*>(x + (size_t)(row0 + r) * D + q * 4);
    *reinterpret_cast<float4*>(X + r * ld + q * 4) = v;
  }
  __syncthreads();
  if (g1) {
    tile_rmsnorm<EMU>(X, Nrm, ld, D, g1, n_valid);
  } else {   // a plain projection of the rows (TeamPMA's keys and values)
    for (int idx = tid; idx < ROWS * D; idx += NTHREADS) {
      const int r = idx / D, cc = idx - r * D;
      Nrm[r * ld + cc] = rnd<EMU>(X[r * ld + cc]);
    }
    __syncthreads();
  }
  for (int c0 = 0; c0 < n_out; c0 += NCHUNK) {
    int cn = min(NCHUNK, n_out - c0);
    float acc[4][4];
    zero_acc(acc);
    tile_linear<EMU>(Nrm, ld, Wqkv + (size_t)c0 * D, D, cn, D, Ws, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = 4 * warp + i;
      if (r < n_valid)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int c = lane + 32 * j;
          if (c < cn) qkv[(size_t)(row0 + r) * n_out + c0 + c] = rnd<EMU>(acc[i][j]);
        }
    }
  }
}

// ------------------------------------------------------------------ spatial, stage 2
// One softmax(q k^T / sqrt(dh) + bias) v over n keys, single pass with a running maximum.
// Key j sits at kbase + j * stride, its value `voff` floats after it.  A masked key scores
// kMaskedScore, so its weight is exactly 0 while any key is live, and when none is live
// every key gets weight 1/n (attention.py:101-112 with finfo.min/2 as the bias).
template <int DH>
__device__ __forceinline__ void attend(const float (&q)[DH], const float* __restrict__ kbase, size_t stride,
                                       int voff, int n, const uint8_t* __restrict__ mask, float scale,
                                       float (&acc)[DH]) {
#pragma unroll
  for (int d = 0; d < DH; ++d) acc[d] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int j = 0; j < n; ++j) {
    const float* kp = kbase + (size_t)j * stride;
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < DH; d += 4) {
      float4 v = *reinterpret_cast<const float4*>(kp + d);
      s = fmaf(q[d], v.x, s); s = fmaf(q[d + 1], v.y, s);
      s = fmaf(q[d + 2], v.z, s); s = fmaf(q[d + 3], v.w, s);
    }
    s *= scale;
    if (mask && !mask[j]) s = kMaskedScore;
    float mn = fmaxf(m, s);
    float corr = expf(m - mn);   // m = -inf on the first key: exp(-inf) = 0
    float pj = expf(s - mn);
    l = l * corr + pj;
    const float* vp = kp + voff;
#pragma unroll
    for (int d = 0; d < DH; d += 4) {
      float4 v = *reinterpret_cast<const float4*>(vp + d);
      acc[d] = fmaf(pj, v.x, acc[d] * corr);
      acc[d + 1] = fmaf(pj, v.y, acc[d + 1] * corr);
      acc[d + 2] = fmaf(pj, v.z, acc[d + 2] * corr);
      acc[d + 3] = fmaf(pj, v.w, acc[d + 3] * corr);
    }
    m = mn;
  }
  float inv = 1.0f / l;
#pragma unroll
  for (int d = 0; d < DH; ++d) acc[d] *= inv;
}

// Masked attention inside each environment, one thread per (query token, head): self-attention
// over the environment's tokens and, when kvb is given, a second softmax over its bullet keys
// (kvb holds nb rows of [k (D) | v (D)] per environment of this launch's slice), gated to zero
// for an environment with no active bullet, and summed before the output projection
// (attention.py:149-166).  env_base is the first environment (group-major) of the slice.
template <bool EMU, int DH>
__global__ void __launch_bounds__(128)
k_attention(const float* __restrict__ qkv, const uint8_t* __restrict__ alive, float* __restrict__ o,
            EnvMap map, int env_base, int D, int H, const float* __restrict__ kvb,
            const uint8_t* __restrict__ bullet_active, int nb) {
  const int env_g = env_base + blockIdx.x;  // group-major environment index
  const int grp = env_g / map.n_envs, e = env_g - grp * map.n_envs;
  const int tok0 = grp * map.total_tokens + map.env_tok_begin(e);
  const int n = map.env_tok_count(e);
  const float scale = rsqrtf((float)DH);
  float gate = 1.f;
  const uint8_t* bmask = nullptr;
  if (kvb && bullet_active) {
    bmask = bullet_active + (size_t)env_g * nb;
    int any = 0;
    for (int j = 0; j < nb; ++j) any |= bmask[j];
    gate = any ? 1.f : 0.f;
  }
  for (int p = blockIdx.y * blockDim.x + threadIdx.x; p < n * H; p += gridDim.y * blockDim.x) {
    const int qi = p / H, h = p - qi * H;
    const float* qp = qkv + (size_t)(tok0 + qi) * 3 * D + h * DH;
    float q[DH], acc[DH];
#pragma unroll
    for (int d = 0; d < DH; d += 4) {
      float4 v = *reinterpret_cast<const float4*>(qp + d);
      q[d] = v.x; q[d + 1] = v.y; q[d + 2] = v.z; q[d + 3] = v.w;
    }
    attend<DH>(q, qkv + (size_t)tok0 * 3 * D + D + h * DH, (size_t)3 * D, D, n,
               alive ? alive + tok0 : nullptr, scale, acc);
    float* op = o + (size_t)(tok0 + qi) * D + h * DH;
#pragma unroll
    for (int d = 0; d < DH; d += 4)
      *reinterpret_cast<float4*>(op + d) = make_float4(rnd<EMU>(acc[d]), rnd<EMU>(acc[d + 1]),
                                                       rnd<EMU>(acc[d + 2]), rnd<EMU>(acc[d + 3]));
    if (kvb) {
      attend<DH>(q, kvb + (size_t)blockIdx.x * nb * 2 * D + h * DH, (size_t)2 * D, D, nb, bmask, scale, acc);
#pragma unroll
      for (int d = 0; d < DH; d += 4) {
        float4 s = *reinterpret_cast<const float4*>(op + d);   // this thread's own write above
        s.x = rnd<EMU>(s.x + rnd<EMU>(acc[d]) * gate);
        s.y = rnd<EMU>(s.y + rnd<EMU>(acc[d + 1]) * gate);
        s.z = rnd<EMU>(s.z + rnd<EMU>(acc[d + 2]) * gate);
        s.w = rnd<EMU>(s.w + rnd<EMU>(acc[d + 3]) * gate);
        *reinterpret_cast<float4*>(op + d) = s;
      }
    }
  }
}

// ------------------------------------------------------------------ spatial, stage 3
// x1 = x + Linear_out(o);  y = x1 + GatedMLP(rmsnorm(x1))
template <bool EMU>
__global__ void __launch_bounds__(NTHREADS)
k_spatial_post(const float* __restrict__ x, const float* __restrict__ o, float* __restrict__ y,
               int n_rows, int D, const float* __restrict__ Wout, const float* __restrict__ g2,
               const float* __restrict__ Wg, const float* __restrict__ Wu, const float* __restrict__ Wd) {
  extern __shared__ __align__(16) float smem[];
  const int ld = max(D, NCHUNK) + 4;
  float* X = smem;
  float* Nrm = X + ROWS * ld;
  float* P = Nrm + ROWS * ld;
  float* Ws = P + ROWS * ld;
  const int row0 = blockIdx.x * ROWS;
  const int n_valid = min(ROWS, n_rows - row0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int idx = tid; idx < ROWS * (D / 4); idx += NTHREADS) {
    int r = idx / (D / 4), q = idx % (D / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f), w = v;
    if (r < n_valid) {
      v = *reinterpret_cast<const float4*>(x + (size_t)(row0 + r) * D + q * 4);
      w = *reinterpret_cast<const float4*>(o + (size_t)(row0 + r) * D + q * 4);
    }
    *reinterpret_cast<float4*>(X + r * ld + q * 4) = v;
    *reinterpret_cast<float4*>(P + r * ld + q * 4) = w;  // o is already rounded for EMU
  }
  float acc[4][4];
  zero_acc(acc);
  tile_linear<EMU>(P, ld, Wout, D, D, D, Ws, acc);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = lane + 32 * j;
      if (c < D) X[(4 * warp + i) * ld + c] += rnd<EMU>(acc[i][j]);
    }
  __syncthreads();
  tile_rmsnorm<EMU>(X, Nrm, ld, D, g2, n_valid);
  float down[4][4];
  tile_gated_mlp<EMU>(Nrm, P, ld, D, Wg, Wu, Wd, Ws, down);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = 4 * warp + i;
    if (r < n_valid)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        if (c < D) y[(size_t)(row0 + r) * D + c] = X[r * ld + c] + rnd<EMU>(down[i][j]);
      }
  }
}

// ------------------------------------------------------------------ temporal
// One temporal sublayer.  FIELD = false: CTA owns ROWS ships and walks t = 0..T-1 with the
// RG-LRU state and conv taps of its (row, column) elements in registers.  FIELD = true:
// rows are (t, field token) pairs, no state, conv+RG-LRU replaced by the field_sub Linear.
template <bool EMU, bool FIELD>
__global__ void __launch_bounds__(NTHREADS, 2)
k_temporal(const float* __restrict__ x, float* __restrict__ y,
           const float* __restrict__ hidden_in, float* __restrict__ hidden_out,
           const uint8_t* __restrict__ done, const uint8_t* __restrict__ reset_env,
           EnvMap map, int T, int D, BnbTemporalWeights w) {
  extern __shared__ __align__(16) float smem[];
  const int ld = max(D, NCHUNK) + 4;
  float* X = smem;                 // residual stream
  float* Nrm = X + ROWS * ld;      // normed input of the current Linear group
  float* P = Nrm + ROWS * ld;      // second operand tile (u, h*b2, gated product)
  float* B2 = P + ROWS * ld;       // gelu(linear2(n))
  float* Ws = B2 + ROWS * ld;
  __shared__ int s_xrow[ROWS];     // token row (within a timestep) of each tile row
  __shared__ int s_env[ROWS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = FIELD ? map.total_fields() * T : map.total_ships;
  const int item0 = blockIdx.x * ROWS;
  const int n_valid = min(ROWS, n_items - item0);
  if (tid < ROWS) {
    int xr = 0, e = 0;
    if (tid < n_valid) {
      int it = item0 + tid;
      if (FIELD) {
        int nf = map.total_fields();
        int t = it / nf, f = it - t * nf;
        xr = t * map.total_tokens + map.field_token_row(f);
      } else {
        xr = map.ship_token_row(it, &e);
      }
    }
    s_xrow[tid] = xr;
    s_env[tid] = e;
  }
  __syncthreads();

  // per-thread state for elements (row 4*warp+i, column lane+32j)
  float hst[4][4], c0[4][4], c1[4][4], c2[4][4];
  int lag_ok[4];  // valid stored lags of each owned row: 3 at t = 0
  if constexpr (!FIELD) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = 4 * warp + i;
      lag_ok[i] = BNB_CONV_KERNEL - 1;
      bool zero = (r >= n_valid) || (reset_env && reset_env[s_env[r]]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        float vh = 0.f, v0 = 0.f, v1 = 0.f, v2 = 0.f;
        if (!zero && c < D) {
          const float* hp = hidden_in + (size_t)(item0 + r) * 4 * D + c;
          vh = hp[0]; v0 = hp[D]; v1 = hp[2 * D]; v2 = hp[3 * D];
        }
        hst[i][j] = vh; c0[i][j] = v0; c1[i][j] = v1; c2[i][j] = v2;
      }
    }
  }

  const int steps = FIELD ? 1 : T;
  for (int t = 0; t < steps; ++t) {
    const size_t tbase = FIELD ? 0 : (size_t)t * map.total_tokens;
    __syncthreads();
    for (int idx = tid; idx < ROWS * (D / 4); idx += NTHREADS) {
      int r = idx / (D / 4), q = idx % (D / 4);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < n_valid) v = *reinterpret_cast<const float4*>(x + (tbase + s_xrow[r]) * D + q * 4);
      *reinterpret_cast<float4*>(X + r * ld + q * 4) = v;
    }
    __syncthreads();
    tile_rmsnorm<EMU>(X, Nrm, ld, D, w.norm1_w, n_valid);

    float b1[4][4], acc[4][4];
    zero_acc(b1);
    tile_linear<EMU>(Nrm, ld, w.linear1_w, D, D, D, Ws, b1);
    zero_acc(acc);
    tile_linear<EMU>(Nrm, ld, w.linear2_w, D, D, D, Ws, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        b1[i][j] = rnd<EMU>(b1[i][j]);
        if (c < D) B2[(4 * warp + i) * ld + c] = rnd<EMU>(gelu_erf(rnd<EMU>(acc[i][j])));
      }

    float br[4][4];  // recurrent-branch output per owned element
    if constexpr (FIELD) {
      // b1 <- field_sub(linear1(n))
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int c = lane + 32 * j;
          if (c < D) P[(4 * warp + i) * ld + c] = b1[i][j];
        }
      zero_acc(acc);
      tile_linear<EMU>(P, ld, w.field_sub_w, D, D, D, Ws, acc);
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int c = lane + 32 * j;
          // bf16 * bf16 -> bf16 under autocast (griffin.py:316)
          br[i][j] = (c < D) ? rnd<EMU>(rnd<EMU>(acc[i][j]) * B2[(4 * warp + i) * ld + c]) : 0.f;
        }
    } else {
      // causal depthwise conv over (tap0, tap1, tap2, b1) with episode-boundary lag masks
      float u[4][4];
      bool reset_a[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int r = 4 * warp + i;
        bool boundary = false;
        if (done && t >= 1 && r < n_valid) boundary = done[(size_t)(t - 1) * map.n_envs + s_env[r]] != 0;
        if (t >= 1) lag_ok[i] = boundary ? 0 : min(lag_ok[i] + 1, BNB_CONV_KERNEL - 1);
        reset_a[i] = boundary;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int c = lane + 32 * j;
          float uu = 0.f;
          if (c < D) {
            const float* cw = w.conv_w + c * BNB_CONV_KERNEL;
            float t0 = lag_ok[i] >= 3 ? __fmul_rn(c0[i][j], cw[0]) : 0.f;
            float t1 = lag_ok[i] >= 2 ? __fmul_rn(c1[i][j], cw[1]) : 0.f;
            float t2 = lag_ok[i] >= 1 ? __fmul_rn(c2[i][j], cw[2]) : 0.f;
            float t3 = __fmul_rn(b1[i][j], cw[3]);
            uu = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(t0, t1), t2), t3), w.conv_b[c]);
            P[(4 * warp + i) * ld + c] = rnd<EMU>(uu);
          }
          u[i][j] = uu;
          c0[i][j] = c1[i][j]; c1[i][j] = c2[i][j]; c2[i][j] = b1[i][j];
        }
      float ga[4][4], gx[4][4];
      zero_acc(ga);
      tile_linear<EMU>(P, ld, w.a_w, D, D, D, Ws, ga);
      zero_acc(gx);
      tile_linear<EMU>(P, ld, w.x_w, D, D, D, Ws, gx);
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int c = lane + 32 * j;
          float out = 0.f;
          if (c < D) {
            float rg = rnd<EMU>(sigmoidf_(rnd<EMU>(ga[i][j] + rnd<EMU>(w.a_b[c]))));
            float ig = rnd<EMU>(sigmoidf_(rnd<EMU>(gx[i][j] + rnd<EMU>(w.x_b[c]))));
            float a = powf(sigmoidf_(w.log_lambda[c]), kRglruC * rg);
            float gate = sqrtf(fmaxf((1.0f - a) * (1.0f + a), kGateFloor));
            float bb = gate * (ig * u[i][j]);
            if (reset_a[i]) a = 0.f;
            hst[i][j] = a * hst[i][j] + bb;
            out = hst[i][j] * B2[(4 * warp + i) * ld + c];  // fp32 * bf16 -> fp32
          }
          br[i][j] = out;
        }
    }
    // x1 = x + linear_out(branch)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        if (c < D) P[(4 * warp + i) * ld + c] = rnd<EMU>(br[i][j]);
      }
    zero_acc(acc);
    tile_linear<EMU>(P, ld, w.out_w, D, D, D, Ws, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        if (c < D) X[(4 * warp + i) * ld + c] += rnd<EMU>(acc[i][j]);
      }
    __syncthreads();
    tile_rmsnorm<EMU>(X, Nrm, ld, D, w.norm2_w, n_valid);
    float down[4][4];
    tile_gated_mlp<EMU>(Nrm, P, ld, D, w.gate_w, w.up_w, w.down_w, Ws, down);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = 4 * warp + i;
      if (r < n_valid)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int c = lane + 32 * j;
          if (c < D) y[(tbase + s_xrow[r]) * D + c] = X[r * ld + c] + rnd<EMU>(down[i][j]);
        }
    }
  }

  if constexpr (!FIELD) {
    if (hidden_out) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int r = 4 * warp + i;
        if (r < n_valid)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int c = lane + 32 * j;
            if (c < D) {
              float* hp = hidden_out + (size_t)(item0 + r) * 4 * D + c;
              hp[0] = hst[i][j]; hp[D] = c0[i][j]; hp[2 * D] = c1[i][j]; hp[3 * D] = c2[i][j];
            }
          }
      }
    }
  }
}

__global__ void k_reset_hidden(const float* __restrict__ in, float* __restrict__ out,
                               const uint8_t* __restrict__ done, EnvMap map, int n_slots, int D) {
  const size_t row_f4 = (size_t)D;  // 4D floats = D float4
  const size_t total = (size_t)n_slots * map.total_ships * row_f4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t row = i / row_f4;
    int s = (int)(row % map.total_ships);
    int e = map.env_of_ship(s);
    float4 v = reinterpret_cast<const float4*>(in)[i];
    if (done[e]) v = make_float4(0.f, 0.f, 0.f, 0.f);
    reinterpret_cast<float4*>(out)[i] = v;
  }
}

// ------------------------------------------------------------------ GatedMLP and RG-LRU on their own
//
// The two sub-modules the reference's own tests call directly (models/yemong/attention.py:21-37,
// griffin.py:169-219).  Inside a trunk call they run fused in the kernels above; these two kernels
// serve the module methods GatedMLP.forward, RGLRU._step and RGLRU.forward_sequence.

// y = down(gelu(gate x) * up x); a Linear casts its input to bf16 under autocast, and so does EMU.
template <bool EMU>
__global__ void __launch_bounds__(NTHREADS)
k_gated_mlp(const float* __restrict__ x, float* __restrict__ y, int n_rows, int D,
            const float* __restrict__ Wg, const float* __restrict__ Wu, const float* __restrict__ Wd) {
  extern __shared__ __align__(16) float smem[];
  const int ld = max(D, NCHUNK) + 4;
  float* X = smem;
  float* P = X + ROWS * ld;
  float* Ws = P + ROWS * ld;
  const int row0 = blockIdx.x * ROWS;
  const int n_valid = min(ROWS, n_rows - row0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int idx = tid; idx < ROWS * (D / 4); idx += NTHREADS) {
    int r = idx / (D / 4), q = idx % (D / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < n_valid) v = *reinterpret_cast<const float4*>(x + (size_t)(row0 + r) * D + q * 4);
    v.x = rnd<EMU>(v.x); v.y = rnd<EMU>(v.y); v.z = rnd<EMU>(v.z); v.w = rnd<EMU>(v.w);
    *reinterpret_cast<float4*>(X + r * ld + q * 4) = v;
  }
  __syncthreads();
  float down[4][4];
  tile_gated_mlp<EMU>(X, P, ld, D, Wg, Wu, Wd, Ws, down);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = 4 * warp + i;
    if (r < n_valid)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        if (c < D) y[(size_t)(row0 + r) * D + c] = rnd<EMU>(down[i][j]);
      }
  }
}

// The RG-LRU over T steps of n_rows independent rows, time-major x (T, n_rows, D):
// r = sigmoid(W_a x + b_a), i = sigmoid(W_x x + b_x), a = sigmoid(Lambda)^(8 r),
// h = a h + sqrt(max((1 - a)(1 + a), 1e-6)) (i x); a_t := 0 where done[t - 1] (griffin.py:213-218).
// The output of a step is its state.  Evaluated as the sequential loop the reference pins its
// parallel scan against.
template <bool EMU>
__global__ void __launch_bounds__(NTHREADS)
k_rglru(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ h0, float* __restrict__ h_out,
        const uint8_t* __restrict__ done, int n_rows, int T, int D, const float* __restrict__ Wa,
        const float* __restrict__ ba, const float* __restrict__ Wx, const float* __restrict__ bx,
        const float* __restrict__ log_lambda) {
  extern __shared__ __align__(16) float smem[];
  const int ld = max(D, NCHUNK) + 4;
  float* X = smem;                 // x_t, float32 (the product i * x uses the unrounded input)
  float* P = X + ROWS * ld;        // x_t as the Linear layers see it
  float* Ws = P + ROWS * ld;
  const int row0 = blockIdx.x * ROWS;
  const int n_valid = min(ROWS, n_rows - row0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float hst[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int r = 4 * warp + i, c = lane + 32 * j;
      hst[i][j] = (r < n_valid && c < D) ? h0[(size_t)(row0 + r) * D + c] : 0.f;
    }
  for (int t = 0; t < T; ++t) {
    __syncthreads();
    for (int idx = tid; idx < ROWS * (D / 4); idx += NTHREADS) {
      int r = idx / (D / 4), q = idx % (D / 4);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < n_valid) v = *reinterpret_cast<const float4*>(x + ((size_t)t * n_rows + row0 + r) * D + q * 4);
      *reinterpret_cast<float4*>(X + r * ld + q * 4) = v;
      v.x = rnd<EMU>(v.x); v.y = rnd<EMU>(v.y); v.z = rnd<EMU>(v.z); v.w = rnd<EMU>(v.w);
      *reinterpret_cast<float4*>(P + r * ld + q * 4) = v;
    }
    __syncthreads();
    float ga[4][4], gx[4][4];
    zero_acc(ga);
    tile_linear<EMU>(P, ld, Wa, D, D, D, Ws, ga);
    zero_acc(gx);
    tile_linear<EMU>(P, ld, Wx, D, D, D, Ws, gx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = 4 * warp + i;
      bool reset = done && t >= 1 && r < n_valid && done[(size_t)(t - 1) * n_rows + row0 + r] != 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int c = lane + 32 * j;
        if (r < n_valid && c < D) {
          float rg = rnd<EMU>(sigmoidf_(rnd<EMU>(ga[i][j] + rnd<EMU>(ba[c]))));
          float ig = rnd<EMU>(sigmoidf_(rnd<EMU>(gx[i][j] + rnd<EMU>(bx[c]))));
          float a = powf(sigmoidf_(log_lambda[c]), kRglruC * rg);
          float gate = sqrtf(fmaxf((1.0f - a) * (1.0f + a), kGateFloor));
          float bb = gate * (ig * X[r * ld + c]);
          if (reset) a = 0.f;
          hst[i][j] = a * hst[i][j] + bb;
          y[((size_t)t * n_rows + row0 + r) * D + c] = hst[i][j];
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int r = 4 * warp + i, c = lane + 32 * j;
      if (r < n_valid && c < D) h_out[(size_t)(row0 + r) * D + c] = hst[i][j];
    }
}

// ------------------------------------------------------------------ encoder MLP
//
// Linear(in, hidden) + b -> RMSNorm(hidden) -> GELU -> Linear(hidden, out) + b [-> RMSNorm(out)]: the chain
// of the reference's ShipEncoder (feature_extractor, or ship_proj / field_proj + shared_proj) and
// BulletEncoder (net), models/yemong/encoder.py:45-51, 84-102, and, without the last norm (g2
// null) and with only the first out_store output columns stored, of the policy's heads
// (models/yemong/policy.py:185-214).  in <= 128 (any width; w1 comes
// padded with zero columns to in_pad, a multiple of 32), hidden <= 256 and out <= 128 multiples of
// 32.  EMU: every stage hands on bfloat16 as under autocast (an RMSNorm of a bf16 input is
// computed in float32 and rounded once), and y holds bfloat16 elements.
template <bool EMU>
__global__ void __launch_bounds__(NTHREADS)
k_encoder_mlp(const float* __restrict__ x, void* __restrict__ y, int n_rows, int in_dim, int in_pad, int hidden, int out_dim,
              int out_store,
              const float* __restrict__ w1, const float* __restrict__ b1, const float* __restrict__ g1,
              const float* __restrict__ w2, const float* __restrict__ b2, const float* __restrict__ g2) {
  extern __shared__ __align__(16) float smem[];
  const int ldx = in_pad + 4, ldh = max(hidden, NCHUNK) + 4;
  float* X = smem;
  float* Hs = X + ROWS * ldx;
  float* Ws = Hs + ROWS * ldh;
  const int row0 = blockIdx.x * ROWS;
  const int n_valid = min(ROWS, n_rows - row0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int idx = tid; idx < ROWS * in_pad; idx += NTHREADS) {
    const int r = idx / in_pad, c = idx - r * in_pad;
    float v = 0.f;
    if (r < n_valid && c < in_dim) v = x[(size_t)(row0 + r) * in_dim + c];
    X[r * ldx + c] = rnd<EMU>(v);
  }
  __syncthreads();
  for (int c0 = 0; c0 < hidden; c0 += NCHUNK) {
    const int cn = min(NCHUNK, hidden - c0);
    float acc[4][4];
    zero_acc(acc);
    tile_linear<EMU>(X, ldx, w1 + (size_t)c0 * in_pad, in_pad, cn, in_pad, Ws, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = lane + 32 * j;
        if (c < cn) Hs[(4 * warp + i) * ldh + c0 + c] = rnd<EMU>(acc[i][j] + rnd<EMU>(b1[c0 + c]));
      }
  }
  __syncthreads();
  tile_rmsnorm<EMU>(Hs, Hs, ldh, hidden, g1, ROWS);
  for (int i = 0; i < 4; ++i)
    for (int c = lane; c < hidden; c += 32) {
      float* p = Hs + (4 * warp + i) * ldh + c;
      *p = rnd<EMU>(gelu_erf(*p));
    }
  __syncthreads();
  float acc[4][4];
  zero_acc(acc);
  tile_linear<EMU>(Hs, ldh, w2, hidden, out_dim, hidden, Ws, acc);
  __syncthreads();  // every warp has read its rows of Hs
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane + 32 * j;
      if (c < out_dim) Hs[(4 * warp + i) * ldh + c] = rnd<EMU>(acc[i][j] + rnd<EMU>(b2[c]));
    }
  __syncthreads();
  if (g2) tile_rmsnorm<EMU>(Hs, Hs, ldh, out_dim, g2, ROWS);   // the encoders end in a norm, the heads do not
  __syncwarp();
  for (int i = 0; i < 4; ++i) {
    const int r = 4 * warp + i;
    if (r >= n_valid) continue;
    for (int c = lane; c < out_store; c += 32) {
      const float v = Hs[r * ldh + c];
      if constexpr (EMU) static_cast<__nv_bfloat16*>(y)[(size_t)(row0 + r) * out_store + c] = __float2bfloat16_rn(v);
      else static_cast<float*>(y)[(size_t)(row0 + r) * out_store + c] = v;
    }
  }
}

// ------------------------------------------------------------------ TeamPMA (policy.py:78-121)
// q[t] = W_q seeds[t] for the two team seeds (one block).
template <bool EMU>
__global__ void k_team_query(const float* __restrict__ seeds, const float* __restrict__ Wq, float* __restrict__ q, int D) {
  // one warp per output: the lanes read a row of Wq contiguously and add their partial sums up
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int o = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; o < 2 * D; o += warps) {
    const int t = o / D, c = o - t * D;
    float acc = 0.f;
    for (int k = lane; k < D; k += 32) acc = fmaf(rnd<EMU>(seeds[t * D + k]), rnd<EMU>(Wq[(size_t)c * D + k]), acc);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) q[o] = rnd<EMU>(acc);
  }
}

// Pooling by attention over the alive ships of each team, 16 environments (32 team rows) per CTA:
// per (environment, team) a softmax per head over that team's alive ships with the team's seed as
// the query, the pooled values through out_proj (a 32-row tile product), zero where the team has no
// ship alive, RMSNorm, and every ship gets its team's row (team_id clamped to 0..1).
template <bool EMU>
__global__ void __launch_bounds__(NTHREADS)
k_team_pool(const float* __restrict__ kv, const float* __restrict__ q, const int32_t* __restrict__ team_id,
            const uint8_t* __restrict__ alive, void* __restrict__ y, int y_bf16, int n_envs, int N, int D, int H,
            const float* __restrict__ Wo, const float* __restrict__ gn) {
  extern __shared__ __align__(16) float smem[];
  const int ld = max(D, NCHUNK) + 4;
  float* P = smem;                   // pooled rows, then the normed team rows
  float* Ws = P + ROWS * ld;
  float* sc = Ws + NCHUNK * WS_STRIDE;   // per warp: N x H softmax weights
  __shared__ float s_has[ROWS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int env0 = blockIdx.x * (ROWS / 2);
  const int dh = D / H;
  const float scale = rsqrtf((float)dh);
  float* my = sc + (size_t)warp * N * H;
  for (int i = 0; i < 4; ++i) {
    const int r = 4 * warp + i;
    const int e = env0 + (r >> 1), t = r & 1;
    bool any = false;
    if (e < n_envs) {
      const size_t base = (size_t)e * N;
      // scores of this team's alive ships, per head
      if ((D & 31) == 0 && D <= 128 && (32 % H) == 0) {
        // the warp reads one ship's key row at a time (contiguous): a lane owns D / 32 consecutive
        // channels, the 32 / H lanes of a head add their partial dot products up
        const int dpl = D >> 5, lph = 32 / H;
        float qv[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < dpl; ++j) qv[j] = q[t * D + lane * dpl + j];
        for (int n = 0; n < N; ++n) {
          const bool ok = team_id[base + n] == t && alive[base + n];   // the same in every lane
          float part = 0.f;
          if (ok) {
            const float* kp = kv + (base + n) * 2 * D + lane * dpl;
            for (int j = 0; j < dpl; ++j) part = fmaf(qv[j], rnd<EMU>(kp[j]), part);
          }
          for (int o = lph >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
          if ((lane & (lph - 1)) == 0) my[n * H + lane / lph] = ok ? part * scale : -INFINITY;
          any |= ok;
        }
      } else {
        for (int n = lane; n < N; n += 32) {
          const bool ok = team_id[base + n] == t && alive[base + n];
          const float* kp = kv + (base + n) * 2 * D;
          for (int h = 0; h < H; ++h) {
            float acc = -INFINITY;
            if (ok) {
              acc = 0.f;
              for (int d = 0; d < dh; ++d) acc = fmaf(q[t * D + h * dh + d], rnd<EMU>(kp[h * dh + d]), acc);
              acc *= scale;
            }
            my[n * H + h] = acc;
          }
          any |= ok;
        }
      }
      any = __any_sync(0xffffffffu, any);
      __syncwarp();
      if (any) {
        for (int h = 0; h < H; ++h) {
          float m = -INFINITY;
          for (int n = lane; n < N; n += 32) m = fmaxf(m, my[n * H + h]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          float l = 0.f;
          for (int n = lane; n < N; n += 32) {
            const float ex = expf(my[n * H + h] - m);   // exp(-inf) = 0 for the masked ships
            my[n * H + h] = ex;
            l += ex;
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
          const float inv = 1.0f / l;
          for (int n = lane; n < N; n += 32) my[n * H + h] *= inv;
        }
        __syncwarp();
      }
    }
    for (int c = lane; c < D; c += 32) {
      float acc = 0.f;
      if (e < n_envs && any) {
        const int h = c / dh;
        for (int n = 0; n < N; ++n) acc = fmaf(my[n * H + h], rnd<EMU>(kv[((size_t)e * N + n) * 2 * D + D + c]), acc);
      }
      P[r * ld + c] = rnd<EMU>(acc);
    }
    if (lane == 0) s_has[r] = (e < n_envs && any) ? 1.f : 0.f;
    __syncwarp();
  }
  __syncthreads();
  float acc[4][4];
  zero_acc(acc);
  tile_linear<EMU>(P, ld, Wo, D, D, D, Ws, acc);
  __syncthreads();   // every warp has read its rows of P
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane + 32 * j;
      if (c < D) P[(4 * warp + i) * ld + c] = rnd<EMU>(acc[i][j]) * s_has[4 * warp + i];
    }
  __syncthreads();
  tile_rmsnorm<EMU>(P, P, ld, D, gn, ROWS);
  __syncthreads();
  const int envs_here = min(ROWS / 2, n_envs - env0);
  for (int idx = tid; idx < envs_here * N * (D / 4); idx += NTHREADS) {
    const int c4 = idx % (D / 4), sn = idx / (D / 4);
    const int el = sn / N;
    const size_t row = (size_t)(env0 + el) * N + (sn - el * N);
    const int t = min(max(team_id[row], 0), 1);
    const float4 v = *reinterpret_cast<const float4*>(P + (2 * el + t) * ld + c4 * 4);
    if (y_bf16) {
      __nv_bfloat162* yp = reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(y) + row * D + c4 * 4);
      yp[0] = __floats2bfloat162_rn(v.x, v.y);
      yp[1] = __floats2bfloat162_rn(v.z, v.w);
    } else {
      *reinterpret_cast<float4*>(static_cast<float*>(y) + row * D + c4 * 4) = v;
    }
  }
}

// ------------------------------------------------------------------ action sampling (policy.py:551-575)
// One thread per ship: three independent categorical draws over the logit slices [0, 3), [3, 10),
// [10, 12) (constants.py:43-48) by inverse CDF from the caller's uniforms, and the sum of the three
// log-probabilities.  EMU: the logits are bfloat16 values and the normalised log-probabilities round
// to bfloat16 like torch.distributions.Categorical's do under autocast.
template <bool EMU>
__global__ void k_sample_action(const float* __restrict__ logits, const float* __restrict__ uniforms,
                                const int64_t* __restrict__ given, int64_t* __restrict__ action, float* __restrict__ logprob,
                                float* __restrict__ entropy, int n_rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  const int lo[3] = {0, 3, 10}, hi[3] = {3, 10, 12};
  float lp_sum = 0.f, ent_sum = 0.f;
  for (int s = 0; s < 3; ++s) {
    float v[7], m = -INFINITY;
    const int n = hi[s] - lo[s];
    for (int k = 0; k < n; ++k) {
      v[k] = rnd<EMU>(logits[(size_t)r * 12 + lo[s] + k]);
      m = fmaxf(m, v[k]);
    }
    float l = 0.f;
    for (int k = 0; k < n; ++k) l += expf(v[k] - m);
    const float lse = rnd<EMU>(m + logf(l));
    int pick;
    if (given) {
      pick = (int)given[(size_t)r * 3 + s];
      pick = min(max(pick, 0), n - 1);
    } else {
      // inverse CDF: the first k with u * l < sum_{j <= k} exp(v_j - m)
      const float target = uniforms[(size_t)r * 3 + s] * l;
      float c = 0.f;
      pick = n - 1;
      for (int k = 0; k < n; ++k) {
        c += expf(v[k] - m);
        if (target < c) { pick = k; break; }
      }
      action[(size_t)r * 3 + s] = pick;
    }
    lp_sum = rnd<EMU>(lp_sum + rnd<EMU>(v[pick] - lse));
    if (entropy) {
      float e = 0.f;
      for (int k = 0; k < n; ++k) {
        const float lg = rnd<EMU>(v[k] - lse);
        e += rnd<EMU>(lg * rnd<EMU>(expf(lg)));
      }
      ent_sum = rnd<EMU>(ent_sum + rnd<EMU>(-rnd<EMU>(e)));
    }
  }
  logprob[r] = lp_sum;
  if (entropy) entropy[r] = ent_sum;
}

// ------------------------------------------------------------------ host launchers

static size_t smem_rows(int D, int tiles) {
  int ld = (D > NCHUNK ? D : NCHUNK) + 4;
  return (size_t)(tiles * ROWS * ld + NCHUNK * WS_STRIDE) * sizeof(float);
}

template <class K>
static bool opt_in(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess;
}

template <bool EMU>
static int launch_attention(const float* qkv, const uint8_t* alive, float* o, const EnvMap& map, int env_base,
                            int n_env, int max_tokens, int D, int H, const float* kvb, const uint8_t* active,
                            int nb, cudaStream_t st) {
  int per_env = max_tokens * H;
  int gy = (per_env + 127) / 128;
  dim3 grid(n_env, gy > 4 ? 4 : (gy < 1 ? 1 : gy));
  count_launch();
  switch (D / H) {
    case 8:  k_attention<EMU, 8><<<grid, 128, 0, st>>>(qkv, alive, o, map, env_base, D, H, kvb, active, nb); break;
    case 16: k_attention<EMU, 16><<<grid, 128, 0, st>>>(qkv, alive, o, map, env_base, D, H, kvb, active, nb); break;
    case 32: k_attention<EMU, 32><<<grid, 128, 0, st>>>(qkv, alive, o, map, env_base, D, H, kvb, active, nb); break;
    case 64: k_attention<EMU, 64><<<grid, 128, 0, st>>>(qkv, alive, o, map, env_base, D, H, kvb, active, nb); break;
    default: return BNB_ERR_UNSUPPORTED_DIMS;
  }
  return BNB_OK;
}

template <bool EMU>
static int spatial_impl(const BnbSpatialWeights& w, int D, int H, const float* x, const uint8_t* alive,
                        const BnbBullets* bul, float* y, const BnbBatch& b, int n_groups, float* qkv, float* o,
                        float* kvb, int kvb_envs, cudaStream_t st) {
  const int n_rows = n_groups * b.total_tokens;
  const int n_tiles = (n_rows + ROWS - 1) / ROWS;
  const size_t sm_qkv = (size_t)(2 * ROWS * (D + 4) + NCHUNK * WS_STRIDE) * sizeof(float);
  if (!opt_in(k_spatial_qkv<EMU>, sm_qkv)) return BNB_ERR_LAUNCH;
  count_launch();
  k_spatial_qkv<EMU><<<n_tiles, NTHREADS, sm_qkv, st>>>(x, qkv, n_rows, D, 3 * D, w.norm1_w, w.qkv_w);
  EnvMap map = make_env_map(b);
  const int total_envs = n_groups * b.n_envs;
  if (bul && w.kv_bullet_w) {
    // keys and values of the bullets, one slice of environments at a time
    const int nb = bul->per_env;
    for (int e0 = 0; e0 < total_envs; e0 += kvb_envs) {
      int ne = total_envs - e0 < kvb_envs ? total_envs - e0 : kvb_envs;
      int rows = ne * nb;
      count_launch();
      k_spatial_qkv<EMU><<<(rows + ROWS - 1) / ROWS, NTHREADS, sm_qkv, st>>>(
          bul->tokens + (size_t)e0 * nb * D, kvb, rows, D, 2 * D, w.norm_bullet_w, w.kv_bullet_w);
      int rc = launch_attention<EMU>(qkv, alive, o, map, e0, ne, b.max_tokens_per_env, D, H, kvb, bul->active, nb, st);
      if (rc) return rc;
    }
  } else if (total_envs > 0) {
    int rc = launch_attention<EMU>(qkv, alive, o, map, 0, total_envs, b.max_tokens_per_env, D, H, nullptr, nullptr, 0, st);
    if (rc) return rc;
  }
  {
    size_t sm = smem_rows(D, 3);
    if (!opt_in(k_spatial_post<EMU>, sm)) return BNB_ERR_LAUNCH;
    count_launch();
    k_spatial_post<EMU><<<n_tiles, NTHREADS, sm, st>>>(x, o, y, n_rows, D, w.out_w, w.norm2_w,
                                                       w.gate_w, w.up_w, w.down_w);
  }
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

int spatial_block(const BnbSpatialWeights& w, int D, int H, const float* x, const uint8_t* alive,
                  const BnbBullets* bullets, float* y, const BnbBatch& b, int n_groups, bool emulate_bf16,
                  float* qkv_scratch, float* o_scratch, float* kvb_scratch, int kvb_envs, cudaStream_t st) {
  return emulate_bf16 ? spatial_impl<true>(w, D, H, x, alive, bullets, y, b, n_groups, qkv_scratch, o_scratch,
                                           kvb_scratch, kvb_envs, st)
                      : spatial_impl<false>(w, D, H, x, alive, bullets, y, b, n_groups, qkv_scratch, o_scratch,
                                            kvb_scratch, kvb_envs, st);
}

template <bool EMU>
static int temporal_impl(const BnbTemporalWeights& w, int D, const float* x, float* y,
                         const float* hin, float* hout, const uint8_t* done, const uint8_t* reset_env,
                         const BnbBatch& b, int T, cudaStream_t st) {
  EnvMap map = make_env_map(b);
  size_t sm = smem_rows(D, 4);
  if (b.total_ships > 0) {
    if (!opt_in(k_temporal<EMU, false>, sm)) return BNB_ERR_LAUNCH;
    int n_tiles = (b.total_ships + ROWS - 1) / ROWS;
    count_launch();
    k_temporal<EMU, false><<<n_tiles, NTHREADS, sm, st>>>(x, y, hin, hout, done, reset_env, map, T, D, w);
  }
  int n_fields = (b.total_tokens - b.total_ships) * T;
  if (n_fields > 0) {
    if (!w.field_sub_w) return BNB_ERR_NULL_POINTER;
    if (!opt_in(k_temporal<EMU, true>, sm)) return BNB_ERR_LAUNCH;
    int n_tiles = (n_fields + ROWS - 1) / ROWS;
    count_launch();
    k_temporal<EMU, true><<<n_tiles, NTHREADS, sm, st>>>(x, y, nullptr, nullptr, nullptr, nullptr, map, T, D, w);
  }
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

int temporal_block(const BnbTemporalWeights& w, int D, const float* x, float* y, const float* hidden_in,
                   float* hidden_out, const uint8_t* done, const uint8_t* reset_env, const BnbBatch& b,
                   int T, bool emulate_bf16, cudaStream_t st) {
  return emulate_bf16 ? temporal_impl<true>(w, D, x, y, hidden_in, hidden_out, done, reset_env, b, T, st)
                      : temporal_impl<false>(w, D, x, y, hidden_in, hidden_out, done, reset_env, b, T, st);
}

template <bool EMU>
static int gated_mlp_impl(const float* gate_w, const float* up_w, const float* down_w, int D, const float* x, float* y,
                          int n_rows, cudaStream_t st) {
  size_t sm = smem_rows(D, 2);
  if (!opt_in(k_gated_mlp<EMU>, sm)) return BNB_ERR_LAUNCH;
  count_launch();
  k_gated_mlp<EMU><<<(n_rows + ROWS - 1) / ROWS, NTHREADS, sm, st>>>(x, y, n_rows, D, gate_w, up_w, down_w);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}
int gated_mlp(const float* gate_w, const float* up_w, const float* down_w, int D, const float* x, float* y,
              int n_rows, bool emulate_bf16, cudaStream_t st) {
  return emulate_bf16 ? gated_mlp_impl<true>(gate_w, up_w, down_w, D, x, y, n_rows, st)
                      : gated_mlp_impl<false>(gate_w, up_w, down_w, D, x, y, n_rows, st);
}

template <bool EMU>
static int rglru_impl(const float* a_w, const float* a_b, const float* x_w, const float* x_b, const float* log_lambda,
                      int D, const float* x, float* y, const float* h0, float* h_out, const uint8_t* done, int n_rows,
                      int T, cudaStream_t st) {
  size_t sm = smem_rows(D, 2);
  if (!opt_in(k_rglru<EMU>, sm)) return BNB_ERR_LAUNCH;
  count_launch();
  k_rglru<EMU><<<(n_rows + ROWS - 1) / ROWS, NTHREADS, sm, st>>>(x, y, h0, h_out, done, n_rows, T, D, a_w, a_b, x_w, x_b,
                                                                 log_lambda);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}
int rglru(const float* a_w, const float* a_b, const float* x_w, const float* x_b, const float* log_lambda, int D,
          const float* x, float* y, const float* h0, float* h_out, const uint8_t* done, int n_rows, int T,
          bool emulate_bf16, cudaStream_t st) {
  return emulate_bf16 ? rglru_impl<true>(a_w, a_b, x_w, x_b, log_lambda, D, x, y, h0, h_out, done, n_rows, T, st)
                      : rglru_impl<false>(a_w, a_b, x_w, x_b, log_lambda, D, x, y, h0, h_out, done, n_rows, T, st);
}

template <bool EMU>
static int encoder_mlp_impl(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2,
                            const float* g2, int in_dim, int in_pad, int hidden, int out_dim, int out_store, const float* x,
                            void* y, int n_rows, cudaStream_t st) {
  const int ldh = (hidden > NCHUNK ? hidden : NCHUNK) + 4;
  const size_t sm = (size_t)(ROWS * (in_pad + 4) + ROWS * ldh + NCHUNK * WS_STRIDE) * sizeof(float);
  if (!opt_in(k_encoder_mlp<EMU>, sm)) return BNB_ERR_LAUNCH;
  count_launch();
  k_encoder_mlp<EMU><<<(n_rows + ROWS - 1) / ROWS, NTHREADS, sm, st>>>(x, y, n_rows, in_dim, in_pad, hidden, out_dim, out_store,
                                                                       w1, b1, g1, w2, b2, g2);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}
int encoder_mlp(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2, const float* g2,
                int in_dim, int in_pad, int hidden, int out_dim, int out_store, const float* x, void* y, int n_rows,
                bool emulate_bf16, cudaStream_t st) {
  return emulate_bf16
             ? encoder_mlp_impl<true>(w1, b1, g1, w2, b2, g2, in_dim, in_pad, hidden, out_dim, out_store, x, y, n_rows, st)
             : encoder_mlp_impl<false>(w1, b1, g1, w2, b2, g2, in_dim, in_pad, hidden, out_dim, out_store, x, y, n_rows, st);
}

template <bool EMU>
static int team_pma_impl(const float* seeds, const float* in_proj_w, const float* out_w, const float* norm_w, int D, int H,
                         const float* x, const int32_t* team_id, const uint8_t* alive, void* y, bool y_bf16, int n_envs, int N,
                         float* kv, float* q, cudaStream_t st) {
  const int n_rows = n_envs * N;
  if (EMU) {
    // keys and values under the bfloat16 contract: operands rounded to bfloat16 inside the tiled
    // product, float32 accumulation; k_team_pool rounds the results as it reads them
    grad::linear_nt(x, in_proj_w + (size_t)D * D, kv, n_rows, 2 * D, D, true, st);
  } else {
    const size_t sm_qkv = (size_t)(2 * ROWS * (D + 4) + NCHUNK * WS_STRIDE) * sizeof(float);
    if (!opt_in(k_spatial_qkv<EMU>, sm_qkv)) return BNB_ERR_LAUNCH;
    count_launch();
    k_spatial_qkv<EMU><<<(n_rows + ROWS - 1) / ROWS, NTHREADS, sm_qkv, st>>>(x, kv, n_rows, D, 2 * D, nullptr,
                                                                            in_proj_w + (size_t)D * D);
  }
  count_launch();
  k_team_query<EMU><<<(2 * D + 7) / 8, 256, 0, st>>>(seeds, in_proj_w, q, D);
  const int ld = (D > NCHUNK ? D : NCHUNK) + 4;
  const size_t sm = (size_t)(ROWS * ld + NCHUNK * WS_STRIDE + (NTHREADS / 32) * N * H) * sizeof(float);
  if (sm > 200 * 1024) return BNB_ERR_TOO_MANY_TOKENS;
  if (!opt_in(k_team_pool<EMU>, sm)) return BNB_ERR_LAUNCH;
  count_launch();
  k_team_pool<EMU><<<(n_envs + ROWS / 2 - 1) / (ROWS / 2), NTHREADS, sm, st>>>(kv, q, team_id, alive, y, y_bf16 ? 1 : 0, n_envs, N,
                                                                             D, H, out_w, norm_w);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}
int team_pma(const float* seeds, const float* in_proj_w, const float* out_w, const float* norm_w, int D, int H, const float* x,
             const int32_t* team_id, const uint8_t* alive, void* y, bool y_bf16, int n_envs, int N, float* kv, float* q,
             bool emulate_bf16, cudaStream_t st) {
  return emulate_bf16 ? team_pma_impl<true>(seeds, in_proj_w, out_w, norm_w, D, H, x, team_id, alive, y, y_bf16, n_envs, N, kv, q, st)
                      : team_pma_impl<false>(seeds, in_proj_w, out_w, norm_w, D, H, x, team_id, alive, y, y_bf16, n_envs, N, kv, q, st);
}

int sample_action(const float* logits, const float* uniforms, const int64_t* given, int64_t* action, float* logprob,
                  float* entropy, int n_rows, bool emulate_bf16, cudaStream_t st) {
  if (n_rows == 0) return BNB_OK;
  count_launch();
  if (emulate_bf16) k_sample_action<true><<<(n_rows + 127) / 128, 128, 0, st>>>(logits, uniforms, given, action, logprob, entropy, n_rows);
  else k_sample_action<false><<<(n_rows + 127) / 128, 128, 0, st>>>(logits, uniforms, given, action, logprob, entropy, n_rows);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

int reset_hidden(const float* in, float* out, const uint8_t* done, int n_slots, int D,
                 const BnbBatch& b, cudaStream_t st) {
  EnvMap map = make_env_map(b);
  size_t total = (size_t)n_slots * b.total_ships * D;
  if (total == 0) return BNB_OK;
  int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  count_launch();
  k_reset_hidden<<<blocks, 256, 0, st>>>(in, out, done, map, n_slots, D);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

}  // namespace exact
}  // namespace bnb
