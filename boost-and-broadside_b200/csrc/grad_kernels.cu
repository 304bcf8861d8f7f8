// Backward pass of the Yemong trunk's sequence forward, float32.
//
// What loss.backward() computes through the trunk loop of evaluate_actions
// (models/yemong/policy.py:422-478, reached from train/rl/ppo.py:1974): gradients with respect to
// the tokens, the initial recurrent state, the bullet tokens and every parameter of
//   TransformerBlock.forward        models/yemong/attention.py:76-169
//   GatedMLP.forward                models/yemong/attention.py:21-37
//   GriffinTemporalBlock.*          models/yemong/griffin.py:249-317
//   RGLRU gates / update            models/yemong/griffin.py:169-219
//   causal conv + tap validity      models/yemong/griffin.py:67-140
//
// Scheme: recompute, as the reference does with grad_checkpoint (policy.py:451-467).  A first pass
// runs the forward sublayer by sublayer and keeps only the input of every sublayer.  The sublayers are then walked in reverse; each recomputes its own intermediates
// into scratch (norms, projections, attention output, gates, recurrent states) and differentiates
// them.  Linear products -- y = x W^T, dx = dy W, dW += dy^T x -- all run on one tensor-core GEMM
// kernel (3 x tf32 m16n8k8 MMAs per product, float32 accumulation: float32-level accuracy; or, for
// a forward that ran under bf16 autocast, one bf16 m16n8k16 MMA with operands rounded on the way
// in, as autocast does to the reference's backward products); the
// weight gradients reduce over all rows with a split over the row dimension and float32 atomics,
// so the caller hands in zeroed (or to-be-accumulated-into) gradient buffers.
//
// Attention gradient: the probabilities are recomputed as exp(s - lse) with lse = max + log(sum)
// in float32 and the row term is <d out, out>, as the fused attention kernels behind
// F.scaled_dot_product_attention do.  For a row with a live key that is the softmax gradient; for
// an environment whose keys are all dead it is the reference's value too (lse rounds to the bias).
#include "grad_kernels.h"

#include "common.cuh"
#include "launch_count.h"

namespace bnb {
namespace grad {

namespace {

// ------------------------------------------------------------------------------ GEMM

constexpr int BM = 128, BN = 128, BK = 32, GT = 256;
// Row strides of the shared tiles, chosen so that the fragment reads of a warp hit 32 different
// banks: [row][k] tiles 36 floats (tf32: 32-bit reads) or 40 (bf16: 64-bit reads of two adjacent
// k), [k][row] tiles 136 or 132.
template <bool BF16> struct Strides { static constexpr int LDK = BF16 ? BK + 8 : BK + 4, LDR = BF16 ? 128 + 4 : 128 + 8; };
constexpr int TILE_FLOATS = BM * (BK + 8);

struct GemmArgs {
  const float* A; int lda;
  const float* B; int ldb;
  float* C; int ldc;
  int M, N, K;
  const float* bias;        // (N) or null
  const float* R; int ldr;  // residual (M, N) or null; may alias C
  int beta;                 // 1: C += product
  int k_per_split;          // K range of one blockIdx.z
  int atomic;               // 1: atomicAdd into C (split over K)
};

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
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two floats -> one register of two bf16, the first in the low half
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// C(m, n) = sum_k A(m, k) B(n, k) [+ bias(n)] [+ R(m, n)] [+ C(m, n)].
// A_KC: A(m, k) = A[m * lda + k], else A[k * lda + m].  B_KC: B(n, k) = B[n * ldb + k], else B[k * ldb + n].
// The contiguous dimension of each operand is a multiple of 4 floats and its base 16-byte aligned.
// 128 x 128 tile per CTA, 8 warps of 64 x 32.  BF16 unset: every float32 operand is split into two
// tf32 numbers and three m16n8k8 MMAs give the float32 product.  BF16 set: operands are rounded to
// bfloat16 on the way into the m16n8k16 MMA (what autocast does to the reference's backward
// products), accumulation in float32 either way.
// 16-byte asynchronous copy into shared memory; bytes = 0 fills the destination with zeros.
__device__ __forceinline__ void cp_async16(float* dst, const float* src, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int GEMM_STAGES = 2;
constexpr size_t GEMM_SMEM = (size_t)GEMM_STAGES * 2 * TILE_FLOATS * sizeof(float);   // 80 KB: two CTAs per SM

template <bool A_KC, bool B_KC, bool BF16>
__global__ void __launch_bounds__(GT, BF16 ? 2 : 1) k_gemm(GemmArgs g) {
  constexpr int LDK = Strides<BF16>::LDK, LDR = Strides<BF16>::LDR;
  extern __shared__ __align__(16) float gemm_smem[];
  static_assert(TILE_FLOATS >= BM * LDK && TILE_FLOATS >= BK * LDR, "either orientation fits the tile buffer");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
  const int wm = (warp & 1) * 64, wn = (warp >> 1) * 32;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kbeg = blockIdx.z * g.k_per_split;
  const int kend = min(g.K, kbeg + g.k_per_split);
  float c[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[i][j][e] = 0.f;

  // one K slice of both operands into a stage; out-of-range pieces are zero-filled
  auto load_stage = [&](int stage, int k0) {
    float* As = gemm_smem + (size_t)stage * 2 * TILE_FLOATS;
    float* Bs = As + TILE_FLOATS;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * GT;
      if constexpr (A_KC) {
        const int row = idx >> 3, c4 = (idx & 7) * 4;
        const int gm = m0 + row, gk = k0 + c4;
        const bool ok = gm < g.M && gk < kend;
        cp_async16(As + row * LDK + c4, ok ? g.A + (size_t)gm * g.lda + gk : g.A, ok ? 16 : 0);
      } else {
        const int kk = idx >> 5, c4 = (idx & 31) * 4;
        const int gk = k0 + kk, gm = m0 + c4;
        const bool ok = gk < kend && gm < g.M;
        cp_async16(As + kk * LDR + c4, ok ? g.A + (size_t)gk * g.lda + gm : g.A, ok ? 16 : 0);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * GT;
      if constexpr (B_KC) {
        const int row = idx >> 3, c4 = (idx & 7) * 4;
        const int gn = n0 + row, gk = k0 + c4;
        const bool ok = gn < g.N && gk < kend;
        cp_async16(Bs + row * LDK + c4, ok ? g.B + (size_t)gn * g.ldb + gk : g.B, ok ? 16 : 0);
      } else {
        const int kk = idx >> 5, c4 = (idx & 31) * 4;
        const int gk = k0 + kk, gn = n0 + c4;
        const bool ok = gk < kend && gn < g.N;
        cp_async16(Bs + kk * LDR + c4, ok ? g.B + (size_t)gk * g.ldb + gn : g.B, ok ? 16 : 0);
      }
    }
    cp_async_commit();
  };

  const int n_it = (kend - kbeg + BK - 1) / BK;
  if (n_it > 0) load_stage(0, kbeg);
  for (int it = 0; it < n_it; ++it) {
    if (it + 1 < n_it) {
      load_stage((it + 1) & 1, kbeg + (it + 1) * BK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* As = gemm_smem + (size_t)(it & 1) * 2 * TILE_FLOATS;
    const float* Bs = As + TILE_FLOATS;
    if constexpr (BF16) {
#pragma unroll
      for (int kk = 0; kk < BK; kk += 16) {
        uint32_t a[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          const int r0 = wm + mt * 16 + gq, kq = kk + 2 * t;
          if constexpr (A_KC) {
            const float2 v0 = *reinterpret_cast<const float2*>(As + r0 * LDK + kq);
            const float2 v1 = *reinterpret_cast<const float2*>(As + (r0 + 8) * LDK + kq);
            const float2 v2 = *reinterpret_cast<const float2*>(As + r0 * LDK + kq + 8);
            const float2 v3 = *reinterpret_cast<const float2*>(As + (r0 + 8) * LDK + kq + 8);
            a[mt][0] = pack_bf16(v0.x, v0.y);
            a[mt][1] = pack_bf16(v1.x, v1.y);
            a[mt][2] = pack_bf16(v2.x, v2.y);
            a[mt][3] = pack_bf16(v3.x, v3.y);
          } else {
            a[mt][0] = pack_bf16(As[kq * LDR + r0], As[(kq + 1) * LDR + r0]);
            a[mt][1] = pack_bf16(As[kq * LDR + r0 + 8], As[(kq + 1) * LDR + r0 + 8]);
            a[mt][2] = pack_bf16(As[(kq + 8) * LDR + r0], As[(kq + 9) * LDR + r0]);
            a[mt][3] = pack_bf16(As[(kq + 8) * LDR + r0 + 8], As[(kq + 9) * LDR + r0 + 8]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int nn = wn + nt * 8 + gq, kq = kk + 2 * t;
          uint32_t b0, b1;
          if constexpr (B_KC) {
            const float2 v0 = *reinterpret_cast<const float2*>(Bs + nn * LDK + kq);
            const float2 v1 = *reinterpret_cast<const float2*>(Bs + nn * LDK + kq + 8);
            b0 = pack_bf16(v0.x, v0.y);
            b1 = pack_bf16(v1.x, v1.y);
          } else {
            b0 = pack_bf16(Bs[kq * LDR + nn], Bs[(kq + 1) * LDR + nn]);
            b1 = pack_bf16(Bs[(kq + 8) * LDR + nn], Bs[(kq + 9) * LDR + nn]);
          }
#pragma unroll
          for (int mt = 0; mt < 4; ++mt) mma_bf16(c[mt][nt], a[mt], b0, b1);
        }
      }
    } else {
#pragma unroll
      for (int kk = 0; kk < BK; kk += 8) {
        uint32_t ah[4][4], al[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          const int r0 = wm + mt * 16 + gq;
          float af[4];
          if constexpr (A_KC) {
            af[0] = As[r0 * LDK + kk + t];
            af[1] = As[(r0 + 8) * LDK + kk + t];
            af[2] = As[r0 * LDK + kk + t + 4];
            af[3] = As[(r0 + 8) * LDK + kk + t + 4];
          } else {
            af[0] = As[(kk + t) * LDR + r0];
            af[1] = As[(kk + t) * LDR + r0 + 8];
            af[2] = As[(kk + t + 4) * LDR + r0];
            af[3] = As[(kk + t + 4) * LDR + r0 + 8];
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) split_tf32(af[e], ah[mt][e], al[mt][e]);
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int nn = wn + nt * 8 + gq;
          float b0, b1;
          if constexpr (B_KC) {
            b0 = Bs[nn * LDK + kk + t];
            b1 = Bs[nn * LDK + kk + t + 4];
          } else {
            b0 = Bs[(kk + t) * LDR + nn];
            b1 = Bs[(kk + t + 4) * LDR + nn];
          }
          uint32_t bh0, bl0, bh1, bl1;
          split_tf32(b0, bh0, bl0);
          split_tf32(b1, bh1, bl1);
#pragma unroll
          for (int mt = 0; mt < 4; ++mt) {
            mma_tf32(c[mt][nt], al[mt], bh0, bh1);
            mma_tf32(c[mt][nt], ah[mt], bl0, bl1);
            mma_tf32(c[mt][nt], ah[mt], bh0, bh1);
          }
        }
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = m0 + wm + mt * 16 + gq + half * 8;
        const int col = n0 + wn + nt * 8 + 2 * t;   // even; N is even, so col + 1 < N whenever col < N
        if (row < g.M && col < g.N) {
          float v0 = c[mt][nt][2 * half], v1 = c[mt][nt][2 * half + 1];
          float* cp = g.C + (size_t)row * g.ldc + col;
          if (g.atomic) {
            atomicAdd(cp, v0);
            atomicAdd(cp + 1, v1);
          } else {
            if (g.bias) { v0 += g.bias[col]; v1 += g.bias[col + 1]; }
            if (g.R) {
              const float2 r = *reinterpret_cast<const float2*>(g.R + (size_t)row * g.ldr + col);
              v0 += r.x; v1 += r.y;
            }
            if (g.beta) {
              const float2 o = *reinterpret_cast<const float2*>(cp);
              v0 += o.x; v1 += o.y;
            }
            *reinterpret_cast<float2*>(cp) = make_float2(v0, v1);
          }
        }
      }
}

// The bf16-operand products: the same tiling, but the operands are converted to bfloat16 once, on
// their way from global memory (through registers) into shared memory, and the fragments come out
// of shared memory with ldmatrix (transposing for the [k][row] orientations), so the inner loop is
// six ldmatrix and sixteen MMAs per 16-wide k step.  Global loads of the next K slice are in flight
// while the current one is multiplied.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const __nv_bfloat16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const __nv_bfloat16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

constexpr int LDKH = BK + 8;     // bf16 per row of a [row][k] tile: 80 bytes, ldmatrix rows fall in distinct bank groups
constexpr int LDRH = 128 + 8;    // bf16 per row of a [k][row] tile: 272 bytes, likewise
constexpr int TILE_H = BM * LDKH;

// A_H / B_H / C_H: that operand lives in global memory as bfloat16 (the 4D-wide buffers of the gated
// MLP in bf16 mode) instead of float32: it is then copied into shared memory as it is, or rounded
// once on the way out.  FULL: every tile of the launch lies inside the matrices and every K slice is
// whole (M, N multiples of the tile, K and the split multiples of the slice), so no load or store
// needs a bounds test.
template <bool A_KC, bool B_KC, bool A_H, bool B_H, bool C_H, bool FULL>
__global__ void __launch_bounds__(GT, 2) k_gemm_bf16(GemmArgs g) {
  static_assert(TILE_H >= BK * LDRH, "either orientation fits the tile buffer");
  // one buffer: two stages of A, two of B; a bfloat16 output tile is staged in it after the loop
  __shared__ __align__(16) __nv_bfloat16 smem_all[4 * TILE_H];
  __nv_bfloat16(*sA)[TILE_H] = reinterpret_cast<__nv_bfloat16(*)[TILE_H]>(smem_all);
  __nv_bfloat16(*sB)[TILE_H] = reinterpret_cast<__nv_bfloat16(*)[TILE_H]>(smem_all + 2 * TILE_H);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
  const int wm = (warp & 1) * 64, wn = (warp >> 1) * 32;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kbeg = blockIdx.z * g.k_per_split;
  const int kend = min(g.K, kbeg + g.k_per_split);
  float c[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[i][j][e] = 0.f;

  // four consecutive elements of an operand: float32 (16 bytes) or bfloat16 (8 bytes, in .x .y)
  auto fetch4 = [](const float* base, size_t elem, bool half) {
    float4 v;
    if (half) {
      const uint2 h = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem);
      v.x = __uint_as_float(h.x);
      v.y = __uint_as_float(h.y);
      v.z = v.w = 0.f;
    } else {
      v = *reinterpret_cast<const float4*>(base + elem);
    }
    return v;
  };
  float4 pa[4], pb[4];
  auto gload = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * GT;
      pa[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      pb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if constexpr (A_KC) {
        const int gm = m0 + (idx >> 3), gk = k0 + (idx & 7) * 4;
        if (FULL || (gm < g.M && gk < kend)) pa[i] = fetch4(g.A, (size_t)gm * g.lda + gk, A_H);
      } else {
        const int gk = k0 + (idx >> 5), gm = m0 + (idx & 31) * 4;
        if (FULL || (gk < kend && gm < g.M)) pa[i] = fetch4(g.A, (size_t)gk * g.lda + gm, A_H);
      }
      if constexpr (B_KC) {
        const int gn = n0 + (idx >> 3), gk = k0 + (idx & 7) * 4;
        if (FULL || (gn < g.N && gk < kend)) pb[i] = fetch4(g.B, (size_t)gn * g.ldb + gk, B_H);
      } else {
        const int gk = k0 + (idx >> 5), gn = n0 + (idx & 31) * 4;
        if (FULL || (gk < kend && gn < g.N)) pb[i] = fetch4(g.B, (size_t)gk * g.ldb + gn, B_H);
      }
    }
  };
  auto sstore = [&](int stage) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * GT;
      const uint2 va = A_H ? make_uint2(__float_as_uint(pa[i].x), __float_as_uint(pa[i].y))
                           : make_uint2(pack_bf16(pa[i].x, pa[i].y), pack_bf16(pa[i].z, pa[i].w));
      const uint2 vb = B_H ? make_uint2(__float_as_uint(pb[i].x), __float_as_uint(pb[i].y))
                           : make_uint2(pack_bf16(pb[i].x, pb[i].y), pack_bf16(pb[i].z, pb[i].w));
      if constexpr (A_KC) *reinterpret_cast<uint2*>(&sA[stage][(idx >> 3) * LDKH + (idx & 7) * 4]) = va;
      else *reinterpret_cast<uint2*>(&sA[stage][(idx >> 5) * LDRH + (idx & 31) * 4]) = va;
      if constexpr (B_KC) *reinterpret_cast<uint2*>(&sB[stage][(idx >> 3) * LDKH + (idx & 7) * 4]) = vb;
      else *reinterpret_cast<uint2*>(&sB[stage][(idx >> 5) * LDRH + (idx & 31) * 4]) = vb;
    }
  };

  const int n_it = (kend - kbeg + BK - 1) / BK;
  const int mat = lane >> 3, r8 = lane & 7;
  if (n_it > 0) {
    gload(kbeg);
    sstore(0);
  }
  __syncthreads();
  for (int it = 0; it < n_it; ++it) {
    const bool more = it + 1 < n_it;
    if (more) gload(kbeg + (it + 1) * BK);
    const __nv_bfloat16* As = sA[it & 1];
    const __nv_bfloat16* Bs = sB[it & 1];
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t a[4][4];
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        const int r0 = wm + mt * 16;
        if constexpr (A_KC) ldmatrix_x4(a[mt], As + (r0 + (mat & 1) * 8 + r8) * LDKH + kk + (mat >> 1) * 8);
        else ldmatrix_x4_trans(a[mt], As + (kk + (mat >> 1) * 8 + r8) * LDRH + r0 + (mat & 1) * 8);
      }
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        const int nb = wn + np * 16;
        uint32_t b[4];   // b0, b1 of n-tile 2 np, then of n-tile 2 np + 1
        if constexpr (B_KC) ldmatrix_x4(b, Bs + (nb + (mat >> 1) * 8 + r8) * LDKH + kk + (mat & 1) * 8);
        else ldmatrix_x4_trans(b, Bs + (kk + (mat & 1) * 8 + r8) * LDRH + nb + (mat >> 1) * 8);
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          mma_bf16(c[mt][2 * np], a[mt], b[0], b[1]);
          mma_bf16(c[mt][2 * np + 1], a[mt], b[2], b[3]);
        }
      }
    }
    if (more) sstore((it + 1) & 1);
    __syncthreads();
  }

  if constexpr (C_H) {
    // plain product, rounded once: the tile goes through shared memory so that every thread
    // writes 16 contiguous bytes of a row (the loop's last barrier has freed the buffer)
    constexpr int LDO = BN + 8;
    static_assert(BM * LDO <= 4 * TILE_H, "the output tile fits the operand buffer");
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half)
          *reinterpret_cast<__nv_bfloat162*>(smem_all + (wm + mt * 16 + gq + half * 8) * LDO + wn + nt * 8 + 2 * t) =
              __floats2bfloat162_rn(c[mt][nt][2 * half], c[mt][nt][2 * half + 1]);
    __syncthreads();
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(g.C);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * GT;
      const int row = idx >> 4, c8 = (idx & 15) * 8;
      if (FULL || (m0 + row < g.M && n0 + c8 < g.N))   // N is a multiple of 8
        *reinterpret_cast<uint4*>(out + (size_t)(m0 + row) * g.ldc + n0 + c8) =
            *reinterpret_cast<const uint4*>(smem_all + row * LDO + c8);
    }
    return;
  }
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = m0 + wm + mt * 16 + gq + half * 8;
        const int col = n0 + wn + nt * 8 + 2 * t;   // even; N is even, so col + 1 < N whenever col < N
        if (FULL || (row < g.M && col < g.N)) {
          float v0 = c[mt][nt][2 * half], v1 = c[mt][nt][2 * half + 1];
          float* cp = g.C + (size_t)row * g.ldc + col;
          if (g.atomic) {
            atomicAdd(cp, v0);
            atomicAdd(cp + 1, v1);
          } else {
            if (g.bias) { v0 += g.bias[col]; v1 += g.bias[col + 1]; }
            if (g.R) {
              const float2 r = *reinterpret_cast<const float2*>(g.R + (size_t)row * g.ldr + col);
              v0 += r.x; v1 += r.y;
            }
            if (g.beta) {
              const float2 o = *reinterpret_cast<const float2*>(cp);
              v0 += o.x; v1 += o.y;
            }
            *reinterpret_cast<float2*>(cp) = make_float2(v0, v1);
          }
        }
      }
}

enum GemmMode { NT, NN, TN };

// Whether no tile of the product needs a bounds test (see k_gemm_bf16's FULL).
inline bool gemm_is_full(const GemmArgs& g) {
  return g.M % BM == 0 && g.N % BN == 0 && g.K % BK == 0 && g.k_per_split % BK == 0;
}

// NT: C (M, N)  = A (M, K) . B (N, K)^T      y = x W^T
// NN: C (M, N)  = A (M, K) . B (K, N)        dx = dy W
// TN: C (M, N) += A (K, M)^T . B (K, N)      dW += dy^T x   (split over K, atomics)
template <bool A_KC, bool B_KC, bool BF16>
void launch_gemm_t(const GemmArgs& g, dim3 grid, cudaStream_t st) {
  static const bool opted =
      cudaFuncSetAttribute(k_gemm<A_KC, B_KC, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM) == cudaSuccess;
  (void)opted;
  k_gemm<A_KC, B_KC, BF16><<<grid, GT, GEMM_SMEM, st>>>(g);
}

template <bool BF16>
void launch_gemm(GemmMode mode, const GemmArgs& g, dim3 grid, cudaStream_t st) {
  if constexpr (BF16) {
    const bool full = gemm_is_full(g);
    if (mode == TN) {
      if (full) k_gemm_bf16<false, false, false, false, false, true><<<grid, GT, 0, st>>>(g);
      else k_gemm_bf16<false, false, false, false, false, false><<<grid, GT, 0, st>>>(g);
    } else if (mode == NT) {
      if (full) k_gemm_bf16<true, true, false, false, false, true><<<grid, GT, 0, st>>>(g);
      else k_gemm_bf16<true, true, false, false, false, false><<<grid, GT, 0, st>>>(g);
    } else {
      if (full) k_gemm_bf16<true, false, false, false, false, true><<<grid, GT, 0, st>>>(g);
      else k_gemm_bf16<true, false, false, false, false, false><<<grid, GT, 0, st>>>(g);
    }
  } else {
    if (mode == TN) launch_gemm_t<false, false, false>(g, grid, st);
    else if (mode == NT) launch_gemm_t<true, true, false>(g, grid, st);
    else launch_gemm_t<true, false, false>(g, grid, st);
  }
}

// Which operands of a bf16-mode product are stored as bfloat16 (a bit mask).
enum : int { H_A = 1, H_B = 2, H_C = 4 };

void split_rows(GemmArgs& g, dim3& grid, int K) {
  const int tiles = grid.x * grid.y;
  int splits = (K + 255) / 256;
  const int cap = tiles >= 592 ? 1 : 592 / tiles;   // about four CTAs per SM in flight
  if (splits > cap) splits = cap;
  if (splits < 1) splits = 1;
  int per = (K + splits - 1) / splits;
  per = (per + BK - 1) / BK * BK;
  grid.z = (K + per - 1) / per;
  g.k_per_split = per;
  g.atomic = 1;
}

// The bf16-mode products that touch a bfloat16 buffer (normed activations; gate / up / gated
// product of the MLP and their gradients): A, B, C point to float32 or, for the operands `halves`
// names, bfloat16 elements.
int gemm_half(GemmMode mode, int halves, const void* A, int lda, const void* B, int ldb, void* C, int ldc, int M, int N, int K,
              const float* bias, const float* R, int ldr, int beta, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return BNB_OK;
  GemmArgs g{static_cast<const float*>(A), lda, static_cast<const float*>(B), ldb, static_cast<float*>(C), ldc, M, N, K,
             bias, R, ldr, beta, K, 0};
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, 1);
  count_launch();
  if (mode == TN) split_rows(g, grid, K);
  const bool full = gemm_is_full(g);
#define BNB_GEMM_CASE(MODE, HALVES, AKC, BKC, AH, BH, CH)                             \
  if (mode == MODE && halves == (HALVES)) {                                           \
    if (full) k_gemm_bf16<AKC, BKC, AH, BH, CH, true><<<grid, GT, 0, st>>>(g);        \
    else k_gemm_bf16<AKC, BKC, AH, BH, CH, false><<<grid, GT, 0, st>>>(g);            \
    return BNB_OK;                                                                    \
  }
  BNB_GEMM_CASE(NT, 0, true, true, false, false, false)
  BNB_GEMM_CASE(NT, H_A, true, true, true, false, false)
  BNB_GEMM_CASE(NT, H_C, true, true, false, false, true)
  BNB_GEMM_CASE(NT, H_A | H_C, true, true, true, false, true)
  BNB_GEMM_CASE(NN, 0, true, false, false, false, false)
  BNB_GEMM_CASE(NN, H_A, true, false, true, false, false)
  BNB_GEMM_CASE(NN, H_C, true, false, false, false, true)
  BNB_GEMM_CASE(TN, 0, false, false, false, false, false)
  BNB_GEMM_CASE(TN, H_A, false, false, true, false, false)
  BNB_GEMM_CASE(TN, H_B, false, false, false, true, false)
  BNB_GEMM_CASE(TN, H_A | H_B, false, false, true, true, false)
#undef BNB_GEMM_CASE
  return BNB_ERR_BAD_ARGUMENT;   // a combination no caller uses
}

void gemm(GemmMode mode, const float* A, int lda, const float* B, int ldb, float* C, int ldc, int M, int N, int K,
          const float* bias, const float* R, int ldr, int beta, cudaStream_t st, bool bf16) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  GemmArgs g{A, lda, B, ldb, C, ldc, M, N, K, bias, R, ldr, beta, K, 0};
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, 1);
  count_launch();
  if (mode == TN) split_rows(g, grid, K);
  if (bf16) launch_gemm<true>(mode, g, grid, st);
  else launch_gemm<false>(mode, g, grid, st);
}

// ------------------------------------------------------------------------------ row-wise pieces

constexpr int MAXW = 128;   // widest normed vector (d_model)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// n = x * rsqrt(mean(x^2) + eps) * g; the reciprocal root is kept for the backward.
template <bool HALF_OUT>
__global__ void __launch_bounds__(256) k_rmsnorm_fwd(const float* __restrict__ x, const float* __restrict__ g,
                                                     float* __restrict__ n, float* __restrict__ inv_out, int rows, int W) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int r = warp; r < rows; r += nwarps) {
    float v[MAXW / 32], ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXW / 32; ++i) {
      const int cidx = lane + 32 * i;
      v[i] = cidx < W ? x[(size_t)r * W + cidx] : 0.f;
      ss = fmaf(v[i], v[i], ss);
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)W + kRmsEps);
    if (lane == 0) inv_out[r] = inv;
#pragma unroll
    for (int i = 0; i < MAXW / 32; ++i) {
      const int cidx = lane + 32 * i;
      if (cidx < W) {
        const float o = v[i] * inv * g[cidx];
        if constexpr (HALF_OUT) reinterpret_cast<__nv_bfloat16*>(n)[(size_t)r * W + cidx] = __float2bfloat16_rn(o);
        else n[(size_t)r * W + cidx] = o;
      }
    }
  }
}

// dx = [dres +] inv * g * dn - x * inv^3 * mean(x * g * dn);  dg += sum_rows dn * x * inv.
// dx may alias dres.
__global__ void __launch_bounds__(256) k_rmsnorm_bwd(const float* __restrict__ x, const float* __restrict__ g,
                                                     const float* __restrict__ inv, const float* __restrict__ dn,
                                                     const float* dres, float* dx, float* __restrict__ dg, int rows, int W) {
  __shared__ float sdg[8][MAXW];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  float acc[MAXW / 32];
#pragma unroll
  for (int i = 0; i < MAXW / 32; ++i) acc[i] = 0.f;
  for (int r = warp; r < rows; r += nwarps) {
    float xv[MAXW / 32], dv[MAXW / 32], gv[MAXW / 32], dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXW / 32; ++i) {
      const int cidx = lane + 32 * i;
      const bool ok = cidx < W;
      xv[i] = ok ? x[(size_t)r * W + cidx] : 0.f;
      dv[i] = ok ? dn[(size_t)r * W + cidx] : 0.f;
      gv[i] = ok ? g[cidx] : 0.f;
      dot = fmaf(xv[i] * gv[i], dv[i], dot);
    }
    dot = warp_sum(dot);
    const float iv = inv[r];
    const float coef = dot * iv * iv * iv / (float)W;
#pragma unroll
    for (int i = 0; i < MAXW / 32; ++i) {
      const int cidx = lane + 32 * i;
      if (cidx < W) {
        float v = iv * gv[i] * dv[i] - xv[i] * coef;
        if (dres) v += dres[(size_t)r * W + cidx];
        dx[(size_t)r * W + cidx] = v;
        acc[i] = fmaf(dv[i] * xv[i], iv, acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXW / 32; ++i) sdg[wib][lane + 32 * i] = acc[i];
  __syncthreads();
  if (dg && (int)threadIdx.x < W) {
    float s = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += sdg[w][threadIdx.x];
    atomicAdd(dg + threadIdx.x, s);
  }
}

// The same for rows of exactly 128 columns: a lane owns four consecutive columns (one 16-byte load per
// array) and a warp keeps two rows in flight.
__global__ void __launch_bounds__(256) k_rmsnorm_bwd_128(const float* __restrict__ x, const float* __restrict__ g,
                                                         const float* __restrict__ inv, const float* __restrict__ dn,
                                                         const float* dres, float* dx, float* __restrict__ dg, int rows) {
  __shared__ float4 sdg[8][32];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  const float4 gv = reinterpret_cast<const float4*>(g)[lane];
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r0 = 2 * warp; r0 < rows; r0 += 2 * nwarps) {
    const bool two = r0 + 1 < rows;
    const size_t o0 = (size_t)r0 * 32 + lane, o1 = o0 + 32;
    const float4 x0 = reinterpret_cast<const float4*>(x)[o0], d0 = reinterpret_cast<const float4*>(dn)[o0];
    float4 x1 = make_float4(0.f, 0.f, 0.f, 0.f), d1 = x1, e0 = x1, e1 = x1;
    if (two) {
      x1 = reinterpret_cast<const float4*>(x)[o1];
      d1 = reinterpret_cast<const float4*>(dn)[o1];
    }
    if (dres) {
      e0 = reinterpret_cast<const float4*>(dres)[o0];
      if (two) e1 = reinterpret_cast<const float4*>(dres)[o1];
    }
    float dot0 = fmaf(x0.x * gv.x, d0.x, fmaf(x0.y * gv.y, d0.y, fmaf(x0.z * gv.z, d0.z, x0.w * gv.w * d0.w)));
    float dot1 = fmaf(x1.x * gv.x, d1.x, fmaf(x1.y * gv.y, d1.y, fmaf(x1.z * gv.z, d1.z, x1.w * gv.w * d1.w)));
    dot0 = warp_sum(dot0);
    dot1 = warp_sum(dot1);
    const float iv0 = inv[r0], iv1 = two ? inv[r0 + 1] : 0.f;
    const float c0 = dot0 * iv0 * iv0 * iv0 * (1.0f / 128.0f), c1 = dot1 * iv1 * iv1 * iv1 * (1.0f / 128.0f);
    reinterpret_cast<float4*>(dx)[o0] = make_float4(iv0 * gv.x * d0.x - x0.x * c0 + e0.x, iv0 * gv.y * d0.y - x0.y * c0 + e0.y,
                                                    iv0 * gv.z * d0.z - x0.z * c0 + e0.z, iv0 * gv.w * d0.w - x0.w * c0 + e0.w);
    if (two)
      reinterpret_cast<float4*>(dx)[o1] = make_float4(iv1 * gv.x * d1.x - x1.x * c1 + e1.x, iv1 * gv.y * d1.y - x1.y * c1 + e1.y,
                                                      iv1 * gv.z * d1.z - x1.z * c1 + e1.z, iv1 * gv.w * d1.w - x1.w * c1 + e1.w);
    acc.x += d0.x * x0.x * iv0 + d1.x * x1.x * iv1;
    acc.y += d0.y * x0.y * iv0 + d1.y * x1.y * iv1;
    acc.z += d0.z * x0.z * iv0 + d1.z * x1.z * iv1;
    acc.w += d0.w * x0.w * iv0 + d1.w * x1.w * iv1;
  }
  sdg[wib][lane] = acc;
  __syncthreads();
  if (dg && threadIdx.x < 128) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += reinterpret_cast<const float*>(&sdg[w][0])[threadIdx.x];
    atomicAdd(dg + threadIdx.x, s);
  }
}

__device__ __forceinline__ float gelu_grad(float v) {
  const float cdf = 0.5f * (1.0f + erff(v * 0.70710678118654752440f));
  return cdf + v * 0.39894228040143267794f * expf(-0.5f * v * v);
}

// h = gelu(g) * u, four elements per thread
__global__ void k_gelu_mul_fwd(const float4* __restrict__ g, const float4* __restrict__ u, float4* __restrict__ h, size_t n4) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 a = g[i], b = u[i];
    h[i] = make_float4(gelu_erf(a.x) * b.x, gelu_erf(a.y) * b.y, gelu_erf(a.z) * b.z, gelu_erf(a.w) * b.w);
  }
}

// dg = dh * u * gelu'(g), du = dh * gelu(g).  dg may alias g, du may alias dh (or u).
__global__ void k_gelu_mul_bwd(const float4* g, const float4* u, const float4* dh, float4* dg, float4* du, size_t n4) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 a = g[i], b = u[i], d = dh[i];
    dg[i] = make_float4(d.x * b.x * gelu_grad(a.x), d.y * b.y * gelu_grad(a.y), d.z * b.z * gelu_grad(a.z),
                        d.w * b.w * gelu_grad(a.w));
    du[i] = make_float4(d.x * gelu_erf(a.x), d.y * gelu_erf(a.y), d.z * gelu_erf(a.z), d.w * gelu_erf(a.w));
  }
}

// The same two on bfloat16 buffers, eight elements per thread; gelu and the product each round to
// bfloat16, as autocast's bf16 tensors do (attention.py:37 under autocast).
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__global__ void k_gelu_mul_fwd_h(const uint4* __restrict__ g, const uint4* __restrict__ u, uint4* __restrict__ h, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float a[8], b[8], o[8];
    unpack8(g[i], a);
    unpack8(u[i], b);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = round_bf16(gelu_erf(a[k])) * b[k];
    h[i] = pack8(o);
  }
}
__global__ void k_gelu_mul_bwd_h(const uint4* g, const uint4* u, const uint4* dh, uint4* dg, uint4* du, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float a[8], b[8], d[8], og[8], ou[8];
    unpack8(g[i], a);
    unpack8(u[i], b);
    unpack8(dh[i], d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      og[k] = d[k] * b[k] * gelu_grad(a[k]);
      ou[k] = d[k] * gelu_erf(a[k]);
    }
    dg[i] = pack8(og);
    du[i] = pack8(ou);
  }
}

// out(n) += sum_rows a(row, n): bias gradients.
__global__ void __launch_bounds__(256) k_colsum(const float* __restrict__ a, float* __restrict__ out, int rows, int N) {
  __shared__ float s[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float acc = 0.f;
  if (col < N) {
    const int step = gridDim.y * 8;
    int r = blockIdx.y * 8 + ry;
    for (; r + 3 * step < rows; r += 4 * step) {   // four loads in flight
      const float v0 = a[(size_t)r * N + col], v1 = a[(size_t)(r + step) * N + col];
      const float v2 = a[(size_t)(r + 2 * step) * N + col], v3 = a[(size_t)(r + 3 * step) * N + col];
      acc += (v0 + v1) + (v2 + v3);
    }
    for (; r < rows; r += step) acc += a[(size_t)r * N + col];
  }
  s[ry][cx] = acc;
  __syncthreads();
  if (ry == 0 && col < N) {
    float v = 0.f;
    for (int i = 0; i < 8; ++i) v += s[i][cx];
    atomicAdd(out + col, v);
  }
}

// Rows of one kind (ships: n0 = 0, per_grp = ships per environment; fields: the rest) between the
// token tensor (groups of NM rows) and a compact buffer.  D4 = D / 4.
__global__ void k_gather_rows(const float4* __restrict__ full, float4* __restrict__ compact, size_t n_rows, int D4,
                              int per_grp, int NM, int n0) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_rows * D4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t q = i / D4;
    const int c = (int)(i - q * D4);
    const size_t grp = q / per_grp;
    const int n = (int)(q - grp * per_grp);
    compact[i] = full[(grp * NM + n0 + n) * D4 + c];
  }
}
__global__ void k_scatter_rows(const float4* __restrict__ compact, float4* __restrict__ full, size_t n_rows, int D4,
                               int per_grp, int NM, int n0) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_rows * D4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t q = i / D4;
    const int c = (int)(i - q * D4);
    const size_t grp = q / per_grp;
    const int n = (int)(q - grp * per_grp);
    full[(grp * NM + n0 + n) * D4 + c] = compact[i];
  }
}

// ------------------------------------------------------------------------------ attention

// Forward: one thread per (query token, head), keys read in sequence with a running maximum;
// o = self-attention [+ gate * bullet attention] (attention.py:131-166).
template <int DH>
__device__ __forceinline__ void attend(const float (&q)[DH], const float* __restrict__ kbase, size_t stride, int voff,
                                       int n, const uint8_t* __restrict__ mask, float scale, float (&acc)[DH]) {
#pragma unroll
  for (int d = 0; d < DH; ++d) acc[d] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int j = 0; j < n; ++j) {
    const float* kp = kbase + (size_t)j * stride;
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < DH; ++d) s = fmaf(q[d], kp[d], s);
    s *= scale;
    if (mask && !mask[j]) s = kMaskedScore;
    const float mn = fmaxf(m, s);
    const float corr = expf(m - mn), pj = expf(s - mn);
    l = l * corr + pj;
    const float* vp = kp + voff;
#pragma unroll
    for (int d = 0; d < DH; ++d) acc[d] = fmaf(pj, vp[d], acc[d] * corr);
    m = mn;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int d = 0; d < DH; ++d) acc[d] *= inv;
}

template <int DH>
__global__ void __launch_bounds__(128) k_attn_fwd(const float* __restrict__ qkv, const uint8_t* __restrict__ alive,
                                                  float* __restrict__ o, int NM, int D, int H,
                                                  const float* __restrict__ kvb, const uint8_t* __restrict__ bactive, int nb,
                                                  int G, int groups_per_block) {
  const float scale = rsqrtf((float)DH);
  const int per_group = NM * H;
  for (int pp = threadIdx.x; pp < groups_per_block * per_group; pp += blockDim.x) {
    const int gl = pp / per_group, p = pp - gl * per_group;
    const size_t grp = (size_t)blockIdx.x * groups_per_block + gl;
    if (grp >= (size_t)G) break;
    const size_t tok0 = grp * NM;
    float gate = 1.f;
    const uint8_t* bmask = nullptr;
    if (kvb && bactive) {
      bmask = bactive + grp * nb;
      int any = 0;
      for (int j = 0; j < nb; ++j) any |= bmask[j];
      gate = any ? 1.f : 0.f;
    }
    const int qi = p / H, h = p - qi * H;
    const float* qp = qkv + (tok0 + qi) * 3 * D + h * DH;
    float q[DH], acc[DH], accb[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) q[d] = qp[d];
    attend<DH>(q, qkv + tok0 * 3 * D + D + h * DH, (size_t)3 * D, D, NM, alive ? alive + tok0 : nullptr, scale, acc);
    if (kvb) {
      attend<DH>(q, kvb + grp * nb * 2 * D + h * DH, (size_t)2 * D, D, nb, bmask, scale, accb);
#pragma unroll
      for (int d = 0; d < DH; ++d) acc[d] += accb[d] * gate;
    }
    float* op = o + (tok0 + qi) * D + h * DH;
#pragma unroll
    for (int d = 0; d < DH; ++d) op[d] = acc[d];
  }
}

struct AttnBwdArgs {
  const float* q; int ldq;                 // query i of group g: q + (g * nq + i) * ldq + h * dh
  const float* kv; int ldkv; int voff;     // key j of group g: kv + (g * nk + j) * ldkv + h * dh, value voff further
  const uint8_t* mask;                     // (groups, nk) or null
  const float* d_o; int ldo;               // gradient of the attention output, rows like q
  float* dq; int lddq; int dq_accumulate;
  float* dkv; int lddkv; int dvoff;        // rows like kv
  int nq, nk, dh;
  float scale;
  int gate_by_mask;                        // the branch is multiplied by any(mask) (bullets)
};

// One CTA per (group, head): keys, values and their gradient accumulators in shared memory, one
// warp per query row.  p = exp(s - lse), ds = p (dp - <do, o>) scale.
__global__ void __launch_bounds__(128) k_attn_bwd(AttnBwdArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int nk = a.nk, dh = a.dh, lds = dh + 1;
  const int nkp = (nk + 31) & ~31;
  float* Ks = sm;
  float* Vs = Ks + nk * lds;
  float* dKs = Vs + nk * lds;
  float* dVs = dKs + nk * dh;
  float* per_warp = dVs + nk * dh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* qs = per_warp + warp * (64 + 2 * nkp);
  float* dos = qs + 32;
  float* ps = dos + 32;
  float* dss = ps + nkp;
  const size_t grp = blockIdx.x;
  const int h = blockIdx.y;
  const uint8_t* mask = a.mask ? a.mask + grp * nk : nullptr;

  for (int idx = tid; idx < nk * dh; idx += blockDim.x) {
    const int j = idx / dh, d = idx - j * dh;
    const float* kp = a.kv + (grp * nk + j) * a.ldkv + h * dh + d;
    Ks[j * lds + d] = kp[0];
    Vs[j * lds + d] = kp[a.voff];
    dKs[idx] = 0.f;
    dVs[idx] = 0.f;
  }
  bool open = true;
  if (a.gate_by_mask && mask) {
    int any = 0;
    for (int j = 0; j < nk; ++j) any |= mask[j];
    open = any != 0;
  }
  __syncthreads();

  if (open) {
    for (int i = warp; i < a.nq; i += (int)(blockDim.x >> 5)) {
      const size_t qrow = grp * a.nq + i;
      float qd = 0.f, dod = 0.f;
      if (lane < dh) {
        qd = a.q[qrow * a.ldq + h * dh + lane];
        dod = a.d_o[qrow * a.ldo + h * dh + lane];
      }
      qs[lane] = qd;
      dos[lane] = dod;
      __syncwarp();
      float mx = -INFINITY;
      for (int j = lane; j < nk; j += 32) {
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < dh; ++d) {
          s = fmaf(qs[d], Ks[j * lds + d], s);
          dp = fmaf(dos[d], Vs[j * lds + d], dp);
        }
        s *= a.scale;
        if (mask && !mask[j]) s = kMaskedScore;
        ps[j] = s;
        dss[j] = dp;
        mx = fmaxf(mx, s);
      }
      mx = warp_max(mx);
      float l = 0.f;
      for (int j = lane; j < nk; j += 32) l += expf(ps[j] - mx);
      l = warp_sum(l);
      const float lse = mx + logf(l);
      const float inv_l = 1.0f / l;
      __syncwarp();
      float od = 0.f;
      if (lane < dh) {
        for (int j = 0; j < nk; ++j) od = fmaf(expf(ps[j] - mx), Vs[j * lds + lane], od);
        od *= inv_l;
      }
      const float delta = warp_sum(dod * od);
      __syncwarp();
      for (int j = lane; j < nk; j += 32) {
        const float p = expf(ps[j] - lse);
        ps[j] = p;
        dss[j] = p * (dss[j] - delta) * a.scale;
      }
      __syncwarp();
      if (lane < dh) {
        float dq = 0.f;
        for (int j = 0; j < nk; ++j) {
          const float dsj = dss[j], pj = ps[j];
          dq = fmaf(dsj, Ks[j * lds + lane], dq);
          atomicAdd(&dKs[j * dh + lane], dsj * qd);
          atomicAdd(&dVs[j * dh + lane], pj * dod);
        }
        float* dqp = a.dq + qrow * a.lddq + h * dh + lane;
        *dqp = a.dq_accumulate ? *dqp + dq : dq;
      }
      __syncwarp();
    }
  } else if (!a.dq_accumulate) {
    for (int idx = tid; idx < a.nq * dh; idx += blockDim.x) {
      const int i = idx / dh, d = idx - i * dh;
      a.dq[(grp * a.nq + i) * a.lddq + h * dh + d] = 0.f;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < nk * dh; idx += blockDim.x) {
    const int j = idx / dh, d = idx - j * dh;
    float* kp = a.dkv + (grp * nk + j) * a.lddkv + h * dh + d;
    kp[0] = dKs[idx];
    kp[a.dvoff] = dVs[idx];
  }
}

// Segmented reductions: lanes are grouped in aligned runs of W (a power of two up to 32).
template <int W>
__device__ __forceinline__ float seg_sum(float v) {
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <int W>
__device__ __forceinline__ float seg_max(float v) {
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Attention for small environments (at most 32 queries and keys, head width 32).  A (group, head)
// pair is served by LPP lanes of a warp (8, 16 or 32: the smallest that holds the keys), so a warp
// serves 32 / LPP pairs at once; lane `sub` of a pair owns key `sub` -- its d k and d v accumulate
// in registers -- and, in the per-channel steps, the channels sub * CPL .. + CPL - 1.  The keys and
// values of the pair sit in the warp's slice of shared memory.
constexpr int SMALL_WARPS = 4;

template <int LPP>
__global__ void __launch_bounds__(32 * SMALL_WARPS) k_attn_bwd_small(AttnBwdArgs a, int n_pairs, int H) {
  constexpr int DH = 32, LDS = DH + 1, PPW = 32 / LPP, CPL = DH / LPP;
  __shared__ float sK[SMALL_WARPS][32 * LDS], sV[SMALL_WARPS][32 * LDS], sDs[SMALL_WARPS][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pw = lane / LPP, sub = lane % LPP;
  const int pair = (blockIdx.x * SMALL_WARPS + warp) * PPW + pw;
  const bool pair_ok = pair < n_pairs;
  const size_t grp = pair_ok ? pair / H : 0;
  const int h = pair_ok ? pair - (int)grp * H : 0;
  const int nk = a.nk, nq = a.nq;
  float* Ks = sK[warp] + pw * LPP * LDS;
  float* Vs = sV[warp] + pw * LPP * LDS;
  float* ds_s = sDs[warp] + pw * LPP;
  const uint8_t* mask = a.mask ? a.mask + grp * nk : nullptr;
  if (pair_ok)
    for (int j = 0; j < nk; ++j)
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) {
        const int d = sub + cc * LPP;   // consecutive lanes, consecutive channels
        const float* kp = a.kv + (grp * nk + j) * a.ldkv + h * DH + d;
        Ks[j * LDS + d] = kp[0];
        Vs[j * LDS + d] = kp[a.voff];
      }
  const bool live = pair_ok && sub < nk;
  bool dead_key = false, open = true;
  if (mask) {
    const int mine = live ? mask[sub] : 0;
    dead_key = live && !mine;
    if (a.gate_by_mask) open = seg_max<LPP>(mine ? 1.f : 0.f) > 0.f;
  }
  __syncwarp();
  float dk[DH], dv[DH];
#pragma unroll
  for (int d = 0; d < DH; ++d) dk[d] = dv[d] = 0.f;
  for (int i = 0; i < nq; ++i) {   // every lane of the warp walks the loop: the shuffles need them all
    const size_t qrow = grp * nq + i;
    float q[DH], go[DH];
    if (pair_ok && open) {
      const float4* qp = reinterpret_cast<const float4*>(a.q + qrow * a.ldq + h * DH);
      const float4* gp = reinterpret_cast<const float4*>(a.d_o + qrow * a.ldo + h * DH);
#pragma unroll
      for (int d4 = 0; d4 < DH / 4; ++d4) {   // the lanes of a pair read the same row
        const float4 v = qp[d4], w = gp[d4];
        q[4 * d4] = v.x; q[4 * d4 + 1] = v.y; q[4 * d4 + 2] = v.z; q[4 * d4 + 3] = v.w;
        go[4 * d4] = w.x; go[4 * d4 + 1] = w.y; go[4 * d4 + 2] = w.z; go[4 * d4 + 3] = w.w;
      }
    } else {
#pragma unroll
      for (int d = 0; d < DH; ++d) q[d] = go[d] = 0.f;
    }
    float sc = 0.f, dp = 0.f;
    if (live) {
#pragma unroll
      for (int d = 0; d < DH; ++d) {
        sc = fmaf(q[d], Ks[sub * LDS + d], sc);
        dp = fmaf(go[d], Vs[sub * LDS + d], dp);
      }
      sc *= a.scale;
      if (dead_key) sc = kMaskedScore;
    }
    const float mx = seg_max<LPP>(live ? sc : -INFINITY);
    const float e = live ? expf(sc - mx) : 0.f;
    const float l = seg_sum<LPP>(e);
    const float lse = mx + logf(l);
    const float delta = seg_sum<LPP>(live ? e / l * dp : 0.f);   // <d out, out>
    const float p = live ? expf(sc - lse) : 0.f;
    const float ds = p * (dp - delta) * a.scale;
    ds_s[sub] = ds;
#pragma unroll
    for (int d = 0; d < DH; ++d) {
      dk[d] = fmaf(ds, q[d], dk[d]);
      dv[d] = fmaf(p, go[d], dv[d]);
    }
    __syncwarp();
    if (pair_ok) {
      float dq[CPL];
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) dq[cc] = 0.f;
      if (open)
        for (int j = 0; j < nk; ++j) {
          const float dsj = ds_s[j];
#pragma unroll
          for (int cc = 0; cc < CPL; ++cc) dq[cc] = fmaf(dsj, Ks[j * LDS + sub * CPL + cc], dq[cc]);
        }
      float* dqp = a.dq + qrow * a.lddq + h * DH + sub * CPL;
      if (open || !a.dq_accumulate)
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) dqp[cc] = a.dq_accumulate ? dqp[cc] + dq[cc] : dq[cc];
    }
    __syncwarp();
  }
  if (live) {
    float4* kp = reinterpret_cast<float4*>(a.dkv + (grp * nk + sub) * a.lddkv + h * DH);
    float4* vp = reinterpret_cast<float4*>(a.dkv + (grp * nk + sub) * a.lddkv + h * DH + a.dvoff);
#pragma unroll
    for (int d4 = 0; d4 < DH / 4; ++d4) {
      kp[d4] = make_float4(dk[4 * d4], dk[4 * d4 + 1], dk[4 * d4 + 2], dk[4 * d4 + 3]);
      vp[d4] = make_float4(dv[4 * d4], dv[4 * d4 + 1], dv[4 * d4 + 2], dv[4 * d4 + 3]);
    }
  }
}

// Forward for the same small environments: o = softmax(q k^T) v [+ gate * the bullet branch], the
// pair's lanes sharing each query: lane `sub` scores key `sub`, then owns CPL output channels.
template <int LPP>
__global__ void __launch_bounds__(32 * SMALL_WARPS) k_attn_fwd_small(const float* __restrict__ qkv, const uint8_t* __restrict__ alive,
                                                                   float* __restrict__ o, int NM, int D, int H, int n_pairs) {
  constexpr int DH = 32, LDS = DH + 1, PPW = 32 / LPP, CPL = DH / LPP;
  __shared__ float sK[SMALL_WARPS][32 * LDS], sV[SMALL_WARPS][32 * LDS], sP[SMALL_WARPS][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pw = lane / LPP, sub = lane % LPP;
  const int pair = (blockIdx.x * SMALL_WARPS + warp) * PPW + pw;
  const bool pair_ok = pair < n_pairs;
  const size_t grp = pair_ok ? pair / H : 0;
  const int h = pair_ok ? pair - (int)grp * H : 0;
  const size_t tok0 = grp * NM;
  float* Ks = sK[warp] + pw * LPP * LDS;
  float* Vs = sV[warp] + pw * LPP * LDS;
  float* p_s = sP[warp] + pw * LPP;
  if (pair_ok)
    for (int j = 0; j < NM; ++j)
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) {
        const int d = sub + cc * LPP;
        const float* kp = qkv + (tok0 + j) * 3 * D + D + h * DH + d;
        Ks[j * LDS + d] = kp[0];
        Vs[j * LDS + d] = kp[D];
      }
  const bool live = pair_ok && sub < NM;
  const bool dead_key = live && alive && !alive[tok0 + sub];
  const float scale = rsqrtf((float)DH);
  __syncwarp();
  for (int i = 0; i < NM; ++i) {
    float sc = 0.f;
    if (live) {
      const float4* qp = reinterpret_cast<const float4*>(qkv + (tok0 + i) * 3 * D + h * DH);
#pragma unroll
      for (int d4 = 0; d4 < DH / 4; ++d4) {
        const float4 v = qp[d4];
        const float* kr = Ks + sub * LDS + 4 * d4;
        sc = fmaf(v.x, kr[0], sc); sc = fmaf(v.y, kr[1], sc); sc = fmaf(v.z, kr[2], sc); sc = fmaf(v.w, kr[3], sc);
      }
      sc *= scale;
      if (dead_key) sc = kMaskedScore;
    }
    const float mx = seg_max<LPP>(live ? sc : -INFINITY);
    const float e = live ? expf(sc - mx) : 0.f;
    const float l = seg_sum<LPP>(e);
    p_s[sub] = e / l;
    __syncwarp();
    if (pair_ok) {
      float acc[CPL];
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) acc[cc] = 0.f;
      for (int j = 0; j < NM; ++j) {
        const float pj = p_s[j];
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) acc[cc] = fmaf(pj, Vs[j * LDS + sub * CPL + cc], acc[cc]);
      }
      float* op = o + (tok0 + i) * D + h * DH + sub * CPL;
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) op[cc] = acc[cc];
    }
    __syncwarp();
  }
}

size_t attn_bwd_smem(int nk, int dh) {
  const int nkp = (nk + 31) & ~31;
  return (size_t)(2 * nk * (dh + 1) + 2 * nk * dh + 4 * (64 + 2 * nkp)) * sizeof(float);
}

// ------------------------------------------------------------------------------ recurrent branch

// Geometry of the ship rows of one temporal sublayer: row s = b * n_rec + n of step t sits at
// (t * Rr + s) * D in the time-major buffers; its state at hid + s * 4 D (h | three taps, oldest first).
struct ShipGeom {
  int T, Rr, D, n_rec, B;
  const uint8_t* done;   // (T, B) or null
};

// u_t = conv bias + sum over lags of tap * padded value, a lag being valid while no episode boundary
// lies between (griffin.py:67-140).
__global__ void __launch_bounds__(256) k_conv_fwd(const float* __restrict__ b1, const float* __restrict__ hid,
                                                  const float* __restrict__ cw, const float* __restrict__ cb,
                                                  float* __restrict__ u, ShipGeom gm) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)gm.Rr * gm.D) return;
  const int s = (int)(idx / gm.D), d = (int)(idx - (size_t)s * gm.D);
  const int b = s / gm.n_rec;
  const float* hp = hid + (size_t)s * 4 * gm.D + d;
  float p3 = hp[gm.D], p2 = hp[2 * gm.D], p1 = hp[3 * gm.D];
  const float w0 = cw[d * 4], w1 = cw[d * 4 + 1], w2 = cw[d * 4 + 2], w3 = cw[d * 4 + 3], bias = cb[d];
  int cur = BNB_CONV_KERNEL - 1;
  for (int t = 0; t < gm.T; ++t) {
    if (t >= 1) {
      const bool boundary = gm.done && gm.done[(size_t)(t - 1) * gm.B + b];
      cur = boundary ? 0 : min(cur + 1, BNB_CONV_KERNEL - 1);
    }
    const size_t at = ((size_t)t * gm.Rr + s) * gm.D + d;
    const float xt = b1[at];
    const float t0 = cur >= 3 ? __fmul_rn(p3, w0) : 0.f;
    const float t1 = cur >= 2 ? __fmul_rn(p2, w1) : 0.f;
    const float t2 = cur >= 1 ? __fmul_rn(p1, w2) : 0.f;
    const float t3 = __fmul_rn(xt, w3);
    u[at] = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(t0, t1), t2), t3), bias);
    p3 = p2; p2 = p1; p1 = xt;
  }
}

// h_t = a_t h_{t-1} + sqrt(1 - a_t^2) (i_t u_t), a_t = sigmoid(lambda)^(8 r_t), zeroed after a boundary
// (griffin.py:169-219); every h_t is kept.
__global__ void __launch_bounds__(256) k_scan_fwd(const float* __restrict__ za, const float* __restrict__ zx,
                                                  const float* __restrict__ u, const float* __restrict__ hid,
                                                  const float* __restrict__ log_lambda, float* __restrict__ hs, ShipGeom gm) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)gm.Rr * gm.D) return;
  const int s = (int)(idx / gm.D), d = (int)(idx - (size_t)s * gm.D);
  const int b = s / gm.n_rec;
  float h = hid[(size_t)s * 4 * gm.D + d];
  const float base = sigmoidf_(log_lambda[d]);
  for (int t = 0; t < gm.T; ++t) {
    const size_t at = ((size_t)t * gm.Rr + s) * gm.D + d;
    const float rg = sigmoidf_(za[at]), ig = sigmoidf_(zx[at]);
    float a = powf(base, kRglruC * rg);
    const float gate = sqrtf(fmaxf((1.0f - a) * (1.0f + a), kGateFloor));
    const float bb = gate * (ig * u[at]);
    if (t >= 1 && gm.done && gm.done[(size_t)(t - 1) * gm.B + b]) a = 0.f;
    h = a * h + bb;
    hs[at] = h;
  }
}

// State after the last step: h_T and the last three padded conv inputs (griffin.py:271-275).
__global__ void __launch_bounds__(256) k_final_state(const float* __restrict__ hs, const float* __restrict__ b1,
                                                     const float* __restrict__ hid, float* __restrict__ hid_out, ShipGeom gm) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)gm.Rr * gm.D) return;
  const int s = (int)(idx / gm.D), d = (int)(idx - (size_t)s * gm.D);
  const size_t step = (size_t)gm.Rr * gm.D, at0 = (size_t)s * gm.D + d;
  float* op = hid_out + (size_t)s * 4 * gm.D + d;
  op[0] = hs[(size_t)(gm.T - 1) * step + at0];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int p = gm.T + k;   // padded index: 0..2 the stored taps, 3 + t the linear1 output of step t
    op[(size_t)(k + 1) * gm.D] = p < 3 ? hid[(size_t)s * 4 * gm.D + (size_t)(p + 1) * gm.D + d] : b1[(size_t)(p - 3) * step + at0];
  }
}

// Reverse-time adjoint of k_scan_fwd.  In: za, zx (with bias), u, hs, dhs (gradient reaching every
// h_t from the output path) and the gradient of the final state.  Out: d za, d zx in place of za,
// zx; the direct part of d u in place of dhs; d h0; d log_lambda (reduced over rows, atomics).
__global__ void __launch_bounds__(256) k_scan_bwd(float* za, float* zx, const float* __restrict__ u,
                                                  const float* __restrict__ hs, float* dhs, const float* __restrict__ hid,
                                                  const float* __restrict__ d_hid_out, float* __restrict__ d_hid_in,
                                                  const float* __restrict__ log_lambda, float* __restrict__ d_log_lambda,
                                                  ShipGeom gm) {
  __shared__ float s_dl[MAXW];
  if ((int)threadIdx.x < gm.D) s_dl[threadIdx.x] = 0.f;
  __syncthreads();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = idx < (size_t)gm.Rr * gm.D;
  const int s = live ? (int)(idx / gm.D) : 0, d = live ? (int)(idx - (size_t)s * gm.D) : 0;
  if (live) {
    const int b = s / gm.n_rec;
    const float lam = log_lambda[d];
    const float base = sigmoidf_(lam);
    const float logb = logf(base);
    float carry = d_hid_out ? d_hid_out[(size_t)s * 4 * gm.D + d] : 0.f;
    float dl = 0.f;
    for (int t = gm.T - 1; t >= 0; --t) {
      const size_t at = ((size_t)t * gm.Rr + s) * gm.D + d;
      const float dh = dhs[at] + carry;
      const float rg = sigmoidf_(za[at]), ig = sigmoidf_(zx[at]), uv = u[at];
      const float a = powf(base, kRglruC * rg);
      const float cc = (1.0f - a) * (1.0f + a);
      const float gate = sqrtf(fmaxf(cc, kGateFloor));
      const bool reset = t >= 1 && gm.done && gm.done[(size_t)(t - 1) * gm.B + b];
      const float hprev = t > 0 ? hs[at - (size_t)gm.Rr * gm.D] : hid[(size_t)s * 4 * gm.D + d];
      float da = reset ? 0.f : dh * hprev;
      carry = reset ? 0.f : dh * a;
      const float dgate = dh * ig * uv;
      const float di = dh * gate * uv;
      if (cc > kGateFloor) da -= dgate * a / gate;
      const float dr = da * a * kRglruC * logb;
      dl = fmaf(da * a * kRglruC * rg, 1.0f - base, dl);
      za[at] = dr * rg * (1.0f - rg);
      zx[at] = di * ig * (1.0f - ig);
      dhs[at] = dh * gate * ig;
    }
    if (d_hid_in) d_hid_in[(size_t)s * 4 * gm.D + d] = carry;
    atomicAdd(&s_dl[d], dl);
  }
  __syncthreads();
  if ((int)threadIdx.x < gm.D) atomicAdd(d_log_lambda + threadIdx.x, s_dl[threadIdx.x]);
}

// Adjoint of k_conv_fwd: d u -> d linear1 output, d stored taps, d conv weight and bias.  The
// new tap buffer is the last three padded values, so its gradient joins there.
__global__ void __launch_bounds__(256) k_conv_bwd(const float* __restrict__ du, const float* __restrict__ b1,
                                                  const float* __restrict__ hid, const float* __restrict__ d_hid_out,
                                                  float* __restrict__ d_hid_in, const float* __restrict__ cw,
                                                  float* __restrict__ db1, float* __restrict__ d_cw, float* __restrict__ d_cb,
                                                  ShipGeom gm) {
  __shared__ float s_w[MAXW * 4], s_b[MAXW];
  for (int i = threadIdx.x; i < gm.D * 4; i += blockDim.x) s_w[i] = 0.f;
  if ((int)threadIdx.x < gm.D) s_b[threadIdx.x] = 0.f;
  __syncthreads();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = idx < (size_t)gm.Rr * gm.D;
  const int s = live ? (int)(idx / gm.D) : 0, d = live ? (int)(idx - (size_t)s * gm.D) : 0;
  if (live) {
    const int b = s / gm.n_rec, T = gm.T, D = gm.D;
    const float* hp = hid + (size_t)s * 4 * D + d;
    // padded index p: 0..2 the stored taps, 3 + t the linear1 output of step t
    auto emit = [&](int p, float v) {
      if (p >= T && d_hid_out) v += d_hid_out[(size_t)s * 4 * D + D + (size_t)(p - T) * D + d];
      if (p < 3) {
        if (d_hid_in) d_hid_in[(size_t)s * 4 * D + D + (size_t)p * D + d] = v;
      } else {
        db1[((size_t)(p - 3) * gm.Rr + s) * D + d] = v;
      }
    };
    const float w[4] = {cw[d * 4], cw[d * 4 + 1], cw[d * 4 + 2], cw[d * 4 + 3]};
    float pad[4] = {hp[D], hp[2 * D], hp[3 * D], 0.f};   // padded[t .. t+3] at step t
    float acc[4] = {0.f, 0.f, 0.f, 0.f};                 // d padded[t .. t+3]
    float dw[4] = {0.f, 0.f, 0.f, 0.f}, dbias = 0.f;
    int cur = BNB_CONV_KERNEL - 1;
    for (int t = 0; t < T; ++t) {
      if (t >= 1) {
        const bool boundary = gm.done && gm.done[(size_t)(t - 1) * gm.B + b];
        cur = boundary ? 0 : min(cur + 1, BNB_CONV_KERNEL - 1);
      }
      const size_t at = ((size_t)t * gm.Rr + s) * D + d;
      pad[3] = b1[at];
      const float g = du[at];
      dbias += g;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool valid = (3 - k) <= cur;   // tap k reads lag 3 - k
        if (valid) {
          acc[k] = fmaf(g, w[k], acc[k]);
          dw[k] = fmaf(g, pad[k], dw[k]);
        }
      }
      emit(t, acc[0]);
      acc[0] = acc[1]; acc[1] = acc[2]; acc[2] = acc[3]; acc[3] = 0.f;
      pad[0] = pad[1]; pad[1] = pad[2]; pad[2] = pad[3];
    }
    emit(T, acc[0]);
    emit(T + 1, acc[1]);
    emit(T + 2, acc[2]);
#pragma unroll
    for (int k = 0; k < 4; ++k) atomicAdd(&s_w[d * 4 + k], dw[k]);
    atomicAdd(&s_b[d], dbias);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < gm.D * 4; i += blockDim.x) atomicAdd(d_cw + i, s_w[i]);
  if ((int)threadIdx.x < gm.D) atomicAdd(d_cb + threadIdx.x, s_b[threadIdx.x]);
}

// ------------------------------------------------------------------------------ host side

struct Arena {
  char* base;
  size_t off = 0;
  float* take(size_t n_floats) {
    float* p = base ? reinterpret_cast<float*>(base + off) : nullptr;
    off += (n_floats * sizeof(float) + 255) & ~(size_t)255;
    return p;
  }
};

constexpr int N_DBUF = 17;

struct Bufs {
  float* bound;        // inputs of sublayers 1 .. S-1
  float* ping[2];      // gradient with respect to a sublayer's input, alternating
  float* d[N_DBUF];    // rows x D each
  float* w3[2];        // rows x 3D
  float* w4[3];        // rows x 4D
  float* inv[2];       // rows
  float *bul_n, *bul_inv, *kvb, *dkvb, *bul_dn;
};

// half_mlp: the three 4D-wide buffers hold bfloat16 (bf16 mode), so they take half the bytes.
void plan(Arena& ar, Bufs& b, int S, size_t R, int D, size_t RB, bool half_mlp) {
  b.bound = ar.take((size_t)(S > 1 ? S - 1 : 0) * R * D);
  for (auto& p : b.ping) p = ar.take(R * D);
  for (auto& p : b.d) p = ar.take(R * D);
  for (auto& p : b.w3) p = ar.take(R * 3 * D);
  for (auto& p : b.w4) p = ar.take(R * 4 * D / (half_mlp ? 2 : 1));
  for (auto& p : b.inv) p = ar.take(R);
  b.bul_n = ar.take(RB * D);
  b.bul_inv = ar.take(RB);
  b.kvb = ar.take(RB * 2 * D);
  b.dkvb = ar.take(RB * 2 * D);
  b.bul_dn = ar.take(RB * D);
}

// The buffers the forward part of one path writes and its backward part reads, taken from an arena
// of their own when the activations are kept between the two (see trunk_sequence_fwd_train).
enum PathKind { P_SPATIAL, P_SHIPS, P_FIELDS };

void bind_forward(Arena& ar, Bufs& b, PathKind kind, size_t rows, int D, size_t RB, bool half_mlp) {
  const int nd = kind == P_SPATIAL ? 3 : kind == P_SHIPS ? 10 : 7;
  // the normed activations (slot 0 of a spatial path, slot 1 of a temporal one, slot 15 before the
  // MLP) are bfloat16 in bf16 mode: half the floats
  const size_t normed = half_mlp ? (rows * D + 1) / 2 : rows * D;
  const int n_slot = kind == P_SPATIAL ? 0 : 1;
  for (int i = 0; i < nd; ++i) b.d[i] = ar.take(i == n_slot ? normed : rows * D);
  b.d[15] = ar.take(normed);
  b.inv[0] = ar.take(rows);
  b.inv[1] = ar.take(rows);
  if (kind == P_SPATIAL) {
    b.w3[0] = ar.take(rows * 3 * D);
    b.bul_n = ar.take(RB * D);
    b.bul_inv = ar.take(RB);
    b.kvb = ar.take(RB * 2 * D);
  }
  for (auto& p : b.w4) p = ar.take(rows * 4 * D / (half_mlp ? 2 : 1));
}

inline int blocks_for(size_t n, int per_block, int cap = 148 * 8) {
  size_t g = (n + per_block - 1) / per_block;
  if (g > (size_t)cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

struct Ctx {
  int D, H;
  bool bf16;   // products round their operands to bfloat16 (the forward ran under autocast)
  cudaStream_t st;
  Bufs b;
};

void mm(const Ctx& c, GemmMode mode, const float* A, int lda, const float* B, int ldb, float* C, int ldc, int M, int N, int K,
        const float* bias = nullptr, const float* R = nullptr, int ldr = 0, int beta = 0) {
  gemm(mode, A, lda, B, ldb, C, ldc, M, N, K, bias, R, ldr, beta, c.st, c.bf16);
}
// The same for products whose operands `halves` names hold bfloat16 in bf16 mode (in float32 mode
// the same buffers hold float32 and the mask is ignored).
void mmh(const Ctx& c, GemmMode mode, int halves, const float* A, int lda, const float* B, int ldb, float* C, int ldc, int M, int N,
         int K, const float* bias = nullptr, const float* R = nullptr, int ldr = 0, int beta = 0) {
  if (c.bf16) gemm_half(mode, halves, A, lda, B, ldb, C, ldc, M, N, K, bias, R, ldr, beta, c.st);
  else gemm(mode, A, lda, B, ldb, C, ldc, M, N, K, bias, R, ldr, beta, c.st, false);
}

void rmsnorm_fwd(const Ctx& c, const float* x, const float* g, float* n, float* inv, size_t rows) {
  if (!rows) return;
  count_launch();
  // the normed activations only ever feed Linear products: in bf16 mode they are stored as bfloat16
  if (c.bf16) k_rmsnorm_fwd<true><<<blocks_for(rows, 8), 256, 0, c.st>>>(x, g, n, inv, (int)rows, c.D);
  else k_rmsnorm_fwd<false><<<blocks_for(rows, 8), 256, 0, c.st>>>(x, g, n, inv, (int)rows, c.D);
}
void rmsnorm_bwd(const Ctx& c, const float* x, const float* g, const float* inv, const float* dn, const float* dres,
                 float* dx, float* dg, size_t rows) {
  if (!rows) return;
  count_launch();
  const auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (c.D == 128 && al(x) && al(g) && al(dn) && al(dx) && (!dres || al(dres)))
    k_rmsnorm_bwd_128<<<blocks_for(rows, 64, 148 * 8), 256, 0, c.st>>>(x, g, inv, dn, dres, dx, dg, (int)rows);
  else
    k_rmsnorm_bwd<<<blocks_for(rows, 64, 148 * 8), 256, 0, c.st>>>(x, g, inv, dn, dres, dx, dg, (int)rows, c.D);
}
void gelu_mul_fwd(const Ctx& c, const float* g, const float* u, float* h, size_t n) {
  if (!n) return;
  count_launch();
  k_gelu_mul_fwd<<<blocks_for(n / 4, 256), 256, 0, c.st>>>(reinterpret_cast<const float4*>(g), reinterpret_cast<const float4*>(u),
                                                           reinterpret_cast<float4*>(h), n / 4);
}
void gelu_mul_bwd(const Ctx& c, const float* g, const float* u, const float* dh, float* dg, float* du, size_t n) {
  if (!n) return;
  count_launch();
  k_gelu_mul_bwd<<<blocks_for(n / 4, 256), 256, 0, c.st>>>(reinterpret_cast<const float4*>(g), reinterpret_cast<const float4*>(u),
                                                           reinterpret_cast<const float4*>(dh), reinterpret_cast<float4*>(dg),
                                                           reinterpret_cast<float4*>(du), n / 4);
}
void colsum(const Ctx& c, const float* a, float* out, size_t rows, int N) {
  if (!rows) return;
  count_launch();
  dim3 grid((N + 31) / 32, blocks_for(rows, 256, 296));
  k_colsum<<<grid, 256, 0, c.st>>>(a, out, (int)rows, N);
}

// Gated MLP at the end of every sublayer, y = x1 + down(gelu(gate n) * up n), n = rmsnorm(x1).
// Leaves n in d[15], the reciprocal roots in inv[1], gate / up / their gated product in w4[0..2];
// writes y when y is given.
void mlp_fwd(const Ctx& c, const float* x1, float* y, size_t rows, const float* g2, const float* Wg, const float* Wu,
             const float* Wd) {
  const int D = c.D, F = 4 * c.D, M = (int)rows;
  float *n2 = c.b.d[15], *gb = c.b.w4[0], *ub = c.b.w4[1], *hb = c.b.w4[2];
  rmsnorm_fwd(c, x1, g2, n2, c.b.inv[1], rows);
  if (c.bf16) {   // gate, up and their gated product are bfloat16 tensors, as under autocast
    gemm_half(NT, H_A | H_C, n2, D, Wg, D, gb, F, M, F, D, nullptr, nullptr, 0, 0, c.st);
    gemm_half(NT, H_A | H_C, n2, D, Wu, D, ub, F, M, F, D, nullptr, nullptr, 0, 0, c.st);
    if (rows) {
      count_launch();
      k_gelu_mul_fwd_h<<<blocks_for(rows * F / 8, 256), 256, 0, c.st>>>(reinterpret_cast<const uint4*>(gb), reinterpret_cast<const uint4*>(ub),
                                                                     reinterpret_cast<uint4*>(hb), rows * F / 8);
    }
    if (y) gemm_half(NT, H_A, hb, F, Wd, F, y, D, M, D, F, nullptr, x1, D, 0, c.st);
    return;
  }
  mm(c, NT, n2, D, Wg, D, gb, F, M, F, D);
  mm(c, NT, n2, D, Wu, D, ub, F, M, F, D);
  gelu_mul_fwd(c, gb, ub, hb, rows * F);
  if (y) mm(c, NT, hb, F, Wd, F, y, D, M, D, F, nullptr, x1, D);
}

// After mlp_fwd: given d y, accumulates the weight gradients and writes d x1.  Uses d[16].
void mlp_bwd(const Ctx& c, const float* x1, const float* dy, float* dx1, size_t rows, const float* g2, const float* Wg,
             const float* Wu, const float* Wd, float* dg2, float* dWg, float* dWu, float* dWd) {
  const int D = c.D, F = 4 * c.D, M = (int)rows;
  float *n2 = c.b.d[15], *dn2 = c.b.d[16], *gb = c.b.w4[0], *ub = c.b.w4[1], *hb = c.b.w4[2];
  if (c.bf16) {
    gemm_half(TN, H_B, dy, D, hb, F, dWd, F, D, F, M, nullptr, nullptr, 0, 0, c.st);
    gemm_half(NN, H_C, dy, D, Wd, F, hb, F, M, F, D, nullptr, nullptr, 0, 0, c.st);
    if (rows) {
      count_launch();
      k_gelu_mul_bwd_h<<<blocks_for(rows * F / 8, 256), 256, 0, c.st>>>(
          reinterpret_cast<const uint4*>(gb), reinterpret_cast<const uint4*>(ub), reinterpret_cast<const uint4*>(hb),
          reinterpret_cast<uint4*>(gb), reinterpret_cast<uint4*>(ub), rows * F / 8);
    }
    gemm_half(TN, H_A | H_B, gb, F, n2, D, dWg, D, F, D, M, nullptr, nullptr, 0, 0, c.st);
    gemm_half(TN, H_A | H_B, ub, F, n2, D, dWu, D, F, D, M, nullptr, nullptr, 0, 0, c.st);
    gemm_half(NN, H_A, gb, F, Wg, D, dn2, D, M, D, F, nullptr, nullptr, 0, 0, c.st);
    gemm_half(NN, H_A, ub, F, Wu, D, dn2, D, M, D, F, nullptr, nullptr, 0, 1, c.st);
    rmsnorm_bwd(c, x1, g2, c.b.inv[1], dn2, dy, dx1, dg2, rows);
    return;
  }
  mm(c, TN, dy, D, hb, F, dWd, F, D, F, M);                 // dWd (D, 4D) += dy^T h
  mm(c, NN, dy, D, Wd, F, hb, F, M, F, D);                  // dh = dy Wd
  gelu_mul_bwd(c, gb, ub, hb, gb, ub, rows * F);            // gb <- d gate, ub <- d up
  mm(c, TN, gb, F, n2, D, dWg, D, F, D, M);
  mm(c, TN, ub, F, n2, D, dWu, D, F, D, M);
  mm(c, NN, gb, F, Wg, D, dn2, D, M, D, F);
  mm(c, NN, ub, F, Wu, D, dn2, D, M, D, F, nullptr, nullptr, 0, 1);
  rmsnorm_bwd(c, x1, g2, c.b.inv[1], dn2, dy, dx1, dg2, rows);
}

template <int DH>
void attn_fwd_t(const Ctx& c, const float* qkv, const uint8_t* alive, float* o, int G, int NM, const float* kvb,
                const uint8_t* bactive, int nb) {
  count_launch();
  const int per_group = NM * c.H;
  const int gpb = per_group >= 128 ? 1 : 128 / per_group;   // small environments share a block
  k_attn_fwd<DH><<<(G + gpb - 1) / gpb, 128, 0, c.st>>>(qkv, alive, o, NM, c.D, c.H, kvb, bactive, nb, G, gpb);
}
void attn_fwd(const Ctx& c, const float* qkv, const uint8_t* alive, float* o, int G, int NM, const float* kvb,
              const uint8_t* bactive, int nb) {
  if (!G) return;
  if (c.D / c.H == 32 && NM <= 32 && !kvb) {
    const int n_pairs = G * c.H;
    const int lpp = NM <= 8 ? 8 : NM <= 16 ? 16 : 32;
    const int per_block = SMALL_WARPS * (32 / lpp);
    const int grid = (n_pairs + per_block - 1) / per_block;
    count_launch();
    if (lpp == 8) k_attn_fwd_small<8><<<grid, 32 * SMALL_WARPS, 0, c.st>>>(qkv, alive, o, NM, c.D, c.H, n_pairs);
    else if (lpp == 16) k_attn_fwd_small<16><<<grid, 32 * SMALL_WARPS, 0, c.st>>>(qkv, alive, o, NM, c.D, c.H, n_pairs);
    else k_attn_fwd_small<32><<<grid, 32 * SMALL_WARPS, 0, c.st>>>(qkv, alive, o, NM, c.D, c.H, n_pairs);
    return;
  }
  switch (c.D / c.H) {
    case 8: attn_fwd_t<8>(c, qkv, alive, o, G, NM, kvb, bactive, nb); break;
    case 16: attn_fwd_t<16>(c, qkv, alive, o, G, NM, kvb, bactive, nb); break;
    default: attn_fwd_t<32>(c, qkv, alive, o, G, NM, kvb, bactive, nb); break;
  }
}
int attn_bwd(const Ctx& c, const AttnBwdArgs& a, int G) {
  if (!G) return BNB_OK;
  if (a.dh == 32 && a.nk <= 32 && a.nq <= 32) {
    const int n_pairs = G * c.H;
    const int lpp = a.nk <= 8 ? 8 : a.nk <= 16 ? 16 : 32;
    const int per_block = SMALL_WARPS * (32 / lpp);
    const int grid = (n_pairs + per_block - 1) / per_block;
    count_launch();
    if (lpp == 8) k_attn_bwd_small<8><<<grid, 32 * SMALL_WARPS, 0, c.st>>>(a, n_pairs, c.H);
    else if (lpp == 16) k_attn_bwd_small<16><<<grid, 32 * SMALL_WARPS, 0, c.st>>>(a, n_pairs, c.H);
    else k_attn_bwd_small<32><<<grid, 32 * SMALL_WARPS, 0, c.st>>>(a, n_pairs, c.H);
    return BNB_OK;
  }
  const size_t sm = attn_bwd_smem(a.nk, a.dh);
  if (sm > 200 * 1024) return BNB_ERR_TOO_MANY_TOKENS;
  if (cudaFuncSetAttribute(k_attn_bwd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm) != cudaSuccess)
    return BNB_ERR_LAUNCH;
  count_launch();
  k_attn_bwd<<<dim3(G, c.H), 128, sm, c.st>>>(a);
  return BNB_OK;
}

// Spatial sublayer, forward part.  Leaves n1 in d[0] (roots in inv[0]), q|k|v in w3[0], the attention
// output in d[1], x1 in d[2], the bullet norm / keys and values in bul_n / bul_inv / kvb, and what
// mlp_fwd leaves; writes y when y is given.
void spatial_fwd(const Ctx& c, const BnbSpatialWeights& w, const float* x, const uint8_t* alive, const BnbBullets* bul,
                 float* y, int G, int NM) {
  const int D = c.D;
  const size_t R = (size_t)G * NM;
  const int M = (int)R;
  const Bufs& b = c.b;
  float *n1 = b.d[0], *o = b.d[1], *x1 = b.d[2], *qkv = b.w3[0];
  const bool reads = bul && w.kv_bullet_w;
  const int nb = reads ? bul->per_env : 0;
  const size_t RB = (size_t)G * nb;
  rmsnorm_fwd(c, x, w.norm1_w, n1, b.inv[0], R);
  mmh(c, NT, H_A, n1, D, w.qkv_w, D, qkv, 3 * D, M, 3 * D, D);
  if (reads) {
    rmsnorm_fwd(c, bul->tokens, w.norm_bullet_w, b.bul_n, b.bul_inv, RB);
    mmh(c, NT, H_A, b.bul_n, D, w.kv_bullet_w, D, b.kvb, 2 * D, (int)RB, 2 * D, D);
  }
  attn_fwd(c, qkv, alive, o, G, NM, reads ? b.kvb : nullptr, reads ? bul->active : nullptr, nb);
  mm(c, NT, o, D, w.out_w, D, x1, D, M, D, D, nullptr, x, D);            // x1 = x + o Wout^T
  mlp_fwd(c, x1, y, R, w.norm2_w, w.gate_w, w.up_w, w.down_w);
}

int spatial_bwd(const Ctx& c, const BnbSpatialWeights& w, const BnbSpatialGrads& dw, const float* x, const uint8_t* alive,
                const BnbBullets* bul, float* d_bullets, const float* dy, float* dx, int G, int NM, bool have_fwd) {
  const int D = c.D;
  const size_t R = (size_t)G * NM;
  const int M = (int)R;
  const Bufs& b = c.b;
  float *n1 = b.d[0], *o = b.d[1], *x1 = b.d[2], *dx1 = b.d[3], *d_o = b.d[4], *dn1 = b.d[5];
  float *qkv = b.w3[0], *dqkv = b.w3[1];
  const bool reads = bul && w.kv_bullet_w;
  const int nb = reads ? bul->per_env : 0;
  const size_t RB = (size_t)G * nb;
  if (reads && (!dw.kv_bullet_w || !dw.norm_bullet_w)) return BNB_ERR_NULL_POINTER;

  if (!have_fwd) spatial_fwd(c, w, x, alive, bul, nullptr, G, NM);
  mlp_bwd(c, x1, dy, dx1, R, w.norm2_w, w.gate_w, w.up_w, w.down_w, dw.norm2_w, dw.gate_w, dw.up_w, dw.down_w);

  mm(c, TN, dx1, D, o, D, dw.out_w, D, D, D, M);
  mm(c, NN, dx1, D, w.out_w, D, d_o, D, M, D, D);
  const int dh = D / c.H;
  const float scale = 1.0f / sqrtf((float)dh);
  AttnBwdArgs self{qkv, 3 * D, qkv + D, 3 * D, D, alive, d_o, D, dqkv, 3 * D, 0, dqkv + D, 3 * D, D, NM, NM, dh, scale, 0};
  int rc = attn_bwd(c, self, G);
  if (rc) return rc;
  if (reads) {
    AttnBwdArgs cross{qkv, 3 * D, b.kvb, 2 * D, D, bul->active, d_o, D, dqkv, 3 * D, 1, b.dkvb, 2 * D, D, NM, nb, dh, scale,
                      bul->active ? 1 : 0};
    rc = attn_bwd(c, cross, G);
    if (rc) return rc;
    mmh(c, TN, H_B, b.dkvb, 2 * D, b.bul_n, D, dw.kv_bullet_w, D, 2 * D, D, (int)RB);
    mm(c, NN, b.dkvb, 2 * D, w.kv_bullet_w, D, b.bul_dn, D, (int)RB, D, 2 * D);
    // the bullet tokens feed every sublayer that reads them: their gradient accumulates
    float* sink = d_bullets ? d_bullets : b.bul_n;   // bul_n is free once the weight gradient above is queued
    rmsnorm_bwd(c, bul->tokens, w.norm_bullet_w, b.bul_inv, b.bul_dn, d_bullets, sink, dw.norm_bullet_w, RB);
  }
  mmh(c, TN, H_B, dqkv, 3 * D, n1, D, dw.qkv_w, D, 3 * D, D, M);
  mm(c, NN, dqkv, 3 * D, w.qkv_w, D, dn1, D, M, D, 3 * D);
  rmsnorm_bwd(c, x, w.norm1_w, b.inv[0], dn1, dx1, dx, dw.norm1_w, R);
  return BNB_OK;
}

void gather(const Ctx& c, const float* full, float* compact, size_t rows, int per_grp, int NM, int n0) {
  if (!rows) return;
  count_launch();
  k_gather_rows<<<blocks_for(rows * (c.D / 4), 256), 256, 0, c.st>>>(reinterpret_cast<const float4*>(full),
                                                                    reinterpret_cast<float4*>(compact), rows, c.D / 4,
                                                                    per_grp, NM, n0);
}
void scatter(const Ctx& c, const float* compact, float* full, size_t rows, int per_grp, int NM, int n0) {
  if (!rows) return;
  count_launch();
  k_scatter_rows<<<blocks_for(rows * (c.D / 4), 256), 256, 0, c.st>>>(reinterpret_cast<const float4*>(compact),
                                                                     reinterpret_cast<float4*>(full), rows, c.D / 4,
                                                                     per_grp, NM, n0);
}

struct TemporalGeom {
  int T, B, NM, n_rec;
  size_t Rs() const { return (size_t)T * B * n_rec; }
  size_t Rf() const { return (size_t)T * B * (NM - n_rec); }
};

// Recurrent path over the ship rows, forward part (griffin.py:249-286).  Buffers: xs d[0], n d[1],
// linear1 out d[2], conv out d[3], gate pre-activations d[4] d[5], states d[6], linear2 out d[7],
// gated branch d[8], x1 d[9]; with y, the sublayer's output goes to d[14] and from there to y's ship rows.
void ships_fwd(const Ctx& c, const BnbTemporalWeights& w, const float* x, const float* hid, const uint8_t* done, float* y,
               float* hid_out, const TemporalGeom& tg) {
  const int D = c.D;
  const Bufs& b = c.b;
  const size_t Rs = tg.Rs();
  const int M = (int)Rs, Rr = tg.B * tg.n_rec;
  ShipGeom gm{tg.T, Rr, D, tg.n_rec, tg.B, done};
  float *xs = b.d[0], *n = b.d[1], *b1 = b.d[2], *u = b.d[3], *za = b.d[4], *zx = b.d[5], *hs = b.d[6], *b2p = b.d[7],
        *m = b.d[8], *x1 = b.d[9];
  const int sblocks = (int)(((size_t)Rr * D + 255) / 256);
  gather(c, x, xs, Rs, tg.n_rec, tg.NM, 0);
  rmsnorm_fwd(c, xs, w.norm1_w, n, b.inv[0], Rs);
  mmh(c, NT, H_A, n, D, w.linear1_w, D, b1, D, M, D, D);
  count_launch();
  k_conv_fwd<<<sblocks, 256, 0, c.st>>>(b1, hid, w.conv_w, w.conv_b, u, gm);
  mm(c, NT, u, D, w.a_w, D, za, D, M, D, D, w.a_b);
  mm(c, NT, u, D, w.x_w, D, zx, D, M, D, D, w.x_b);
  count_launch();
  k_scan_fwd<<<sblocks, 256, 0, c.st>>>(za, zx, u, hid, w.log_lambda, hs, gm);
  if (hid_out) {
    count_launch();
    k_final_state<<<sblocks, 256, 0, c.st>>>(hs, b1, hid, hid_out, gm);
  }
  mmh(c, NT, H_A, n, D, w.linear2_w, D, b2p, D, M, D, D);
  gelu_mul_fwd(c, b2p, hs, m, Rs * D);                                  // m = h * gelu(linear2 n)
  mm(c, NT, m, D, w.out_w, D, x1, D, M, D, D, nullptr, xs, D);
  mlp_fwd(c, x1, y ? b.d[14] : nullptr, Rs, w.norm2_w, w.gate_w, w.up_w, w.down_w);
  if (y) scatter(c, b.d[14], y, Rs, tg.n_rec, tg.NM, 0);
}

// Non-recurrent path over the field rows (griffin.py:288-317).  Buffers: xf d[0], n d[1], linear1 out
// d[2], field_sub out d[3], linear2 out d[4], gated branch d[5], x1 d[6]; y as in ships_fwd.
void fields_fwd(const Ctx& c, const BnbTemporalWeights& w, const float* x, float* y, const TemporalGeom& tg) {
  const int D = c.D;
  const Bufs& b = c.b;
  const size_t Rf = tg.Rf();
  const int M = (int)Rf, nf = tg.NM - tg.n_rec;
  float *xf = b.d[0], *n = b.d[1], *c1 = b.d[2], *b1 = b.d[3], *b2p = b.d[4], *m = b.d[5], *x1 = b.d[6];
  gather(c, x, xf, Rf, nf, tg.NM, tg.n_rec);
  rmsnorm_fwd(c, xf, w.norm1_w, n, b.inv[0], Rf);
  mmh(c, NT, H_A, n, D, w.linear1_w, D, c1, D, M, D, D);
  mm(c, NT, c1, D, w.field_sub_w, D, b1, D, M, D, D);
  mmh(c, NT, H_A, n, D, w.linear2_w, D, b2p, D, M, D, D);
  gelu_mul_fwd(c, b2p, b1, m, Rf * D);
  mm(c, NT, m, D, w.out_w, D, x1, D, M, D, D, nullptr, xf, D);
  mlp_fwd(c, x1, y ? b.d[14] : nullptr, Rf, w.norm2_w, w.gate_w, w.up_w, w.down_w);
  if (y) scatter(c, b.d[14], y, Rf, nf, tg.NM, tg.n_rec);
}

int temporal_fwd(const Ctx& cs, const Ctx& cf, const BnbTemporalWeights& w, const float* x, const float* hid,
                 const uint8_t* done, float* y, float* hid_out, const TemporalGeom& tg) {
  if (tg.Rs()) ships_fwd(cs, w, x, hid, done, y, hid_out, tg);
  if (tg.Rf()) {
    if (!w.field_sub_w) return BNB_ERR_NULL_POINTER;
    fields_fwd(cf, w, x, y, tg);
  }
  return BNB_OK;
}

// One temporal sublayer: the recurrent path over the ship rows, the non-recurrent one over the
// field rows, both sharing every parameter but field_sub.
int temporal_bwd(const Ctx& cs, const Ctx& cf, const BnbTemporalWeights& w, const BnbTemporalGrads& dw, const float* x,
                 const float* hid, const float* d_hid_out, float* d_hid_in, const uint8_t* done, const float* dy, float* dx,
                 const TemporalGeom& tg, bool have_fwd) {
  const int D = cs.D;
  const size_t Rs = tg.Rs(), Rf = tg.Rf();
  if (Rs) {
    const Ctx& c = cs;
    const Bufs& b = c.b;
    const int M = (int)Rs, Rr = tg.B * tg.n_rec;
    ShipGeom gm{tg.T, Rr, D, tg.n_rec, tg.B, done};
    float *xs = b.d[0], *n = b.d[1], *b1 = b.d[2], *u = b.d[3], *za = b.d[4], *zx = b.d[5], *hs = b.d[6], *b2p = b.d[7],
          *m = b.d[8], *x1 = b.d[9], *dys = b.d[10], *dx1 = b.d[11], *dm = b.d[12], *dn = b.d[13], *dxs = b.d[14];
    const int sblocks = (int)(((size_t)Rr * D + 255) / 256);
    if (!have_fwd) ships_fwd(c, w, x, hid, done, nullptr, nullptr, tg);
    gather(c, dy, dys, Rs, tg.n_rec, tg.NM, 0);
    mlp_bwd(c, x1, dys, dx1, Rs, w.norm2_w, w.gate_w, w.up_w, w.down_w, dw.norm2_w, dw.gate_w, dw.up_w, dw.down_w);

    mm(c, TN, dx1, D, m, D, dw.out_w, D, D, D, M);
    mm(c, NN, dx1, D, w.out_w, D, dm, D, M, D, D);
    gelu_mul_bwd(c, b2p, hs, dm, b2p, dm, Rs * D);                      // b2p <- d linear2 out, dm <- d h
    mmh(c, TN, H_B, b2p, D, n, D, dw.linear2_w, D, D, D, M);
    mm(c, NN, b2p, D, w.linear2_w, D, dn, D, M, D, D);
    count_launch();
    k_scan_bwd<<<sblocks, 256, 0, c.st>>>(za, zx, u, hs, dm, hid, d_hid_out, d_hid_in, w.log_lambda, dw.log_lambda, gm);
    // za, zx hold d za, d zx; dm the direct part of d u
    mm(c, TN, za, D, u, D, dw.a_w, D, D, D, M);
    mm(c, TN, zx, D, u, D, dw.x_w, D, D, D, M);
    colsum(c, za, dw.a_b, Rs, D);
    colsum(c, zx, dw.x_b, Rs, D);
    mm(c, NN, za, D, w.a_w, D, dm, D, M, D, D, nullptr, nullptr, 0, 1);
    mm(c, NN, zx, D, w.x_w, D, dm, D, M, D, D, nullptr, nullptr, 0, 1);
    float* db1 = za;   // free now
    count_launch();
    k_conv_bwd<<<sblocks, 256, 0, c.st>>>(dm, b1, hid, d_hid_out, d_hid_in, w.conv_w, db1, dw.conv_w, dw.conv_b, gm);
    mmh(c, TN, H_B, db1, D, n, D, dw.linear1_w, D, D, D, M);
    mm(c, NN, db1, D, w.linear1_w, D, dn, D, M, D, D, nullptr, nullptr, 0, 1);
    rmsnorm_bwd(c, xs, w.norm1_w, b.inv[0], dn, dx1, dxs, dw.norm1_w, Rs);
    scatter(c, dxs, dx, Rs, tg.n_rec, tg.NM, 0);
  }
  if (Rf) {
    const Ctx& c = cf;
    const Bufs& b = c.b;
    if (!w.field_sub_w || !dw.field_sub_w) return BNB_ERR_NULL_POINTER;
    const int M = (int)Rf, nf = tg.NM - tg.n_rec;
    float *xf = b.d[0], *n = b.d[1], *c1 = b.d[2], *b1 = b.d[3], *b2p = b.d[4], *m = b.d[5], *x1 = b.d[6], *dyf = b.d[7],
          *dx1 = b.d[8], *dm = b.d[9], *dc1 = b.d[10], *dn = b.d[11], *dxf = b.d[12];
    if (!have_fwd) fields_fwd(c, w, x, nullptr, tg);
    gather(c, dy, dyf, Rf, nf, tg.NM, tg.n_rec);
    mlp_bwd(c, x1, dyf, dx1, Rf, w.norm2_w, w.gate_w, w.up_w, w.down_w, dw.norm2_w, dw.gate_w, dw.up_w, dw.down_w);

    mm(c, TN, dx1, D, m, D, dw.out_w, D, D, D, M);
    mm(c, NN, dx1, D, w.out_w, D, dm, D, M, D, D);
    gelu_mul_bwd(c, b2p, b1, dm, b2p, dm, Rf * D);                      // b2p <- d linear2 out, dm <- d b1
    mm(c, TN, dm, D, c1, D, dw.field_sub_w, D, D, D, M);
    mm(c, NN, dm, D, w.field_sub_w, D, dc1, D, M, D, D);
    mmh(c, TN, H_B, dc1, D, n, D, dw.linear1_w, D, D, D, M);
    mm(c, NN, dc1, D, w.linear1_w, D, dn, D, M, D, D);
    mmh(c, TN, H_B, b2p, D, n, D, dw.linear2_w, D, D, D, M);
    mm(c, NN, b2p, D, w.linear2_w, D, dn, D, M, D, D, nullptr, nullptr, 0, 1);
    rmsnorm_bwd(c, xf, w.norm1_w, b.inv[0], dn, dx1, dxf, dw.norm1_w, Rf);
    scatter(c, dxf, dx, Rf, nf, tg.NM, tg.n_rec);
  }
  return BNB_OK;
}

bool dims_ok(int D, int H) {
  if (D <= 0 || D > MAXW || D % 32 != 0 || H <= 0 || D % H != 0) return false;
  const int dh = D / H;
  return dh == 8 || dh == 16 || dh == 32;
}

// Everything both entry points derive from the call's geometry, and the walk over the sublayers
// that hands each path its buffers: from the shared scratch, or (kept activations) from the arena
// the training forward filled.
struct Walk {
  int D, T, B, NM, n_rec, G, S, nb;
  size_t R, RB, Rr;
  TemporalGeom tgm;
};

int make_walk(Walk& wk, int n_blocks, int n_spatial, int n_temporal, int D, int H, const BnbBatch& bt, int T,
              const BnbBullets* bullets) {
  if (bt.tok_off || bt.ship_off) return BNB_ERR_UNSUPPORTED_DIMS;   // environments of one size only
  if (!dims_ok(D, H)) return BNB_ERR_UNSUPPORTED_DIMS;
  wk.D = D; wk.T = T; wk.B = bt.n_envs; wk.NM = bt.tokens_per_env; wk.n_rec = bt.ships_per_env;
  if (T < 1 || wk.B < 0 || wk.NM < 1 || wk.n_rec < 0 || wk.n_rec > wk.NM) return BNB_ERR_BAD_ARGUMENT;
  wk.G = T * wk.B;
  wk.R = (size_t)wk.G * wk.NM;
  if (wk.R > (size_t)INT32_MAX / 2) return BNB_ERR_TOO_MANY_TOKENS;
  wk.S = n_blocks * (n_spatial + n_temporal);
  if (wk.S > 256) return BNB_ERR_BAD_ARGUMENT;
  wk.nb = bullets ? bullets->per_env : 0;
  wk.RB = (size_t)wk.G * wk.nb;
  wk.Rr = (size_t)wk.B * wk.n_rec;
  wk.tgm = TemporalGeom{T, wk.B, wk.NM, wk.n_rec};
  return BNB_OK;
}

// Layout of the kept activations: the outputs of sublayers 0 .. S-2, then per sublayer the buffers
// of bind_forward (a temporal sublayer: ships, then fields).
struct Kept {
  float* bound = nullptr;
  Bufs first[256], second[256];   // spatial or ships | fields
};

void layout_kept(Arena& ar, Kept& k, const Walk& wk, int n_blocks, int n_spatial, int n_temporal, const Bufs& shared,
                 bool half_mlp) {
  k.bound = ar.take((size_t)(wk.S > 1 ? wk.S - 1 : 0) * wk.R * wk.D);
  int s = 0;
  for (int blk = 0; blk < n_blocks; ++blk) {
    for (int j = 0; j < n_spatial; ++j, ++s) {
      k.first[s] = shared;
      bind_forward(ar, k.first[s], P_SPATIAL, wk.R, wk.D, wk.RB, half_mlp);
    }
    for (int j = 0; j < n_temporal; ++j, ++s) {
      k.first[s] = shared;
      k.second[s] = shared;
      bind_forward(ar, k.first[s], P_SHIPS, wk.tgm.Rs(), wk.D, 0, half_mlp);
      bind_forward(ar, k.second[s], P_FIELDS, wk.tgm.Rf(), wk.D, 0, half_mlp);
    }
  }
}

}  // namespace

void linear_nt(const float* x, const float* W, float* y, int M, int N, int K, bool bf16_operands, cudaStream_t st) {
  gemm(NT, x, K, W, K, y, N, M, N, K, nullptr, nullptr, 0, 0, st, bf16_operands);
}

size_t scratch_bytes(int n_blocks, int n_spatial, int n_temporal, int D, const BnbBatch& bt, int T, int bullets_per_env,
                     bool bf16) {
  Arena ar{nullptr};
  Bufs b;
  const int S = n_blocks * (n_spatial + n_temporal);
  const size_t G = (size_t)T * bt.n_envs;
  plan(ar, b, S, G * bt.tokens_per_env, D, G * (bullets_per_env > 0 ? bullets_per_env : 0), bf16);
  return ar.off + 256;
}

size_t kept_bytes(int n_blocks, int n_spatial, int n_temporal, int D, int H, const BnbBatch& bt, int T, int bullets_per_env,
                  bool bf16) {
  Walk wk;
  BnbBullets bul{nullptr, nullptr, bullets_per_env};
  if (make_walk(wk, n_blocks, n_spatial, n_temporal, D, H, bt, T, bullets_per_env > 0 ? &bul : nullptr)) return 0;
  Arena ar{nullptr};
  static thread_local Kept k;
  layout_kept(ar, k, wk, n_blocks, n_spatial, n_temporal, Bufs{}, bf16);
  return ar.off + 256;
}

namespace {

// Shared scratch and, when given, the kept-activation arena of a call.
int open_buffers(Ctx& c, Kept* kept, const Walk& wk, int n_blocks, int n_spatial, int n_temporal, void* scratch,
                 size_t scratch_bytes, void* kept_ptr, size_t kept_size) {
  uintptr_t base = (reinterpret_cast<uintptr_t>(scratch) + 255) & ~(uintptr_t)255;
  Arena ar{reinterpret_cast<char*>(base)};
  plan(ar, c.b, kept_ptr ? 0 : wk.S, wk.R, wk.D, wk.RB, c.bf16);
  if (ar.off + (base - reinterpret_cast<uintptr_t>(scratch)) > scratch_bytes) return BNB_ERR_SCRATCH_TOO_SMALL;
  if (kept_ptr) {
    uintptr_t kb = (reinterpret_cast<uintptr_t>(kept_ptr) + 255) & ~(uintptr_t)255;
    Arena ka{reinterpret_cast<char*>(kb)};
    layout_kept(ka, *kept, wk, n_blocks, n_spatial, n_temporal, c.b, c.bf16);
    if (ka.off + (kb - reinterpret_cast<uintptr_t>(kept_ptr)) > kept_size) return BNB_ERR_SCRATCH_TOO_SMALL;
  }
  return BNB_OK;
}

}  // namespace

// The forward of a call that will be differentiated: the same sublayer forward parts the backward
// recomputes from, run once with every path's intermediates written to `kept`, plus the trunk's
// output and final state.
int trunk_sequence_fwd_train(const TrunkFwdTrainArgs& a) {
  Walk wk;
  int rc = make_walk(wk, a.n_blocks, a.n_spatial, a.n_temporal, a.D, a.H, *a.batch, a.T, a.bullets);
  if (rc) return rc;
  if (wk.R == 0) return BNB_OK;
  const int D = wk.D;
  Ctx c;
  c.D = D; c.H = a.H; c.bf16 = a.bf16_products; c.st = a.stream;
  static thread_local Kept kept;
  if ((rc = open_buffers(c, &kept, wk, a.n_blocks, a.n_spatial, a.n_temporal, a.scratch, a.scratch_bytes, a.kept, a.kept_bytes)))
    return rc;
  if (wk.S == 0) {
    cudaMemcpyAsync(a.y, a.x, wk.R * D * sizeof(float), cudaMemcpyDeviceToDevice, a.stream);
    return BNB_OK;
  }
  const float* cur = a.x;
  int s = 0;
  for (int blk = 0; blk < a.n_blocks; ++blk) {
    for (int j = 0; j < a.n_spatial; ++j, ++s) {
      float* out = s + 1 == wk.S ? a.y : kept.bound + (size_t)s * wk.R * D;
      Ctx cs = c;
      cs.b = kept.first[s];
      spatial_fwd(cs, a.spatial[blk * a.n_spatial + j], cur, a.alive, a.bullets, out, wk.G, wk.NM);
      cur = out;
    }
    for (int j = 0; j < a.n_temporal; ++j, ++s) {
      float* out = s + 1 == wk.S ? a.y : kept.bound + (size_t)s * wk.R * D;
      const int slot = blk * a.n_temporal + j;
      const size_t hoff = (size_t)slot * wk.Rr * 4 * D;
      Ctx cs = c, cf = c;
      cs.b = kept.first[s];
      cf.b = kept.second[s];
      rc = temporal_fwd(cs, cf, a.temporal[slot], cur, a.hidden_in + hoff, a.done, out,
                        a.hidden_out ? a.hidden_out + hoff : nullptr, wk.tgm);
      if (rc) return rc;
      cur = out;
    }
  }
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

int trunk_sequence_bwd(const TrunkBwdArgs& a) {
  Walk wk;
  int rc = make_walk(wk, a.n_blocks, a.n_spatial, a.n_temporal, a.D, a.H, *a.batch, a.T, a.bullets);
  if (rc) return rc;
  if (wk.R == 0) return BNB_OK;
  const int D = wk.D, S = wk.S, G = wk.G, NM = wk.NM;
  const size_t R = wk.R, Rr = wk.Rr;
  cudaStream_t st = a.stream;
  Ctx c;
  c.D = D; c.H = a.H; c.bf16 = a.bf16_products; c.st = st;
  static thread_local Kept kept;
  const bool have_fwd = a.kept != nullptr;
  if ((rc = open_buffers(c, &kept, wk, a.n_blocks, a.n_spatial, a.n_temporal, a.scratch, a.scratch_bytes, a.kept, a.kept_bytes)))
    return rc;

  if (S == 0) {
    cudaMemcpyAsync(a.dx, a.dy, R * D * sizeof(float), cudaMemcpyDeviceToDevice, st);
    return BNB_OK;
  }

  // the input of every sublayer: kept by the training forward, or from a first pass here
  const float* inputs[256];
  if (have_fwd) {
    for (int s = 0; s < S; ++s) inputs[s] = s == 0 ? a.x : kept.bound + (size_t)(s - 1) * R * D;
  } else {
    const float* cur = a.x;
    int s = 0;
    for (int blk = 0; blk < a.n_blocks; ++blk) {
      for (int j = 0; j < a.n_spatial; ++j, ++s) {
        inputs[s] = cur;
        if (s + 1 == S) break;
        float* out = c.b.bound + (size_t)s * R * D;
        spatial_fwd(c, a.spatial[blk * a.n_spatial + j], cur, a.alive, a.bullets, out, G, NM);
        cur = out;
      }
      for (int j = 0; j < a.n_temporal; ++j, ++s) {
        inputs[s] = cur;
        if (s + 1 == S) break;
        float* out = c.b.bound + (size_t)s * R * D;
        const int slot = blk * a.n_temporal + j;
        rc = temporal_fwd(c, c, a.temporal[slot], cur, a.hidden_in + (size_t)slot * Rr * 4 * D, a.done, out, nullptr, wk.tgm);
        if (rc) return rc;
        cur = out;
      }
    }
  }

  if (a.d_bullets && wk.RB) cudaMemsetAsync(a.d_bullets, 0, wk.RB * D * sizeof(float), st);

  // sublayers in reverse
  const float* dcur = a.dy;
  for (int blk = a.n_blocks - 1; blk >= 0; --blk) {
    for (int j = a.n_temporal - 1; j >= 0; --j) {
      const int s = blk * (a.n_spatial + a.n_temporal) + a.n_spatial + j;
      float* dout = s == 0 ? a.dx : c.b.ping[s & 1];
      const int slot = blk * a.n_temporal + j;
      const size_t hoff = (size_t)slot * Rr * 4 * D;
      Ctx cs = c, cf = c;
      if (have_fwd) {
        cs.b = kept.first[s];
        cf.b = kept.second[s];
      }
      rc = temporal_bwd(cs, cf, a.temporal[slot], a.d_temporal[slot], inputs[s], a.hidden_in + hoff,
                        a.d_hidden_out ? a.d_hidden_out + hoff : nullptr, a.d_hidden_in ? a.d_hidden_in + hoff : nullptr,
                        a.done, dcur, dout, wk.tgm, have_fwd);
      if (rc) return rc;
      dcur = dout;
    }
    for (int j = a.n_spatial - 1; j >= 0; --j) {
      const int s = blk * (a.n_spatial + a.n_temporal) + j;
      float* dout = s == 0 ? a.dx : c.b.ping[s & 1];
      const int k = blk * a.n_spatial + j;
      Ctx cs = c;
      if (have_fwd) cs.b = kept.first[s];
      rc = spatial_bwd(cs, a.spatial[k], a.d_spatial[k], inputs[s], a.alive, a.bullets, a.d_bullets, dcur, dout, G, NM,
                       have_fwd);
      if (rc) return rc;
      dcur = dout;
    }
  }
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

}  // namespace grad
}  // namespace bnb
