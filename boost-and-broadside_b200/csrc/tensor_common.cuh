// Shared pieces of the tensor-core trunk kernels (sm_100a): the sublayer program a launch
// runs, the layout constants of the packed weight image, and the inline-PTX wrappers
// (tcgen05 / mbarrier / bulk copy / ldmatrix / mma.sync) both tile kernels are written with.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "common.cuh"

namespace bnb {
namespace tensor {

constexpr int D = 128;
constexpr int HEADS = 4;
constexpr int DH = 32;
constexpr int TILE = 128;
constexpr int CHUNK_BYTES = 16384;       // one weight chunk: up to 128 rows x 64 bf16
constexpr int N_SPATIAL_CHUNKS = 34;       // chunks of a spatial sublayer proper
constexpr int N_BULLET_CHUNKS = 4;         // kv_bullet: keys (2 K atoms), values (2 K atoms); zero when absent
constexpr int N_SPATIAL_IMAGE = N_SPATIAL_CHUNKS + N_BULLET_CHUNKS;
constexpr int N_TEMPORAL_CHUNKS = 36;
constexpr int STAGE_STRIDE = 208;        // bytes per staged q|k|v row (96 bf16 + pad)
constexpr int MAX_SUBLAYERS = 8;

// shared memory map (offsets from a 1024-aligned base)
constexpr int OFF_A = 0;                 // 32 KB
constexpr int OFF_P = 32768;             // 16 KB
constexpr int OFF_RING = 49152;          // 2 x 16 KB
constexpr int OFF_STAGE = 81920;         // 128 x 208 = 26624
constexpr int OFF_META = 108544;         // env_first[128], env_n[128], alive[128], items[128]
constexpr int OFF_BAR = 109056;          // full[2], empty[2], acc, tmem base
constexpr int OFF_SS = 109120;           // partial sums of squares, up to 4 x 128 floats
constexpr int OFF_ROWINFO = 111168;      // hidden row of each tile row (int, -1 = no state), then flags
constexpr int SMEM_BYTES = 111168 + 512 + 128 + 1024;

constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t COL_RESID = 0;
constexpr uint32_t COL_ACC = 128;

// SUB_SPATIAL_PRE / _POST split a spatial sublayer around a separate attention kernel
// (environments larger than one tile): PRE = norm1 + QKV to global scratch, POST = attention
// output from scratch + out_proj + norm2 + GatedMLP.
// SUB_BULLET_KV runs over bullet rows instead of token rows: norm_bullet + kv_bullet, keys and
// values written as bf16 to global scratch for the attention kernel; it leaves no residual.
enum : int { SUB_SPATIAL = 0, SUB_TEMPORAL = 1, SUB_SPATIAL_PRE = 2, SUB_SPATIAL_POST = 3, SUB_BULLET_KV = 4 };
enum : int { ST_TIMEOUT_FULL = 101, ST_TIMEOUT_EMPTY = 102, ST_TIMEOUT_ACC = 103 };

struct SubLayer {
  int type;
  const uint8_t* packed;
  const float* conv_w;
  const float* conv_b;
  const float* a_b;
  const float* x_b;
  const float* decay_log2;   // 8 * log2(sigmoid(log_lambda)), written by the pack kernel
  const float* hid_in;
  float* hid_out;
  __nv_bfloat16* qkv_out;        // PRE: (rows, 384) q|k|v, head-major inside each third
  const __nv_bfloat16* o_in;     // POST: (rows, 128) attention output
  __nv_bfloat16* kvb_out;        // BULLET_KV: (rows, 256) k | v of the bullet rows
};

struct TrunkArgs {
  const float* x;
  float* y;
  const uint8_t* alive;
  const uint8_t* done;
  const uint8_t* reset_env;
  EnvMap map;
  int n_groups;       // replication of the batch for the spatial fold (T for a sequence)
  int t_loop;         // timesteps walked inside the kernel (temporal programs of a sequence)
  int n_sub;
  int n_tiles;
  int envs_per_tile;
  int env_tiles;      // tiles per group
  int has_fields;
  int flat_rows;      // 1: tiles are plain 128-row slices of the token rows (no attention inside)
  const int* tile_env_begin;  // ragged batches: range of each tile in tile_env_ids (+ end), else null
  const int* tile_env_ids;    // ragged batches: environments in tile order
  // Bullet key/value program only: tile row r reads input row row_index[r], and only the first
  // *n_rows_dev rows exist (the active bullets, compacted on the device); null = all rows, in order.
  const int* row_index;
  const int* n_rows_dev;
  int* status;
  // Test hooks of the bounded waits (0 / -1 in normal use): the poll limit of this launch, and the
  // ring operation of CTA 0 whose weight copy the fetching lane leaves out, so that the issuing
  // lane's wait for it runs out and the kernel has to drain and return with a status code.
  int poll_limit;
  int skip_op;
  int io_bf16;   // x and y hold bfloat16 (BNB_BF16_IO) instead of float32
  SubLayer sub[MAX_SUBLAYERS];
};
// Process-wide values of the two hooks, set by bnb_debug_wait_test and copied into every launch.
extern int g_debug_poll_limit;
extern int g_debug_skip_op;

// ------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after a number of polls, records `code` in the status word and lets the
// caller go on.  `aborted` points at two shared ints: [0] is set once any wait of the CTA has run
// out (later waits then give up after four polls, so the kernel drains quickly), [1] is the poll
// limit of this launch.
constexpr int DEFAULT_POLL_LIMIT = 1 << 20;
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int* status, volatile int* aborted, int code) {
  if (mbar_try_wait(bar, parity)) return;   // the common case costs one instruction
  const int limit = aborted[0] ? 4 : aborted[1];
  for (int i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return;
  *aborted = 1;
  atomicCAS(status, 0, code);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Named barriers of the epilogue threads (ids 1 and 2; id 0 is __syncthreads).
template <int NQ>
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(128 * NQ) : "memory"); }
template <int NQ>
__device__ __forceinline__ void wake_barrier() { asm volatile("bar.sync 2, %0;" ::"n"(128 * NQ) : "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, bf16 operands, fp32 accumulate, M = 128.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8_nowait(uint32_t taddr, uint32_t* v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr) : "memory");
}
// N consecutive columns of this thread's lane (N a multiple of 8, at most 64); no wait.
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[N]) {
  static_assert(N % 8 == 0 && N <= 64, "column count");
  int done = 0;
  if constexpr (N >= 32) {
    tmem_ld32_nowait(taddr, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
    done = 32;
    if constexpr (N >= 64) {
      tmem_ld32_nowait(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      done = 64;
    }
  }
  if constexpr ((N % 32) >= 16) {
    tmem_ld16_nowait(taddr + done, *reinterpret_cast<uint32_t(*)[16]>(&v[N - (N % 32)]));
    done += 16;
  }
  if constexpr ((N % 16) == 8) tmem_ld8_nowait(taddr + done, &v[N - 8]);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  tmem_ld32_nowait(taddr, v);
  tmem_wait_ld();
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// MUFU-based elementwise functions for the bf16 path.  Their results are rounded to bf16 (or
// feed products that are), so approximations a few 1e-4 relative are below the rounding.
__device__ __forceinline__ float tanh_fast(float v) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float ex2_fast(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float sqrt_fast(float v) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
// erf GeLU as 0.5 x (1 + tanh(x (c1 + c3 x^2 + c5 x^4))): the inner polynomial is a minimax
// fit to x * Phi(x) (max abs error 2.5e-5, max relative error 1.2e-3 where |gelu| > 1e-2).
__device__ __forceinline__ float gelu_fast(float v) {
  const float x2 = fminf(v * v, 100.0f);  // beyond |x| = 10 the polynomial stays positive and tanh saturates
  float p = fmaf(x2, -3.51516841e-4f, 3.70056464e-2f);
  p = fmaf(x2, p, 7.97507884e-1f);
  const float t = tanh_fast(v * p);
  const float h = 0.5f * v;
  return fmaf(h, t, h);
}
// gelu(g) * u for two elements at once in half precision (11 mantissa bits against the 8 of the
// bf16 result), packed as two bf16: one tanh.approx.f16x2 and about half the instructions of two
// float evaluations.  g * g saturates at 100 as in gelu_fast (an overflow to inf lands there too).
__device__ __forceinline__ uint32_t gelu_mul_bf16x2(float g0, float g1, float u0, float u1) {
  const __half2 g = __floats2half2_rn(g0, g1);
  const __half2 u = __floats2half2_rn(u0, u1);
  const __half2 x2 = __hmin2(__hmul2(g, g), __float2half2_rn(100.0f));
  __half2 p = __hfma2(x2, __float2half2_rn(-3.51516841e-4f), __float2half2_rn(3.70056464e-2f));
  p = __hfma2(x2, p, __float2half2_rn(7.97507884e-1f));
  const __half2 a = __hmul2(g, p);
  uint32_t ti, to;
  ti = *reinterpret_cast<const uint32_t*>(&a);
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(to) : "r"(ti));
  const __half2 t = *reinterpret_cast<const __half2*>(&to);
  const __half2 h = __hmul2(g, __float2half2_rn(0.5f));
  const __half2 r = __hmul2(__hfma2(h, t, h), u);
  const float2 f = __half22float2(r);
  return pack_bf16(f.x, f.y);
}
__device__ __forceinline__ float sigmoid_fast(float v) { return fmaf(0.5f, tanh_fast(0.5f * v), 0.5f); }

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// Byte offset of the 16-byte group holding columns [8*c8, 8*c8+8) of row r inside a
// 128-row x 64-column bf16 atom with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(int r, int c8) { return (uint32_t)(r * 128 + ((c8 ^ (r & 7)) << 4)); }

// The fused one-CTA-per-SM kernel (pipelined_tile_kernel.cu): programs of whole-environment tiles
// made of SUB_SPATIAL and SUB_TEMPORAL sublayers only.
int launch_pipelined(const TrunkArgs& a, cudaStream_t st);

}  // namespace tensor
}  // namespace bnb
