// Tensor-core trunk kernels for sm_100a: tcgen05.mma (bf16 x bf16 -> fp32 in TMEM) for every
// projection, mma.sync for the tiny per-environment attention problems, bulk async copies
// (cp.async.bulk + mbarrier) for the pre-tiled weight stream.
//
// One CTA owns one tile of 128 token rows made of whole environments and walks it through
// a program of sublayers (S = spatial, T = temporal) with the residual stream resident in
// tensor memory:
//
//   TMEM columns [0,128)    residual stream, fp32, lane = tile row.  out_proj, linear_out and
//                           down_proj accumulate straight into it (x + W h with one rounding
//                           instead of bf16(W h) + x: closer to the float32 result than the
//                           autocast reference, well inside the bf16 tolerance).
//   TMEM columns [128,256)  projection accumulators (q|k|v of one head, gate|up chunk, ...).
//
//   shared memory           A operand 128x128 bf16 (two 64-wide swizzled K atoms), second
//                           operand 128x64 bf16, 2-slot ring of 16 KB weight chunks, q|k|v
//                           staging for the attention warps.
//
// 256 threads, two per tile row (TMEM lane = row, half of the columns each), do every epilogue;
// thread 0 also issues the MMAs and the bulk copies of the weight stream.  Two CTAs fit one SM (256 TMEM
// columns, about 108 KB of shared memory each) so one CTA's epilogue overlaps the other's MMAs.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in the status
// word and the kernel drains without hanging.
//
// Reference arithmetic: models/yemong/attention.py:76-169, models/yemong/griffin.py:67-317.
#include "bullet_slices.h"
#include "tensor_kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "launch_count.h"

#include "tensor_common.cuh"

namespace bnb {
namespace tensor {

int g_debug_poll_limit = 0;
int g_debug_skip_op = -1;

// ------------------------------------------------------------------ weight image

// Source of row `r` (0..127) of chunk `c` of a sublayer image: pointer to 64 consecutive
// floats, or nullptr for a zero row.
__device__ __forceinline__ const float* ffn_chunk_row(int c, int r, const float* gate, const float* up, const float* down) {
  int cc = c / 3, i = c % 3;
  if (i < 2) return (r < 64 ? gate + (size_t)(64 * cc + r) * D : up + (size_t)(64 * cc + r - 64) * D) + i * 64;
  return down + (size_t)r * 4 * D + 64 * cc;
}
__device__ __forceinline__ const float* spatial_chunk_row(const BnbSpatialWeights& w, int c, int r) {
  if (c < 10) {
    int p = c / 5, i = c % 5;
    if (i < 4) {
      int h = 2 * p + i / 2, kh = i % 2;
      if (r >= 96) return nullptr;
      return w.qkv_w + (size_t)((r / 32) * D + h * DH + (r % 32)) * D + kh * 64;
    }
    return w.out_w + (size_t)r * D + 64 * p;
  }
  if (c >= N_SPATIAL_CHUNKS) {
    // kv_bullet (2D, D): rows 0..127 are the keys of all heads, 128..255 the values
    if (!w.kv_bullet_w) return nullptr;
    const int i = c - N_SPATIAL_CHUNKS;
    return w.kv_bullet_w + (size_t)((i >> 1) * D + r) * D + (i & 1) * 64;
  }
  return ffn_chunk_row(c - 10, r, w.gate_w, w.up_w, w.down_w);
}
__device__ __forceinline__ const float* temporal_chunk_row(const BnbTemporalWeights& w, int c, int r) {
  int kh = c & 1;
  switch (c >> 1) {
    case 0: return w.linear2_w + (size_t)r * D + kh * 64;
    case 1: return w.linear1_w + (size_t)r * D + kh * 64;
    case 2: return (r < 64 ? w.a_w + (size_t)r * D : w.x_w + (size_t)(r - 64) * D) + kh * 64;
    case 3: return (r < 64 ? w.a_w + (size_t)(64 + r) * D : w.x_w + (size_t)r * D) + kh * 64;
    case 4: return w.field_sub_w ? w.field_sub_w + (size_t)r * D + kh * 64 : nullptr;
    case 5: return w.out_w + (size_t)r * D + kh * 64;
    default: return ffn_chunk_row(c - 12, r, w.gate_w, w.up_w, w.down_w);
  }
}

// RMSNorm gain folded into chunk `c`: the 64 gains of the chunk's K columns when the chunk's
// input is a normed activation, else nullptr.  The kernels then feed x * rsqrt(mean x^2 + eps)
// without the gain, and the products see W[n][k] * g[k] rounded to bf16 once.
__device__ __forceinline__ const float* spatial_chunk_gain(const BnbSpatialWeights& w, int c) {
  if (c < 10) { const int i = c % 5; return i < 4 ? w.norm1_w + (i % 2) * 64 : nullptr; }
  if (c >= N_SPATIAL_CHUNKS) return w.norm_bullet_w ? w.norm_bullet_w + ((c - N_SPATIAL_CHUNKS) & 1) * 64 : nullptr;
  const int i = (c - 10) % 3;
  return i < 2 ? w.norm2_w + i * 64 : nullptr;
}
__device__ __forceinline__ const float* temporal_chunk_gain(const BnbTemporalWeights& w, int c) {
  if (c < 4) return w.norm1_w + (c & 1) * 64;        // linear2, linear1
  if (c < 12) return nullptr;                         // gates, field_sub, linear_out: not fed by a norm
  const int i = (c - 12) % 3;
  return i < 2 ? w.norm2_w + i * 64 : nullptr;
}

template <class W, class F, class G>
__device__ __forceinline__ void pack_image(const W& w, int n_chunks, uint8_t* out, F row_of, G gain_of) {
  // one thread per 16-byte group: (chunk, row, group of 8 columns)
  const int total = n_chunks * TILE * 8;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    int c = i / (TILE * 8), r = (i / 8) % TILE, g = i % 8;
    const float* src = row_of(w, c, r);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (src) {
      float4 a = *reinterpret_cast<const float4*>(src + g * 8);
      float4 b = *reinterpret_cast<const float4*>(src + g * 8 + 4);
      if (const float* gain = gain_of(w, c)) {
        const float4 ga = *reinterpret_cast<const float4*>(gain + g * 8), gb = *reinterpret_cast<const float4*>(gain + g * 8 + 4);
        a.x *= ga.x; a.y *= ga.y; a.z *= ga.z; a.w *= ga.w;
        b.x *= gb.x; b.y *= gb.y; b.z *= gb.z; b.w *= gb.w;
      }
      v = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
    }
    *reinterpret_cast<uint4*>(out + (size_t)c * CHUNK_BYTES + swz(r, g)) = v;
  }
}
__global__ void k_pack_spatial(BnbSpatialWeights w, uint8_t* out) {
  pack_image(w, N_SPATIAL_IMAGE, out, [](const BnbSpatialWeights& ww, int c, int r) { return spatial_chunk_row(ww, c, r); },
             [](const BnbSpatialWeights& ww, int c) { return spatial_chunk_gain(ww, c); });
}
__global__ void k_pack_temporal(BnbTemporalWeights w, uint8_t* out) {
  if (blockIdx.x == 0 && threadIdx.x < D) {
    float sg = 1.0f / (1.0f + expf(-w.log_lambda[threadIdx.x]));
    reinterpret_cast<float*>(out + (size_t)N_TEMPORAL_CHUNKS * CHUNK_BYTES)[threadIdx.x] = kRglruC * log2f(sg);
  }
  pack_image(w, N_TEMPORAL_CHUNKS, out, [](const BnbTemporalWeights& ww, int c, int r) { return temporal_chunk_row(ww, c, r); },
             [](const BnbTemporalWeights& ww, int c) { return temporal_chunk_gain(ww, c); });
}

// Every image of a trunk in one launch: blockIdx.y selects the sublayer.
constexpr int MAX_PACK_JOBS = 8;
struct PackJobs {
  int n_spatial, n_temporal;
  BnbSpatialWeights sw[MAX_PACK_JOBS];
  BnbTemporalWeights tw[MAX_PACK_JOBS];
};
__global__ void k_pack_trunk(const __grid_constant__ PackJobs jobs) {
  const int j = blockIdx.y;
  if (j < jobs.n_spatial) {
    const BnbSpatialWeights& w = jobs.sw[j];
    pack_image(w, N_SPATIAL_IMAGE, static_cast<uint8_t*>(const_cast<void*>(w.packed)),
               [](const BnbSpatialWeights& ww, int c, int r) { return spatial_chunk_row(ww, c, r); },
               [](const BnbSpatialWeights& ww, int c) { return spatial_chunk_gain(ww, c); });
  } else {
    const BnbTemporalWeights& w = jobs.tw[j - jobs.n_spatial];
    uint8_t* out = static_cast<uint8_t*>(const_cast<void*>(w.packed));
    if (blockIdx.x == 0 && threadIdx.x < D) {
      float sg = 1.0f / (1.0f + expf(-w.log_lambda[threadIdx.x]));
      reinterpret_cast<float*>(out + (size_t)N_TEMPORAL_CHUNKS * CHUNK_BYTES)[threadIdx.x] = kRglruC * log2f(sg);
    }
    pack_image(w, N_TEMPORAL_CHUNKS, out, [](const BnbTemporalWeights& ww, int c, int r) { return temporal_chunk_row(ww, c, r); },
               [](const BnbTemporalWeights& ww, int c) { return temporal_chunk_gain(ww, c); });
  }
}

// ------------------------------------------------------------------ the tile kernel
//
// Thread layout: 256 epilogue threads, two per tile row.  Thread (row, half) owns TMEM lane
// `row` (warps w and w+4 both reach lanes 32*(w%4)..) and half of the columns of whatever is
// being read: K atom `half` of a 128-wide operand, 32 of the 64 columns of a gate|up chunk, ...

// Optional cycle accounting (compile with -DBNB_TIMING): thread 64 of every CTA adds up the
// cycles it spends in each phase and stores them behind the status word.
#ifdef BNB_TIMING
#define T_BEGIN(c) long long _t0 = clock64()
#define T_END(c, slot) (c).tacc[slot] += clock64() - _t0
#else
#define T_BEGIN(c)
#define T_END(c, slot)
#endif
enum : int { TM_WAIT = 0, TM_BARRIER, TM_NORM, TM_FFN_EPI, TM_QKV_EPI, TM_ATTN, TM_TEMPORAL_EPI, TM_IO, TM_TOTAL, TM_FULL_WAIT, TM_REFILL, TM_EXPECT, TM_BULK, TM_ISSUE, TM_COUNT };

struct Ctx {
#ifdef BNB_TIMING
  long long tacc[TM_COUNT];
#endif
  uint8_t* smem;
  uint32_t sA, sP, sRing, sStage;   // shared addresses
  uint32_t bar_full[3], bar_acc;
  uint32_t tmem;                    // base tensor-memory address
  uint32_t lane_addr;               // tmem + (row's lane << 16)
  int* status;
  volatile int* aborted;
  uint32_t acc_phase;
  int row;                          // tile row owned by this thread
  int part;                         // which slice of the columns (0 .. NQ-1)
  float* ss_part;                   // [NQ][128] partial sums of squares
  // Weight stream.  Three ring slots: two dedicated, the third is the q|k|v staging area,
  // which only the GatedMLP chunks use (attention is over by then).  Every call site knows
  // the slot of the chunk it consumes; the fetching thread walks a schedule table.
  uint32_t parity;                  // consumer (thread 0): per-slot phase bit of the full barrier
  int cons_count;                   // consumer: chunks consumed so far
  volatile int* s_cons;             // shared copy of cons_count, published before each commit
  const uint16_t* sched;            // fetcher: schedule of one pass over the sublayers
  int sched_len, p_idx, p_seq, p_left;
  int occ[3];                       // fetcher: sequence number of the chunk in each slot (-1 = none)
  const SubLayer* subs;             // sublayer table in shared memory
};

// The last warp fetches weights; thread 0 issues the MMAs.

__device__ __forceinline__ uint32_t slot_addr(const Ctx& c, uint32_t slot) {
  return slot < 2 ? c.sRing + slot * CHUNK_BYTES : c.sStage;
}
__device__ __forceinline__ uint32_t chunk_slot(int type, int ch) {
  if (type == SUB_TEMPORAL) return ch < 12 ? (uint32_t)(ch & 1) : (uint32_t)((ch - 12) % 3);
  if (type == SUB_BULLET_KV) return (uint32_t)(ch & 1);
  if (ch >= 10) return (uint32_t)((ch - 10) % 3);
  if (type == SUB_SPATIAL) return (uint32_t)(ch & 1);
  if (type == SUB_SPATIAL_PRE) return (uint32_t)((ch < 5 ? ch : ch - 1) & 1);  // q|k|v chunks only: K atom 0 -> slot 0
  return ch == 4 ? 0u : 1u;                                                    // POST: the two out_proj chunks
}
// Does a sublayer of `type` consume chunk `ch` of its weight image?
__device__ __forceinline__ bool chunk_used(int type, int ch, bool has_fields) {
  if (type == SUB_TEMPORAL) return has_fields || (ch != 8 && ch != 9);
  if (type == SUB_BULLET_KV) return ch >= N_SPATIAL_CHUNKS;
  if (ch >= N_SPATIAL_CHUNKS) return false;
  if (type == SUB_SPATIAL_PRE) return ch < 10 && ch != 4 && ch != 9;
  if (type == SUB_SPATIAL_POST) return ch == 4 || ch >= 9;
  return true;
}

// Fetching warp: bring the next chunks of the stream into every slot whose previous chunk has
// been retired.  Called right after the accumulator barrier, when all MMAs issued so far are
// complete, so a chunk with sequence number < *s_cons is retired.  The whole warp runs the
// bookkeeping (warp-uniform); lanes 0..2 each issue one of up to three copies.
__device__ __forceinline__ void refill(Ctx& c) {
  const int lane = threadIdx.x & 31;
  const int retired = *c.s_cons;
  // candidate of this lane: the lane-th next chunk of the schedule
  int idx = c.p_idx + lane;
  if (idx >= c.sched_len) idx -= c.sched_len;
  if (idx >= c.sched_len) idx -= c.sched_len;
  const bool in_range = lane < 3 && lane < c.p_left;
  const uint32_t e = c.sched[in_range ? idx : 0];
  const uint32_t slot = e & 3u;
  const int occ = slot == 0 ? c.occ[0] : (slot == 1 ? c.occ[1] : c.occ[2]);
  // a chunk may go out if its slot is free and no earlier chunk of this batch takes the same slot
  const uint32_t s0 = __shfl_sync(0xffffffffu, slot, 0), s1 = __shfl_sync(0xffffffffu, slot, 1);
  bool ok = in_range && occ < retired;
  if (lane == 1 && slot == s0) ok = false;
  if (lane == 2 && (slot == s0 || slot == s1)) ok = false;
  const uint32_t okmask = __ballot_sync(0xffffffffu, ok);
  const int n = (okmask & 1u) ? ((okmask & 2u) ? ((okmask & 4u) ? 3 : 2) : 1) : 0;  // leading run
  if (lane < n) {
    const SubLayer& s = c.subs[(e >> 2) & 15u];
    mbar_expect_tx(c.bar_full[slot], CHUNK_BYTES);
    bulk_g2s(slot_addr(c, slot), s.packed + (size_t)(e >> 6) * CHUNK_BYTES, CHUNK_BYTES, c.bar_full[slot]);
  }
#pragma unroll
  for (int l = 0; l < 3; ++l) {
    const uint32_t sl = __shfl_sync(0xffffffffu, slot, l);
    if (l < n) {
      if (sl == 0) c.occ[0] = c.p_seq + l; else if (sl == 1) c.occ[1] = c.p_seq + l; else c.occ[2] = c.p_seq + l;
    }
  }
  c.p_seq += n;
  c.p_left -= n;
  c.p_idx += n;
  if (c.p_idx >= c.sched_len) c.p_idx -= c.sched_len;
}

template <int NQ>
__device__ __forceinline__ void round_begin(Ctx& c) {
  T_BEGIN(c);
  fence_proxy_async();
  tc_fence_before();
  epi_barrier<NQ>();
  if (threadIdx.x == 0) tc_fence_after();
  T_END(c, TM_BARRIER);
}
// Thread 0: D[128 x n] (+)= A[128 x 64] * W[n x 64]^T with the next weight chunk of the stream,
// which the schedule placed in ring slot `slot`.
__device__ __forceinline__ void issue_chunk(Ctx& c, uint32_t a_addr, uint32_t n, uint32_t d_col, uint32_t accumulate, uint32_t slot) {
  {
    T_BEGIN(c);
    mbar_wait(c.bar_full[slot], (c.parity >> slot) & 1u, c.status, c.aborted, ST_TIMEOUT_FULL);
    T_END(c, TM_FULL_WAIT);
  }
  c.parity ^= 1u << slot;
  tc_fence_after();
  const uint32_t b_addr = slot_addr(c, slot);
  const uint32_t idesc = instr_desc(n);
  {
    T_BEGIN(c);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      tc_mma(c.tmem + d_col, smem_desc(a_addr + k * 32), smem_desc(b_addr + k * 32), idesc, (accumulate | (uint32_t)k) ? 1u : 0u);
    T_END(c, TM_ISSUE);
  }
  ++c.cons_count;
}
template <int NQ>
__device__ __forceinline__ void round_end(Ctx& c) {
  T_BEGIN(c);
  if (threadIdx.x == 0) {
    *c.s_cons = c.cons_count;
    __threadfence_block();
    tc_commit(c.bar_acc);
  }
  // Warp 0 polls the mbarrier; everybody else sleeps on a hardware barrier instead of spending
  // issue slots of the co-resident CTA on a spin loop.
  if (threadIdx.x < 32) {
    __syncwarp();
    mbar_wait(c.bar_acc, c.acc_phase, c.status, c.aborted, ST_TIMEOUT_ACC);
  }
  c.acc_phase ^= 1u;
  wake_barrier<NQ>();
  if ((threadIdx.x >> 5) == 4 * NQ - 1) {
    T_BEGIN(c);
    refill(c);
    T_END(c, TM_REFILL);
  }
  __syncwarp();
  tc_fence_after();
  T_END(c, TM_WAIT);
}

// Thread layout of the epilogues: NQ threads per tile row (2 or 4), thread (row, part) owns
// TMEM lane `row` and columns [part * 128/NQ, ...) of a 128-wide row, [part * 64/NQ, ...) of a
// 64-wide block and [part * 96/NQ, ...) of a q|k|v accumulator.

// residual (TMEM) -> x * rsqrt(mean x^2 + eps) -> bf16 A operand (the RMSNorm gain is in the weights)
template <int NQ>
__device__ __forceinline__ void norm_to_A(Ctx& c) {
  constexpr int CPT = 128 / NQ;
  T_BEGIN(c);
  uint32_t v[CPT];
  tmem_ld_cols<CPT>(c.lane_addr + COL_RESID + c.part * CPT, v);
  tmem_wait_ld();
  // Sum of squares in chains of 32 columns, combined pairwise, so that the result has the same
  // bits whether a row is shared by two threads or by four.
  float ss = 0.f;
#pragma unroll
  for (int h = 0; h < CPT / 32; ++h) {
    float sh = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float a = __uint_as_float(v[h * 32 + i]);
      sh = fmaf(a, a, sh);
    }
    ss = h == 0 ? sh : ss + sh;
  }
  c.ss_part[c.part * TILE + c.row] = ss;
  // only the NQ warps that share these 32 rows exchange partial sums: a barrier of their own
  // (named barriers 3..6, one per group of 32 rows)
  asm volatile("bar.sync %0, %1;" ::"r"(3 + ((threadIdx.x >> 5) & 3)), "n"(32 * NQ) : "memory");
  if constexpr (NQ == 2) ss = c.ss_part[c.row] + c.ss_part[TILE + c.row];
  else ss = (c.ss_part[c.row] + c.ss_part[TILE + c.row]) + (c.ss_part[2 * TILE + c.row] + c.ss_part[3 * TILE + c.row]);
  const float inv = rsqrtf(ss * (1.0f / D) + kRmsEps);
#pragma unroll
  for (int q = 0; q < CPT / 8; ++q) {
    const int col = c.part * CPT + q * 8;
    const uint32_t* src = &v[q * 8];
    uint4 o;
    // the gain lives in the weights that consume this operand (see *_chunk_gain)
    o.x = pack_bf16(__uint_as_float(src[0]) * inv, __uint_as_float(src[1]) * inv);
    o.y = pack_bf16(__uint_as_float(src[2]) * inv, __uint_as_float(src[3]) * inv);
    o.z = pack_bf16(__uint_as_float(src[4]) * inv, __uint_as_float(src[5]) * inv);
    o.w = pack_bf16(__uint_as_float(src[6]) * inv, __uint_as_float(src[7]) * inv);
    *reinterpret_cast<uint4*>(c.smem + OFF_A + (col >> 6) * CHUNK_BYTES + swz(c.row, (col & 63) >> 3)) = o;
  }
  T_END(c, TM_NORM);
}

// GatedMLP on the A operand (already normed): residual += down(gelu(gate) * up).
template <int NQ>
__device__ __forceinline__ void ffn(Ctx& c) {
  constexpr int GC = 64 / NQ;
  round_begin<NQ>(c);
  if (threadIdx.x == 0) {
    issue_chunk(c, c.sA, 128, COL_ACC, 0, 0);
    issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_ACC, 1, 1);
  }
  round_end<NQ>(c);
  for (int cc = 0; cc < 8; ++cc) {
    // gate = acc[0,64), up = acc[64,128); this thread: hidden columns [GC part, GC part + GC)
    T_BEGIN(c);
    uint32_t gv[GC], uv[GC];
    tmem_ld_cols<GC>(c.lane_addr + COL_ACC + c.part * GC, gv);
    tmem_ld_cols<GC>(c.lane_addr + COL_ACC + 64 + c.part * GC, uv);
    tmem_wait_ld();
#pragma unroll
    for (int q = 0; q < GC / 8; ++q) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = gelu_mul_bf16x2(__uint_as_float(gv[q * 8 + 2 * j]), __uint_as_float(gv[q * 8 + 2 * j + 1]),
                               __uint_as_float(uv[q * 8 + 2 * j]), __uint_as_float(uv[q * 8 + 2 * j + 1]));
      *reinterpret_cast<uint4*>(c.smem + OFF_P + swz(c.row, c.part * (GC / 8) + q)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    T_END(c, TM_FFN_EPI);
    // one round: this chunk's down projection into the residual, then the next chunk's
    // gate|up (the accumulator has been read, the product operand is only read by `down`)
    round_begin<NQ>(c);
    if (threadIdx.x == 0) {
      issue_chunk(c, c.sP, 128, COL_RESID, 1, 2);
      if (cc < 7) {
        issue_chunk(c, c.sA, 128, COL_ACC, 0, 0);
        issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_ACC, 1, 1);
      }
    }
    round_end<NQ>(c);
  }
}

// Attention of one head for every environment of the tile, from the staged q|k|v rows
// (row-major, q at bf16 column 0, k at 32, v at 64) into columns [32*hh, 32*hh+32) of the
// second operand.  One warp per block of 16 query rows of one environment; MAXKB blocks of
// 16 keys at most.
template <int NQ, int MAXKB>
__device__ __forceinline__ void attention_head(Ctx& c, int hh, int n_items) {
  const uint8_t* meta = c.smem + OFF_META;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const float scale = 0.17677669529663687f;  // 1/sqrt(32)
  for (int it = warp; it < n_items; it += 4 * NQ) {
    const int r0 = meta[384 + it];
    const int e0 = meta[r0], n = meta[128 + r0] + 1;   // first tile row and size of the environment
    const int last = e0 + n - 1;
    uint32_t qa[2][4];
    {
      int row = min(r0 + (lane & 7) + ((lane >> 3) & 1) * 8, last);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks)
        ldsm_x4(c.sStage + row * STAGE_STRIDE + (ks * 16 + (lane >> 4) * 8) * 2, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
    }
    const int nkb = (n + 15) >> 4;
    float s[MAXKB][2][4];
#pragma unroll
    for (int kb = 0; kb < MAXKB; ++kb) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[kb][nt][i] = 0.f;
      if (kb < nkb) {
        int krow = min(e0 + kb * 16 + (lane >> 4) * 8 + (lane & 7), last);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(c.sStage + krow * STAGE_STRIDE + (DH + ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
          mma_bf16(s[kb][0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
          mma_bf16(s[kb][1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
        }
      }
    }
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int kb = 0; kb < MAXKB; ++kb)
      if (kb < nkb) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            int j = kb * 16 + nt * 8 + 2 * t + i;
            bool valid = j < n;
            bool live = valid && meta[256 + e0 + j];
            float a = valid ? (live ? s[kb][nt][i] * scale : kMaskedScore) : -INFINITY;
            float b = valid ? (live ? s[kb][nt][2 + i] * scale : kMaskedScore) : -INFINITY;
            s[kb][nt][i] = a;
            s[kb][nt][2 + i] = b;
            m0 = fmaxf(m0, a);
            m1 = fmaxf(m1, b);
          }
      }
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int kb = 0; kb < MAXKB; ++kb)
      if (kb < nkb) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            float a = __expf(s[kb][nt][i] - m0), b = __expf(s[kb][nt][2 + i] - m1);  // exp(-inf) = 0 for padding
            s[kb][nt][i] = a;
            s[kb][nt][2 + i] = b;
            l0 += a;
            l1 += b;
          }
      }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float o[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[nt][i] = 0.f;
#pragma unroll
    for (int kb = 0; kb < MAXKB; ++kb)
      if (kb < nkb) {
        uint32_t a0 = pack_bf16(s[kb][0][0], s[kb][0][1]), a1 = pack_bf16(s[kb][0][2], s[kb][0][3]);
        uint32_t a2 = pack_bf16(s[kb][1][0], s[kb][1][1]), a3 = pack_bf16(s[kb][1][2], s[kb][1][3]);
        int vrow = min(e0 + kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), last);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(c.sStage + vrow * STAGE_STRIDE + (2 * DH + (np * 2 + (lane >> 4)) * 8) * 2, b0, b1, b2, b3);
          mma_bf16(o[np * 2], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[np * 2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    const int q0 = r0 + g, q1 = r0 + g + 8;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      int col = hh * DH + nt * 8 + 2 * t;
      if (q0 <= last)
        *reinterpret_cast<uint32_t*>(c.smem + OFF_P + swz(q0, col >> 3) + (col & 7) * 2) = pack_bf16(o[nt][0] * i0, o[nt][1] * i0);
      if (q1 <= last)
        *reinterpret_cast<uint32_t*>(c.smem + OFF_P + swz(q1, col >> 3) + (col & 7) * 2) = pack_bf16(o[nt][2] * i1, o[nt][3] * i1);
    }
  }
}

// bf16 pack of N accumulator columns into 16-byte groups
__device__ __forceinline__ uint4 pack8(const uint32_t* src) {
  return make_uint4(pack_bf16(__uint_as_float(src[0]), __uint_as_float(src[1])), pack_bf16(__uint_as_float(src[2]), __uint_as_float(src[3])),
                    pack_bf16(__uint_as_float(src[4]), __uint_as_float(src[5])), pack_bf16(__uint_as_float(src[6]), __uint_as_float(src[7])));
}

template <int NQ, int MAXKB>
__device__ __forceinline__ void run_spatial(Ctx& c, const SubLayer& s, int n_items, bool row_valid) {
  constexpr int QC = 96 / NQ, GC = 64 / NQ;
  norm_to_A<NQ>(c);
  for (int p = 0; p < 2; ++p) {
    for (int hh = 0; hh < 2; ++hh) {
      round_begin<NQ>(c);
      if (threadIdx.x == 0) {
        issue_chunk(c, c.sA, 96, COL_ACC, 0, (uint32_t)(p & 1));          // chunks 5p+2hh, 5p+2hh+1
        issue_chunk(c, c.sA + CHUNK_BYTES, 96, COL_ACC, 1, (uint32_t)((p & 1) ^ 1));
      }
      round_end<NQ>(c);
      // q|k|v of this head -> bf16 staging rows; this thread: accumulator columns [QC part, QC part + QC)
      {
        T_BEGIN(c);
        uint32_t v[QC];
        tmem_ld_cols<QC>(c.lane_addr + COL_ACC + c.part * QC, v);
        tmem_wait_ld();
        uint8_t* dst = c.smem + OFF_STAGE + c.row * STAGE_STRIDE + c.part * QC * 2;
#pragma unroll
        for (int q = 0; q < QC / 8; ++q) *reinterpret_cast<uint4*>(dst + q * 16) = pack8(&v[q * 8]);
        T_END(c, TM_QKV_EPI);
      }
      if (!row_valid && hh == 0) {
        // rows outside every environment contribute a zero operand row
#pragma unroll
        for (int q = 0; q < GC / 8; ++q)
          *reinterpret_cast<uint4*>(c.smem + OFF_P + swz(c.row, c.part * (GC / 8) + q)) = make_uint4(0u, 0u, 0u, 0u);
      }
      tc_fence_before();
      {
        T_BEGIN(c);
        epi_barrier<NQ>();
        attention_head<NQ, MAXKB>(c, hh, n_items);
        epi_barrier<NQ>();  // staging rows are free again
        T_END(c, TM_ATTN);
      }
    }
    round_begin<NQ>(c);
    if (threadIdx.x == 0) issue_chunk(c, c.sP, 128, COL_RESID, 1, (uint32_t)(p & 1));  // chunk 5p+4
    round_end<NQ>(c);
  }
  norm_to_A<NQ>(c);
  ffn<NQ>(c);
}

// Spatial sublayer, first part, for environments that span several tiles: norm1 and the
// q|k|v projection of every head, written as bf16 to global scratch for the attention kernel.
template <int NQ>
__device__ __forceinline__ void run_spatial_pre(Ctx& c, const SubLayer& s, size_t grow, bool row_valid) {
  constexpr int QC = 96 / NQ;
  norm_to_A<NQ>(c);
  for (int hd = 0; hd < HEADS; ++hd) {
    round_begin<NQ>(c);
    if (threadIdx.x == 0) {
      issue_chunk(c, c.sA, 96, COL_ACC, 0, 0);
      issue_chunk(c, c.sA + CHUNK_BYTES, 96, COL_ACC, 1, 1);
    }
    round_end<NQ>(c);
    uint32_t v[QC];
    tmem_ld_cols<QC>(c.lane_addr + COL_ACC + c.part * QC, v);
    tmem_wait_ld();
    if (row_valid) {
      __nv_bfloat16* dst = s.qkv_out + grow * (3 * D);
#pragma unroll
      for (int q = 0; q < QC / 8; ++q) {
        const int j = c.part * QC + q * 8;                 // accumulator column: q (0-31), k (32-63), v (64-95)
        const int col = (j >> 5) * D + hd * DH + (j & 31);
        *reinterpret_cast<uint4*>(dst + col) = pack8(&v[q * 8]);
      }
    }
  }
}

// Spatial sublayer, second part: attention output from global scratch -> out_proj into the
// residual -> norm2 -> GatedMLP.
template <int NQ>
__device__ __forceinline__ void run_spatial_post(Ctx& c, const SubLayer& s, size_t grow, bool row_valid) {
  constexpr int CPT = 128 / NQ;
  {
    const uint4* src = reinterpret_cast<const uint4*>(s.o_in + grow * D + c.part * CPT);
#pragma unroll
    for (int q = 0; q < CPT / 8; ++q) {
      const int col = c.part * CPT + q * 8;
      uint4 o = make_uint4(0u, 0u, 0u, 0u);
      if (row_valid) o = src[q];
      *reinterpret_cast<uint4*>(c.smem + OFF_A + (col >> 6) * CHUNK_BYTES + swz(c.row, (col & 63) >> 3)) = o;
    }
  }
  round_begin<NQ>(c);
  if (threadIdx.x == 0) {
    issue_chunk(c, c.sA, 128, COL_RESID, 1, 0);
    issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_RESID, 1, 1);
  }
  round_end<NQ>(c);
  norm_to_A<NQ>(c);
  ffn<NQ>(c);
}

// Bullet rows: norm_bullet and the kv_bullet projection, keys and values of all heads, written
// as bf16 to global scratch (models/yemong/attention.py:151 of the reference).  This program
// runs alone in its launch and its four weight chunks are the same for every tile, so they are
// loaded once per CTA (ring slots 0 and 1: keys; staging area and P: values) and stay put.
// The residual is dead after the norm, so one round projects the keys into the accumulator
// columns and the values into the residual columns.
template <int NQ>
__device__ __forceinline__ void run_bullet_kv(Ctx& c, const SubLayer& s, size_t grow, bool row_valid) {
  constexpr int CPT = 128 / NQ;
  norm_to_A<NQ>(c);
  round_begin<NQ>(c);
  if (threadIdx.x == 0) {
    if (!(c.parity & 1u)) {   // first tile of this CTA: the resident chunks are still arriving
      mbar_wait(c.bar_full[0], 0, c.status, c.aborted, ST_TIMEOUT_FULL);
      c.parity |= 1u;
    }
    tc_fence_after();
    const uint32_t idesc = instr_desc(128);
    const uint32_t wk[2] = {c.sRing, c.sRing + CHUNK_BYTES}, wv[2] = {c.sStage, c.sP};
#pragma unroll
    for (int atom = 0; atom < 2; ++atom)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        tc_mma(c.tmem + COL_ACC, smem_desc(c.sA + atom * CHUNK_BYTES + k * 32), smem_desc(wk[atom] + k * 32), idesc, (atom | k) ? 1u : 0u);
        tc_mma(c.tmem + COL_RESID, smem_desc(c.sA + atom * CHUNK_BYTES + k * 32), smem_desc(wv[atom] + k * 32), idesc, (atom | k) ? 1u : 0u);
      }
  }
  round_end<NQ>(c);
#pragma unroll
  for (int half = 0; half < 2; ++half)
#pragma unroll
    for (int ch = 0; ch < CPT / 32; ++ch) {
      uint32_t v[32];
      tmem_ld32(c.lane_addr + (half ? COL_RESID : COL_ACC) + c.part * CPT + ch * 32, v);
      if (row_valid) {
        __nv_bfloat16* dst = s.kvb_out + grow * (2 * D) + half * D + c.part * CPT + ch * 32;
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + q * 8) = pack8(&v[q * 8]);
      }
    }
}

struct RowState {
  int hrow;        // row of the packed hidden state, -1 for field / invalid rows
  int lag_ok;      // stored conv lags still inside the current episode (0..3)
  bool zero_in;    // incoming state taken as zero (reset_env)
};

// One temporal sublayer on the tile at one timestep.  In the gate rounds thread (row, part)
// works on hidden columns [64 rnd + GC part, +GC), GC = 64 / NQ, and parks b2 for exactly those.
template <int NQ>
__device__ __forceinline__ void run_temporal(Ctx& c, const SubLayer& s, const RowState& rs, bool is_field, bool boundary,
                                             bool has_fields, const float* hid_in) {
  constexpr int CPT = 128 / NQ, GC = 64 / NQ, WARPS = 4 * NQ;
  const bool is_ship = rs.hrow >= 0;
  norm_to_A<NQ>(c);
  // b2 = bf16(gelu(linear2 n)) for this thread's columns, parked as packed bf16 pairs
  uint32_t b2p[2][GC / 2];
  round_begin<NQ>(c);
  if (threadIdx.x == 0) {
    issue_chunk(c, c.sA, 128, COL_ACC, 0, 0);
    issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_ACC, 1, 1);
  }
  round_end<NQ>(c);
  {
    T_BEGIN(c);
#pragma unroll
    for (int rnd = 0; rnd < 2; ++rnd) {
      uint32_t v[GC];
      tmem_ld_cols<GC>(c.lane_addr + COL_ACC + rnd * 64 + c.part * GC, v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < GC / 2; ++j)
        b2p[rnd][j] = pack_bf16(gelu_fast(__uint_as_float(v[2 * j])), gelu_fast(__uint_as_float(v[2 * j + 1])));
    }
    T_END(c, TM_TEMPORAL_EPI);
  }
  // b1 = bf16(linear1 n); ships: causal conv with the stored taps -> u; fields: keep b1.
  round_begin<NQ>(c);
  if (threadIdx.x == 0) {
    issue_chunk(c, c.sA, 128, COL_ACC, 0, 0);
    issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_ACC, 1, 1);
  }
  round_end<NQ>(c);
  const float* hin = is_ship ? hid_in + (size_t)rs.hrow * 4 * D : nullptr;
  float* hout = is_ship ? s.hid_out + (size_t)rs.hrow * 4 * D : nullptr;
  T_BEGIN(c);
  // (1) every thread parks bf16(b1) of its CPT columns in the A operand
#pragma unroll
  for (int ch = 0; ch < CPT / 32; ++ch) {
    uint32_t v[32];
    tmem_ld_cols<32>(c.lane_addr + COL_ACC + c.part * CPT + ch * 32, v);
    tmem_wait_ld();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int col = c.part * CPT + ch * 32 + q * 8;
      *reinterpret_cast<uint4*>(c.smem + OFF_A + (col >> 6) * CHUNK_BYTES + swz(c.row, (col & 63) >> 3)) = pack8(&v[q * 8]);
    }
  }
  tc_fence_before();
  epi_barrier<NQ>();
  // (2) causal conv, one warp per ship row and four columns per lane, so that the stored taps
  // are read and written as whole 512-byte rows.  u = bias + w0 tap0 + w1 tap1 + w2 tap2 + w3 b1,
  // summed in the reference's order; new taps = (tap1, tap2, b1); bf16(u) replaces b1 in A.
  {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = lane * 4;
    float cw[4][4], cb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 w4 = __ldg(reinterpret_cast<const float4*>(s.conv_w + (col + i) * 4));
      cw[i][0] = w4.x; cw[i][1] = w4.y; cw[i][2] = w4.z; cw[i][3] = w4.w;
      cb[i] = __ldg(s.conv_b + col + i);
    }
    const int* row_hrow = reinterpret_cast<const int*>(c.smem + OFF_ROWINFO);
    const uint8_t* row_flags = c.smem + OFF_ROWINFO + 512;
    // Four rows at a time: all loads of the group are issued before any store, because the
    // state may be updated in place and the compiler must otherwise keep loads behind stores.
    for (int r0 = warp; r0 < TILE; r0 += 4 * WARPS) {
      float4 t0[4], t1[4], t2[4];
      uint2 bw[4];
      int hr[4], lag[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int r = r0 + WARPS * k;
        hr[k] = row_hrow[r];
        const int flags = row_flags[r];
        lag[k] = flags & 3;
        t0[k] = t1[k] = t2[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        bw[k] = make_uint2(0u, 0u);
        if (hr[k] >= 0) {
          if (!(flags & 4)) {
            const float* hi = hid_in + (size_t)hr[k] * 4 * D + col;
            t0[k] = *reinterpret_cast<const float4*>(hi + D);
            t1[k] = *reinterpret_cast<const float4*>(hi + 2 * D);
            t2[k] = *reinterpret_cast<const float4*>(hi + 3 * D);
          }
          bw[k] = *reinterpret_cast<const uint2*>(c.smem + OFF_A + (lane >> 4) * CHUNK_BYTES + swz(r, (lane & 15) >> 1) + (lane & 1) * 8);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (hr[k] < 0) continue;
        const int r = r0 + WARPS * k;
        float* ho = s.hid_out + (size_t)hr[k] * 4 * D + col;
        const float b1[4] = {bf16_lo(bw[k].x), bf16_hi(bw[k].x), bf16_lo(bw[k].y), bf16_hi(bw[k].y)};
        *reinterpret_cast<float4*>(ho + D) = t1[k];
        *reinterpret_cast<float4*>(ho + 2 * D) = t2[k];
        *reinterpret_cast<float4*>(ho + 3 * D) = make_float4(b1[0], b1[1], b1[2], b1[3]);
        const float a0[4] = {t0[k].x, t0[k].y, t0[k].z, t0[k].w}, a1[4] = {t1[k].x, t1[k].y, t1[k].z, t1[k].w},
                    a2[4] = {t2[k].x, t2[k].y, t2[k].z, t2[k].w};
        float u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float p0 = lag[k] >= 3 ? __fmul_rn(a0[i], cw[i][0]) : 0.f;
          float p1 = lag[k] >= 2 ? __fmul_rn(a1[i], cw[i][1]) : 0.f;
          float p2 = lag[k] >= 1 ? __fmul_rn(a2[i], cw[i][2]) : 0.f;
          float p3 = __fmul_rn(b1[i], cw[i][3]);
          u[i] = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(p0, p1), p2), p3), cb[i]);
        }
        *reinterpret_cast<uint2*>(c.smem + OFF_A + (lane >> 4) * CHUNK_BYTES + swz(r, (lane & 15) >> 1) + (lane & 1) * 8) =
            make_uint2(pack_bf16(u[0], u[1]), pack_bf16(u[2], u[3]));
      }
    }
  }
  T_END(c, TM_TEMPORAL_EPI);
  // gates and state update, 64 hidden columns per round: acc[0,64) = W_a u, acc[64,128) = W_x u
#pragma unroll
  for (int rnd = 0; rnd < 2; ++rnd) {
    round_begin<NQ>(c);
    if (threadIdx.x == 0) {
      issue_chunk(c, c.sA, 128, COL_ACC, 0, 0);
      issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_ACC, 1, 1);
    }
    // previous state of this thread's columns, requested before waiting for the gates
    float4 hprev[GC / 4];
#pragma unroll
    for (int q = 0; q < GC / 4; ++q) {
      hprev[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (is_ship && !rs.zero_in) hprev[q] = *reinterpret_cast<const float4*>(hin + rnd * 64 + c.part * GC + q * 4);
    }
    round_end<NQ>(c);
    T_BEGIN(c);
    // sixteen columns at a time keeps the gate accumulators, the parked b2 and the prefetched
    // state inside the register budget
#pragma unroll
    for (int sc = 0; sc < GC / 16; ++sc) {
      uint32_t rv[16], iv[16];
      tmem_ld_cols<16>(c.lane_addr + COL_ACC + c.part * GC + sc * 16, rv);       // executed by every lane of the warp
      tmem_ld_cols<16>(c.lane_addr + COL_ACC + 64 + c.part * GC + sc * 16, iv);
      tmem_wait_ld();
      if (is_ship) {
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          const int q = sc * 2 + q2;
          const int col = rnd * 64 + c.part * GC + q * 8;
          // u (bf16) back from the A operand (K atom rnd)
          uint8_t* ua = c.smem + OFF_A + rnd * CHUNK_BYTES + swz(c.row, c.part * (GC / 8) + q);
          const uint4 ub = *reinterpret_cast<const uint4*>(ua);
          const uint32_t uw[4] = {ub.x, ub.y, ub.z, ub.w};
          uint32_t ob[4];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int cc = col + hf * 4;
            const float4 hv = hprev[q * 2 + hf];
            const float4 ab = __ldg(reinterpret_cast<const float4*>(s.a_b + cc));
            const float4 xb = __ldg(reinterpret_cast<const float4*>(s.x_b + cc));
            const float4 dl = __ldg(reinterpret_cast<const float4*>(s.decay_log2 + cc));
            const float abv[4] = {ab.x, ab.y, ab.z, ab.w}, xbv[4] = {xb.x, xb.y, xb.z, xb.w}, dlv[4] = {dl.x, dl.y, dl.z, dl.w};
            float hn[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int k = q2 * 8 + hf * 4 + i;
              float rg = round_bf16(sigmoid_fast(__uint_as_float(rv[k]) + abv[i]));
              float ig = round_bf16(sigmoid_fast(__uint_as_float(iv[k]) + xbv[i]));
              // sigmoid(Lambda)^(8 r) = 2^(r * 8 log2 sigmoid(Lambda)); the table is part of the weight image
              float a = ex2_fast(rg * dlv[i]);
              float gate = sqrt_fast(fmaxf((1.0f - a) * (1.0f + a), kGateFloor));
              uint32_t uword = uw[hf * 2 + (i >> 1)];
              float uu = (i & 1) ? bf16_hi(uword) : bf16_lo(uword);
              float bb = gate * (ig * uu);
              if (boundary) a = 0.f;
              hn[i] = fmaf(a, hn[i], bb);
            }
            *reinterpret_cast<float4*>(hout + cc) = make_float4(hn[0], hn[1], hn[2], hn[3]);
            const int bi = q * 4 + hf * 2;
            ob[hf * 2] = pack_bf16(hn[0] * bf16_lo(b2p[rnd][bi]), hn[1] * bf16_hi(b2p[rnd][bi]));
            ob[hf * 2 + 1] = pack_bf16(hn[2] * bf16_lo(b2p[rnd][bi + 1]), hn[3] * bf16_hi(b2p[rnd][bi + 1]));
          }
          // branch operand for linear_out: K atom 0 lives in the second operand, K atom 1 in place
          uint8_t* dst = rnd == 0 ? c.smem + OFF_P + swz(c.row, c.part * (GC / 8) + q) : ua;
          *reinterpret_cast<uint4*>(dst) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
        }
      }
    }
    T_END(c, TM_IO);
  }
  if (has_fields) {
    // field rows: branch = bf16(bf16(field_sub b1) * b2)
    round_begin<NQ>(c);
    if (threadIdx.x == 0) {
      issue_chunk(c, c.sA, 128, COL_ACC, 0, 0);
      issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_ACC, 1, 1);
    }
    round_end<NQ>(c);
#pragma unroll
    for (int rnd = 0; rnd < 2; ++rnd) {
      uint32_t v[GC];
      tmem_ld_cols<GC>(c.lane_addr + COL_ACC + rnd * 64 + c.part * GC, v);        // executed by every lane of the warp
      tmem_wait_ld();
      if (!is_ship) {
#pragma unroll
        for (int q = 0; q < GC / 8; ++q) {
          uint32_t ob[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int bi = q * 4 + j;
            float f0 = is_field ? round_bf16(__uint_as_float(v[q * 8 + 2 * j])) * bf16_lo(b2p[rnd][bi]) : 0.f;
            float f1 = is_field ? round_bf16(__uint_as_float(v[q * 8 + 2 * j + 1])) * bf16_hi(b2p[rnd][bi]) : 0.f;
            ob[j] = pack_bf16(f0, f1);
          }
          uint8_t* dst = rnd == 0 ? c.smem + OFF_P + swz(c.row, c.part * (GC / 8) + q)
                                  : c.smem + OFF_A + CHUNK_BYTES + swz(c.row, c.part * (GC / 8) + q);
          *reinterpret_cast<uint4*>(dst) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
        }
      }
    }
  } else if (!is_ship) {
    // rows outside every environment: zero operand rows
#pragma unroll
    for (int q = 0; q < GC / 8; ++q) {
      *reinterpret_cast<uint4*>(c.smem + OFF_P + swz(c.row, c.part * (GC / 8) + q)) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(c.smem + OFF_A + CHUNK_BYTES + swz(c.row, c.part * (GC / 8) + q)) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  // residual += linear_out(branch): K atom 0 from the second operand, K atom 1 from A
  round_begin<NQ>(c);
  if (threadIdx.x == 0) {
    issue_chunk(c, c.sP, 128, COL_RESID, 1, 0);
    issue_chunk(c, c.sA + CHUNK_BYTES, 128, COL_RESID, 1, 1);
  }
  round_end<NQ>(c);
  norm_to_A<NQ>(c);
  ffn<NQ>(c);
}

template <int NQ, int MAXKB>
__global__ void __launch_bounds__(128 * NQ, NQ == 4 ? 1 : 2) k_trunk_tiles(const __grid_constant__ TrunkArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ int s_aborted[2];
  __shared__ int s_items;
  __shared__ SubLayer s_sub[MAX_SUBLAYERS];  // kernel parameters are slow to index dynamically
  __shared__ uint16_t s_sched[MAX_SUBLAYERS * N_TEMPORAL_CHUNKS];  // (chunk << 6) | (sublayer << 2) | slot
  __shared__ int s_sched_len;
  __shared__ int s_cons;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid < args.n_sub) s_sub[tid] = args.sub[tid];
  if (tid == 32) {
    int n = 0;
    for (int si = 0; si < args.n_sub; ++si) {
      const int type = args.sub[si].type;
      const int n_chunks = type == SUB_TEMPORAL ? N_TEMPORAL_CHUNKS : N_SPATIAL_IMAGE;
      for (int ch = 0; ch < n_chunks; ++ch) {
        if (!chunk_used(type, ch, args.has_fields != 0)) continue;
        s_sched[n++] = (uint16_t)((ch << 6) | (si << 2) | chunk_slot(type, ch));
      }
    }
    s_sched_len = n;
    s_cons = 0;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 48);

  if (tid == 0) {
    s_aborted[0] = (*args.status != 0) ? 1 : 0;
    s_aborted[1] = args.poll_limit > 0 ? args.poll_limit : DEFAULT_POLL_LIMIT;
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    mbar_init(smem_u32(&bars[2]), 1);
    mbar_init(smem_u32(&bars[3]), 1);
    mbar_init(smem_u32(&bars[4]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  {
    // ---------------------------------------------------------------- tile owners
    Ctx c;
    c.smem = smem;
    c.sA = smem_u32(smem + OFF_A);
    c.sP = smem_u32(smem + OFF_P);
    c.sRing = smem_u32(smem + OFF_RING);
    c.sStage = smem_u32(smem + OFF_STAGE);
    c.bar_full[0] = smem_u32(&bars[0]);
    c.bar_full[1] = smem_u32(&bars[1]);
    c.bar_full[2] = smem_u32(&bars[2]);
    c.bar_acc = smem_u32(&bars[4]);
    c.tmem = tmem_base;
    c.row = tid & (TILE - 1);
    c.part = tid >> 7;
    c.lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    c.status = args.status;
    c.aborted = s_aborted;
    c.acc_phase = 0;
    c.ss_part = reinterpret_cast<float*>(smem + OFF_SS);
#ifdef BNB_TIMING
    for (int i = 0; i < TM_COUNT; ++i) c.tacc[i] = 0;
    const long long t_kernel0 = clock64();
#endif
    c.subs = s_sub;
    c.parity = 0;
    c.cons_count = 0;
    c.s_cons = &s_cons;
    c.sched = s_sched;
    c.sched_len = s_sched_len;
    c.p_idx = 0;
    c.p_seq = 0;
    {
      const int my_tiles = blockIdx.x < args.n_tiles ? (args.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      c.p_left = my_tiles * args.t_loop * s_sched_len;
    }
    c.occ[0] = c.occ[1] = c.occ[2] = -1;
    // A bullet key/value program keeps its four weight chunks resident instead of streaming them.
    const bool kv_resident = args.n_sub == 1 && s_sub[0].type == SUB_BULLET_KV;
    if (kv_resident) {
      c.p_left = 0;
      if (warp == 4 * NQ - 1 && blockIdx.x < args.n_tiles) {
        const int lane = tid & 31;
        if (lane == 0) mbar_expect_tx(c.bar_full[0], N_BULLET_CHUNKS * CHUNK_BYTES);
        __syncwarp();
        if (lane < N_BULLET_CHUNKS) {
          const uint32_t dst = lane == 0 ? c.sRing : (lane == 1 ? c.sRing + CHUNK_BYTES : (lane == 2 ? c.sStage : c.sP));
          bulk_g2s(dst, s_sub[0].packed + (size_t)(N_SPATIAL_CHUNKS + lane) * CHUNK_BYTES, CHUNK_BYTES, c.bar_full[0]);
        }
      }
    }
    if (warp == 4 * NQ - 1) refill(c);
    uint8_t* meta = smem + OFF_META;
    const EnvMap& map = args.map;
    const int NM = map.tokens_per_env;
    const int row = c.row;

    const int flat_limit = args.n_rows_dev ? *args.n_rows_dev : map.total_tokens;
    for (int tile = blockIdx.x; tile < args.n_tiles; tile += gridDim.x) {
      // ---- rows of this tile: whole environments, ships first then fields in each
      const int grp = tile / args.env_tiles, eb = tile - grp * args.env_tiles;
      if (args.flat_rows && eb * TILE >= flat_limit) continue;   // same decision in every thread of the CTA
      bool valid;
      int env, tok, env_first, env_n, env_ships;
      size_t grow = 0;
      int hrow_if_ship;
      if (args.flat_rows) {
        // plain slices of the token rows; the environment of a row is looked up
        const int r = eb * TILE + row;
        if (kv_resident) {
          // ask L2 for this thread's share of the next tile's input rows
          const long long rn = (long long)r + (long long)gridDim.x * TILE;
          if (rn < flat_limit) {
            const size_t src = args.row_index ? (size_t)args.row_index[rn] : (size_t)rn;
            const char* nx = reinterpret_cast<const char*>(args.x) + src * D * (args.io_bf16 ? 2 : 4) + c.part * (512 / NQ);
#pragma unroll
            for (int l = 0; l < 4 / NQ; ++l) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + l * 128));
          }
        }
        valid = r < flat_limit;
        env = valid ? map.env_of_token(r) : 0;
        env_first = 0;
        env_n = 1;
        tok = valid ? r - map.env_tok_begin(env) : 0;
        env_ships = valid ? map.env_ship_count(env) : 0;
        grow = (size_t)grp * map.total_tokens + (size_t)r;
        hrow_if_ship = map.env_ship_begin(env) + tok;
      } else if (args.tile_env_begin) {
        // ragged: the tile holds the environments tile_env_ids[k_lo .. k_hi), rows in that order
        const int k_lo = args.tile_env_begin[eb], k_hi = args.tile_env_begin[eb + 1];
        int k = k_lo, first = 0;
        env = args.tile_env_ids[k];
        int cnt = map.tok_off[env + 1] - map.tok_off[env];
        while (row >= first + cnt && k + 1 < k_hi) {
          first += cnt;
          ++k;
          env = args.tile_env_ids[k];
          cnt = map.tok_off[env + 1] - map.tok_off[env];
        }
        valid = row < first + cnt;
        env_first = first;
        env_n = cnt;
        env_ships = map.ship_off[env + 1] - map.ship_off[env];
        tok = row - first;
        grow = (size_t)grp * map.total_tokens + (size_t)(map.tok_off[env] + tok);
        hrow_if_ship = map.ship_off[env] + tok;
      } else {
        const int env0 = eb * args.envs_per_tile;
        const int env_cnt = min(args.envs_per_tile, map.n_envs - env0);
        const int el = row / NM;
        tok = row - el * NM;
        valid = el < env_cnt;
        env = env0 + el;
        env_first = el * NM;
        env_n = NM;
        env_ships = map.ships_per_env;
        grow = (size_t)grp * map.total_tokens + (size_t)env * NM + tok;
        hrow_if_ship = env * map.ships_per_env + tok;
      }
      if (!valid) { grow = 0; env = 0; }
      // input row of this tile row (differs from the output row only for compacted bullet rows)
      const size_t xrow0 = (args.row_index && valid) ? (size_t)args.row_index[grow] : grow;
      const bool is_ship = valid && tok < env_ships;
      const bool is_field = valid && !is_ship;
      RowState rs;
      rs.hrow = is_ship ? hrow_if_ship : -1;
      rs.lag_ok = BNB_CONV_KERNEL - 1;
      rs.zero_in = is_ship && args.reset_env && args.reset_env[env];
      epi_barrier<NQ>();  // previous tile's readers of the meta arrays are done
      if (c.part == 0) {
        meta[row] = (uint8_t)(valid ? env_first : row);
        meta[128 + row] = (uint8_t)(valid ? env_n - 1 : 0);
      }
      if (c.part == 0) reinterpret_cast<int*>(smem + OFF_ROWINFO)[row] = rs.hrow;
      if (tid == 0) s_items = 0;
      epi_barrier<NQ>();
      if (c.part == 0 && valid && (tok & 15) == 0) meta[384 + atomicAdd(&s_items, 1)] = (uint8_t)row;

      for (int t = 0; t < args.t_loop; ++t) {
        const size_t trow = grow + (size_t)t * map.total_tokens;
        if (c.part == 0) meta[256 + row] = valid ? (args.alive ? args.alive[trow] : (uint8_t)1) : (uint8_t)0;
        // residual <- x (this thread: columns [CPT part, CPT part + CPT))
        constexpr int CPT = 128 / NQ;
#pragma unroll
        for (int ch = 0; ch < CPT / 32; ++ch) {
          uint32_t v[32];
          const size_t xoff = (xrow0 + (size_t)t * map.total_tokens) * D + c.part * CPT + ch * 32;
          if (args.io_bf16) {   // input rows held as bfloat16 (this kernel's y, when it has one, stays float32)
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(args.x) + xoff);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w = make_uint4(0u, 0u, 0u, 0u);
              if (valid) w = src[q];
              const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                v[q * 8 + 2 * j] = ws[j] << 16;              // a bfloat16 is the upper half of its float
                v[q * 8 + 2 * j + 1] = ws[j] & 0xFFFF0000u;
              }
            }
          } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
              if (valid) f = *reinterpret_cast<const float4*>(args.x + xoff + q * 4);
              v[q * 4 + 0] = __float_as_uint(f.x); v[q * 4 + 1] = __float_as_uint(f.y);
              v[q * 4 + 2] = __float_as_uint(f.z); v[q * 4 + 3] = __float_as_uint(f.w);
            }
          }
          tmem_st32(c.lane_addr + COL_RESID + c.part * CPT + ch * 32, v);
        }
        bool boundary = false;
        if (t >= 1) {
          boundary = is_ship && args.done && args.done[(size_t)(t - 1) * map.n_envs + env];
          rs.lag_ok = boundary ? 0 : min(rs.lag_ok + 1, BNB_CONV_KERNEL - 1);
          rs.zero_in = false;
        }
        if (c.part == 0) smem[OFF_ROWINFO + 512 + row] = (uint8_t)(rs.lag_ok | (rs.zero_in ? 4 : 0));
        tc_fence_before();
        epi_barrier<NQ>();
        tc_fence_after();
        const int n_items = s_items;
        for (int si = 0; si < args.n_sub; ++si) {
          const SubLayer& s = s_sub[si];
          // Ask L2 for the recurrent state of the temporal sublayer that follows this one: every
          // CTA reaches it at about the same time, and the rows are needed one sublayer from now.
          if (is_ship && t == 0 && si + 1 < args.n_sub && s_sub[si + 1].type == SUB_TEMPORAL && s.type != SUB_TEMPORAL) {
            const char* base = reinterpret_cast<const char*>(s_sub[si + 1].hid_in + (size_t)rs.hrow * 4 * D) + c.part * (2048 / NQ);
#pragma unroll
            for (int l = 0; l < 16 / NQ; ++l) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + l * 128));
          }
          if (s.type == SUB_SPATIAL) run_spatial<NQ, MAXKB>(c, s, n_items, valid);
          else if (s.type == SUB_SPATIAL_PRE) run_spatial_pre<NQ>(c, s, trow, valid);
          else if (s.type == SUB_SPATIAL_POST) run_spatial_post<NQ>(c, s, trow, valid);
          else if (s.type == SUB_BULLET_KV) run_bullet_kv<NQ>(c, s, trow, valid);
          else run_temporal<NQ>(c, s, rs, is_field, boundary, args.has_fields != 0, t == 0 ? s.hid_in : s.hid_out);
        }
        // y <- residual
#pragma unroll
        for (int ch = 0; ch < CPT / 32; ++ch) {
          uint32_t v[32];
          tmem_ld32(c.lane_addr + COL_RESID + c.part * CPT + ch * 32, v);
          if (valid && args.y) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(args.y + trow * D + c.part * CPT + ch * 32 + q * 4) =
                  make_float4(__uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]), __uint_as_float(v[q * 4 + 2]), __uint_as_float(v[q * 4 + 3]));
          }
        }
      }
    }
    // a CTA whose tiles were all beyond the compacted row count has not yet waited for its
    // resident weight chunks; they must have landed before the CTA gives up its shared memory
    if (kv_resident && tid == 0 && blockIdx.x < args.n_tiles && !(c.parity & 1u))
      mbar_wait(c.bar_full[0], 0, c.status, c.aborted, ST_TIMEOUT_FULL);
#ifdef BNB_TIMING
  if (tid == 64 || tid == 0) {
    c.tacc[TM_TOTAL] = clock64() - t_kernel0;
    for (int i = 0; i < TM_COUNT; ++i)
      if (tid == 64 ? i < TM_FULL_WAIT : i >= TM_FULL_WAIT)
        reinterpret_cast<long long*>(args.status)[32 + blockIdx.x * TM_COUNT + i] = c.tacc[i];
  }
#endif
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ attention kernel of the split path
//
// One CTA per (environment, head): q, k, v of that head are staged from the bf16 scratch the
// PRE phase wrote, then each warp takes blocks of 16 query rows and walks the keys in blocks of
// 32 with a running maximum (mma.sync, fp32 softmax).  Dead keys score kMaskedScore, so their
// weight is exactly 0 unless no key of the environment is alive, in which case every key gets
// the same weight (models/yemong/attention.py:101-112 of the reference).  When the sublayer
// reads bullets, the environment's bullet keys and values (written by the BULLET_KV phase) are
// staged too and get a softmax of their own; its output, gated to zero when the environment has
// no active bullet, is added to the self-attention output (attention.py:149-166).
// A CTA stages HPC heads of one environment (all four when they fit in shared memory, else one):
// a staged row holds HPC x 32 bf16 plus 16 bytes of padding, which keeps ldmatrix conflict-free.
__host__ __device__ constexpr int flash_stride(int hpc) { return hpc * 64 + 16; }

// One softmax pass of a block of 16 queries (fragments qa) over n keys staged at sK / sV; returns
// the normalised output fragments in acc.  Keys are walked 32 at a time.  `bias` holds one float
// per key, padded to a multiple of 32: 0 for a live key, kMaskedScore for a dead one, -inf beyond
// n.  Scores are carried in the log2 domain: t = (q.k) * log2(e) / sqrt(32) + bias, p = 2^(t - max).
__device__ __forceinline__ void flash_pass(const uint32_t (&qa)[2][4], uint32_t sK, uint32_t sV, int stride,
                                           const float* __restrict__ bias, int n, int lane, float (&acc)[4][4]) {
  const int t = lane & 3;
  const float c2 = 0.17677669529663687f * 1.4426950408889634f;
  const int last = n - 1;
  const int nkb = (n + 31) >> 5;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
  for (int kb = 0; kb < nkb; ++kb) {
    float sc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[nt][i] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int krow = min(kb * 32 + h * 16 + (lane >> 4) * 8 + (lane & 7), last);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sK + krow * stride + (ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
        mma_bf16(sc[2 * h], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16(sc[2 * h + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
    }
    float bm0 = -INFINITY, bm1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      // a dead key's bias swallows its score: kMaskedScore exactly (weight 0 unless every key is dead)
      const float2 bj = *reinterpret_cast<const float2*>(bias + kb * 32 + nt * 8 + 2 * t);
      sc[nt][0] = fmaf(sc[nt][0], c2, bj.x);
      sc[nt][1] = fmaf(sc[nt][1], c2, bj.y);
      sc[nt][2] = fmaf(sc[nt][2], c2, bj.x);
      sc[nt][3] = fmaf(sc[nt][3], c2, bj.y);
      bm0 = fmaxf(bm0, fmaxf(sc[nt][0], sc[nt][1]));
      bm1 = fmaxf(bm1, fmaxf(sc[nt][2], sc[nt][3]));
    }
    bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1));
    bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
    bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1));
    bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
    const float n0 = fmaxf(m0, bm0), n1 = fmaxf(m1, bm1);       // finite: every block holds a valid key
    const float c0 = ex2_fast(m0 - n0), c1 = ex2_fast(m1 - n1); // 2^(-inf) = 0 on the first block
    m0 = n0;
    m1 = n1;
    l0 *= c0;
    l1 *= c1;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      acc[nt][0] *= c0; acc[nt][1] *= c0;
      acc[nt][2] *= c1; acc[nt][3] *= c1;
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      sc[nt][0] = ex2_fast(sc[nt][0] - m0);
      sc[nt][1] = ex2_fast(sc[nt][1] - m0);
      sc[nt][2] = ex2_fast(sc[nt][2] - m1);
      sc[nt][3] = ex2_fast(sc[nt][3] - m1);
      l0 += sc[nt][0] + sc[nt][1];
      l1 += sc[nt][2] + sc[nt][3];
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t a0 = pack_bf16(sc[2 * h][0], sc[2 * h][1]), a1 = pack_bf16(sc[2 * h][2], sc[2 * h][3]);
      const uint32_t a2 = pack_bf16(sc[2 * h + 1][0], sc[2 * h + 1][1]), a3 = pack_bf16(sc[2 * h + 1][2], sc[2 * h + 1][3]);
      const int vrow = min(kb * 32 + h * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), last);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sV + vrow * stride + ((np * 2 + (lane >> 4)) * 8) * 2, b0, b1, b2, b3);
        mma_bf16(acc[np * 2], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[np * 2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    acc[nt][0] *= i0; acc[nt][1] *= i0;
    acc[nt][2] *= i1; acc[nt][3] *= i1;
  }
}

// env_base: first environment (group-major) of this launch.  kvb holds the bullet keys and values
// of the launch's environments (null: none): with env_off, the rows of the active bullets only,
// environment i of the launch owning rows [env_off[i], env_off[i+1]) (an inactive bullet has
// weight exactly 0 and an environment without active bullets is gated off, so neither needs a
// row); without env_off, nb rows per environment, all of them keys (no mask was given).
// blockIdx.y selects a group of hpc heads; the warps (4 to 8, chosen by the launcher so that the
// (head, query block) pairs divide evenly) share the pairs out.
__global__ void __launch_bounds__(256) k_attention_flash(const __nv_bfloat16* __restrict__ qkv, const uint8_t* __restrict__ alive,
                                                         __nv_bfloat16* __restrict__ o, EnvMap map, int env_base, int hpc,
                                                         const __nv_bfloat16* __restrict__ kvb,
                                                         const int* __restrict__ env_off, int nb) {
  extern __shared__ __align__(16) uint8_t fs[];
  const int env_g = env_base + blockIdx.x, hd0 = blockIdx.y * hpc;
  const int grp = env_g / map.n_envs, e = env_g - grp * map.n_envs;
  const size_t tok0 = (size_t)grp * map.total_tokens + map.env_tok_begin(e);
  const int n = map.env_tok_count(e);
  size_t brow0 = 0;
  if (!kvb) {
    nb = 0;
  } else if (env_off) {
    brow0 = (size_t)env_off[blockIdx.x];
    nb = env_off[blockIdx.x + 1] - (int)brow0;
  } else {
    brow0 = (size_t)blockIdx.x * nb;
  }
  const int stride = flash_stride(hpc);
  uint8_t* Qs = fs;
  uint8_t* Ks = Qs + (size_t)n * stride;
  uint8_t* Vs = Ks + (size_t)n * stride;
  uint8_t* Kb = Vs + (size_t)n * stride;
  uint8_t* Vb = Kb + (size_t)nb * stride;
  float* bias_s = reinterpret_cast<float*>(Vb + (size_t)nb * stride);   // strides are multiples of 16 bytes
  const int n32 = (n + 31) & ~31, nb32 = (nb + 31) & ~31;
  float* bias_b = bias_s + n32;
  const int gpr = hpc * 4;   // 16-byte groups per staged row
  // asynchronous 16-byte copies: all of them are in flight before the first one is waited for
  for (int i = threadIdx.x; i < n * 3 * gpr; i += blockDim.x) {
    const int r = i / (3 * gpr), rem = i - r * 3 * gpr, part = rem / gpr, q = rem - part * gpr;
    cp_async16(smem_u32(fs + ((size_t)part * n + r) * stride + q * 16),
               qkv + (tok0 + r) * (3 * D) + part * D + hd0 * DH + q * 8);
  }
  for (int i = threadIdx.x; i < nb * 2 * gpr; i += blockDim.x) {
    const int r = i / (2 * gpr), rem = i - r * 2 * gpr, part = rem / gpr, q = rem - part * gpr;
    cp_async16(smem_u32(Kb + ((size_t)part * nb + r) * stride + q * 16),
               kvb + (brow0 + r) * (2 * D) + part * D + hd0 * DH + q * 8);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int i = threadIdx.x; i < n32; i += blockDim.x)
    bias_s[i] = i < n ? ((!alive || alive[tok0 + i]) ? 0.f : kMaskedScore) : -INFINITY;
  for (int i = threadIdx.x; i < nb32; i += blockDim.x) bias_b[i] = i < nb ? 0.f : -INFINITY;
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int last = n - 1;
  const int nqb = (n + 15) >> 4;
  const int n_warps = blockDim.x >> 5;
  for (int item = warp; item < hpc * nqb; item += n_warps) {
    const int hl = item % hpc, qb = item / hpc;
    const uint32_t hoff = (uint32_t)hl * 64;
    const uint32_t sQ = smem_u32(Qs) + hoff, sK = smem_u32(Ks) + hoff, sV = smem_u32(Vs) + hoff;
    uint32_t qa[2][4];
    {
      const int row = min(qb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, last);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks)
        ldsm_x4(sQ + row * stride + (ks * 16 + (lane >> 4) * 8) * 2, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
    }
    float acc[4][4];
    flash_pass(qa, sK, sV, stride, bias_s, n, lane, acc);
    if (nb > 0) {
      float accb[4][4];
      flash_pass(qa, smem_u32(Kb) + hoff, smem_u32(Vb) + hoff, stride, bias_b, nb, lane, accb);
      // both outputs are bf16 tensors in the reference; so is their sum
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = round_bf16(acc[nt][i]) + round_bf16(accb[nt][i]);
    }
    const int q0 = qb * 16 + g, q1 = q0 + 8;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int col = (hd0 + hl) * DH + nt * 8 + 2 * t;
      if (q0 <= last) *reinterpret_cast<uint32_t*>(o + (tok0 + q0) * D + col) = pack_bf16(acc[nt][0], acc[nt][1]);
      if (q1 <= last) *reinterpret_cast<uint32_t*>(o + (tok0 + q1) * D + col) = pack_bf16(acc[nt][2], acc[nt][3]);
    }
  }
}

// ------------------------------------------------------------------ compaction of the active bullets
//
// Three small kernels turn the active mask of a slice of environments into (a) env_off, the
// exclusive prefix sum of the per-environment active counts (n_env + 1 entries), and (b) idx,
// the bullet rows of the slice that are active, in order.  The key/value projection then runs
// over idx only and the attention kernel stages rows [env_off[e], env_off[e+1]).

// one warp per environment: cnt[e] = number of active slots
__global__ void __launch_bounds__(256) k_bullet_count(const uint8_t* __restrict__ active, int n_env, int nb, int* __restrict__ cnt) {
  const int lane = threadIdx.x & 31;
  for (int e = blockIdx.x * 8 + (threadIdx.x >> 5); e < n_env; e += gridDim.x * 8) {
    int c = 0;
    for (int j0 = 0; j0 < nb; j0 += 32) {
      const int j = j0 + lane;
      const bool a = j < nb && active[(size_t)e * nb + j];
      c += __popc(__ballot_sync(0xffffffffu, a));
    }
    if (lane == 0) cnt[e] = c;
  }
}
// one CTA: env_off = exclusive scan of cnt, in place (env_off[n_env] = total)
__global__ void __launch_bounds__(1024) k_bullet_scan(int* __restrict__ env_off, int n_env) {
  __shared__ int warp_sum[32];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n_env; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < n_env ? env_off[i] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += u;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sum[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += u;
      }
      warp_sum[lane] = w;
    }
    __syncthreads();
    const int before = carry + (warp ? warp_sum[warp - 1] : 0) + inc - v;
    if (i < n_env) env_off[i] = before;
    __syncthreads();
    if (threadIdx.x == 1023) carry = before + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) env_off[n_env] = carry;
}
// one warp per environment: the active slots of environment e, in order, at idx[env_off[e]...]
__global__ void __launch_bounds__(256) k_bullet_fill(const uint8_t* __restrict__ active, int n_env, int nb,
                                                     const int* __restrict__ env_off, int* __restrict__ idx) {
  const int lane = threadIdx.x & 31;
  for (int e = blockIdx.x * 8 + (threadIdx.x >> 5); e < n_env; e += gridDim.x * 8) {
    int off = env_off[e];
    for (int j0 = 0; j0 < nb; j0 += 32) {
      const int j = j0 + lane;
      const bool a = j < nb && active[(size_t)e * nb + j];
      const uint32_t m = __ballot_sync(0xffffffffu, a);
      if (a) idx[off + __popc(m & ((1u << lane) - 1u))] = e * nb + j;
      off += __popc(m);
    }
  }
}

// ------------------------------------------------------------------ host side

constexpr int MAX_ENV_TOKENS = 512;  // split-attention path: q, k, v of one head of one environment in shared memory

bool supported(int d_model, int n_heads, int max_tokens_per_env) {
  return d_model == D && n_heads == HEADS && max_tokens_per_env >= 1 && max_tokens_per_env <= MAX_ENV_TOKENS;
}
// Environments that fit one 128-row tile run fully fused; larger ones take the split path.
static bool fits_tile(const BnbBatch& b) { return b.max_tokens_per_env <= TILE; }
bool supported_batch(int d_model, int n_heads, const BnbBatch& b) {
  if (!supported(d_model, n_heads, b.max_tokens_per_env)) return false;
  if (b.tok_off) return fits_tile(b) && b.tile_env_begin != nullptr && b.tile_env_ids != nullptr && b.n_tiles > 0;
  return b.tokens_per_env >= 1;
}

int plan_tiles(const int32_t* tok_off, int n_envs, int32_t* tile_env_begin, int32_t* tile_env_ids, int capacity,
               int* n_tiles) {
  // Best-fit decreasing: environments sorted by size (counting sort, sizes 1..128), each put into
  // the open tile with the least room that still takes it.  Tiles are then listed as ranges of
  // tile_env_ids.  Near-full tiles matter: a tile costs about the same whatever its fill.
  if (capacity < n_envs + 1) return BNB_ERR_SCRATCH_TOO_SMALL;
  std::vector<int> order;
  order.reserve(n_envs);
  {
    std::vector<std::vector<int>> by_size(TILE + 1);
    for (int e = 0; e < n_envs; ++e) {
      const int n = tok_off[e + 1] - tok_off[e];
      if (n <= 0 || n > TILE) return BNB_ERR_TOO_MANY_TOKENS;
      by_size[n].push_back(e);
    }
    for (int n = TILE; n >= 1; --n) order.insert(order.end(), by_size[n].begin(), by_size[n].end());
  }
  std::vector<std::vector<int>> tiles;                   // environments of each tile
  std::vector<std::vector<int>> open_by_room(TILE + 1);  // tiles with exactly r free rows
  for (int e : order) {
    const int n = tok_off[e + 1] - tok_off[e];
    int room = -1;
    for (int r = n; r <= TILE; ++r)
      if (!open_by_room[r].empty()) { room = r; break; }
    int t;
    if (room < 0) {
      t = (int)tiles.size();
      tiles.emplace_back();
      room = TILE;
    } else {
      t = open_by_room[room].back();
      open_by_room[room].pop_back();
    }
    tiles[t].push_back(e);
    open_by_room[room - n].push_back(t);
  }
  int k = 0;
  for (size_t t = 0; t < tiles.size(); ++t) {
    tile_env_begin[t] = k;
    for (int e : tiles[t]) tile_env_ids[k++] = e;
  }
  tile_env_begin[tiles.size()] = k;
  *n_tiles = (int)tiles.size();
  return BNB_OK;
}

static size_t round256(size_t v) { return (v + 255) / 256 * 256; }
// Shared memory of the attention kernel for environments of up to max_tokens tokens and nb bullets.
static size_t flash_smem(int max_tokens, int nb, int hpc) {
  // staged q, k, v (and bullet k, v) rows, then one bias float per key, each set padded to 32 keys
  return (size_t)(3 * max_tokens + 2 * nb) * flash_stride(hpc) + 4 * (size_t)(((max_tokens + 31) & ~31) + ((nb + 31) & ~31)) + 16;
}
constexpr size_t FLASH_SMEM_MAX = 227 * 1024;
// All four heads in one CTA while that leaves room for three CTAs per SM, else one head per CTA.
static int flash_heads_per_cta(int max_tokens, int nb) {
  return flash_smem(max_tokens, nb, HEADS) <= 72 * 1024 ? HEADS : 1;
}
bool supported_bullets(const BnbBatch& b, int bullets_per_env) {
  return bullets_per_env >= 1 && flash_smem(b.max_tokens_per_env, bullets_per_env, 1) <= FLASH_SMEM_MAX;
}

// Layout: status area | q|k|v and attention output of every row (split path: environments larger
// than a tile, or any sublayer reading bullets) | bullet keys and values of one slice of environments.
size_t scratch_bytes(int, const BnbBatch& b, int T, int bullets_per_env) {
  size_t bytes = 65536;  // status word (and cycle accounting)
  if (!fits_tile(b) || bullets_per_env > 0)
    bytes += round256((size_t)T * b.total_tokens * 4 * D * sizeof(__nv_bfloat16));
  bytes += round256(bullet_slice_bytes((long long)T * b.n_envs, bullets_per_env, D, sizeof(__nv_bfloat16)));
  if (bullets_per_env > 0) {
    // env_off (slice environments + 1) and idx (one int per bullet row of a slice)
    const size_t envs = (size_t)bullet_slice_envs((long long)T * b.n_envs, bullets_per_env, D, sizeof(__nv_bfloat16));
    bytes += round256((envs + 1) * sizeof(int)) + round256(envs * bullets_per_env * sizeof(int));
  }
  return bytes;
}
size_t packed_spatial_bytes(int d_model) { return d_model == D ? (size_t)N_SPATIAL_IMAGE * CHUNK_BYTES : 0; }
size_t packed_temporal_bytes(int d_model) { return d_model == D ? (size_t)N_TEMPORAL_CHUNKS * CHUNK_BYTES + 1024 : 0; }

int pack_spatial(const BnbSpatialWeights& w, int d_model, int n_heads, void* packed, cudaStream_t st) {
  if (d_model != D || n_heads != HEADS) return BNB_ERR_UNSUPPORTED_DIMS;
  count_launch();
  k_pack_spatial<<<148, 256, 0, st>>>(w, static_cast<uint8_t*>(packed));
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}
int pack_temporal(const BnbTemporalWeights& w, int d_model, void* packed, cudaStream_t st) {
  if (d_model != D) return BNB_ERR_UNSUPPORTED_DIMS;
  count_launch();
  k_pack_temporal<<<148, 256, 0, st>>>(w, static_cast<uint8_t*>(packed));
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

int pack_trunk(const BnbSpatialWeights* spatial, int n_spatial, const BnbTemporalWeights* temporal, int n_temporal,
               int d_model, int n_heads, cudaStream_t st) {
  if (d_model != D || n_heads != HEADS) return BNB_ERR_UNSUPPORTED_DIMS;
  // as many launches as it takes at MAX_PACK_JOBS sublayers of each kind per launch (one for the
  // trunks of the shipped profiles)
  for (int s0 = 0, t0 = 0; s0 < n_spatial || t0 < n_temporal;) {
    PackJobs jobs{};
    for (; s0 < n_spatial && jobs.n_spatial < MAX_PACK_JOBS; ++s0) {
      if (!spatial[s0].packed) return BNB_ERR_NULL_POINTER;
      jobs.sw[jobs.n_spatial++] = spatial[s0];
    }
    for (; t0 < n_temporal && jobs.n_temporal < MAX_PACK_JOBS; ++t0) {
      if (!temporal[t0].packed) return BNB_ERR_NULL_POINTER;
      jobs.tw[jobs.n_temporal++] = temporal[t0];
    }
    count_launch();
    k_pack_trunk<<<dim3(24, jobs.n_spatial + jobs.n_temporal), 256, 0, st>>>(jobs);
    if (cudaGetLastError() != cudaSuccess) return BNB_ERR_LAUNCH;
  }
  return BNB_OK;
}

// ------------------------------------------------------------------ status word on the host
//
// The bounded waits record a code in the status word at the head of the scratch buffer.  Every
// call copies that word to a pinned host word of its device when its kernels are done
// (asynchronously, on the call's stream); whoever asks later -- the next call, or
// bnb_last_status -- finds a non-zero code there and keeps it until it is cleared.
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_status_mutex;
int* g_host_status[kMaxDevices] = {};
int g_sticky_status[kMaxDevices] = {};

void latch_status(int dev) {
  if (g_host_status[dev]) {
    const int v = *static_cast<volatile int*>(g_host_status[dev]);
    if (v != 0 && g_sticky_status[dev] == 0) g_sticky_status[dev] = v;
  }
}
}  // namespace

int report_status(const int* status, cudaStream_t st) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return BNB_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_host_status[dev]) {
    // the first call on a device allocates the word; it should not come during a stream capture
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return BNB_OK;
    void* p = nullptr;
    if (cudaHostAlloc(&p, 64, cudaHostAllocDefault) != cudaSuccess) { (void)cudaGetLastError(); return BNB_OK; }
    g_host_status[dev] = static_cast<int*>(p);
    *g_host_status[dev] = 0;
  }
  latch_status(dev);
  if (cudaMemcpyAsync(g_host_status[dev], status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return BNB_ERR_LAUNCH;
  return BNB_OK;
}
int last_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  latch_status(dev);
  return g_sticky_status[dev];
}
void clear_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  g_sticky_status[dev] = 0;
  if (g_host_status[dev]) *g_host_status[dev] = 0;
}
void debug_wait_test(int skip_op, int poll_limit) {
  g_debug_skip_op = skip_op;
  g_debug_poll_limit = poll_limit;
}

static int launch(TrunkArgs& a, const BnbBatch& b, cudaStream_t st) {
  a.map = make_env_map(b);
  if (a.flat_rows) {
    a.tile_env_begin = nullptr;
    a.envs_per_tile = 0;
    a.env_tiles = (b.total_tokens + TILE - 1) / TILE;
  } else if (b.tok_off) {
    a.tile_env_begin = b.tile_env_begin;
    a.tile_env_ids = b.tile_env_ids;
    a.envs_per_tile = 0;
    a.env_tiles = b.n_tiles;
  } else {
    a.tile_env_begin = nullptr;
    a.envs_per_tile = TILE / b.tokens_per_env;
    a.env_tiles = (b.n_envs + a.envs_per_tile - 1) / a.envs_per_tile;
  }
  a.n_tiles = a.env_tiles * a.n_groups;
  a.has_fields = b.total_tokens > b.total_ships ? 1 : 0;
  a.poll_limit = g_debug_poll_limit;
  a.skip_op = g_debug_skip_op;
  if (a.n_tiles == 0) return BNB_OK;
  {
    // the pipelined kernel runs every program of spatial (whole or split around the attention
    // kernel) and temporal sublayers; whole spatial sublayers need tiles of whole environments
    bool fused = !a.row_index && !a.n_rows_dev;
    for (int i = 0; i < a.n_sub; ++i) {
      const int t = a.sub[i].type;
      fused = fused && ((t == SUB_SPATIAL && !a.flat_rows) || t == SUB_TEMPORAL || t == SUB_SPATIAL_PRE || t == SUB_SPATIAL_POST);
    }
    const char* force_old = getenv("BNB_OLD_TILE_KERNEL");
    if (fused && !(force_old && force_old[0] == '1')) return launch_pipelined(a, st);
  }
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BNB_ERR_NO_DEVICE;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(k_trunk_tiles<2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(k_trunk_tiles<2, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(k_trunk_tiles<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(k_trunk_tiles<4, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return BNB_ERR_LAUNCH;
    configured[dev] = true;
  }
  // Two variants: two CTAs per SM with two threads per row (four threads per row would have 64
  // registers each and spill), or one CTA per SM with four threads per row and the full register
  // budget, in which a tile takes about 0.6 of the time but only one runs per SM: it wins when
  // the tiles fit one per SM (measured no better at 297..444 tiles, three of its rounds against
  // two of the other's).
  const bool one_per_sm = a.n_tiles <= 148;
  int grid = one_per_sm ? (a.n_tiles < 148 ? a.n_tiles : 148) : (a.n_tiles < 2 * 148 ? a.n_tiles : 2 * 148);
  count_launch();
  const bool small_keys = b.max_tokens_per_env <= 64 || a.flat_rows;
  if (one_per_sm) {
    if (small_keys) k_trunk_tiles<4, 4><<<grid, 512, SMEM_BYTES, st>>>(a);
    else k_trunk_tiles<4, 8><<<grid, 512, SMEM_BYTES, st>>>(a);
  } else if (small_keys) {
    k_trunk_tiles<2, 4><<<grid, 256, SMEM_BYTES, st>>>(a);
  } else {
    k_trunk_tiles<2, 8><<<grid, 256, SMEM_BYTES, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

static int prepare_status(void* scratch, size_t scratch_bytes, cudaStream_t st, int** status) {
  if (!scratch) return BNB_ERR_NULL_POINTER;
  if (scratch_bytes < 65536) return BNB_ERR_SCRATCH_TOO_SMALL;
  *status = static_cast<int*>(scratch);
  if (cudaMemsetAsync(scratch, 0, 256, st) != cudaSuccess) return BNB_ERR_LAUNCH;
  return BNB_OK;
}

static void fill_spatial(SubLayer& s, const BnbSpatialWeights& w) {
  s = SubLayer{};
  s.type = SUB_SPATIAL;
  s.packed = static_cast<const uint8_t*>(w.packed);
}
static void fill_temporal(SubLayer& s, const BnbTemporalWeights& w, const float* hin, float* hout) {
  s = SubLayer{};
  s.type = SUB_TEMPORAL;
  s.packed = static_cast<const uint8_t*>(w.packed);
  s.conv_w = w.conv_w;
  s.conv_b = w.conv_b;
  s.a_b = w.a_b;
  s.x_b = w.x_b;
  s.decay_log2 = reinterpret_cast<const float*>(static_cast<const uint8_t*>(w.packed) + (size_t)N_TEMPORAL_CHUNKS * CHUNK_BYTES);
  s.hid_in = hin;
  s.hid_out = hout;
}

// Attention of the environments [env_base, env_base + n_env) (group-major), with the bullet keys
// of the same environments in kvb when nb > 0.
static int launch_attention(const __nv_bfloat16* qkv, const uint8_t* alive, __nv_bfloat16* o, const BnbBatch& b,
                            int env_base, int n_env, const __nv_bfloat16* kvb, const int* env_off, int nb,
                            cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BNB_ERR_NO_DEVICE;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(k_attention_flash, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FLASH_SMEM_MAX) != cudaSuccess)
      return BNB_ERR_LAUNCH;
    configured[dev] = true;
  }
  if (n_env <= 0) return BNB_OK;
  const int hpc = flash_heads_per_cta(b.max_tokens_per_env, kvb ? nb : 0);
  const size_t smem = flash_smem(b.max_tokens_per_env, kvb ? nb : 0, hpc);
  if (smem > FLASH_SMEM_MAX) return BNB_ERR_TOO_MANY_TOKENS;
  dim3 grid(n_env, HEADS / hpc);
  // warps per CTA: the fewest idle warp-rounds over the (head, query block) pairs of a full environment
  const int items = hpc * ((b.max_tokens_per_env + 15) / 16);
  int n_warps = 4, best_idle = 1 << 30;
  for (int w = 4; w <= 8; ++w) {
    const int idle = (items + w - 1) / w * w - items;
    if (idle < best_idle) { best_idle = idle; n_warps = w; }
  }
  count_launch();
  k_attention_flash<<<grid, 32 * n_warps, smem, st>>>(qkv, alive, o, make_env_map(b), env_base, hpc, kvb, env_off, nb);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

// env_off / idx of the active bullets of n_env environments (see the compaction kernels).
static int launch_compact(const uint8_t* active, int n_env, int nb, int* env_off, int* idx, cudaStream_t st) {
  if (n_env <= 0) return BNB_OK;
  const int blocks = (n_env + 7) / 8 < 148 * 8 ? (n_env + 7) / 8 : 148 * 8;
  count_launch();
  k_bullet_count<<<blocks, 256, 0, st>>>(active, n_env, nb, env_off);
  count_launch();
  k_bullet_scan<<<1, 1024, 0, st>>>(env_off, n_env);
  count_launch();
  k_bullet_fill<<<blocks, 256, 0, st>>>(active, n_env, nb, env_off, idx);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

// norm_bullet + kv_bullet of bullet rows (a slice of whole environments) into kvb: all `rows`
// rows in order, or, with idx / n_rows_dev, the first *n_rows_dev rows of idx.
static int launch_bullet_kv(const BnbSpatialWeights& w, const float* bullet_rows, bool rows_bf16, int rows, const int* idx,
                            const int* n_rows_dev, __nv_bfloat16* kvb, int* status, cudaStream_t st) {
  if (rows <= 0) return BNB_OK;
  TrunkArgs a{};
  a.x = bullet_rows;
  a.row_index = idx;
  a.n_rows_dev = n_rows_dev;
  a.y = nullptr;              // nothing but the keys and values leaves this program
  a.io_bf16 = rows_bf16 ? 1 : 0;
  a.status = status;
  a.n_groups = 1;
  a.t_loop = 1;
  a.n_sub = 1;
  a.flat_rows = 1;
  a.sub[0].type = SUB_BULLET_KV;
  a.sub[0].packed = static_cast<const uint8_t*>(w.packed);
  a.sub[0].kvb_out = kvb;
  BnbBatch rb{};              // every bullet row is a one-token environment without state
  rb.n_envs = rows;
  rb.tokens_per_env = 1;
  rb.max_tokens_per_env = 1;
  rb.total_tokens = rows;
  return launch(a, rb, st);
}

// Accumulates sublayers into tile-kernel launches.  In split mode (environments larger than
// one tile) a spatial sublayer becomes PRE | attention kernel | POST, and the tile kernel
// walks plain 128-row slices.  A sublayer that reads bullets takes the same three-part form
// whatever the environment size, with the bullet key/value projection and the attention kernel
// run once per slice of environments.
struct Plan {
  const BnbBatch& b;
  cudaStream_t st;
  int* status;
  bool split;
  const uint8_t* alive;
  const uint8_t* done;
  const uint8_t* reset_env;
  const float* cur;      // where the residual stream currently lives
  float* y;
  const BnbBullets* bullets;
  __nv_bfloat16* qkv;
  __nv_bfloat16* o;
  __nv_bfloat16* kvb;    // bullet keys and values of one slice
  int kvb_envs;          // environments per slice
  int* env_off;          // compaction of the slice's active bullets (see launch_compact)
  int* idx;
  int compacted_e0;      // first environment of the slice env_off / idx currently describe, -1 = none
  bool io_bf16 = false;  // x and y (and so the stream between launches) hold bfloat16
  int n_groups, t_loop;  // geometry of the pending program
  TrunkArgs a;
  int n;

  void begin(int groups, int tl) {
    a = TrunkArgs{};
    n = 0;
    n_groups = groups;
    t_loop = tl;
  }
  int flush() {
    if (n == 0) return BNB_OK;
    a.status = status;
    a.alive = split ? nullptr : alive;
    a.done = done;
    a.reset_env = reset_env;
    a.n_groups = n_groups;
    a.t_loop = t_loop;
    a.n_sub = n;
    a.flat_rows = split ? 1 : 0;
    a.io_bf16 = io_bf16 ? 1 : 0;
    a.x = cur;
    a.y = y;
    int rc = launch(a, b, st);
    cur = y;
    const int g = n_groups, tl = t_loop;
    begin(g, tl);
    return rc;
  }
  int ensure(int groups, int tl) {
    if (n > 0 && (groups != n_groups || tl != t_loop)) {
      int rc = flush();
      if (rc) return rc;
    }
    n_groups = groups;
    t_loop = tl;
    return BNB_OK;
  }
  int add_spatial(const BnbSpatialWeights& w, int groups) {
    int rc = ensure(groups, 1);
    if (rc) return rc;
    if (n == MAX_SUBLAYERS && (rc = flush())) return rc;
    const bool reads = bullets && w.kv_bullet_w;
    fill_spatial(a.sub[n], w);
    if (!split && !reads) { ++n; return BNB_OK; }
    a.sub[n].type = SUB_SPATIAL_PRE;
    a.sub[n].qkv_out = qkv;
    ++n;
    if ((rc = flush())) return rc;
    const int total_envs = groups * b.n_envs;
    if (reads) {
      const int nb = bullets->per_env;
      for (int e0 = 0; e0 < total_envs; e0 += kvb_envs) {
        const int ne = total_envs - e0 < kvb_envs ? total_envs - e0 : kvb_envs;
        const bool masked = bullets->active != nullptr;
        if (masked && compacted_e0 != e0) {
          // the mask is the same for every reading sublayer of the call: one slice -> compact once
          if ((rc = launch_compact(bullets->active + (size_t)e0 * nb, ne, nb, env_off, idx, st))) return rc;
          compacted_e0 = e0;
        }
        const bool rows_bf16 = bullets->tokens_bf16 != 0;
        const float* rows0 = rows_bf16
            ? reinterpret_cast<const float*>(reinterpret_cast<const __nv_bfloat16*>(bullets->tokens) + (size_t)e0 * nb * D)
            : bullets->tokens + (size_t)e0 * nb * D;
        if ((rc = launch_bullet_kv(w, rows0, rows_bf16, ne * nb, masked ? idx : nullptr,
                                   masked ? env_off + ne : nullptr, kvb, status, st)))
          return rc;
        if ((rc = launch_attention(qkv, alive, o, b, e0, ne, kvb, masked ? env_off : nullptr, nb, st))) return rc;
      }
    } else if ((rc = launch_attention(qkv, alive, o, b, 0, total_envs, nullptr, nullptr, 0, st))) {
      return rc;
    }
    fill_spatial(a.sub[n], w);
    a.sub[n].type = SUB_SPATIAL_POST;
    a.sub[n].o_in = o;
    ++n;
    return BNB_OK;
  }
  int add_temporal(const BnbTemporalWeights& w, const float* hin, float* hout, int tl) {
    int rc = ensure(tl > 1 ? 1 : n_groups, tl);
    if (rc) return rc;
    if (tl > 1 && n > 0 && (rc = flush())) return rc;   // a time walk runs alone
    if (n == MAX_SUBLAYERS && (rc = flush())) return rc;
    fill_temporal(a.sub[n++], w, hin, hout);
    if (tl > 1) return flush();
    return BNB_OK;
  }
};

static int make_plan(Plan& p, void* scratch, size_t scratch_bytes, int T) {
  int rc = prepare_status(scratch, scratch_bytes, p.st, &p.status);
  if (rc) return rc;
  p.split = !fits_tile(p.b);
  p.qkv = nullptr;
  p.o = nullptr;
  p.kvb = nullptr;
  p.kvb_envs = 0;
  const int nb = p.bullets ? p.bullets->per_env : 0;
  if (nb > 0 && !supported_bullets(p.b, nb)) return BNB_ERR_UNSUPPORTED_DIMS;
  if (scratch_bytes < tensor::scratch_bytes(D, p.b, T, nb)) return BNB_ERR_SCRATCH_TOO_SMALL;
  uint8_t* base = static_cast<uint8_t*>(scratch) + 65536;
  if (p.split || nb > 0) {
    const size_t rows = (size_t)T * p.b.total_tokens;
    p.qkv = reinterpret_cast<__nv_bfloat16*>(base);
    p.o = p.qkv + rows * 3 * D;
    base += round256(rows * 4 * D * sizeof(__nv_bfloat16));
  }
  p.env_off = nullptr;
  p.idx = nullptr;
  p.compacted_e0 = -1;
  if (nb > 0) {
    p.kvb = reinterpret_cast<__nv_bfloat16*>(base);
    p.kvb_envs = bullet_slice_envs((long long)T * p.b.n_envs, nb, D, sizeof(__nv_bfloat16));
    base += round256(bullet_slice_bytes((long long)T * p.b.n_envs, nb, D, sizeof(__nv_bfloat16)));
    p.env_off = reinterpret_cast<int*>(base);
    base += round256(((size_t)p.kvb_envs + 1) * sizeof(int));
    p.idx = reinterpret_cast<int*>(base);
  }
  p.begin(1, 1);
  return BNB_OK;
}

int spatial_block(const BnbSpatialWeights& w, int d_model, int n_heads, const float* x, const uint8_t* alive,
                  const BnbBullets* bullets, float* y, const BnbBatch& b, int n_groups, void* scratch,
                  size_t scratch_bytes, cudaStream_t st) {
  if (!supported_batch(d_model, n_heads, b) || !w.packed) return BNB_ERR_UNSUPPORTED_DIMS;
  Plan p{b, st, nullptr, false, alive, nullptr, nullptr, x, y, bullets};
  int rc = make_plan(p, scratch, scratch_bytes, n_groups);
  if (rc) return rc;
  if ((rc = p.add_spatial(w, n_groups))) return rc;
  if ((rc = p.flush())) return rc;
  return report_status(p.status, st);
}

int temporal_block(const BnbTemporalWeights& w, int d_model, const float* x, float* y, const float* hidden_in,
                   float* hidden_out, const uint8_t* done, const uint8_t* reset_env, const BnbBatch& b, int T,
                   void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (!supported_batch(d_model, HEADS, b) || !w.packed) return BNB_ERR_UNSUPPORTED_DIMS;
  Plan p{b, st, nullptr, false, nullptr, done, reset_env, x, y, nullptr};
  int rc = make_plan(p, scratch, scratch_bytes, T);
  if (rc) return rc;
  if ((rc = p.add_temporal(w, hidden_in, hidden_out, T))) return rc;
  if ((rc = p.flush())) return rc;
  return report_status(p.status, st);
}

int trunk(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal, int n_blocks, int n_spatial,
          int n_temporal, int d_model, int n_heads, const float* x, const uint8_t* alive, const BnbBullets* bullets,
          float* y, const float* hidden_in, float* hidden_out, const uint8_t* done, const uint8_t* reset_env,
          const BnbBatch& b, int T, void* scratch, size_t scratch_bytes, cudaStream_t st, bool io_bf16) {
  if (!supported_batch(d_model, n_heads, b)) return BNB_ERR_UNSUPPORTED_DIMS;
  // bfloat16 x / y: every tile-kernel launch of the call reads and writes bfloat16 rows, so the
  // residual stream is rounded where one launch hands over to the next (the reference, given
  // bfloat16 tokens, rounds it after every sublayer)
  for (int i = 0; i < n_blocks * n_spatial; ++i) if (!spatial[i].packed) return BNB_ERR_UNSUPPORTED_DIMS;
  for (int i = 0; i < n_blocks * n_temporal; ++i) if (!temporal[i].packed) return BNB_ERR_UNSUPPORTED_DIMS;
  // a time walk carries its state through hidden_out between timesteps
  if (T > 1 && n_blocks * n_temporal > 0 && b.total_ships > 0 && !hidden_out) return BNB_ERR_NULL_POINTER;
  Plan p{b, st, nullptr, false, alive, done, reset_env, x, y, bullets};
  p.io_bf16 = io_bf16;
  int rc = make_plan(p, scratch, scratch_bytes, T);
  if (rc) return rc;
  const size_t slot_stride = (size_t)b.total_ships * 4 * D;
  for (int i = 0; i < n_blocks; ++i) {
    for (int j = 0; j < n_spatial; ++j)
      if ((rc = p.add_spatial(spatial[i * n_spatial + j], T))) return rc;
    for (int j = 0; j < n_temporal; ++j) {
      const int slot = i * n_temporal + j;
      if ((rc = p.add_temporal(temporal[slot], hidden_in ? hidden_in + slot * slot_stride : nullptr,
                               hidden_out ? hidden_out + slot * slot_stride : nullptr, T))) return rc;
    }
  }
  if ((rc = p.flush())) return rc;
  if (p.cur == x && y != x) {
    if (cudaMemcpyAsync(y, x, (size_t)T * b.total_tokens * D * (io_bf16 ? 2 : sizeof(float)), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return BNB_ERR_LAUNCH;
  }
  return report_status(p.status, st);
}

}  // namespace tensor
}  // namespace bnb
