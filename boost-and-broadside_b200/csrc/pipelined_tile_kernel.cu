// The fused trunk kernel for sm_100a: one CTA per SM walks a tile of 128 token rows (whole
// environments) through a program of spatial and temporal sublayers, with the residual stream
// resident in tensor memory and three warp roles that only meet at mbarriers:
//
//   16 epilogue warps   four threads per tile row (thread (row, part): TMEM lane = row, a quarter
//                       of whatever columns are being read).  RMSNorm, q|k|v staging, attention
//                       (mma.sync), gelu(gate) * up, causal conv, RG-LRU gates and state update.
//   1 issuing warp      one lane issues every tcgen05.mma.  It waits for "operand ready" (the
//                       epilogue warps arrive on an mbarrier after fence.proxy.async) and for
//                       "chunk landed" (the bulk copy's complete_tx), and signals "accumulator
//                       ready" / "slot free" with tcgen05.commit.
//   1 fetching warp     one lane streams the pre-tiled weight image through a ring of nine
//                       16 KB slots with cp.async.bulk, following a static schedule.
//
//   TMEM  [0,128)    residual stream, fp32, lane = tile row (out_proj, linear_out and down_proj
//                    accumulate straight into it)
//         [128,512)  three 128-column accumulators.  q|k|v of all four heads fill them in one
//                    round; the GatedMLP runs them as a three-deep pipeline: gate|up of chunk
//                    c + 3 is issued as soon as chunk c has been read, so the tensor pipe works
//                    on chunks c + 1 .. c + 3 while the epilogue warps turn chunk c into the bf16
//                    operand of its down projection.
//
//   SMEM  A (32 KB)  normed activations (K-major, 128-byte swizzle); q of all heads during
//                    attention.   P (2 x 16 KB)  gelu(gate) * up, double buffered; attention
//                    output; RG-LRU branch.   KV (64 KB)  keys and values of all heads during
//                    attention, four more ring slots otherwise.   Ring (5 x 16 KB).
//
// Every mbarrier wait is bounded: a wait that runs out records a code in the status word, later
// waits give up at once, and the kernel drains and returns.
//
// Reference arithmetic: models/yemong/attention.py:76-169, models/yemong/griffin.py:67-317.
#include "launch_count.h"
#include "tensor_common.cuh"
#include "tensor_kernels.h"

namespace bnb {
namespace tensor {
namespace pipe {

constexpr int EPI_WARPS = 16;
constexpr int EPI_THREADS = 32 * EPI_WARPS;
constexpr int MMA_WARP = EPI_WARPS;
constexpr int LOAD_WARP = EPI_WARPS + 1;
constexpr int THREADS = EPI_THREADS + 64;
// Weight ring: three pair slots (32 KB: both K atoms of one 128-row weight block, consumed by
// eight MMAs) and three single slots (16 KB: one down-projection chunk).  Slots 0, 1 (pairs) and
// 3 (single) are dedicated; 2, 4 and 5 live in the key/value staging area and carry weights only
// while no attention runs.
constexpr int N_SLOTS = 6;
constexpr int RING_BYTES = 5 * CHUNK_BYTES;

constexpr int OFF_A = 0;
constexpr int OFF_P = 32768;
constexpr int OFF_KV = 65536;
constexpr int OFF_RING = 131072;
constexpr int OFF_META = OFF_RING + RING_BYTES;  // env_first[128], env_n[128], alive[128], items[128]
constexpr int OFF_ROWINFO = OFF_META + 512;                     // hidden row of each tile row (int), then flags[128]
constexpr int OFF_SS = OFF_ROWINFO + 640;                       // partial sums of squares [4][128]
constexpr int OFF_BIAS = OFF_SS + 2048;                         // attention bias of each tile row as a key (float), + 16 of slack
constexpr int OFF_BAR = OFF_BIAS + 576;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;

// mbarrier indices
// OP: operand ready (epilogue warps -> issuing lane).  KVREL: the key/value area may take weights
// again (epilogue warps -> fetching lane).  FULL[s]: the weights of slot s have landed.  DONE[s]:
// the MMAs that read slot s are complete (tcgen05.commit) -- the fetching lane takes it as "slot
// free" and, inside the GatedMLP pipeline, the epilogue warps as "accumulator ready" / "product
// buffer read": one commit per ring operation serves both.  ACC: every MMA of a round outside the
// GatedMLP pipeline is complete (one more commit per round).  DRAIN: every MMA of the CTA is
// complete (once, at the end).
enum : int { B_OP0 = 0, B_OP1, B_KVREL, B_ACC, B_DRAIN, B_FULL0, B_DONE0 = B_FULL0 + N_SLOTS, B_COUNT = B_DONE0 + N_SLOTS };
static_assert(B_COUNT * 8 + 8 <= 256, "barrier area");

constexpr uint32_t COL_RESID = 0;
constexpr uint32_t COL_ACC0 = 128, COL_ACC1 = 256, COL_ACC2 = 384;
constexpr uint32_t TMEM_COLS = 512;

enum : int { ST_TIMEOUT_FULL = 101, ST_TIMEOUT_FREE = 102, ST_TIMEOUT_ACC = 103, ST_TIMEOUT_OPERAND = 104 };

// Optional cycle accounting (compile with -DBNB_TIMING): thread 0 (an epilogue thread), the
// issuing lane and the fetching lane of every CTA add up the cycles they spend in each phase and
// store them behind the status word: 32 counters per CTA from byte 256 on.
enum : int { TE_ACC_WAIT = 0, TE_FFN_ACC_WAIT, TE_FFN_PF_WAIT, TE_FFN_MATH, TE_NORM, TE_STAGE, TE_ATTN, TE_SYNC, TE_TEMPORAL,
             TE_IO, TE_TOTAL, TM_FULL_WAIT, TM_OP_WAIT, TM_ISSUE, TM_TOTAL, TL_FREE_WAIT, TL_KV_WAIT, TL_TOTAL, T_COUNT };
#ifdef BNB_TIMING
#define T_BEGIN() const long long _t0 = clock64()
#define T_END(acc, slot) (acc)[slot] += clock64() - _t0
#define T_WAITSLOT(e, s) (e).wait_slot = (s)
#define T_MARK(name) long long name = clock64()
#define T_RESET(name) name = clock64()
#define T_SINCE(acc, slot, name) do { const long long _n = clock64(); (acc)[slot] += _n - name; name = _n; } while (0)
#define T_STORE(args, acc, lo, hi) for (int _i = lo; _i < hi; ++_i) reinterpret_cast<long long*>((args).status)[32 + blockIdx.x * 32 + _i] = (acc)[_i]
#else
#define T_BEGIN()
#define T_END(acc, slot)
#define T_WAITSLOT(e, s)
#define T_MARK(name)
#define T_RESET(name)
#define T_SINCE(acc, slot, name)
#define T_STORE(args, acc, lo, hi)
#endif

// Optional event trace (compile with -DBNB_TRACE): CTA 0 records (event id, clock) pairs of one
// epilogue thread, the issuing lane and the fetching lane from byte 16384 of the status area on,
// 1500 events per role.
#ifdef BNB_TRACE
struct Trace { unsigned long long* buf; int n; };
__device__ __forceinline__ void trace_init(Trace& t, int* status, int role) {
  t.buf = reinterpret_cast<unsigned long long*>(status) + 2048 + role * 1500;
  t.n = blockIdx.x == 0 ? 0 : 1500;
}
__device__ __forceinline__ void trace(Trace& t, int id) {
  if (t.n < 1500) t.buf[t.n++] = ((unsigned long long)id << 48) | ((unsigned long long)clock64() & 0xFFFFFFFFFFFFull);
}
#define TRACE(t, id) trace(t, id)
#else
#define TRACE(t, id)
#endif

// Schedule entry of one ring operation: slot (3 bits) | sublayer (3) | first chunk (6) | second
// chunk (6; 63 = none: a single) | wait for the key/value area first (1).
constexpr uint32_t NO_CHUNK = 63;
__device__ __forceinline__ uint32_t sched_entry(int slot, int si, int ch0, int ch1, bool kvwait) {
  return (uint32_t)slot | ((uint32_t)si << 3) | ((uint32_t)ch0 << 6) | ((uint32_t)ch1 << 12) | (kvwait ? 1u << 18 : 0u);
}
constexpr int MAX_SCHED = MAX_SUBLAYERS * 22;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Ring operations of a sublayer in the order the issuing lane consumes them.  GatedMLP with
// image base b: gate|up of chunk c are chunks b + 3c, b + 3c + 1 (a pair), its down projection is
// b + 3c + 2 (a single); the three-deep pipeline consumes GU0 GU1 GU2 D0 GU3 D1 GU4 D2 ... GU7 D5 D6 D7.
struct SlotRotation {
  int pair, single;
  __device__ __forceinline__ int next_pair() { const int r = pair; pair = pair == 2 ? 0 : pair + 1; return r; }
  __device__ __forceinline__ int next_single() { const int r = single; single = single == 5 ? 3 : single + 1; return r; }
};
__device__ __forceinline__ int ffn_ops(uint32_t* out, int n, int si, int base, SlotRotation& rot, int first_flagged) {
  // first_flagged: index (in GU order) of the first gate|up pair that must wait for the key/value area, or -1
  for (int c = 0; c < 3; ++c) out[n++] = sched_entry(rot.next_pair(), si, base + 3 * c, base + 3 * c + 1, c == first_flagged);
  for (int c = 0; c < 8; ++c) {
    out[n++] = sched_entry(rot.next_single(), si, base + 3 * c + 2, NO_CHUNK, false);
    if (c + 3 < 8) out[n++] = sched_entry(rot.next_pair(), si, base + 3 * (c + 3), base + 3 * (c + 3) + 1, false);
  }
  return n;
}
__device__ __forceinline__ int build_schedule(const SubLayer* subs, int n_sub, bool has_fields, uint32_t* out) {
  int n = 0;
  SlotRotation rot{0, 3};
  for (int si = 0; si < n_sub; ++si) {
    if (subs[si].type == SUB_SPATIAL) {
      for (int h = 0; h < HEADS; ++h) {
        const int ch = 5 * (h >> 1) + 2 * (h & 1);
        out[n++] = sched_entry(rot.next_pair(), si, ch, ch + 1, false);
      }
      // fetched while the attention runs: the dedicated slots only.  out_proj -> pair slot 0, the
      // first gate|up -> pair slot 1 and the first down projection -> single slot 3; the second
      // gate|up is the first operation that goes to the key/value area and waits for it.
      out[n++] = sched_entry(0, si, 4, 9, false);
      rot.pair = 1;
      rot.single = 3;
      n = ffn_ops(out, n, si, 10, rot, 1);
    } else if (subs[si].type == SUB_SPATIAL_PRE) {
      // q|k|v only: the attention runs in a kernel of its own between this launch and the next
      for (int h = 0; h < HEADS; ++h) {
        const int ch = 5 * (h >> 1) + 2 * (h & 1);
        out[n++] = sched_entry(rot.next_pair(), si, ch, ch + 1, false);
      }
    } else if (subs[si].type == SUB_SPATIAL_POST) {
      // out_proj on the attention output read back from global memory, then the GatedMLP; nothing
      // of this sublayer uses the key/value area, so no operation waits for it
      out[n++] = sched_entry(rot.next_pair(), si, 4, 9, false);
      n = ffn_ops(out, n, si, 10, rot, -1);
    } else {
      for (int i = 0; i < 6; ++i) {
        if (!has_fields && i == 4) continue;
        out[n++] = sched_entry(rot.next_pair(), si, 2 * i, 2 * i + 1, false);
      }
      n = ffn_ops(out, n, si, 12, rot, -1);
    }
  }
  return n;
}

__device__ __forceinline__ uint32_t slot_offset(uint32_t slot) {
  switch (slot) {
    case 0: return OFF_RING;
    case 1: return OFF_RING + 2 * CHUNK_BYTES;
    case 2: return OFF_KV;
    case 3: return OFF_RING + 4 * CHUNK_BYTES;
    case 4: return OFF_KV + 2 * CHUNK_BYTES;
    default: return OFF_KV + 3 * CHUNK_BYTES;
  }
}

// ------------------------------------------------------------------ epilogue side

struct Epi {
#ifdef BNB_TRACE
  Trace tr;
#endif
#ifdef BNB_TIMING
  long long tacc[T_COUNT];
  int wait_slot;
#endif
  uint8_t* smem;
  uint32_t sbase;       // shared address of smem
  uint32_t bars;        // shared address of the barrier array
  uint32_t lane_addr;   // tensor-memory address of this thread's lane, column 0
  uint32_t par;         // phase bits of the DONE barriers, one per ring slot
  const uint32_t* sched;
  int sched_len, cur;   // cursor into the schedule: the next ring operation this thread waits for
  int row, part;
  int* status;
  volatile int* aborted;
  float* ss_part;
};

// "My share of the operand is written and my reads of the accumulator are done."
__device__ __forceinline__ void post(Epi& e, int bar) {
  TRACE(e.tr, 200 + bar);
  fence_proxy_async();
  tc_fence_before();
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(e.bars + 8 * bar);
  TRACE(e.tr, 210 + bar);
}
// The epilogue threads walk the schedule of ring operations with a cursor of their own and keep
// one phase bit per DONE barrier.
//
// wait_round: a round outside the GatedMLP pipeline (n operations, then a commit on ACC).  The
// threads wait on ACC and flip the phase bits of the n operations, which are complete by then.
__device__ __forceinline__ void wait_round(Epi& e, int n) {
  T_BEGIN();
  mbar_wait(e.bars + 8 * B_ACC, (e.par >> 8) & 1u, e.status, e.aborted, ST_TIMEOUT_ACC);
  e.par ^= 1u << 8;
  for (int i = 0; i < n; ++i) {
    const uint32_t slot = e.sched[e.cur] & 7u;
    e.cur = e.cur + 1 == e.sched_len ? 0 : e.cur + 1;
    e.par ^= 1u << slot;
  }
  tc_fence_after();
  T_END(e.tacc, e.wait_slot);
  TRACE(e.tr, 110 + n);
}
// wait_ops: inside the GatedMLP pipeline the threads wait for each operation on its own DONE
// barrier, in schedule order.  A slot is not reused before the threads have seen its previous
// operation complete: the reuse distance is three operations of a kind, and the issuing lane
// issues gate|up of chunk c + 3 and the down projection of chunk c only after the post of chunk c.
__device__ __forceinline__ void wait_ops(Epi& e, int n) {
  T_BEGIN();
  for (int i = 0; i < n; ++i) {
    const uint32_t slot = e.sched[e.cur] & 7u;
    e.cur = e.cur + 1 == e.sched_len ? 0 : e.cur + 1;
    mbar_wait(e.bars + 8 * (B_DONE0 + slot), (e.par >> slot) & 1u, e.status, e.aborted, ST_TIMEOUT_ACC);
    e.par ^= 1u << slot;
  }
  tc_fence_after();
  T_END(e.tacc, e.wait_slot);
  TRACE(e.tr, 100 + n);
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory"); }

// residual (TMEM) -> x * rsqrt(mean x^2 + eps) -> bf16 A operand (the RMSNorm gain is in the weights)
__device__ __forceinline__ void norm_to_A(Epi& e) {
  TRACE(e.tr, 300);
  T_BEGIN();
  uint32_t v[32];
  tmem_ld32(e.lane_addr + COL_RESID + e.part * 32, v);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float a = __uint_as_float(v[i]);
    ss = fmaf(a, a, ss);
  }
  e.ss_part[e.part * TILE + e.row] = ss;
  // the four warps that share these 32 rows exchange partial sums (named barriers 3..6)
  asm volatile("bar.sync %0, 128;" ::"r"(3 + ((threadIdx.x >> 5) & 3)) : "memory");
  ss = (e.ss_part[e.row] + e.ss_part[TILE + e.row]) + (e.ss_part[2 * TILE + e.row] + e.ss_part[3 * TILE + e.row]);
  const float inv = rsqrtf(ss * (1.0f / D) + kRmsEps);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int col = e.part * 32 + q * 8;
    const uint32_t* s = &v[q * 8];
    uint4 o;
    o.x = pack_bf16(__uint_as_float(s[0]) * inv, __uint_as_float(s[1]) * inv);
    o.y = pack_bf16(__uint_as_float(s[2]) * inv, __uint_as_float(s[3]) * inv);
    o.z = pack_bf16(__uint_as_float(s[4]) * inv, __uint_as_float(s[5]) * inv);
    o.w = pack_bf16(__uint_as_float(s[6]) * inv, __uint_as_float(s[7]) * inv);
    *reinterpret_cast<uint4*>(e.smem + OFF_A + (col >> 6) * CHUNK_BYTES + swz(e.row, (col & 63) >> 3)) = o;
  }
  // the partial sums are read again by the next norm only after at least one full barrier
  T_END(e.tacc, TE_NORM);
}

__device__ __forceinline__ uint4 pack8(const uint32_t* s) {
  return make_uint4(pack_bf16(__uint_as_float(s[0]), __uint_as_float(s[1])), pack_bf16(__uint_as_float(s[2]), __uint_as_float(s[3])),
                    pack_bf16(__uint_as_float(s[4]), __uint_as_float(s[5])), pack_bf16(__uint_as_float(s[6]), __uint_as_float(s[7])));
}

// GatedMLP on the A operand (already normed and posted on OP0): residual += down(gelu(gate) * up).
// Chunk c: gate = acc[c % 3][0,64), up = acc[c % 3][64,128); this thread: hidden columns
// [16 part, 16 part + 16) of the chunk.
__device__ __forceinline__ void ffn(Epi& e) {
#pragma unroll 1
  for (int c = 0; c < 8; ++c) {
    const int ai = c % 3, pi = c & 1;
    T_WAITSLOT(e, TE_FFN_ACC_WAIT);
    wait_ops(e, 1);   // gate|up of chunk c
    T_BEGIN();
    uint32_t gv[16], uv[16];
    const uint32_t acc = e.lane_addr + COL_ACC0 + ai * 128 + e.part * 16;
    tmem_ld16_nowait(acc, gv);
    tmem_ld16_nowait(acc + 64, uv);
    tmem_wait_ld();
    uint4 o[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        w[j] = gelu_mul_bf16x2(__uint_as_float(gv[q * 8 + 2 * j]), __uint_as_float(gv[q * 8 + 2 * j + 1]),
                               __uint_as_float(uv[q * 8 + 2 * j]), __uint_as_float(uv[q * 8 + 2 * j + 1]));
      o[q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    T_END(e.tacc, TE_FFN_MATH);
    // the down projection of chunk c - 2 is next in the schedule: its wait keeps the cursor in step
    T_WAITSLOT(e, TE_FFN_PF_WAIT);
    if (c >= 2) wait_ops(e, 1);
    // The gated product stays in tensor memory as the A operand of the down projection: this
    // thread's 16 k (8 columns of packed bf16 pairs) over the first half of its own 16 gate
    // columns, which it has just read; K step `part` of the MMA reads exactly those columns.
    {
      const uint32_t w8[8] = {o[0].x, o[0].y, o[0].z, o[0].w, o[1].x, o[1].y, o[1].z, o[1].w};
      tmem_st8(e.lane_addr + COL_ACC0 + ai * 128 + e.part * 16, w8);
    }
    post(e, B_OP0 + pi);
  }
  // residual complete: the down projections of chunks 6 and 7
  wait_ops(e, 2);
  T_WAITSLOT(e, TE_ACC_WAIT);
}

// Attention of every head and environment of the tile from the staged q (A area), k and v (KV
// area), all in the swizzled operand layout (128 rows x 64 bf16 atoms; head h sits in atom h / 2,
// columns 32 (h % 2) ..).  Warp w serves head w % 4 and every fourth block of 16 query rows;
// keys are walked in blocks of 16 with a running maximum.  Output: bf16 into the P area as the
// A operand of out_proj.
__device__ __forceinline__ void attention(Epi& e, int n_items) {
  TRACE(e.tr, 310);
  const uint8_t* meta = e.smem + OFF_META;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int h = warp & 3;
  const uint32_t atom = (uint32_t)(h >> 1) * CHUNK_BYTES;
  const int c8h = (h & 1) * 4;
  const uint32_t sQ = e.sbase + OFF_A + atom, sK = e.sbase + OFF_KV + atom, sV = sK + 2 * CHUNK_BYTES;
  const float* key_bias = reinterpret_cast<const float*>(e.smem + OFF_BIAS);
  const float c2 = 0.17677669529663687f * 1.4426950408889634f;  // log2(e) / sqrt(32): scores in the log2 domain
  for (int it = warp >> 2; it < n_items; it += EPI_WARPS / 4) {
    const int r0 = meta[384 + it];
    const int e0 = meta[r0], n = meta[128 + r0] + 1;   // first tile row and size of the environment
    const int last = e0 + n - 1;
    uint32_t qa[2][4];
    {
      const int row = min(r0 + (lane & 7) + ((lane >> 3) & 1) * 8, last);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks)
        ldsm_x4(sQ + swz(row, c8h + ks * 2 + (lane >> 4)), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
    }
    const int nkb = (n + 15) >> 4;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
#pragma unroll 1
    for (int kb = 0; kb < nkb; ++kb) {
      float sc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[nt][i] = 0.f;
      const int krow = min(e0 + kb * 16 + (lane >> 4) * 8 + (lane & 7), last);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sK + swz(krow, c8h + ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma_bf16(sc[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16(sc[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
      float bm0 = -INFINITY, bm1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int j = kb * 16 + nt * 8 + 2 * t + i;
          const bool valid = j < n;
          // a dead key's bias (kMaskedScore) swallows its score: weight exactly 0 unless every key is
          // dead, then uniform; rows past the environment's last are no keys at all
          const float bj = key_bias[e0 + j];
          const float a = valid ? fmaf(sc[nt][i], c2, bj) : -INFINITY;
          const float b = valid ? fmaf(sc[nt][2 + i], c2, bj) : -INFINITY;
          sc[nt][i] = a;
          sc[nt][2 + i] = b;
          bm0 = fmaxf(bm0, a);
          bm1 = fmaxf(bm1, b);
        }
      bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1));
      bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
      bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1));
      bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
      const float n0 = fmaxf(m0, bm0), n1 = fmaxf(m1, bm1);   // finite: every block holds a valid key
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
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float a = ex2_fast(sc[nt][i] - m0), b = ex2_fast(sc[nt][2 + i] - m1);
          sc[nt][i] = a;
          sc[nt][2 + i] = b;
          l0 += a;
          l1 += b;
        }
      const uint32_t a0 = pack_bf16(sc[0][0], sc[0][1]), a1 = pack_bf16(sc[0][2], sc[0][3]);
      const uint32_t a2 = pack_bf16(sc[1][0], sc[1][1]), a3 = pack_bf16(sc[1][2], sc[1][3]);
      const int vrow = min(e0 + kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), last);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sV + swz(vrow, c8h + np * 2 + (lane >> 4)), b0, b1, b2, b3);
        mma_bf16(acc[np * 2], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[np * 2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    const int q0 = r0 + g, q1 = r0 + g + 8;
    uint8_t* po = e.smem + OFF_P + atom;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      if (q0 <= last) *reinterpret_cast<uint32_t*>(po + swz(q0, c8h + nt) + t * 4) = pack_bf16(acc[nt][0] * i0, acc[nt][1] * i0);
      if (q1 <= last) *reinterpret_cast<uint32_t*>(po + swz(q1, c8h + nt) + t * 4) = pack_bf16(acc[nt][2] * i1, acc[nt][3] * i1);
    }
  }
}

__device__ __forceinline__ void run_spatial(Epi& e, int n_items, bool row_valid) {
  norm_to_A(e);
  post(e, B_OP0);
  wait_round(e, HEADS);   // q|k|v of head h in columns [128 + 96 h, +96)
  {
    T_BEGIN();
    // this thread stages head `part` of its row: q into the A area (the normed operand has been
    // consumed), k and v into the KV area, all in the swizzled atom layout
    const int h = e.part;
    const uint32_t atom = (uint32_t)(h >> 1) * CHUNK_BYTES;
    const int c8h = (h & 1) * 4;
    const uint32_t dst[3] = {OFF_A + atom, OFF_KV + atom, OFF_KV + 2 * CHUNK_BYTES + atom};
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      uint32_t v[32];
      tmem_ld32(e.lane_addr + COL_ACC0 + h * 96 + p * 32, v);
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(e.smem + dst[p] + swz(e.row, c8h + q)) = pack8(&v[q * 8]);
    }
    if (!row_valid) {
      // rows outside every environment contribute a zero operand row to out_proj
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(e.smem + OFF_P + atom + swz(e.row, c8h + q)) = make_uint4(0u, 0u, 0u, 0u);
    }
    T_END(e.tacc, TE_STAGE);
  }
  tc_fence_before();
  {
    T_BEGIN();
    epi_sync();
    T_END(e.tacc, TE_SYNC);
  }
  {
    T_BEGIN();
    attention(e, n_items);
    T_END(e.tacc, TE_ATTN);
  }
  // keys and values are dead: the area may take weight chunks again
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(e.bars + 8 * B_KVREL);
  post(e, B_OP0);   // attention output in P
  wait_round(e, 1);   // out_proj accumulated into the residual
  norm_to_A(e);
  post(e, B_OP0);
  ffn(e);
}

// A spatial sublayer around a separate attention kernel (environments larger than a tile, or a
// sublayer that reads bullets).  First part: norm1 and q|k|v of every head, written as bf16 to
// global scratch, (rows, 384) = q | k | v with the heads side by side inside each third.
__device__ __forceinline__ void run_spatial_pre(Epi& e, const SubLayer& s, size_t grow, bool row_valid) {
  norm_to_A(e);
  post(e, B_OP0);
  wait_round(e, HEADS);   // q|k|v of head h in columns [128 + 96 h, +96)
  const int h = e.part;
  __nv_bfloat16* dst = s.qkv_out + grow * (3 * D) + h * DH;
#pragma unroll
  for (int p = 0; p < 3; ++p) {
    uint32_t v[32];
    tmem_ld32(e.lane_addr + COL_ACC0 + h * 96 + p * 32, v);
    if (row_valid) {
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + p * D + q * 8) = pack8(&v[q * 8]);
    }
  }
  tc_fence_before();
}
// Second part: the attention output (bf16, (rows, 128)) becomes the A operand of out_proj, which
// accumulates into the residual; then norm2 and the GatedMLP.
__device__ __forceinline__ void run_spatial_post(Epi& e, const SubLayer& s, size_t grow, bool row_valid) {
  const uint4* src = reinterpret_cast<const uint4*>(s.o_in + grow * D + e.part * 32);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int col = e.part * 32 + q * 8;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (row_valid) o = src[q];
    *reinterpret_cast<uint4*>(e.smem + OFF_A + (col >> 6) * CHUNK_BYTES + swz(e.row, (col & 63) >> 3)) = o;
  }
  post(e, B_OP0);
  wait_round(e, 1);   // out_proj accumulated into the residual
  norm_to_A(e);
  post(e, B_OP0);
  ffn(e);
}

struct RowState {
  int hrow;        // row of the packed hidden state, -1 for field / invalid rows
  int lag_ok;      // stored conv lags still inside the current episode (0..3)
  bool zero_in;    // incoming state taken as zero (reset_env)
};

// One temporal sublayer on the tile at one timestep.  In the gate epilogue thread (row, part)
// works on hidden columns [64 rnd + 16 part, +16), and parks b2 for exactly those.
__device__ __forceinline__ void run_temporal(Epi& e, const SubLayer& s, const RowState& rs, bool is_field, bool boundary,
                                             bool has_fields, const float* hid_in) {
  const bool is_ship = rs.hrow >= 0;
  norm_to_A(e);
  post(e, B_OP0);
  wait_round(e, 2);   // acc0 = linear2 n, acc1 = linear1 n
  T_MARK(tt);
  // b2 = bf16(gelu(linear2 n)) for this thread's columns, parked as packed bf16 pairs
  uint32_t b2p[2][8];
#pragma unroll
  for (int rnd = 0; rnd < 2; ++rnd) {
    uint32_t v[16];
    tmem_ld16_nowait(e.lane_addr + COL_ACC0 + rnd * 64 + e.part * 16, v);
    tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 8; ++j) b2p[rnd][j] = pack_bf16(gelu_fast(__uint_as_float(v[2 * j])), gelu_fast(__uint_as_float(v[2 * j + 1])));
  }
  // b1 = bf16(linear1 n) into the A operand; ships: causal conv with the stored taps -> u
  {
    uint32_t v[32];
    tmem_ld32(e.lane_addr + COL_ACC1 + e.part * 32, v);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int col = e.part * 32 + q * 8;
      *reinterpret_cast<uint4*>(e.smem + OFF_A + (col >> 6) * CHUNK_BYTES + swz(e.row, (col & 63) >> 3)) = pack8(&v[q * 8]);
    }
  }
  tc_fence_before();
  T_SINCE(e.tacc, TE_TEMPORAL, tt);
  epi_sync();
  T_SINCE(e.tacc, TE_SYNC, tt);
  const float* hin = is_ship ? hid_in + (size_t)rs.hrow * 4 * D : nullptr;
  float* hout = is_ship ? s.hid_out + (size_t)rs.hrow * 4 * D : nullptr;
  // Causal conv, one warp per ship row and four columns per lane, so that the stored taps are
  // read and written as whole 512-byte rows.  u = bias + w0 tap0 + w1 tap1 + w2 tap2 + w3 b1,
  // summed in the reference's order; new taps = (tap1, tap2, b1); bf16(u) replaces b1 in A.
  {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = lane * 4;
    float cw[4][4], cb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 w4 = __ldg(reinterpret_cast<const float4*>(s.conv_w + (col + i) * 4));
      cw[i][0] = w4.x; cw[i][1] = w4.y; cw[i][2] = w4.z; cw[i][3] = w4.w;
      cb[i] = __ldg(s.conv_b + col + i);
    }
    const int* row_hrow = reinterpret_cast<const int*>(e.smem + OFF_ROWINFO);
    const uint8_t* row_flags = e.smem + OFF_ROWINFO + 512;
    // Four rows at a time: all loads of the group are issued before any store, because the
    // state may be updated in place and the compiler must otherwise keep loads behind stores.
#pragma unroll 1
    for (int r0 = warp; r0 < TILE; r0 += 4 * EPI_WARPS) {
      float4 t0[4], t1[4], t2[4];
      uint2 bw[4];
      int hr[4], lag[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int r = r0 + EPI_WARPS * k;
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
          bw[k] = *reinterpret_cast<const uint2*>(e.smem + OFF_A + (lane >> 4) * CHUNK_BYTES + swz(r, (lane & 15) >> 1) + (lane & 1) * 8);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (hr[k] < 0) continue;
        const int r = r0 + EPI_WARPS * k;
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
          const float p0 = lag[k] >= 3 ? __fmul_rn(a0[i], cw[i][0]) : 0.f;
          const float p1 = lag[k] >= 2 ? __fmul_rn(a1[i], cw[i][1]) : 0.f;
          const float p2 = lag[k] >= 1 ? __fmul_rn(a2[i], cw[i][2]) : 0.f;
          const float p3 = __fmul_rn(b1[i], cw[i][3]);
          u[i] = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(p0, p1), p2), p3), cb[i]);
        }
        *reinterpret_cast<uint2*>(e.smem + OFF_A + (lane >> 4) * CHUNK_BYTES + swz(r, (lane & 15) >> 1) + (lane & 1) * 8) =
            make_uint2(pack_bf16(u[0], u[1]), pack_bf16(u[2], u[3]));
      }
    }
  }
  post(e, B_OP0);   // A = u (ship rows) / b1 (field rows)
  T_SINCE(e.tacc, TE_TEMPORAL, tt);
  // previous state of this thread's columns of the first half, requested before the gates arrive
  float4 hprev[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    hprev[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (is_ship && !rs.zero_in) hprev[q] = *reinterpret_cast<const float4*>(hin + e.part * 16 + q * 4);
  }
  wait_round(e, has_fields ? 3 : 2);   // acc0 / acc1 = [W_a u | W_x u] of hidden columns [0,64) / [64,128); acc2 = field_sub b1
  T_MARK(tu);
  // gates and state update
#pragma unroll
  for (int rnd = 0; rnd < 2; ++rnd) {
    uint32_t rv[16], iv[16];
    const uint32_t acc = e.lane_addr + COL_ACC0 + rnd * 128 + e.part * 16;
    tmem_ld16_nowait(acc, rv);        // executed by every lane of the warp
    tmem_ld16_nowait(acc + 64, iv);
    tmem_wait_ld();
    float4 hnext[4];
    if (rnd == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        hnext[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (is_ship && !rs.zero_in) hnext[q] = *reinterpret_cast<const float4*>(hin + 64 + e.part * 16 + q * 4);
      }
    }
    if (is_ship) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int col = rnd * 64 + e.part * 16 + q * 8;
        // u (bf16) back from the A operand (K atom rnd)
        uint8_t* ua = e.smem + OFF_A + rnd * CHUNK_BYTES + swz(e.row, e.part * 2 + q);
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
            const int k = q * 8 + hf * 4 + i;
            const float rg = round_bf16(sigmoid_fast(__uint_as_float(rv[k]) + abv[i]));
            const float ig = round_bf16(sigmoid_fast(__uint_as_float(iv[k]) + xbv[i]));
            // sigmoid(Lambda)^(8 r) = 2^(r * 8 log2 sigmoid(Lambda)); the table is part of the weight image
            float a = ex2_fast(rg * dlv[i]);
            const float gate = sqrt_fast(fmaxf((1.0f - a) * (1.0f + a), kGateFloor));
            const uint32_t uword = uw[hf * 2 + (i >> 1)];
            const float uu = (i & 1) ? bf16_hi(uword) : bf16_lo(uword);
            const float bb = gate * (ig * uu);
            if (boundary) a = 0.f;
            hn[i] = fmaf(a, hn[i], bb);
          }
          *reinterpret_cast<float4*>(hout + cc) = make_float4(hn[0], hn[1], hn[2], hn[3]);
          const int bi = q * 4 + hf * 2;
          ob[hf * 2] = pack_bf16(hn[0] * bf16_lo(b2p[rnd][bi]), hn[1] * bf16_hi(b2p[rnd][bi]));
          ob[hf * 2 + 1] = pack_bf16(hn[2] * bf16_lo(b2p[rnd][bi + 1]), hn[3] * bf16_hi(b2p[rnd][bi + 1]));
        }
        // branch operand of linear_out: K atom 0 lives in P0, K atom 1 in place in A
        uint8_t* dst = rnd == 0 ? e.smem + OFF_P + swz(e.row, e.part * 2 + q) : ua;
        *reinterpret_cast<uint4*>(dst) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
      }
    }
    if (rnd == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) hprev[q] = hnext[q];
    }
  }
  if (has_fields) {
    // field rows: branch = bf16(bf16(field_sub b1) * b2)
#pragma unroll
    for (int rnd = 0; rnd < 2; ++rnd) {
      uint32_t v[16];
      tmem_ld16_nowait(e.lane_addr + COL_ACC2 + rnd * 64 + e.part * 16, v);        // executed by every lane of the warp
      tmem_wait_ld();
      if (!is_ship) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint32_t ob[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int bi = q * 4 + j;
            const float f0 = is_field ? round_bf16(__uint_as_float(v[q * 8 + 2 * j])) * bf16_lo(b2p[rnd][bi]) : 0.f;
            const float f1 = is_field ? round_bf16(__uint_as_float(v[q * 8 + 2 * j + 1])) * bf16_hi(b2p[rnd][bi]) : 0.f;
            ob[j] = pack_bf16(f0, f1);
          }
          uint8_t* dst = rnd == 0 ? e.smem + OFF_P + swz(e.row, e.part * 2 + q)
                                  : e.smem + OFF_A + CHUNK_BYTES + swz(e.row, e.part * 2 + q);
          *reinterpret_cast<uint4*>(dst) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
        }
      }
    }
  } else if (!is_ship) {
    // rows outside every environment: zero operand rows
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      *reinterpret_cast<uint4*>(e.smem + OFF_P + swz(e.row, e.part * 2 + q)) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(e.smem + OFF_A + CHUNK_BYTES + swz(e.row, e.part * 2 + q)) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  post(e, B_OP0);   // branch operand
  T_SINCE(e.tacc, TE_TEMPORAL, tu);
  wait_round(e, 1);   // residual += linear_out(branch)
  norm_to_A(e);
  post(e, B_OP0);
  ffn(e);
}

// ------------------------------------------------------------------ issuing side (one lane)

struct Issuer {
#ifdef BNB_TRACE
  Trace tr;
#endif
#ifdef BNB_TIMING
  long long tacc[T_COUNT];
#endif
  uint32_t sbase, bars, tmem;
  uint32_t full_par;   // per-slot phase bits of the full barriers
  uint32_t op_par;     // phase bits of OP0, OP1
  const uint32_t* sched;
  int sched_len, idx;
  uint32_t next_slot;  // ring slot of the next chunk of the schedule
  int* status;
  volatile int* aborted;
};

__device__ __forceinline__ void wait_operand(Issuer& m, int i) {
  T_BEGIN();
  mbar_wait(m.bars + 8 * (B_OP0 + i), (m.op_par >> i) & 1u, m.status, m.aborted, ST_TIMEOUT_OPERAND);
  m.op_par ^= 1u << i;
  tc_fence_after();
  T_END(m.tacc, TM_OP_WAIT);
  TRACE(m.tr, 400 + i);
}
// tcgen05.mma with both shared-memory descriptors built from 32-bit halves inside the asm block
// (K-major, 128-byte swizzle, 8-row groups 1024 B apart: the high word is a constant), which keeps
// the issuing lane's register count low.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ void tc_mma_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(0x40004040u) : "memory");
}

// The next ring operation of the schedule: wait for its weights, issue its MMAs
// (D[128 x n] (+)= A[128 x 64] * W[n x 64]^T per K atom: a pair reads K atom 0 of the operand at
// a_off0 and K atom 1 at a_off1), and commit on the slot's DONE barrier.
__device__ __forceinline__ void issue_op(Issuer& m, bool pair, uint32_t a_off0, uint32_t a_off1, uint32_t n, uint32_t d_col,
                                         uint32_t accumulate) {
  const uint32_t slot = m.next_slot;
  m.idx = m.idx + 1 == m.sched_len ? 0 : m.idx + 1;
  m.next_slot = m.sched[m.idx] & 7u;   // not needed before the next call: the load's latency is hidden
  T_MARK(tw);
  mbar_wait(m.bars + 8 * (B_FULL0 + slot), (m.full_par >> slot) & 1u, m.status, m.aborted, ST_TIMEOUT_FULL);
  m.full_par ^= 1u << slot;
  T_SINCE(m.tacc, TM_FULL_WAIT, tw);
  TRACE(m.tr, 410);
  const uint32_t b_lo = desc_lo(m.sbase + slot_offset(slot));
  const uint32_t idesc = instr_desc(n);
  // a step of 16 K columns = 32 bytes = 2 in descriptor units; a K atom = 16 KB = 1024 units
  const uint32_t a0 = desc_lo(m.sbase + a_off0);
#pragma unroll
  for (uint32_t k = 0; k < 4; ++k) tc_mma_lo(m.tmem + d_col, a0 + 2 * k, b_lo + 2 * k, idesc, (accumulate | k) ? 1u : 0u);
  if (pair) {
    const uint32_t a1 = desc_lo(m.sbase + a_off1);
#pragma unroll
    for (uint32_t k = 0; k < 4; ++k) tc_mma_lo(m.tmem + d_col, a1 + 2 * k, b_lo + 1024 + 2 * k, idesc, 1u);
  }
  tc_commit(m.bars + 8 * (B_DONE0 + slot));
  T_SINCE(m.tacc, TM_ISSUE, tw);
  TRACE(m.tr, 420);
}
// The same with the A operand in tensor memory: K step k reads the 8 columns at a_col + 16 k
// (lane = row, a 32-bit column = two consecutive k as bfloat16).
__device__ __forceinline__ void tc_mma_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(0x40004040u) : "memory");
}
__device__ __forceinline__ void issue_down_tmem(Issuer& m, uint32_t a_col) {
  const uint32_t slot = m.next_slot;
  m.idx = m.idx + 1 == m.sched_len ? 0 : m.idx + 1;
  m.next_slot = m.sched[m.idx] & 7u;
  mbar_wait(m.bars + 8 * (B_FULL0 + slot), (m.full_par >> slot) & 1u, m.status, m.aborted, ST_TIMEOUT_FULL);
  m.full_par ^= 1u << slot;
  const uint32_t b_lo = desc_lo(m.sbase + slot_offset(slot));
  const uint32_t idesc = instr_desc(128);
#pragma unroll
  for (uint32_t k = 0; k < 4; ++k) tc_mma_tmem_a(m.tmem + COL_RESID, m.tmem + a_col + 16 * k, b_lo + 2 * k, idesc, 1u);
  tc_commit(m.bars + 8 * (B_DONE0 + slot));
}
__device__ __forceinline__ void issue_pair(Issuer& m, uint32_t a_off, uint32_t n, uint32_t d_col) {
  issue_op(m, true, a_off, a_off + CHUNK_BYTES, n, d_col, 0);
}
__device__ __forceinline__ void commit_round(const Issuer& m) { tc_commit(m.bars + 8 * B_ACC); }

__device__ __forceinline__ void issue_ffn(Issuer& m) {
  wait_operand(m, 0);
#pragma unroll 1
  for (int c = 0; c < 3; ++c) issue_pair(m, OFF_A, 128, COL_ACC0 + 128 * c);
#pragma unroll 1
  for (int c = 0; c < 8; ++c) {
    wait_operand(m, c & 1);   // product of chunk c written, accumulator c % 3 read
    issue_down_tmem(m, COL_ACC0 + 128 * (c % 3));
    if (c + 3 < 8) issue_pair(m, OFF_A, 128, COL_ACC0 + 128 * (c % 3));
  }
}
__device__ __forceinline__ void issue_spatial(Issuer& m) {
  wait_operand(m, 0);
#pragma unroll 1
  for (int h = 0; h < HEADS; ++h) issue_pair(m, OFF_A, 96, COL_ACC0 + 96 * h);
  commit_round(m);
  wait_operand(m, 0);   // attention output: K atom 0 = heads 0, 1; K atom 1 = heads 2, 3
  issue_op(m, true, OFF_P, OFF_P + CHUNK_BYTES, 128, COL_RESID, 1);
  commit_round(m);
  issue_ffn(m);
}
__device__ __forceinline__ void issue_spatial_pre(Issuer& m) {
  wait_operand(m, 0);
#pragma unroll 1
  for (int h = 0; h < HEADS; ++h) issue_pair(m, OFF_A, 96, COL_ACC0 + 96 * h);
  commit_round(m);
}
__device__ __forceinline__ void issue_spatial_post(Issuer& m) {
  wait_operand(m, 0);   // attention output in A: K atom 0 = heads 0, 1; K atom 1 = heads 2, 3
  issue_op(m, true, OFF_A, OFF_A + CHUNK_BYTES, 128, COL_RESID, 1);
  commit_round(m);
  issue_ffn(m);
}
__device__ __forceinline__ void issue_temporal(Issuer& m, bool has_fields) {
  wait_operand(m, 0);
  issue_pair(m, OFF_A, 128, COL_ACC0);   // linear2
  issue_pair(m, OFF_A, 128, COL_ACC1);   // linear1
  commit_round(m);
  wait_operand(m, 0);
  issue_pair(m, OFF_A, 128, COL_ACC0);   // gates of hidden columns [0,64)
  issue_pair(m, OFF_A, 128, COL_ACC1);   // gates of hidden columns [64,128)
  if (has_fields) issue_pair(m, OFF_A, 128, COL_ACC2);   // field_sub
  commit_round(m);
  wait_operand(m, 0);
  issue_op(m, true, OFF_P, OFF_A + CHUNK_BYTES, 128, COL_RESID, 1);   // linear_out: K atom 0 from P0, K atom 1 in place in A
  commit_round(m);
  issue_ffn(m);
}

// ------------------------------------------------------------------ the kernel

__global__ void __launch_bounds__(THREADS, 1) k_trunk_pipelined(const __grid_constant__ TrunkArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ int s_aborted[2];
  __shared__ int s_items;
  __shared__ SubLayer s_sub[MAX_SUBLAYERS];  // kernel parameters are slow to index dynamically
  __shared__ uint32_t s_sched[MAX_SCHED];
  __shared__ int s_sched_len;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid < args.n_sub) s_sub[tid] = args.sub[tid];
  if (tid == 32) s_sched_len = build_schedule(args.sub, args.n_sub, args.has_fields != 0, s_sched);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 8 * B_COUNT);
  if (tid == 0) {
    s_aborted[0] = (*args.status != 0) ? 1 : 0;
    s_aborted[1] = args.poll_limit > 0 ? args.poll_limit : DEFAULT_POLL_LIMIT;
    mbar_init(smem_u32(&bars[B_OP0]), EPI_WARPS);
    mbar_init(smem_u32(&bars[B_OP1]), EPI_WARPS);
    mbar_init(smem_u32(&bars[B_KVREL]), EPI_WARPS);
    for (int i = B_ACC; i < B_COUNT; ++i) mbar_init(smem_u32(&bars[i]), 1);
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
  const int my_tiles = blockIdx.x < args.n_tiles ? (args.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int passes = my_tiles * args.t_loop;

  if (warp == LOAD_WARP) {
    // ---------------------------------------------------------------- weight stream
    if ((tid & 31) == 0) {
      const uint32_t sbase = smem_u32(smem), bar0 = smem_u32(bars);
      uint32_t free_par = (1u << N_SLOTS) - 1u;   // a fresh barrier passes a wait on parity 1: every slot starts free
      uint32_t kv_par = 0;
      const int len = s_sched_len;
#ifdef BNB_TIMING
      long long tacc[T_COUNT];
      for (int i = 0; i < T_COUNT; ++i) tacc[i] = 0;
#endif
      T_MARK(t_start);
#ifdef BNB_TRACE
      Trace ltr;
      trace_init(ltr, args.status, 2);
#endif
      for (int pass = 0; pass < passes; ++pass)
        for (int i = 0; i < len; ++i) {
          const uint32_t en = s_sched[i];
          const uint32_t slot = en & 7u;
          T_MARK(tw);
          if (en & (1u << 18)) {
            mbar_wait(bar0 + 8 * B_KVREL, kv_par, args.status, s_aborted, ST_TIMEOUT_FREE);
            kv_par ^= 1u;
          }
          T_SINCE(tacc, TL_KV_WAIT, tw);
          mbar_wait(bar0 + 8 * (B_DONE0 + slot), (free_par >> slot) & 1u, args.status, s_aborted, ST_TIMEOUT_FREE);
          free_par ^= 1u << slot;
          // Once a wait of this CTA has run out nothing is in step any more: stop fetching.  Arming a
          // FULL barrier again before its previous copy has landed would arrive on it twice in one
          // phase, which is undefined; the other roles' waits give up at once and the kernel drains.
          if (*static_cast<volatile int*>(s_aborted)) { pass = passes; break; }
          T_SINCE(tacc, TL_FREE_WAIT, tw);
          TRACE(ltr, 500 + slot);
          const uint32_t full = bar0 + 8 * (B_FULL0 + slot);
          const uint8_t* image = s_sub[(en >> 3) & 7u].packed;
          const uint32_t ch0 = (en >> 6) & 63u, ch1 = (en >> 12) & 63u;
          const uint32_t dst = sbase + slot_offset(slot);
          if (blockIdx.x == 0 && pass * len + i == args.skip_op) {
            // test hook: this operation's weights never arrive
          } else if (ch1 == NO_CHUNK) {
            mbar_expect_tx(full, CHUNK_BYTES);
            bulk_g2s(dst, image + (size_t)ch0 * CHUNK_BYTES, CHUNK_BYTES, full);
          } else if (ch1 == ch0 + 1) {
            mbar_expect_tx(full, 2 * CHUNK_BYTES);
            bulk_g2s(dst, image + (size_t)ch0 * CHUNK_BYTES, 2 * CHUNK_BYTES, full);
          } else {
            mbar_expect_tx(full, 2 * CHUNK_BYTES);
            bulk_g2s(dst, image + (size_t)ch0 * CHUNK_BYTES, CHUNK_BYTES, full);
            bulk_g2s(dst + CHUNK_BYTES, image + (size_t)ch1 * CHUNK_BYTES, CHUNK_BYTES, full);
          }
        }
#ifdef BNB_TIMING
      tacc[TL_TOTAL] = clock64() - t_start;
      T_STORE(args, tacc, TL_FREE_WAIT, T_COUNT);
#endif
    }
  } else if (warp == MMA_WARP) {
    // ---------------------------------------------------------------- tensor-core issue
    if ((tid & 31) == 0) {
      Issuer m;
      m.sbase = smem_u32(smem);
      m.bars = smem_u32(bars);
      m.tmem = tmem_base;
      m.full_par = 0;
      m.op_par = 0;
      m.sched = s_sched;
      m.sched_len = s_sched_len;
      m.idx = 0;
      m.next_slot = s_sched[0] & 7u;
      m.status = args.status;
      m.aborted = s_aborted;
#ifdef BNB_TRACE
      trace_init(m.tr, args.status, 1);
#endif
#ifdef BNB_TIMING
      for (int i = 0; i < T_COUNT; ++i) m.tacc[i] = 0;
#endif
      T_MARK(t_start);
      for (int pass = 0; pass < passes; ++pass)
        for (int si = 0; si < args.n_sub; ++si) {
          const int type = s_sub[si].type;
          if (type == SUB_SPATIAL) issue_spatial(m);
          else if (type == SUB_SPATIAL_PRE) issue_spatial_pre(m);
          else if (type == SUB_SPATIAL_POST) issue_spatial_post(m);
          else issue_temporal(m, args.has_fields != 0);
        }
      // Nothing issued here may outlive the CTA: its tensor memory is freed and its barriers go
      // away at the end.  In a normal run the epilogue warps' last waits already imply this; after
      // a wait has run out nobody has waited for anything, so wait here, with the full limit.
      tc_commit(m.bars + 8 * B_DRAIN);
      for (int i = 0; i < DEFAULT_POLL_LIMIT && !mbar_try_wait(m.bars + 8 * B_DRAIN, 0); ++i) {
      }
#ifdef BNB_TIMING
      m.tacc[TM_TOTAL] = clock64() - t_start;
      T_STORE(args, m.tacc, TM_FULL_WAIT, TL_FREE_WAIT);
#endif
    }
  } else {
    // ---------------------------------------------------------------- tile owners
    Epi e;
    e.smem = smem;
    e.sbase = smem_u32(smem);
    e.bars = smem_u32(bars);
    e.row = tid & (TILE - 1);
    e.part = tid >> 7;
    e.lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    e.par = 0;
    e.sched = s_sched;
    e.sched_len = s_sched_len;
    e.cur = 0;
    e.status = args.status;
    e.aborted = s_aborted;
    e.ss_part = reinterpret_cast<float*>(smem + OFF_SS);
#ifdef BNB_TRACE
    trace_init(e.tr, args.status, 0);
    if (tid != 0) e.tr.n = 1500;
#endif
#ifdef BNB_TIMING
    for (int i = 0; i < T_COUNT; ++i) e.tacc[i] = 0;
    e.wait_slot = TE_ACC_WAIT;
#endif
    T_MARK(t_start);
    uint8_t* meta = smem + OFF_META;
    const EnvMap& map = args.map;
    const int NM = map.tokens_per_env;
    const int row = e.row;

    for (int tile = blockIdx.x; tile < args.n_tiles; tile += gridDim.x) {
      // ---- rows of this tile: whole environments, ships first then fields in each
      T_MARK(t_io);
      const int grp = tile / args.env_tiles, eb = tile - grp * args.env_tiles;
      bool valid;
      int env, tok, env_first, env_n, env_ships;
      size_t grow = 0;
      int hrow_if_ship;
      if (args.flat_rows) {
        // plain 128-row slices of the token rows (programs without attention inside: the
        // environments are larger than a tile); the environment of a row is looked up
        const int r = eb * TILE + row;
        valid = r < map.total_tokens;
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
      const bool is_ship = valid && tok < env_ships;
      const bool is_field = valid && !is_ship;
      RowState rs;
      rs.hrow = is_ship ? hrow_if_ship : -1;
      rs.lag_ok = BNB_CONV_KERNEL - 1;
      rs.zero_in = is_ship && args.reset_env && args.reset_env[env];
      epi_sync();  // previous tile's readers of the meta arrays are done
      if (e.part == 0) {
        meta[row] = (uint8_t)(valid ? env_first : row);
        meta[128 + row] = (uint8_t)(valid ? env_n - 1 : 0);
        reinterpret_cast<int*>(smem + OFF_ROWINFO)[row] = rs.hrow;
      }
      if (tid == 0) s_items = 0;
      epi_sync();
      if (e.part == 0 && valid && (tok & 15) == 0) meta[384 + atomicAdd(&s_items, 1)] = (uint8_t)row;

      for (int t = 0; t < args.t_loop; ++t) {
        const size_t trow = grow + (size_t)t * map.total_tokens;
        if (e.part == 0) {
          const bool live = valid && (!args.alive || args.alive[trow]);
          meta[256 + row] = live ? (uint8_t)1 : (uint8_t)0;
          reinterpret_cast<float*>(smem + OFF_BIAS)[row] = live ? 0.f : kMaskedScore;
        }
        // residual <- x (this thread: columns [32 part, 32 part + 32))
        {
          uint32_t v[32];
          if (args.io_bf16) {
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(args.x) + trow * D + e.part * 32);
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
              if (valid) f = *reinterpret_cast<const float4*>(args.x + trow * D + e.part * 32 + q * 4);
              v[q * 4 + 0] = __float_as_uint(f.x); v[q * 4 + 1] = __float_as_uint(f.y);
              v[q * 4 + 2] = __float_as_uint(f.z); v[q * 4 + 3] = __float_as_uint(f.w);
            }
          }
          tmem_st32(e.lane_addr + COL_RESID + e.part * 32, v);
        }
        bool boundary = false;
        if (t >= 1) {
          boundary = is_ship && args.done && args.done[(size_t)(t - 1) * map.n_envs + env];
          rs.lag_ok = boundary ? 0 : min(rs.lag_ok + 1, BNB_CONV_KERNEL - 1);
          rs.zero_in = false;
        }
        if (e.part == 0) smem[OFF_ROWINFO + 512 + row] = (uint8_t)(rs.lag_ok | (rs.zero_in ? 4 : 0));
        epi_sync();
        T_SINCE(e.tacc, TE_IO, t_io);
        const int n_items = s_items;
        for (int si = 0; si < args.n_sub; ++si) {
          const SubLayer& s = s_sub[si];
          // Ask L2 for the recurrent state of the temporal sublayer that follows this one: the
          // rows are needed one sublayer from now.
          if (is_ship && t == 0 && si + 1 < args.n_sub && s_sub[si + 1].type == SUB_TEMPORAL && s.type != SUB_TEMPORAL) {
            const char* base = reinterpret_cast<const char*>(s_sub[si + 1].hid_in + (size_t)rs.hrow * 4 * D) + e.part * 512;
#pragma unroll
            for (int l = 0; l < 4; ++l) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + l * 128));
          }
          if (s.type == SUB_SPATIAL) run_spatial(e, n_items, valid);
          else if (s.type == SUB_SPATIAL_PRE) run_spatial_pre(e, s, trow, valid);
          else if (s.type == SUB_SPATIAL_POST) run_spatial_post(e, s, trow, valid);
          else run_temporal(e, s, rs, is_field, boundary, args.has_fields != 0, t == 0 ? s.hid_in : s.hid_out);
        }
        // y <- residual
        T_RESET(t_io);
        {
          uint32_t v[32];
          tmem_ld32(e.lane_addr + COL_RESID + e.part * 32, v);
          if (valid && args.io_bf16) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(args.y) + trow * D + e.part * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = pack8(&v[q * 8]);
          } else if (valid) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(args.y + trow * D + e.part * 32 + q * 4) =
                  make_float4(__uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]), __uint_as_float(v[q * 4 + 2]), __uint_as_float(v[q * 4 + 3]));
          }
        }
        T_SINCE(e.tacc, TE_IO, t_io);
      }
    }
#ifdef BNB_TIMING
    e.tacc[TE_TOTAL] = clock64() - t_start;
    if (tid == 0) T_STORE(args, e.tacc, 0, TM_FULL_WAIT);
#endif
  }
  tc_fence_before();
  __syncthreads();
  if (s_aborted[0] && warp == LOAD_WARP) {
    // a wait ran out: copies may still be in flight towards this CTA's shared memory; give them
    // time to land before the CTA gives it up
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace pipe

int launch_pipelined(const TrunkArgs& a, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BNB_ERR_NO_DEVICE;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(pipe::k_trunk_pipelined, cudaFuncAttributeMaxDynamicSharedMemorySize, pipe::SMEM_BYTES) != cudaSuccess)
      return BNB_ERR_LAUNCH;
    configured[dev] = true;
  }
  const int grid = a.n_tiles < 148 ? a.n_tiles : 148;
  count_launch();
  pipe::k_trunk_pipelined<<<grid, pipe::THREADS, pipe::SMEM_BYTES, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? BNB_OK : BNB_ERR_LAUNCH;
}

}  // namespace tensor
}  // namespace bnb
