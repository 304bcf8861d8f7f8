/*
 * C ABI of the B200 YemongPolicy trunk kernels.
 *
 * The reference (AvesNova/boost-and-broadside) is pure PyTorch and has no FFI layer;
 * its trunk hot path sits behind nn.Module methods.  Each entry point below replaces
 * the body of one of those methods and is what a binding on the reference side calls
 * (a ctypes stub is enough: plain pointers, ints and one opaque stream handle).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - float tensors are float32, row-major, innermost stride 1, 16-byte aligned;
 *   - bool tensors are one byte per element (torch.bool storage);
 *   - Linear weights are (out_features, in_features) exactly as nn.Linear stores them;
 *   - calls are asynchronous on `stream` (a cudaStream_t passed as void*), never
 *     synchronise, never allocate, never free; scratch memory comes from the caller;
 *   - the return value is a BnbStatus; nothing throws.
 *
 * Precision
 *   BNB_FP32  every operation in float32 (the reference without autocast).
 *   BNB_BF16  the reference under torch.autocast(bfloat16): Linear operands and outputs,
 *             attention q/k/v/out, GeLU and gate*up rounded to bf16; norms, residual
 *             stream, conv taps, pow, recurrence and hidden state float32.
 */
#ifndef BNB_TRUNK_H_
#define BNB_TRUNK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BNB_ABI_VERSION 3 /* 3: BnbBullets.tokens_bf16; BNB_BF16_IO accepted by bnb_head_mlp_fwd and on multi-launch trunk calls */
#define BNB_CONV_KERNEL 4 /* models/yemong/griffin.py:22 */

typedef enum {
  BNB_OK = 0,
  BNB_ERR_NULL_POINTER = 1,
  BNB_ERR_MISALIGNED = 2,
  BNB_ERR_UNSUPPORTED_DIMS = 3,   /* d_model / n_heads / head width outside the built set */
  BNB_ERR_TOO_MANY_TOKENS = 4,    /* an environment holds more tokens than the kernels take */
  BNB_ERR_BAD_ARGUMENT = 5,
  BNB_ERR_SCRATCH_TOO_SMALL = 6,
  BNB_ERR_LAUNCH = 7,             /* the CUDA runtime refused a launch; see cudaGetLastError */
  BNB_ERR_NO_DEVICE = 8,
  BNB_ERR_EXCEEDS_STATIC_LIMIT = 9, /* more rows than bnb_spatial_block_fwd_static's fixed scratch holds */
  /* Codes a tensor-core kernel leaves in the status word (below) when one of its bounded waits
   * ran out; entry points never return them, bnb_last_status does. */
  BNB_STATUS_WAIT_WEIGHTS = 101,  /* a weight copy did not land */
  BNB_STATUS_WAIT_SLOT = 102,     /* a weight slot (or the key/value area) was not released */
  BNB_STATUS_WAIT_MMA = 103,      /* tensor-core results did not arrive */
  BNB_STATUS_WAIT_OPERAND = 104   /* an operand was not posted */
} BnbStatus;

/* The status word.  Every wait inside the tensor-core kernels is bounded.  A wait that runs out
 * writes one of the BNB_STATUS_WAIT_* codes into the first 4 bytes of the call's scratch buffer
 * (an int at byte offset 0; each call zeroes it first), the kernel drains and returns, and the
 * call's outputs are then unspecified.  The entry point has returned BNB_OK long before, so every
 * BNB_BF16 call also copies the word to a pinned host word of its device, asynchronously on its
 * stream; bnb_last_status() reports the first non-zero code seen there since the last
 * bnb_clear_status().  The first BNB_BF16 call on a device allocates the host word and should
 * come before any stream capture (a call that finds itself capturing without it skips the copy). */
int bnb_last_status(void);
void bnb_clear_status(void);

/* Test hook for the above, never needed in production: the next launches of the fused tile
 * kernel use `poll_limit` polls per wait (0 = default) and CTA 0 leaves out the weight copy of
 * its `skip_op`-th ring operation (-1 = none), so that exactly one wait runs out, nothing
 * faults or spins, and the status word reads BNB_STATUS_WAIT_WEIGHTS. */
void bnb_debug_wait_test(int skip_op, int poll_limit);

typedef enum {
  BNB_FP32 = 0,
  BNB_BF16 = 1,
  /* BNB_BF16 with the token tensors themselves in bfloat16: `x` and `y` of bnb_trunk_step /
   * bnb_trunk_sequence then point to bfloat16 elements (the declared float type notwithstanding);
   * hidden state and parameters stay float32.  This is what the reference's trunk sees on the GPU:
   * under torch.autocast("cuda", bfloat16) its encoder ends in an RMSNorm of a bf16 Linear output,
   * which is bf16, and its heads cast what the trunk returns to bf16.  The residual stream is still
   * carried in float32 inside a launch and rounded on the way out (the reference adds in
   * bf16 after every sublayer).  Halves the bytes of the token tensors.  Served by the tensor-core
   * kernels only (d_model 128, 4 heads); any other call returns BNB_ERR_UNSUPPORTED_DIMS and the
   * caller converts.  A call that takes several launches (environments larger than a tile, sublayers
   * that read bullets, a time walk) rounds the residual stream where one launch hands over to the
   * next. */
  BNB_BF16_IO = 2
} BnbPrecision;

/* Which engine runs a BNB_BF16 call.
 *   BNB_ENGINE_AUTO   the fused tcgen05 kernels where the shapes are built for them, else SIMT
 *   BNB_ENGINE_SIMT   the exact kernels: float32 elementwise math on the CUDA cores, Linear
 *                     products float32-accurate (3 x tf32 MMAs), bf16 roundings applied in software
 *   BNB_ENGINE_TENSOR the fused tcgen05 kernels or BNB_ERR_UNSUPPORTED_DIMS
 * BNB_FP32 always runs on the exact kernels. */
typedef enum { BNB_ENGINE_AUTO = 0, BNB_ENGINE_SIMT = 1, BNB_ENGINE_TENSOR = 2 } BnbEngine;

/* Parameters of one spatial sublayer.
 * Replaces: TransformerBlock parameters, models/yemong/attention.py:51-74. */
typedef struct {
  const float* norm1_w;   /* (D)            norm1.weight          */
  const float* qkv_w;     /* (3D, D)        qkv.weight            */
  const float* out_w;     /* (D, D)         out_proj.weight       */
  const float* norm2_w;   /* (D)            norm2.weight          */
  const float* gate_w;    /* (4D, D)        ffn.gate_proj.weight  */
  const float* up_w;      /* (4D, D)        ffn.up_proj.weight    */
  const float* down_w;    /* (D, 4D)        ffn.down_proj.weight  */
  /* Only for a sublayer built with reads_bullets (attention.py:64-71); both NULL otherwise. */
  const float* norm_bullet_w; /* (D)        norm_bullet.weight    */
  const float* kv_bullet_w;   /* (2D, D)    kv_bullet.weight      */
  const void*  packed;    /* optional: image written by bnb_pack_spatial, or NULL */
} BnbSpatialWeights;

/* Encoded bullet tokens of a call: keys and values of the cross-attention branch of the
 * sublayers that read bullets, never queries (models/yemong/attention.py:149-166).
 * Every environment of every group holds the same number of ring-buffer slots. */
typedef struct {
  const float* tokens;    /* (n_groups * n_envs, per_env, D) float32, group-major like x */
  const uint8_t* active;  /* (n_groups * n_envs, per_env) bytes, or NULL: every slot is a key and
                             the branch is never gated off (bullet_mask=None in the reference) */
  int32_t per_env;        /* NB >= 1 */
  int32_t tokens_bf16;    /* 0: tokens are float32.  1: tokens point to bfloat16 elements (what the
                             reference's BulletEncoder returns under CUDA autocast); only calls the
                             tensor-core kernels serve take them (BNB_BF16 forward, supported shapes),
                             any other call returns BNB_ERR_UNSUPPORTED_DIMS */
} BnbBullets;

/* Parameters of one temporal sublayer plus its field substitute.
 * Replaces: GriffinTemporalBlock / RGLRU parameters, models/yemong/griffin.py:160-247,
 * and YemongBlock.field_sub, griffin.py:359-368. */
typedef struct {
  const float* norm1_w;     /* (D)       norm1.weight            */
  const float* linear1_w;   /* (D, D)    linear1.weight          */
  const float* conv_w;      /* (D, 4)    conv.weight (D,1,4)     */
  const float* conv_b;      /* (D)       conv.bias               */
  const float* log_lambda;  /* (D)       rg_lru.log_lambda       */
  const float* a_w;         /* (D, D)    rg_lru.linear_a.weight  */
  const float* a_b;         /* (D)       rg_lru.linear_a.bias    */
  const float* x_w;         /* (D, D)    rg_lru.linear_x.weight  */
  const float* x_b;         /* (D)       rg_lru.linear_x.bias    */
  const float* linear2_w;   /* (D, D)    linear2.weight          */
  const float* out_w;       /* (D, D)    linear_out.weight       */
  const float* norm2_w;     /* (D)       norm2.weight            */
  const float* gate_w;      /* (4D, D)   gated_mlp.gate_proj     */
  const float* up_w;        /* (4D, D)   gated_mlp.up_proj       */
  const float* down_w;      /* (D, 4D)   gated_mlp.down_proj     */
  const float* field_sub_w; /* (D, D)    field_sub[j].weight; may be NULL when no fields */
  const void*  packed;      /* optional: image written by bnb_pack_temporal, or NULL */
} BnbTemporalWeights;

/* Geometry of one batch of environments.
 *
 * Uniform batch (tok_off == NULL): every environment holds tokens_per_env tokens, the
 * first ships_per_env of which are ships (recurrent), the rest fields.  Token rows are
 * env-major: row = env * tokens_per_env + token.  Hidden rows are env-major over ships:
 * row = env * ships_per_env + ship (models/yemong/policy.py:284).
 *
 * Ragged batch (tok_off != NULL): environment e owns token rows
 * [tok_off[e], tok_off[e+1]) and hidden rows [ship_off[e], ship_off[e+1]); its first
 * ship_off[e+1]-ship_off[e] tokens are ships.  Both arrays hold n_envs+1 int32 on the
 * device.  max_tokens_per_env must bound every environment.
 */
typedef struct {
  int32_t n_envs;
  int32_t tokens_per_env;
  int32_t ships_per_env;
  int32_t max_tokens_per_env;
  int32_t total_tokens;        /* rows of x per timestep  */
  int32_t total_ships;         /* rows of hidden          */
  const int32_t* tok_off;
  const int32_t* ship_off;
  /* Ragged batches on the tensor-core engine only: tile plan written by bnb_plan_tiles and
   * copied to the device: tile t holds the environments tile_env_ids[tile_env_begin[t] ..
   * tile_env_begin[t+1]) (n_tiles + 1 and n_envs int32).  NULL / 0 keeps a ragged batch on
   * the SIMT engine. */
  const int32_t* tile_env_begin;
  const int32_t* tile_env_ids;
  int32_t n_tiles;
} BnbBatch;

int bnb_abi_version(void);
const char* bnb_status_string(int status);

/* Kernels launched by this library in this process so far (instrumentation for the
 * benchmark's launch accounting; no counterpart in the reference). */
unsigned long long bnb_launch_count(void);

/* BNB_BF16 calls so far that asked for BNB_ENGINE_AUTO and ran on the exact kernels (several times
 * slower) because the tensor-core kernels are not built for their shape: d_model other than 128,
 * other than 4 heads, more than 512 tokens in an environment, a ragged batch without a tile plan,
 * more bullets per environment than the attention kernel stages.  The choice is made per call and
 * is otherwise silent; the Python binding warns once when this counter moves. */
unsigned long long bnb_auto_fallback_count(void);

/* Host-only query: 1 if (d_model, n_heads, max tokens per environment) can run with the
 * given precision and engine, else 0.  No device is touched. */
int bnb_supported(int d_model, int n_heads, int max_tokens_per_env, int precision, int engine);

/* Host-only: group the environments of a ragged batch into tiles of whole environments (at
 * most 128 token rows each, best-fit decreasing) for the tensor-core engine.
 *   tok_off_host        n_envs + 1 prefix sums on the HOST
 *   tile_env_begin_host receives n_tiles + 1 offsets into tile_env_ids_host; capacity is the
 *                       number of int32 it can hold and must be at least n_envs + 1
 *   tile_env_ids_host   receives the n_envs environment indices in tile order
 * Returns BNB_ERR_TOO_MANY_TOKENS when an environment has more than 128 tokens.
 * No counterpart in the reference (it cannot express per-environment fleet sizes in one call,
 * models/yemong/griffin.py:398-399). */
int bnb_plan_tiles(const int32_t* tok_off_host, int n_envs, int32_t* tile_env_begin_host,
                   int32_t* tile_env_ids_host, int capacity, int* n_tiles);

/* Bytes of scratch a call with this geometry may use (upper bound over all entry points).
 * `timesteps` is 1 for a step; `bullets_per_env` is 0 for calls without bullets.  The bullet
 * keys and values are projected in slices of environments, so their share of the scratch is
 * capped (512 MiB) whatever the batch. */
size_t bnb_scratch_bytes(int d_model, const BnbBatch* batch, int timesteps, int bullets_per_env);

/* y = TransformerBlock.forward(x, alive_mask, bullets, bullet_mask)
 * Replaces: models/yemong/attention.py:76-99 (with _attn 114-169 and GatedMLP 21-37).
 *   x, y    (n_rows, D) with n_rows = n_groups * batch->total_tokens; y may alias x
 *   alive   (n_rows) bytes or NULL (no key masking, attention.py:142-145)
 *   bullets NULL, or the bullet tokens; read only when w->kv_bullet_w is set
 *           (attention.py:149: reads_bullets and bullets is not None)
 *   n_groups replicates the batch geometry (the T*B fold of griffin.py:443-449). */
int bnb_spatial_block_fwd(const BnbSpatialWeights* w, int d_model, int n_heads,
                          const float* x, const uint8_t* alive, const BnbBullets* bullets, float* y,
                          const BnbBatch* batch, int n_groups, int precision, int engine,
                          void* scratch, size_t scratch_bytes, void* stream);

/* The same spatial sublayer for callers that cannot allocate device memory at all: a bare
 * ctypes / cgo / JNI stub that owns no allocator, or a host that has given the whole device
 * to another framework's pool and must not cudaMalloc around it.  The scratch that
 * bnb_spatial_block_fwd takes from the caller lives here in a fixed array inside the library
 * image, so this call (and everything under it) performs no cudaMalloc / cudaFree and uses
 * no allocating library routine.  It has no counterpart in the reference.
 *   - limit: n_groups * batch->total_tokens <= BNB_STATIC_MAX_ROWS, else
 *     BNB_ERR_EXCEEDS_STATIC_LIMIT and nothing is launched; d_model <= 128;
 *   - cost: every GPU that loads the library holds BNB_STATIC_SCRATCH_BYTES until exit;
 *   - always the exact (BNB_ENGINE_SIMT) kernels, in either precision;
 *   - the first call on each device looks up the array's device address (that device must
 *     be current); make that first call before starting any stream capture;
 *   - all calls share the one array: two calls that may overlap on the GPU (different
 *     streams, no dependency between them) race on it.  Calls on one stream are safe.
 *     Nothing in the array needs clearing between calls.
 * Arguments as bnb_spatial_block_fwd, without bullets, engine and scratch. */
#define BNB_STATIC_MAX_ROWS 2048
#define BNB_STATIC_SCRATCH_BYTES ((size_t)BNB_STATIC_MAX_ROWS * 4 * 128 * sizeof(float)) /* 4 MiB */
int bnb_spatial_block_fwd_static(const BnbSpatialWeights* w, int d_model, int n_heads,
                                 const float* x, const uint8_t* alive, float* y,
                                 const BnbBatch* batch, int n_groups, int precision, void* stream);

/* One temporal sublayer over T >= 1 timesteps for every token of the batch.
 * Replaces: GriffinTemporalBlock.forward_sequence (griffin.py:249-286) on the ship tokens,
 * GriffinTemporalBlock.forward_nonrecurrent (288-317) on the field tokens, and the
 * split / permute / cat around them in YemongBlock.step (403-415) and .sequence (451-470).
 *   x, y        (T, total_tokens, D); y may alias x
 *   hidden_in   (total_ships, 4D) packed [h | tap0 | tap1 | tap2], taps oldest first
 *               (models/yemong/policy.py:27-34); one slot of the policy's hidden tensor
 *   hidden_out  same layout; may alias hidden_in
 *   done        (T, n_envs) bytes or NULL; done[t] ends the episode at t, so step t+1
 *               starts from a zero state and ignores conv taps from before it
 *               (griffin.py:67-93, 213-218).  The taps written to hidden_out are the
 *               last three linear1 outputs unmasked (griffin.py:277). */
int bnb_temporal_block_fwd(const BnbTemporalWeights* w, int d_model,
                           const float* x, float* y,
                           const float* hidden_in, float* hidden_out,
                           const uint8_t* done, const BnbBatch* batch, int timesteps,
                           int precision, int engine,
                           void* scratch, size_t scratch_bytes, void* stream);

/* The whole trunk for one rollout step: n_blocks x (n_spatial spatial sublayers, then
 * n_temporal temporal sublayers), hidden slot i*n_temporal+j for temporal sublayer j of
 * block i.
 * Replaces: the trunk loop and hidden unpack/repack of YemongPolicy.get_action_and_value,
 * models/yemong/policy.py:315-354, with YemongBlock.step, griffin.py:376-417.
 *   spatial   n_blocks*n_spatial entries, block-major
 *   temporal  n_blocks*n_temporal entries, block-major
 *   x, y      (total_tokens, D); y may alias x
 *   hidden_in/out (n_blocks*n_temporal, total_ships, 4D); may alias
 *   bullets   NULL or the step's bullet tokens (n_groups = 1), passed to every spatial
 *             sublayer as griffin.py:400-401 does
 *   reset_env (n_envs) bytes or NULL: environments whose incoming state is taken as zero,
 *             i.e. reset_hidden_for_envs (policy.py:268-285) folded into the load. */
int bnb_trunk_step(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal,
                   int n_blocks, int n_spatial, int n_temporal, int d_model, int n_heads,
                   const float* x, const uint8_t* alive, const BnbBullets* bullets, float* y,
                   const float* hidden_in, float* hidden_out, const uint8_t* reset_env,
                   const BnbBatch* batch, int precision, int engine,
                   void* scratch, size_t scratch_bytes, void* stream);

/* The whole trunk over T timesteps from one initial state.
 * Replaces: the trunk loop of YemongPolicy.evaluate_actions, models/yemong/policy.py:422-478,
 * with YemongBlock.sequence, griffin.py:419-472.
 *   x, y    (T, total_tokens, D); alive (T, total_tokens) or NULL; done (T, n_envs) or NULL
 *   bullets NULL or the bullet tokens of all T * n_envs environments (n_groups = T)
 *   hidden_out receives the final state (the reference computes and drops it); may be NULL. */
int bnb_trunk_sequence(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal,
                       int n_blocks, int n_spatial, int n_temporal, int d_model, int n_heads,
                       const float* x, const uint8_t* alive, const BnbBullets* bullets, float* y,
                       const float* hidden_in, float* hidden_out, const uint8_t* done,
                       const BnbBatch* batch, int timesteps, int precision, int engine,
                       void* scratch, size_t scratch_bytes, void* stream);

/* hidden_out = hidden_in * keep, keep = 0 for every ship row of a done environment.
 * Replaces: YemongPolicy.reset_hidden_for_envs, models/yemong/policy.py:268-285.
 *   hidden_in/out (n_slots, total_ships, 4D); may alias;  done (n_envs) bytes */
int bnb_reset_hidden(const float* hidden_in, float* hidden_out, const uint8_t* done,
                     int n_slots, int d_model, const BnbBatch* batch, void* stream);

/* GatedMLP on its own: y = down(gelu_erf(gate x) * up x), no biases.
 * Replaces: GatedMLP.forward, models/yemong/attention.py:36-37 (inside a sublayer it runs fused).
 *   x, y (n_rows, D) float32; gate_w, up_w (4D, D); down_w (D, 4D).  BNB_BF16 applies the autocast
 *   roundings (input, every Linear output, the gelu and the product) and leaves bf16 values in y. */
int bnb_gated_mlp_fwd(const float* gate_w, const float* up_w, const float* down_w, int d_model,
                      const float* x, float* y, int n_rows, int precision, void* stream);

/* The RG-LRU on its own over `timesteps` steps of n_rows independent rows.
 * Replaces: RGLRU._step (timesteps = 1, done = NULL) and RGLRU.forward_sequence,
 * models/yemong/griffin.py:169-219 (inside a temporal sublayer it runs fused).
 *   x, y (timesteps, n_rows, D) time-major float32: y[t] is the state after step t;
 *   h0, h_out (n_rows, D); done (timesteps, n_rows) bytes or NULL: done[t] cuts the state
 *   before step t + 1.  The recurrence is evaluated step by step, which is what the reference
 *   pins its parallel scan against. */
int bnb_rglru_fwd(const float* a_w, const float* a_b, const float* x_w, const float* x_b,
                  const float* log_lambda, int d_model, const float* x, float* y, const float* h0,
                  float* h_out, const uint8_t* done, int n_rows, int timesteps, int precision,
                  void* stream);

/* The encoder chain Linear + b -> RMSNorm -> GELU(erf) -> Linear + b -> RMSNorm on rows of raw
 * feature vectors: the token encoders in front of the trunk.
 * Replaces: ShipEncoder.feature_extractor (or ship_proj / field_proj followed by shared_proj) and
 * BulletEncoder.net, models/yemong/encoder.py:45-51, 84-102.  The FeatureCoordinator that builds
 * the raw vectors from an observation stays the caller's.
 *   x (n_rows, in_dim) float32, 1 <= in_dim <= 128, rows need no alignment;
 *   w1 (hidden, in_pad) float32 = the first Linear's weight with zero columns appended up to
 *   in_pad, a multiple of 32; b1, g1 (hidden), hidden a multiple of 32 up to 256;
 *   w2 (out_dim, hidden), b2, g2 (out_dim), out_dim a multiple of 32 up to 128;
 *   y (n_rows, out_dim): float32 for BNB_FP32; **bfloat16 elements** for BNB_BF16, where every
 *   stage hands on bfloat16 as under torch.autocast (the RMSNorm of a bf16 input is computed in
 *   float32 with the float32 eps and rounded once) -- the tensor bnb_trunk_step takes with
 *   BNB_BF16_IO. */
int bnb_encoder_mlp_fwd(const float* w1, const float* b1, const float* g1, const float* w2,
                        const float* b2, const float* g2, int in_dim, int in_pad, int hidden,
                        int out_dim, const float* x, void* y, int n_rows, int precision, void* stream);

/* Gradient buffers of one sublayer: the fields of BnbSpatialWeights / BnbTemporalWeights, same
 * shapes, float32, written by accumulation (+=), so the caller zeroes them or hands in running
 * sums.  The bullet fields may be NULL for a sublayer that does not read bullets, field_sub_w when
 * the batch has no field tokens. */
typedef struct {
  float* norm1_w; float* qkv_w; float* out_w; float* norm2_w; float* gate_w; float* up_w; float* down_w;
  float* norm_bullet_w; float* kv_bullet_w;
} BnbSpatialGrads;

typedef struct {
  float* norm1_w; float* linear1_w; float* conv_w; float* conv_b; float* log_lambda; float* a_w; float* a_b;
  float* x_w; float* x_b; float* linear2_w; float* out_w; float* norm2_w; float* gate_w; float* up_w;
  float* down_w; float* field_sub_w;
} BnbTemporalGrads;

/* Scratch bytes of bnb_trunk_sequence_bwd for this structure and batch. */
size_t bnb_trunk_bwd_scratch_bytes(int n_blocks, int n_spatial, int n_temporal, int d_model,
                                   const BnbBatch* batch, int timesteps, int bullets_per_env, int precision);

/* Backward of bnb_trunk_sequence (and, with timesteps = 1 and no done, of bnb_trunk_step without
 * reset_env).  Every tensor is float32.  precision BNB_FP32: float32-accurate products (3 x tf32).
 * BNB_BF16: the Linear products of the recomputed forward and of the gradients round their operands
 * to bfloat16 and accumulate in float32, as autocast makes the reference's backward do; everything
 * else (norms, softmax, gates, recurrence, residual stream) stays float32.
 * Replaces: what loss.backward() runs through the trunk loop of YemongPolicy.evaluate_actions,
 * models/yemong/policy.py:422-478 (reached from train/rl/ppo.py:1974), with or without
 * grad_checkpoint (policy.py:451-467; this entry always recomputes).
 *   x, alive, bullets, hidden_in, done, batch, timesteps: the forward call's arguments (environments
 *   of one size only: batch->tok_off must be NULL).
 *   dy (T, total_tokens, D): gradient of the loss with respect to the forward's y.
 *   d_hidden_out (L, total_ships, 4D) or NULL (= zero): gradient with respect to the final state.
 *   dx (T, total_tokens, D): written.  d_hidden_in (L, total_ships, 4D) or NULL: written.
 *   d_bullets (T * n_envs, NB, D) or NULL: written (zeroed here, then accumulated over the sublayers
 *   that read bullets).
 *   d_spatial / d_temporal: one entry per sublayer, indexed like spatial / temporal; accumulated into.
 *   kept / kept_bytes: the buffer bnb_trunk_sequence_fwd_train filled for this call, or NULL / 0:
 *   the backward then recomputes every sublayer's intermediates itself.
 * The attention gradient follows the fused attention kernels behind F.scaled_dot_product_attention
 * (probabilities recomputed from the float32 log-sum-exp); d_model a multiple of 32 up to 128,
 * head width 8, 16 or 32.  Weight gradients reduce with float32 atomics: run-to-run bits may differ
 * in the last places. */
int bnb_trunk_sequence_bwd(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal,
                           const BnbSpatialGrads* d_spatial, const BnbTemporalGrads* d_temporal,
                           int n_blocks, int n_spatial, int n_temporal, int d_model, int n_heads,
                           const float* x, const uint8_t* alive, const BnbBullets* bullets,
                           const float* hidden_in, const uint8_t* done, const BnbBatch* batch, int timesteps,
                           int precision, const float* dy, const float* d_hidden_out, float* dx, float* d_hidden_in,
                           float* d_bullets, void* kept, size_t kept_bytes, void* scratch, size_t scratch_bytes,
                           void* stream);

/* Bytes of activations bnb_trunk_sequence_fwd_train keeps for the backward (for two blocks of two
 * spatial and one temporal sublayer at d_model 128: about 65 KB per token row with BNB_FP32, 47 KB
 * with BNB_BF16, where the 4 d_model-wide buffers of the gated MLPs hold bfloat16); 0 for a geometry
 * the backward does not cover.  Sizes depend on the precision: query with the call's. */
size_t bnb_trunk_kept_bytes(int n_blocks, int n_spatial, int n_temporal, int d_model, int n_heads,
                            const BnbBatch* batch, int timesteps, int bullets_per_env, int precision);

/* The sequence forward for a call that will be differentiated: y and hidden_out as
 * bnb_trunk_sequence computes them (same arithmetic contract per precision: float32, or bfloat16
 * operands in every Linear product), run sublayer by sublayer with each sublayer's intermediates
 * written to `kept`, so that bnb_trunk_sequence_bwd given the same `kept` skips its recomputation.
 * Replaces: the forward half of evaluate_actions' trunk loop without grad_checkpoint
 * (models/yemong/policy.py:422-478), where autograd stores the activations.
 * `kept` is consumed by the backward (it overwrites parts of it): one backward per forward.
 * scratch: bnb_trunk_bwd_scratch_bytes. */
int bnb_trunk_sequence_fwd_train(const BnbSpatialWeights* spatial, const BnbTemporalWeights* temporal,
                                 int n_blocks, int n_spatial, int n_temporal, int d_model, int n_heads,
                                 const float* x, const uint8_t* alive, const BnbBullets* bullets, float* y,
                                 const float* hidden_in, float* hidden_out, const uint8_t* done,
                                 const BnbBatch* batch, int timesteps, int precision, void* kept,
                                 size_t kept_bytes, void* scratch, size_t scratch_bytes, void* stream);

/* One head of the policy: Linear + b -> RMSNorm -> GELU(erf) -> Linear + b on the trunk's output.
 * Replaces: YemongPolicy.action_head, .value_head_local, .value_head_win and NextStateHead.net,
 * models/yemong/policy.py:56-72, 185-214 (all four have this shape).
 *   x (n_rows, in_dim) float32, in_dim a multiple of 32 up to 128; w1 (hidden, in_dim), b1, g1
 *   (hidden); w2 (out_pad, hidden) and b2 (out_pad): the second Linear with zero rows / entries
 *   appended up to out_pad, a multiple of 32; y (n_rows, out_dim), float32 for BNB_FP32,
 *   **bfloat16 elements** for BNB_BF16 (what the last Linear returns under autocast).
 *   precision BNB_BF16_IO: the BNB_BF16 contract with x holding bfloat16 elements too (the trunk's
 *   output under autocast), on a 16-byte boundary; served by the tiled kernel only
 *   (BNB_ERR_UNSUPPORTED_DIMS otherwise, and the caller converts). */
int bnb_head_mlp_fwd(const float* w1, const float* b1, const float* g1, const float* w2, const float* b2,
                     int in_dim, int hidden, int out_dim, int out_pad, const float* x, void* y, int n_rows,
                     int precision, void* stream);

/* TeamPMA: for each team t in {0, 1} a learned seed attends over the trunk outputs of that team's
 * alive ships (an nn.MultiheadAttention without biases), the result goes through out_proj, is zeroed
 * where the team has no ship alive, RMS-normed, and every ship receives its team's row.
 * Replaces: TeamPMA.forward, models/yemong/policy.py:78-121.
 *   seeds (2, D); in_proj_w (3D, D) = attn.in_proj_weight; out_w (D, D) = attn.out_proj.weight;
 *   norm_w (D); x (n_envs, n_ships, D) float32; team_id (n_envs, n_ships) int32; alive bytes;
 *   y (n_envs, n_ships, D): float32, or bfloat16 elements when y_is_bf16 (the reference writes into a
 *   tensor of x's dtype).  scratch: bnb_team_pma_scratch_bytes. */
size_t bnb_team_pma_scratch_bytes(int d_model, int n_envs, int n_ships);
int bnb_team_pma_fwd(const float* seeds, const float* in_proj_w, const float* out_w, const float* norm_w,
                     int d_model, int n_heads, const float* x, const int32_t* team_id, const uint8_t* alive,
                     void* y, int y_is_bf16, int n_envs, int n_ships, int precision, void* scratch,
                     size_t scratch_bytes, void* stream);

/* The factored categorical over the 12 action logits [power 0:3 | turn 3:10 | shoot 10:12]
 * (constants.py:43-48).
 * Replaces: _sample_action and _evaluate_action, models/yemong/policy.py:551-602 (forward only).
 *   logits (n_rows, 12) float32 (bfloat16 values under BNB_BF16).
 *   given_action NULL: one inverse-CDF draw per slice from uniforms (n_rows, 3) in [0, 1) into
 *   action (n_rows, 3) int64; the caller supplies the uniforms (torch.rand on the device), so the
 *   draws follow the caller's generator, not torch.multinomial's stream.
 *   given_action (n_rows, 3) int64: those actions are scored instead.
 *   logprob (n_rows): sum of the three log-probabilities; entropy (n_rows) or NULL. */
int bnb_action_dist_fwd(const float* logits, const float* uniforms, const int64_t* given_action,
                        int64_t* action, float* logprob, float* entropy, int n_rows, int precision,
                        void* stream);

/* Bytes of the tensor-core weight image of one sublayer (bf16, pre-tiled). */
size_t bnb_packed_spatial_bytes(int d_model);
size_t bnb_packed_temporal_bytes(int d_model);

/* Write the tensor-core image of a sublayer's float32 parameters into `packed`.
 * Re-run after every parameter update; the image is derived data, never saved.  It holds the
 * Linear weights pre-tiled in bf16 with the RMSNorm gains of their inputs multiplied in (and the
 * decay table of log_lambda), so an update of any parameter of the sublayer, gains included,
 * needs a new image.
 * No counterpart in the reference (it casts weights per call under autocast). */
int bnb_pack_spatial(const BnbSpatialWeights* w, int d_model, int n_heads, void* packed, void* stream);
int bnb_pack_temporal(const BnbTemporalWeights* w, int d_model, void* packed, void* stream);

/* The same for every sublayer of a trunk in one launch: each struct's `packed` names the
 * destination of its image.  Cheap enough (about 10 MB of traffic) to run before every call, which
 * is what the Python binding does: an image then never goes stale, whatever updated the
 * parameters (an optimizer step, an in-place copy that bumps no version counter, a replayed CUDA
 * graph whose captured work includes this launch). */
int bnb_pack_trunk(const BnbSpatialWeights* spatial, int n_spatial_total, const BnbTemporalWeights* temporal,
                   int n_temporal_total, int d_model, int n_heads, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BNB_TRUNK_H_ */
