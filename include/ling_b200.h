/* ling_b200.h -- C ABI of the B200 (sm_100a) ragged speculative verify step.
 *
 * The reference engine (dreamference/ling-engine) is one statically linked C++ program with no FFI; the
 * boundary it offers for this path is the public C++ surface its scheduler calls.  Every entry point below
 * names the reference declaration it stands in for (file:line inside the reference project).  A C++ facade
 * with the reference's own names (ling::Engine, ling::KvPool, ling::serve::*) lives beside the kernels and
 * forwards to these functions.
 *
 * Conventions: plain pointers and sizes, int status codes (0 = LING_B200_OK), never throws, no allocation
 * after ling_b200_create() unless a function says otherwise.  One thread drives one context, one step in
 * flight (src/serve/main.cpp:357-377 in the reference: a single engine thread).
 */
#ifndef LING_B200_H_
#define LING_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------ limits */
#define LING_B200_MAX_LAYERS 128
#define LING_B200_MAX_SEQS 64        /* sequences per step (reference: kernels.cuh:52 kMaxSeqs = 4)          */
#define LING_B200_MAX_TREE_ROWS 32   /* rows of one sequence's tree (kernels.cuh:107 kMaxStreamRows = 32)    */
#define LING_B200_MAX_TREE_VARIANTS 32 /* kernels.cuh:118 kMaxTreeVariants                                   */
#define LING_B200_MAX_ROWS 2048      /* packed rows of one step (all sequences)                              */

/* ------------------------------------------------------------------------------------------------ status */
enum {
  LING_B200_OK = 0,
  LING_B200_ERR_ARG = 1,          /* bad argument: nothing was launched or changed                          */
  LING_B200_ERR_CUDA = 2,         /* a CUDA call failed: see ling_b200_last_error()                          */
  LING_B200_ERR_POOL = 3,         /* KvPoolExhausted (engine.hpp:227-232): nothing launched, nothing changed */
  LING_B200_ERR_DEVICE_FLAG = 4,  /* a kernel's bounded wait ran out or a bounds check tripped               */
  LING_B200_ERR_UNSUPPORTED = 5
};
/* per-sequence status in ling_b200_seq_result */
enum { LING_B200_SEQ_OK = 0, LING_B200_SEQ_NONFINITE = 1 /* NonFiniteLogits, sampling.hpp:22-25 */ };

/* ------------------------------------------------------------------------------------------------ model  */
/* ModelConfig of the reference (src/core/model.hpp:43-62), as a POD. */
typedef struct ling_b200_model_config {
  int hidden, intermediate, layers, vocab;
  int heads, kv_heads, head_dim, rotary_dim;
  float rope_theta, eps;
  int lin_k_heads, lin_v_heads, lin_k_dim, lin_v_dim, conv_kernel; /* conv_kernel must be 4 */
  unsigned char full_attention[LING_B200_MAX_LAYERS];             /* per layer: 1 = gated GQA attention  */
} ling_b200_model_config;

/* EngineOptions (src/core/engine.hpp:56-187), the fields this path reads. */
typedef struct ling_b200_options {
  int sessions;      /* resident session slots: each owns a page table, DeltaNet state and conv window */
  int max_context;   /* positions one session's page table can map                                    */
  int page_tokens;   /* positions per KV page: 16 or 64 (reference: compile-time 64, kernels.cuh:57)  */
  int pool_pages;    /* usable pages (ids 1..pool_pages); page 0 is reserved (kv_pool.hpp:4-5)         */
  int max_seqs;      /* most sequences in one step  (<= LING_B200_MAX_SEQS)                            */
  int max_rows;      /* most packed rows in one step (<= LING_B200_MAX_ROWS)                           */
  int gemm_impl;     /* 0 = tcgen05/TMEM/TMA (the product path); 1 = plain CUDA-core GEMM (cross-check) */
  int use_graph;     /* 1 = replay the step as one CUDA graph (engine.hpp:125 step_graphs)             */
  int device;        /* CUDA device ordinal                                                           */
  int debug_rows;    /* rows for which logits and per-layer taps can be kept (0: neither is available)   */
  int pdl;           /* 1 = programmatic dependent launch (launch.cuh:1-98 in the reference): a GEMM prefetches its
                        weight tiles while the kernel before it finishes                                 */
  int chain;         /* 1 = steps of at most 32 packed rows run each layer's segments (norm + in projection; out projection +
                        norm + gate|up + SiLU + down) as persistent kernels with counter dependencies, the reference's
                        ffn_persistent / gdn_persistent idea (stream_gemm.cu:841-851,1074-1086); bit-identical results,
                        but on B200 slower than the separate launches (10.1 vs 7.6 ms per 27B step): off by default     */
  int gating_stream; /* 0 (default) or 1 = the DeltaNet gating projections (a, b -> g, beta: needed only by the DeltaNet kernel)
                        run on a second stream beside the in projection, forked after the norm and joined before the DeltaNet
                        kernel (7.61 -> 7.52 ms per 27B step; the same kernels, the same results); -1 = in the step's one stream   */
  int attn_positions; /* 0, or the cached positions summed over a step's sequences that the attention's partial buffers are
                        sized for, when larger than the pool's positions: sessions that share pages (the prefix KV store)
                        can hold more context between them than the pool has pages for                              */
  int fuse_swiglu;   /* 1 = silu(gate) * up and its FP8 copy are written by the gate|up GEMM itself: the CTA that completes a pair
                        of gate and up tiles last (a ticket per pair) adds the K splits' planes and applies them; one launch
                        less per layer, the same bits.  Measured slower than the kernel of its own behind the GEMM (7.96
                        against 7.49 ms per 27B step: the last CTA's round trips to L2 sit on the critical path, the
                        separate kernel's launch is hidden by dependent launch): 0 = off (default)                  */
  int reserved[1];
} ling_b200_options;

typedef struct ling_b200_ctx ling_b200_ctx;

/* Engine::Engine (src/core/engine.cpp:129-434): everything is allocated here, nothing while serving. */
int ling_b200_create(const ling_b200_model_config* cfg, const ling_b200_options* opt, ling_b200_ctx** out);
/* A second set of step buffers (activations, descriptors, streams, graphs) on a context's weights, KV pool, page tables and state
 * slots: for work that runs beside that context's verify steps on the same GPU without touching its staged step (a prefill
 * chunk's attention layers).  The sibling owns none of the shared memory: destroy it before the parent; it takes no weight
 * uploads.  No counterpart of its own in the reference, where the prefill and the verify path share one engine's buffers in
 * turn. */
int ling_b200_create_sibling(const ling_b200_ctx* parent, int max_seqs, int max_rows, ling_b200_ctx** out);
void ling_b200_destroy(ling_b200_ctx* ctx);
/* The last error's text (thread-local for calls without a context). */
const char* ling_b200_last_error(void);
/* Library/ABI version, and whether the CUDA kernels are present (always 1: there is no CPU path). */
int ling_b200_abi_version(void);
/* kernels::set_pdl / pdl_enabled (src/core/kernels.cuh:82-83): programmatic dependent launch for launches that the calling
 * host thread makes outside a context's step (the kernel-level entry points below).  A context's step follows its own
 * options.pdl and leaves this setting as it found it. */
void ling_b200_set_pdl(int on);
int ling_b200_pdl_enabled(void);

/* Tensor names for ling_b200_set_tensor (LayerWeights, src/core/model.hpp:86-104). */
enum {
  LING_B200_T_EMBED = 0,   /* [vocab][hidden]   kept BF16                                   */
  LING_B200_T_FINAL_NORM,  /* [hidden]          BF16                                        */
  LING_B200_T_LM_HEAD,     /* [vocab][hidden]   FP8 E4M3 + fp32 scale per 1x128             */
  LING_B200_T_INPUT_NORM,  /* [hidden]                                                      */
  LING_B200_T_POST_NORM,   /* [hidden]                                                      */
  LING_B200_T_GATE,        /* [intermediate][hidden] FP8                                    */
  LING_B200_T_UP,          /* [intermediate][hidden] FP8                                    */
  LING_B200_T_DOWN,        /* [hidden][intermediate] FP8                                    */
  LING_B200_T_IN_QKV,      /* [C][hidden] FP8, C = 2*Hk*Dk + HV*Dv, channels q|k|v          */
  LING_B200_T_IN_Z,        /* [HV*Dv][hidden] FP8                                           */
  LING_B200_T_OUT,         /* [hidden][HV*Dv] FP8                                           */
  LING_B200_T_IN_A,        /* [HV][hidden] BF16                                             */
  LING_B200_T_IN_B,        /* [HV][hidden] BF16                                             */
  LING_B200_T_CONV,        /* [C][4] BF16                                                   */
  LING_B200_T_A_LOG,       /* [HV] BF16                                                     */
  LING_B200_T_DT_BIAS,     /* [HV] BF16                                                     */
  LING_B200_T_LIN_NORM,    /* [Dv] BF16                                                     */
  LING_B200_T_Q,           /* [Hq*2*D][hidden] FP8, per head: D query rows then D gate rows */
  LING_B200_T_K,           /* [Hkv*D][hidden] FP8                                           */
  LING_B200_T_V,           /* [Hkv*D][hidden] FP8                                           */
  LING_B200_T_O,           /* [hidden][Hq*D] FP8                                            */
  LING_B200_T_Q_NORM,      /* [D] BF16                                                      */
  LING_B200_T_K_NORM,      /* [D] BF16                                                      */
  LING_B200_T_COUNT
};

/* Model::Model upload (src/core/model.cu:265-276): one tensor from host fp32 [rows][cols]; matrices are
 * rounded to BF16 first and then to FP8 E4M3 with one fp32 scale (amax/448) per row per 128 columns, on the
 * device; the rest are kept as BF16.  `layer` is ignored for the three global tensors. */
int ling_b200_set_tensor(ling_b200_ctx* ctx, int layer, int tensor, const float* host, int rows, int cols);
/* Every tensor filled on the device from the counter-based generator keyed by (seed, layer, tensor, index):
 * matrices N(0, 0.02) rounded to BF16 (an Irwin-Hall sum of 12 uniforms, exact integer arithmetic, so the
 * host restates any element bit for bit); norms N(0, 0.02); conv N(0, 0.3); A_log, dt_bias N(0, 0.5).
 * Stands in for the checkpoints (absent). */
int ling_b200_synth_weights(ling_b200_ctx* ctx, uint64_t seed);
/* A matrix's device encoding back on the host (parity of the quantizer): codes [rows][cols] and scales
 * [rows][ceil(cols/128)].  Either pointer may be NULL. */
int ling_b200_get_matrix(ling_b200_ctx* ctx, int layer, int tensor, uint8_t* codes, float* scales, int rows, int cols);
/* Bytes of weights one step streams (GEMM codes + block scales + BF16 extras + nothing of the embedding). */
size_t ling_b200_weight_bytes(const ling_b200_ctx* ctx);

/* ------------------------------------------------------------------------------------------------ sessions */
/* kv_table_set (src/core/kernels.cuh:156-161, kernels.cu:501-509): table[slot][idx[i]] = page[i]; the entries
 * are ordered on the step stream before the next step reads them.  page 0 = unmapped. */
int ling_b200_kv_table_set(ling_b200_ctx* ctx, int slot, const int* idx, const int* page, int n);
/* Copy-on-write page copies returned by KvPool::ensure (kv_pool.hpp:24-26, engine.cpp:858-866): whole pages,
 * every full-attention layer's K and V codes and scales, src[i] into dst[i]. */
int ling_b200_kv_pages_copy(ling_b200_ctx* ctx, const int* src, const int* dst, int n);
/* The K and V of positions [from, from+n) of one full-attention layer (index among the attention layers)
 * written through the slot's page table from host fp32 [n][kv_heads][head_dim] (K already normed and
 * rotated).  Quantized as the step quantizes them: E4M3 codes, one fp32 scale amax/448 per (position, head).
 * What a prefill would have left; tests and benches build contexts with it. */
int ling_b200_kv_write(ling_b200_ctx* ctx, int slot, int attn_layer, int from, int n, const float* k, const float* v);
/* The same positions read back dequantized (fp32), or as codes+scales when the float pointers are NULL. */
int ling_b200_kv_read(ling_b200_ctx* ctx, int slot, int attn_layer, int from, int n, float* k, float* v,
                      uint8_t* kcodes, float* kscales, uint8_t* vcodes, float* vscales);
/* Positions [0, n) of every attention layer of a slot filled on the device from the generator (N(0,1) values). */
int ling_b200_synth_kv(ling_b200_ctx* ctx, int slot, int n, uint64_t seed);
/* The same over positions [from, from + n) only (a prefill stand-in that resumed at `from` must not write the positions it
 * shares with another holder); values are a function of the seed, the slot, the layer and the position. */
int ling_b200_synth_kv_range(ling_b200_ctx* ctx, int slot, int from, int n, uint64_t seed);
/* One DeltaNet layer's (index among the DeltaNet layers) state [HV][Dk][Dv] and conv window [C][3] of a slot
 * (engine.cpp:226-229).  NULL pointers are skipped. */
int ling_b200_state_write(ling_b200_ctx* ctx, int slot, int gdn_layer, const float* state, const float* conv);
int ling_b200_state_read(ling_b200_ctx* ctx, int slot, int gdn_layer, float* state, float* conv);
int ling_b200_synth_state(ling_b200_ctx* ctx, int slot, uint64_t seed); /* state N(0,0.1), window N(0,1) */
/* Engine::state_hash (engine.cpp:954-971): FNV-1a over every DeltaNet and conv state of a slot, bit for bit. */
int ling_b200_state_hash(ling_b200_ctx* ctx, int slot, uint64_t* hash);

/* A session's whole recurrent state (every DeltaNet layer's state, then every conv window) saved to and restored from a
 * device arena, as the prefix KV store keeps states at its nodes' ends (Engine::copy_slot / state_view,
 * engine.cpp:1061-1068,1125-1137; the arena is EngineOptions::prefix_kv_mb's, engine.cpp:380-425).  The arena is reserved once;
 * offsets into it are the caller's bookkeeping (ling_b200_arena_*), multiples of 16.  The copies are queued on the
 * context's stream, in order with the steps.  ling_b200_state_reset zeroes a slot (Engine::reset_state). */
size_t ling_b200_state_bytes(const ling_b200_ctx* ctx);
int ling_b200_state_arena_reserve(ling_b200_ctx* ctx, size_t bytes);
int ling_b200_state_save(ling_b200_ctx* ctx, int slot, size_t offset);
int ling_b200_state_restore(ling_b200_ctx* ctx, int slot, size_t offset);
int ling_b200_state_reset(ling_b200_ctx* ctx, int slot);

/* ------------------------------------------------------------------------------------------------ the step */
/* One sequence of a step: Engine::SeqStep (engine.hpp:337-344) after the drafter has produced its tree
 * (DraftTree, tree.hpp:41-48: parent index < child index, row 0 the anchor, rows 1..chain the chain). */
typedef struct ling_b200_seq_step {
  int slot;          /* session slot                                                           */
  int pos;           /* positions already in the cache: the anchor's slot (Session::pos)        */
  int rope_delta;    /* DevPos::rdelta (kernels.cuh:27-29)                                      */
  int n_rows;        /* 1..32                                                                   */
  int chain;         /* DraftTree::E                                                            */
  const int* tokens; /* [n_rows]                                                                */
  const int* parent; /* [n_rows], parent[0] = -1                                                */
  const int* force_argmax; /* NULL, or [n_rows]: replaces the device argmax before acceptance (a test and
                              benchmark hook that imposes an accepted length); a negative entry leaves
                              that row's own argmax                                              */
} ling_b200_seq_step;

typedef struct ling_b200_seq_result {
  int status;                                   /* LING_B200_SEQ_*                                  */
  int n_path;                                   /* accepted path rows, the anchor included (>= 1)   */
  int path[LING_B200_MAX_TREE_ROWS];            /* accept_tree_greedy's rows (tree.cpp:148-166)      */
  int next_token;                               /* the token after the path                          */
  int n_out;                                    /* = n_path                                          */
  int out[LING_B200_MAX_TREE_ROWS + 1];         /* SeqStep::out: accepted drafts, then next_token    */
} ling_b200_seq_result;

/* The attention kernels keep one partial result per (kv head, 512-key chunk of a sequence's context) of a step: the slots a
 * sequence with `pos` cached positions takes, and the slots the context has.  A step whose sequences need more is refused
 * (LING_B200_ERR_ARG) before anything is launched; a scheduler counts them when it chooses a pass's partners.  No counterpart
 * in the reference, whose attention scratch is sized for the rows and the context capacity of a pass (engine.cpp:109-111). */
int ling_b200_attn_slot_need(const ling_b200_ctx* ctx, int pos);
int ling_b200_attn_slot_capacity(const ling_b200_ctx* ctx);

/* Flags of ling_b200_verify_step. */
enum {
  LING_B200_STEP_COMMIT = 1,       /* compaction + DeltaNet commit inside the step (speculate.cpp:1004-1020,516-529) */
  LING_B200_STEP_KEEP_LOGITS = 2,  /* also materialize logits[rows][vocab] (SeqStep::row_logits)                    */
  LING_B200_STEP_KEEP_TAPS = 4     /* keep per-layer residual rows for ling_b200_read_tap (debug / parity)          */
};

/* Engine::speculate_batch (speculate.cpp:1101-1282) from its verify on: pack the trees, one forward pass over
 * all rows, argmax, greedy tree acceptance, KV compaction and DeltaNet commit.  Host buffers in, host buffers
 * out; the page tables must already map [pos, pos + n_rows) of every sequence (kv_ensure, engine.cpp:841-869).
 * Returns after the result is on the host. */
int ling_b200_verify_step(ling_b200_ctx* ctx, const ling_b200_seq_step* seqs, int n_seqs, int flags,
                          ling_b200_seq_result* results);
/* The same step split for measurement with inputs resident in HBM: stage() copies the descriptors,
 * launch() enqueues the step (graph replay) on the context's stream, fetch() waits and reads the results. */
int ling_b200_step_stage(ling_b200_ctx* ctx, const ling_b200_seq_step* seqs, int n_seqs, int flags);
int ling_b200_step_launch(ling_b200_ctx* ctx);
int ling_b200_step_fetch(ling_b200_ctx* ctx, ling_b200_seq_result* results);

/* kernels::TreeDesc (src/core/kernels.cuh:119-130), the same field order, so a describe_tree result compares
 * with memcmp. */
typedef struct ling_b200_tree_desc {
  int n;
  int depth[LING_B200_MAX_TREE_ROWS];
  int var[LING_B200_MAX_TREE_ROWS];
  int nvar;
  int path[LING_B200_MAX_TREE_VARIANTS][LING_B200_MAX_TREE_ROWS];
  int ngdn;
  int gdn_len[LING_B200_MAX_TREE_VARIANTS];
  int gdn_step[LING_B200_MAX_TREE_VARIANTS][2 * LING_B200_MAX_TREE_ROWS];
} ling_b200_tree_desc;
#define LING_B200_TREE_LEAF (1 << 8)
#define LING_B200_TREE_WRITE (1 << 9)

/* What the last step built and computed, read back for parity checks. */
/* describe_tree's result for sequence i of the last step, built on the device (tree.cpp:81-146). */
int ling_b200_read_tree_desc(ling_b200_ctx* ctx, int seq, ling_b200_tree_desc* out);
/* Packing of the last step (speculate.cpp:1190-1201; kernels.cuh:58-78): row0[n_seqs+1], and per packed row its
 * sequence, depth, RoPE position, cache slot and ancestor mask (bit j set: row row0+j of its sequence is on the
 * row's root-to-row path, the row itself included).  NULL pointers are skipped. */
int ling_b200_read_packing(ling_b200_ctx* ctx, int* row0, int* token, int* seq_of, int* depth, int* rope_pos,
                           int* cache_slot, uint32_t* anc_mask);
/* Per packed row: argmax id and value (topk_rows K=1, topk.cu:83-129). */
int ling_b200_read_argmax(ling_b200_ctx* ctx, int* ids, float* vals);
/* logits[rows][vocab] of the last step (needs LING_B200_STEP_KEEP_LOGITS). */
int ling_b200_read_logits(ling_b200_ctx* ctx, float* out);
/* Residual stream after layer `layer` (0..layers-1), or the final-normed rows for layer = layers;
 * [rows][hidden] (needs LING_B200_STEP_KEEP_TAPS). */
int ling_b200_read_tap(ling_b200_ctx* ctx, int layer, float* out);

/* ------------------------------------------------------------------------------------------------ timing */
/* Device time of the last n launch() calls, measured with CUDA events on the context's stream. */
int ling_b200_timer_begin(ling_b200_ctx* ctx);
int ling_b200_timer_end(ling_b200_ctx* ctx, float* ms);
/* Per-kernel-family device time of one eager (non-graph) replay of the staged step, by CUDA events around each
 * family's launches: [0] weight GEMMs, [1] attention, [2] DeltaNet, [3] norms/quant/elementwise,
 * [4] head+argmax, [5] pack/accept/compact/commit.  Also the number of kernel launches in one step. */
int ling_b200_profile_step(ling_b200_ctx* ctx, float ms[8], int* launches);
/* The weight GEMMs of one step (4 per layer + the LM head, in the step's order, on the staged step's row class and the
 * activations the last step left) captured as one graph and replayed `iters` times on the context's stream between two
 * CUDA events after one warm-up replay: ms per pass.  The GEMM's streaming rate with nothing between the launches. */
int ling_b200_gemm_chain_ms(ling_b200_ctx* ctx, int iters, float* ms);
int ling_b200_step_launch_count(ling_b200_ctx* ctx);
/* Debugging aid (the reference's LING_MK_TIMES, engine.hpp:637-642): with LING_B200_TIMELINE=1 in the environment when
 * the context is created, replays the staged step once and returns four GPU-timer stamps (ns) per weight-GEMM launch:
 * first CTA start, first and last producer past the dependency wait, last CTA end.  Returns the launches written. */
int ling_b200_gemm_timeline(ling_b200_ctx* ctx, unsigned long long* out, int max_launches);
/* Writes more than L2 between timed steps (the bench's flush). */
int ling_b200_flush_l2(ling_b200_ctx* ctx);
int ling_b200_sync(ling_b200_ctx* ctx);

/* ------------------------------------------------------------------------------------------------ kernels */
/* The kernel layer of the reference is free functions over raw device pointers (src/core/kernels.cuh:82-578).
 * These take HOST buffers, run the kernel once on the device and copy the result back, for parity tests. */

/* y[M][N] = x[M][K] . W[N][K]^T with x quantized to E4M3 per row per 128 columns and W per row per 128 columns
 * (stream_gemm_fp8, stream_gemm.cu:674-703, at this build's numerics).  impl as ling_b200_options.gemm_impl.
 * splits: the K split (0 = the library's choice for the shape). */
int ling_b200_gemm_fp8_host(int device, int impl, int splits, const float* x, const float* w, float* y, int M, int N, int K);
/* The same GEMM timed on the device with resident operands: ms per launch over `iters` launches. */
int ling_b200_gemm_fp8_bench(int device, int impl, int splits, int M, int N, int K, int iters, float* ms_per_launch);
/* The FP8 tensor pipe's sustained dense rate on this GPU, measured: one CTA per SM issues `iters` groups of tcgen05.mma
 * kind::f8f6f4 (128 x 256 x 128 each) on operands resident in shared memory, no loads and no epilogue, between two CUDA
 * events.  The denominator for the many-row, tensor-bound configurations (the reference quotes none for B200). */
int ling_b200_fp8_tensor_peak(int device, int iters, float* tflops, float* ms);

/* ---- NVFP4 operands of the prefill chunk: E2M1 values two a byte (the first in the low nibble), one E4M3 scale per 16
 * values, one fp32 scale per tensor.  The entry points below take the reference's layouts (values [rows][K/2], scales
 * [rows][K/16] row-major, HOST buffers); on the device the library keeps the scales in the order tcgen05.cp reads. ---- */

/* quantize_nvfp4 (src/core/model.hpp:29-41; model.cu:188-249): BF16 weights [N][K] (bit patterns) to NVFP4 in the
 * checkpoints' rounding: *scale2 = amax / (448 * 6), block scales max(amax16 / 6 / scale2, 2^-9) as E4M3, codes nearest
 * with a value halfway between two codes taking the smaller magnitude.  K % 16 == 0. */
int ling_b200_quantize_nvfp4_host(int device, const uint16_t* w_bf16, int N, int K, uint8_t* values, uint8_t* scales, float* scale2);
/* quant_act_nvfp4 and, with up != NULL, silu_mul_quant_nvfp4 (src/core/kernels.cuh:190-197; prefill_gemm.cu:383-420,
 * 607-618): x (or silu(x) * up) [M][K] rounded to BF16, then NVFP4 under the global scale 1 / input_scale. */
int ling_b200_quant_act_nvfp4_host(int device, const float* x, const float* up, int M, int K, float input_scale, uint8_t* q, uint8_t* sf);
/* rmsnorm_quant with nvfp4 = true (src/core/kernels.cuh:203-204; prefill_gemm.cu:426-459,632-638): x * rstd * (1 + w) per row,
 * into NVFP4 and, when out != NULL, into fp32 too.  w: BF16 bit patterns [H]. */
int ling_b200_rmsnorm_quant_nvfp4_host(int device, const float* x, const uint16_t* w_bf16, float* out, int M, int H, float eps,
                                       float input_scale, uint8_t* q, uint8_t* sf);
/* prefill_gemm_nvfp4 (src/core/kernels.cuh:206-210; prefill_gemm.cu:685-690): y[m * ldy + n] = alpha * xq[m] . w[n] (or += with
 * accumulate) over n < N; columns N .. ldy of y are left alone.  The weight is given in the checkpoint layout (the
 * reference passes its tiled copy of the same values).  N % 128 == 0, K % 128 == 0, M = 0 returns at once. */
int ling_b200_prefill_gemm_nvfp4_host(int device, const uint8_t* xq, const uint8_t* xs, int M, const uint8_t* wq, const uint8_t* ws,
                                      float alpha, float* y, int ldy, int N, int K, int accumulate);
/* prefill_swiglu_nvfp4 (src/core/kernels.cuh:215-221; prefill_gemm.cu:700-715): NVFP4(silu(alpha_gate * xq . G^T) *
 * (alpha_up * xq . U^T)) under the global scale 1 / out_input_scale into q_out [M][N/2], sf_out [M][N/16]; byte for byte
 * what the two plain GEMMs followed by ling_b200_quant_act_nvfp4_host(up != NULL) give. */
int ling_b200_prefill_swiglu_nvfp4_host(int device, const uint8_t* xq, const uint8_t* xs, int M, const uint8_t* gate_q,
                                        const uint8_t* gate_s, float alpha_gate, const uint8_t* up_q, const uint8_t* up_s, float alpha_up,
                                        int N, int K, float out_input_scale, uint8_t* q_out, uint8_t* sf_out);
/* Which form of the NVFP4 GEMM the entry points below launch (process-wide): 0 = one CTA per 128 x 256 tile, 1 = the
 * two-CTA form (tcgen05 cta_group::2 over a cluster of two: 256 x 256 per pair, each CTA loading its own rows of the
 * activations and half of the weight tile by ordinary, non-multicast TMA).  Same results bit for bit.  Returns the previous
 * setting. */
int ling_b200_nvfp4_pair_mode(int mode);
/* The NVFP4 GEMM (fused != 0: the gate|up form) timed on the device with resident operands: ms per launch.  cycle_shares
 * (optional, 3 doubles): from one more launch with the kernel's cycle counters on, the shares of a CTA's time that the MMA
 * issuer spent waiting for operand stages, that it spent waiting for the epilogue to free the accumulator, and that one
 * epilogue warp was busy. */
int ling_b200_nvfp4_gemm_bench(int device, int M, int N, int K, int fused, int iters, float* ms_per_launch, double* cycle_shares);

/* The NVFP4 tensor pipe's dense rate on this GPU, measured like ling_b200_fp8_tensor_peak: tcgen05.mma kind::mxf4nvf4.block_scale
 * (128 x 256 x 64, block scales of 16 in tensor memory) on resident operands.  mode 0 is the denominator for the NVFP4 GEMMs.
 * The other modes price the GEMM's scale copies (tcgen05.cp, shared -> tensor memory, 48 columns per group of four MMAs):
 * 1 = twelve 32x128b.warpx4 copies before every group into the region the MMAs read; 2 = into two regions in turn; 3 = issued
 * by a thread of another warp into a region the running MMAs do not read; 4 = the same 48 columns written by six 128x256b
 * copies.  All four cost the pipe the same third: the price is per column written, whoever issues it and in whatever shape. */
int ling_b200_fp4_tensor_peak(int device, int iters, int mode, float* tflops, float* ms);

/* The prefill chunk's feed-forward stack held on the device: per layer h += down(swiglu(gate, up)(norm(h))), the three
 * matrices NVFP4 with synthetic BF16 N(0, 0.02) values rounded as quantize_nvfp4 rounds (the quantized branch of the
 * layer loop's MLP section, src/core/engine.cpp:1238-1247,1704-1711, taken for a chunk of more than 32 rows).  It owns a stream: launch() enqueues the whole stack
 * over the resident residual `repeats` times and returns, wait() joins it and reports the device time between its events, so the stack can run
 * beside a verify step of a ling_b200_ctx; forward() is the host-buffer call (pinned staging, copies inside). */
typedef struct ling_b200_nvfp4_ffn ling_b200_nvfp4_ffn;
int ling_b200_nvfp4_ffn_create(int device, int layers, int hidden, int intermediate, int max_rows, uint64_t seed,
                               ling_b200_nvfp4_ffn** out);
void ling_b200_nvfp4_ffn_destroy(ling_b200_nvfp4_ffn* f);
/* Adds the DeltaNet layers' prefill-path mixers (see ling_b200_prefill_gdn below) in front of their feed-forward blocks: every
 * layer except each full_every-th (0: every layer) gets synthetic mixer weights and a zero state.  The full-attention layers'
 * mixer on the prefill path is not built: those layers keep their feed-forward block only. */
int ling_b200_nvfp4_ffn_add_mixers(ling_b200_nvfp4_ffn* f, int k_heads, int v_heads, int full_every, uint64_t seed);
int ling_b200_nvfp4_ffn_set_residual(ling_b200_nvfp4_ffn* f, const float* h, int rows);
int ling_b200_nvfp4_ffn_launch(ling_b200_nvfp4_ffn* f, int rows, int repeats);
/* CTAs of each GEMM launch of the stack (0 = one per SM): fewer leave SMs to a verify step running beside it. */
int ling_b200_nvfp4_ffn_set_ctas(ling_b200_nvfp4_ffn* f, int ctas);
int ling_b200_nvfp4_ffn_wait(ling_b200_nvfp4_ffn* f, float* device_ms);
int ling_b200_nvfp4_ffn_forward(ling_b200_nvfp4_ffn* f, const float* h_in, int rows, float* h_out);
/* One layer's operands back on the host in the reference's layouts (any pointer may be NULL); scales5 = the static
 * activation scales of the two GEMMs' inputs, then the tensor scales of gate, up and down. */
int ling_b200_nvfp4_ffn_read_layer(ling_b200_nvfp4_ffn* f, int layer, uint16_t* norm_bf16, uint8_t* gate_q, uint8_t* gate_s,
                                   uint8_t* up_q, uint8_t* up_s, uint8_t* down_q, uint8_t* down_s, float* scales5);

/* The kernels' bounded wait made to run out on purpose, harmlessly: one CTA waits at most limit_us microseconds on a barrier
 * that nobody arrives at, records the code of an expired wait in the error word and returns.  The call returns
 * LING_B200_ERR_DEVICE_FLAG with that code in *code (1) and the time the kernel waited in *waited_us; the device and its
 * contexts stay usable.  (The reference's persistent kernels trap after 50 ms instead, stream_gemm.cu:865-882.) */
int ling_b200_wait_probe(int device, unsigned limit_us, int* code, unsigned* waited_us);

/* No counterpart in the reference.  The same block-scaled FP8 GEMM for hosts that must not allocate device memory on
 * this path: a serving loop that gave the whole device to its own arena at start-up, a real-time thread for which an
 * allocation's implicit synchronization is not acceptable, a sandboxed plugin that receives buffers but may not create
 * them.  The K splits' partial-sum planes, which the other entry points allocate, live in a 16 MiB __device__ array built
 * into the library (every GPU that loads it carries the array until the process exits).  This call makes no cudaMalloc /
 * cudaFree and calls no allocating library routine.
 *   All pointers are DEVICE pointers in the library's operand layouts, padded with zero codes:
 *   w_codes [N_pad][K_pad] E4M3, w_scales [K_pad/128][N_pad] fp32, x_codes [128][K_pad] E4M3 (rows >= M unused),
 *   x_scales [K_pad/128][128] fp32, y [M][N] fp32; N_pad, K_pad = N, K rounded up to 128.
 *   Limits: M <= LING_B200_NOALLOC_MAX_ROWS and N_pad <= 32768 (one plane must fit the array); beyond them the call
 *   returns LING_B200_ERR_ARG and touches nothing.  The K split is the regular one unless the array holds fewer planes.
 *   The first call on a device looks the array's address up (cudaGetSymbolAddress) and sets kernel attributes.  Every
 *   call enqueues on `stream` (NULL = the default stream), waits for the stream and returns the status; the device that owns the operands and `stream` must be the calling thread's current device.  Every call shares
 *   the array: calls that overlap on the GPU race.  Nothing in it needs clearing by the caller. */
#define LING_B200_NOALLOC_MAX_ROWS 128
#define LING_B200_NOALLOC_SCRATCH_BYTES (16u << 20)
int ling_b200_gemm_fp8_noalloc(const uint8_t* w_codes, const float* w_scales, const uint8_t* x_codes, const float* x_scales,
                               float* y, int M, int N, int K, void* stream);

/* attention_rows(_seqs) + attention_combine (kernels.cuh:223-290; kernels.cu:919-961) for one full-attention layer (index
 * among the attention layers): q [rows][heads][head_dim] (normed, rotated); every row attends to its sequence's context
 * [0, pos) and to the in-flight positions pos + j of its own root-to-row path, as the slot's cache holds them (write them
 * with ling_b200_kv_write first); out [rows][heads][head_dim], before the output gate. */
int ling_b200_attention_host(ling_b200_ctx* ctx, const ling_b200_seq_step* seqs, int n_seqs, int attn_layer, const float* q,
                             float* out);

/* attn_prepare(_seqs) (kernels.cuh:223-236; kernels.cu:558-596, attention_body.cuh:54-99) for one full-attention layer:
 * qkv [rows][heads * 2 * head_dim + 2 * kv_heads * head_dim] is the q|k|v projection's output (per q head: head_dim query
 * values, then head_dim gate values); every row's K (normed, rotated at pos + depth + rope_delta) and V (raw) go to cache
 * slot pos + row index of its sequence's slot (read them back with ling_b200_kv_read); q_out [rows][heads][head_dim] is
 * the normed, rotated query as the attention kernel receives it (rounded to FP16). */
int ling_b200_attn_prepare_host(ling_b200_ctx* ctx, const ling_b200_seq_step* seqs, int n_seqs, int attn_layer,
                                const float* qkv, float* q_out);

/* gdn_conv_tree + gdn_recurrent_tree + gated_rmsnorm (kernels.cuh:131-136, 478-480) as the step's single DeltaNet kernel
 * runs them, for n_seqs sequences of one layer (the kernel covers key dim = value dim = 64 or 128).  n_rows, chain
 * [n_seqs]; parent [rows] the sequences' trees one after another (a sequence's row 0 is its anchor); in [rows][C + HV*Dv]
 * the in projection's output (conv channels q|k|v, then z); convw [C][4]; g, beta [rows][HV]; state [n_seqs][HV][Dk][Dv]
 * and conv [n_seqs][C][3] (read, never written); norm_w [Dv].  Out: pre [rows][C] (the raw conv inputs kept for the
 * commit), post [rows][C] (as ling_b200_gdn_tree_host), core [rows][HV*Dv] (the recurrence's output before the gated
 * norm), and the out projection's FP8 input: out_codes [rows][HV*Dv], out_scales [rows][HV*Dv/128]. */
int ling_b200_gdn_fused_host(int device, int Hk, int HV, int Dk, int Dv, int n_seqs, const int* n_rows, const int* chain,
                             const int* parent, const float* in, const float* convw, const float* g, const float* beta,
                             const float* state, const float* conv, const float* norm_w, float eps, float* pre, float* post,
                             float* core, uint8_t* out_codes, float* out_scales);

/* gdn_conv_tree + gdn_recurrent_tree (kernels.cuh:131-136): one sequence, one layer.  pre [n][C], g and beta
 * [n][HV] (g = log decay), state [HV][Dk][Dv], conv [C][3]; out core [n][HV*Dv] and post [n][C] (the conv outputs with
 * the q and k channels already L2-normalized per head, q also scaled by 1/sqrt(Dk): what the recurrence consumes). */
int ling_b200_gdn_tree_host(int device, int Hk, int HV, int Dk, int Dv, const ling_b200_tree_desc* td,
                            const float* pre, const float* convw, const float* g, const float* beta,
                            const float* state, const float* conv, float* post, float* core);
/* Engine::commit (speculate.cpp:516-529) for one layer: rows path[0..n) replayed, state and window written.
 * `post` as ling_b200_gdn_tree_host returns it. */
int ling_b200_gdn_commit_host(int device, int Hk, int HV, int Dk, int Dv, const int* path, int n, int rows,
                              const float* pre, const float* post, const float* g, const float* beta,
                              float* state, float* conv);
/* topk_rows K=1 (topk.cu:83-129): ids/vals per row, ties to the lower id, NaN skipped. */
int ling_b200_argmax_host(int device, const float* logits, int rows, int vocab, int* ids, float* vals);

/* ------------------------------------------------------------------------------------------------ host logic */
/* describe_tree (tree.cpp:81-146) on the host: returns 0 or LING_B200_ERR_ARG (too many rows/leaves/paths). */
int ling_b200_describe_tree(const int* parent, int n_rows, int chain, ling_b200_tree_desc* out);
/* accept_tree_greedy (tree.cpp:148-166): path out (<= n_rows entries), returns the path length. */
int ling_b200_accept_tree_greedy(const int* parent, const int* token, int n_rows, const int* argmax, int* path,
                                 int* next);
/* lookup_propose (lookup.cpp:7-24): returns the number of proposed tokens written to out (<= max). */
int ling_b200_lookup_propose(const int* seq, int len, int max, int ngram, int* out, int* match);
/* build_tree (tree.cpp:30-79). shape = {nodes, width, max_depth, chain}; returns rows, fills parent/depth/token/pick. */
int ling_b200_build_tree(int anchor, const int* cand, const float* scores, int E, int K16, const int* chain_tokens,
                         const int* chain_picks, int nodes, double temp, int width, int max_depth, int chain,
                         int max_rows, int* parent, int* depth, int* token, int* pick, double* extra_mass);

/* KvPool (src/core/kv_pool.hpp:20-83), handle based.  Tables are caller-owned int arrays with their length. */
typedef struct ling_b200_kvpool ling_b200_kvpool;
ling_b200_kvpool* ling_b200_kvpool_create(int pages, int page_tokens);
void ling_b200_kvpool_destroy(ling_b200_kvpool* p);
int ling_b200_kvpool_capacity(const ling_b200_kvpool* p);
int ling_b200_kvpool_free_pages(const ling_b200_kvpool* p);
int ling_b200_kvpool_pending_pages(const ling_b200_kvpool* p);
int ling_b200_kvpool_refs(const ling_b200_kvpool* p, int page);
int ling_b200_kvpool_needed(const ling_b200_kvpool* p, const int* table, int len, int from, int to);
/* ensure: table has room for cap entries; *len is updated. copies: [2*max_copies] (src,dst); returns 1/0, or <0 on a bad range. */
int ling_b200_kvpool_ensure(ling_b200_kvpool* p, int* table, int* len, int cap, int from, int to, int* copies,
                            int max_copies, int* n_copies);
int ling_b200_kvpool_share(ling_b200_kvpool* p, int* dst, int* dst_len, int cap, const int* src, int src_len, int n);
void ling_b200_kvpool_truncate(ling_b200_kvpool* p, int* table, int len, int n);
void ling_b200_kvpool_unshare(ling_b200_kvpool* p, int* table, int len, int n);
int ling_b200_kvpool_net_need(const ling_b200_kvpool* p, const int* table, int len, int pages);
int ling_b200_kvpool_resume_need(const ling_b200_kvpool* p, const int* table, int len, int reuse, int pages,
                                 const int* donor, int donor_len);
int ling_b200_kvpool_reclaimable(const ling_b200_kvpool* p, const int* const* tables, const int* lens, int n);
int ling_b200_kvpool_retain(ling_b200_kvpool* p, int page);
int ling_b200_kvpool_release(ling_b200_kvpool* p, int page);
void ling_b200_kvpool_retire(ling_b200_kvpool* p);

/* ArenaAlloc (src/core/prefix_kv.hpp:35-49): first-fit byte offsets inside one region whose size is fixed at the start, freed
 * ranges merged with their neighbours.  Host bookkeeping only; the region itself is the caller's (the saved DeltaNet states of
 * the prefix KV store live in one: ling_b200_state_arena_reserve).  alloc returns the offset, or -1 when no free range fits. */
typedef struct ling_b200_arena ling_b200_arena;
ling_b200_arena* ling_b200_arena_create(size_t size, size_t align);
void ling_b200_arena_destroy(ling_b200_arena* a);
long long ling_b200_arena_alloc(ling_b200_arena* a, size_t bytes);
void ling_b200_arena_release(ling_b200_arena* a, size_t offset);
size_t ling_b200_arena_size(const ling_b200_arena* a);
size_t ling_b200_arena_in_use(const ling_b200_arena* a);

/* PrefixKvTree in its paged mode (src/core/prefix_kv.hpp:12-22,51-124; src/core/prefix_kv.cpp): a radix tree of token runs
 * whose nodes hold a reference to each KV pool page their run overlaps, and at some node ends a saved recurrent state.  The
 * byte budget covers the states only.  The reference's std::function Ops are C callbacks over one user pointer:
 *   hold(user, from, to, pages, cap)  the active session's page ids for page indices from / page_tokens .. (to - 1) / page_tokens
 *                                     into pages[], a reference taken on each; returns how many it wrote.  Another count than
 *                                     the range's, or an id 0 among them, is a failure: the tree gives back the ids it got
 *                                     and the insert stops there, keeping the nodes already made.
 *   retain / drop(user, page)         take / give back one reference.
 *   state_alloc(user, bytes)          storage for one saved state (any non-NULL token the caller can map to it), or NULL.
 *   state_release(user, state)
 * The reference's buffer mode (KV copied into the store's own buffers: an engine without a page pool) has no counterpart: the
 * KV here always lives in pool pages.  Node ids are small integers; 0 is the root. */
typedef struct ling_b200_prefix ling_b200_prefix;
typedef struct ling_b200_prefix_ops {
  void* user;
  int (*hold)(void* user, int from, int to, int* pages, int cap);
  void (*retain)(void* user, int page);
  void (*drop)(void* user, int page);
  void* (*state_alloc)(void* user, size_t bytes);
  void (*state_release)(void* user, void* state);
} ling_b200_prefix_ops;
ling_b200_prefix* ling_b200_prefix_create(size_t budget_bytes, size_t state_bytes, int page_tokens, const ling_b200_prefix_ops* ops);
void ling_b200_prefix_destroy(ling_b200_prefix* t); /* clears first */
/* match (prefix_kv.hpp:82-83): the prompt's leading tokens held under `scope`; the nodes along them into path[] (as many as fit
 * in cap), their number into *n_path.  Returns the matched length. */
int ling_b200_prefix_match(const ling_b200_prefix* t, const int* prompt, int n, uint64_t scope, int* path, int cap, int* n_path);
/* best_state (prefix_kv.hpp:84-85): the deepest node end on the path, at most min(len, limit), that has a state: its position
 * (0: none) and, into *state, what state_alloc returned for it. */
int ling_b200_prefix_best_state(const ling_b200_prefix* t, const int* path, int n_path, int len, int limit, void** state);
/* pages (prefix_kv.hpp:88-95): one page id per page index below ceil(n / page_tokens), the deepest node's on the path where two
 * overlap.  Returns the count, or -1 when cap is too small. */
int ling_b200_prefix_pages(const ling_b200_prefix* t, const int* path, int n_path, int n, int* pages, int cap);
void ling_b200_prefix_touch(ling_b200_prefix* t, const int* path, int n_path, uint64_t epoch);
/* insert (prefix_kv.hpp:98-105): prompt[0, q) with every position of the ascending cuts[] in (0, q] a node end.  The cut nodes
 * that have no state yet come back as (node, position) pairs; returns their number (at most cap are written). */
int ling_b200_prefix_insert(ling_b200_prefix* t, const int* prompt, int n, int q, const int* cuts, int n_cuts, uint64_t epoch,
                            uint64_t scope, int* want_node, int* want_pos, int cap);
/* add_state (prefix_kv.hpp:106-107): makes room in the budget (evicting least recently used leaves stamped before `epoch`) and
 * returns the node's new state storage, or NULL. */
void* ling_b200_prefix_add_state(ling_b200_prefix* t, int node, uint64_t epoch);
/* evict_lru_leaf (prefix_kv.hpp:109-112): 1 when a leaf outside keep[] went, 0 when none is left. */
int ling_b200_prefix_evict_lru_leaf(ling_b200_prefix* t, const int* keep, int n_keep);
void ling_b200_prefix_clear(ling_b200_prefix* t);
size_t ling_b200_prefix_bytes(const ling_b200_prefix* t);
size_t ling_b200_prefix_budget(const ling_b200_prefix* t);
int ling_b200_prefix_nodes(const ling_b200_prefix* t);
int ling_b200_prefix_states(const ling_b200_prefix* t);
int ling_b200_prefix_pages_held(const ling_b200_prefix* t);
/* page_lists (prefix_kv.hpp:122-124): every live node's page ids outside skip[], concatenated into pages[] with each node's
 * count in lens[].  Returns the number of lists, or -1 when either array is too small. */
int ling_b200_prefix_page_lists(const ling_b200_prefix* t, const int* skip, int n_skip, int* pages, int cap_pages, int* lens,
                                int cap_lists);

/* select_batch / pair_order (src/serve/pairing.hpp:46-75): candidates as three parallel arrays. Returns the count. */
int ling_b200_pair_order(const int* batchable, const int* recent, const long* last, int n, int fair, int* order);
int ling_b200_select_batch(const int* batchable, const int* recent, const long* last, int n, int self, int fit,
                           int fair, int* batch);
/* kv_verdict / kv_last_resort (src/serve/kv_policy.hpp:38-93): verdict 0 Go, 1 Retire, 2 Reclaim, 3 Wait. */
int ling_b200_kv_verdict(int need, int free_pages, int pending, int idle);
int ling_b200_kv_last_resort(const long* admitted, const int* waiting, const int* need, int n, int free_pages,
                             int pending, int idle);
/* plan_memory + plan_kv_pool + refusal (src/serve/admission.hpp:94-124,202-232): returns pages; fills the plan. */
typedef struct ling_b200_memory_plan {
  size_t weights, per_session, sessions, scratch, kv_pool;
  int session_count;
  long kv_pool_pages;
  size_t total;
  int refused; /* start_plan's refusal is non-empty */
} ling_b200_memory_plan;
int ling_b200_start_plan(const ling_b200_model_config* cfg, size_t weight_bytes, size_t scratch, int drafter,
                         int sessions, int max_context, long avail_mb, long reserve_mb, int kv_on,
                         size_t store_bytes, long pool_mb, int page_tokens, int kv_elem_bytes,
                         ling_b200_memory_plan* out);
/* choose_size (admission.hpp:262-310): given values < 0 mean "not given". */
int ling_b200_choose_size(const ling_b200_model_config* cfg, size_t weight_bytes, size_t scratch, int drafter,
                          long avail_mb, long reserve_mb, int full_context, int sessions, int max_context,
                          int auto_size, int kv_on, size_t store_bytes, long pool_mb, int page_tokens,
                          int kv_elem_bytes, int* out_sessions, int* out_context, int* sessions_auto,
                          int* context_auto, int* sized);
/* refuse_request (admission.hpp:312-319): the 503 text of a request that arrives while the host is below the admission
 * reserve, into buf; returns its length, 0 when the request may run, -1 when buf is too small. */
int ling_b200_refuse_request(long avail_mb, long reserve_mb, char* buf, int buf_len);
/* kv_reclaim (src/serve/kv_policy.hpp:58-72) with the reference's std::function arguments as C callbacks over one user
 * pointer: need / have return the unit's need and the free + pending pages now; evict(user, group) evicts the next holder
 * of a group (1) or reports the group empty (0).  Groups [0, n_kept) may go without moving the unit's resume point,
 * groups [n_kept, n_kept + n_source) are the unit's own source.  Returns 1 when the unit fits at the end. */
typedef int (*ling_b200_count_fn)(void* user);
typedef int (*ling_b200_evict_fn)(void* user, int group);
int ling_b200_kv_reclaim(ling_b200_count_fn need, ling_b200_count_fn have, ling_b200_evict_fn evict, void* user, int n_kept,
                         int need_kept, int reach_kept, int n_source, int need_all, int reach_all, int must);
/* format_step (src/serve/step_trace.hpp:66-87): one trace line into buf; returns its length. */
int ling_b200_format_step(double t, long pass, const char* kind, size_t turn, const int* sessions, const int* rows,
                          const int* tokens, const int* left, int n,
                          const int* cand /* [n_cand][3]: session, state, recent */, const long* cand_request,
                          const long* cand_last, int n_cand, double ms, int side, char* buf, int buf_len);

/* Attention over the M rows of a prefill chunk of one session (positions pos0 .. pos0 + M - 1) in one attention layer, through
 * the step's own prepare / attention / combine kernels in slices of 32 query rows, as the reference's prefill runs its rows
 * kernel "in slices of queries" (src/core/kernels.cuh:486-490; Engine::forward's full-attention branch, engine.cpp:1395-1460):
 * qkv [M][Hq * 2 D + 2 Hkv D] are the q|gate, k, v projection's rows; the rows' K and V go into the session's cache (its page
 * table must map [0, pos0 + M)), out [M][Hq * D] is the gated attention output in front of the o projection.  Correct, not
 * fast: every slice reads the whole context again. */
int ling_b200_prefill_attention_host(ling_b200_ctx* ctx, int slot, int attn_layer, int pos0, int M, const float* qkv, float* out);
/* A full-attention layer's whole mixer over a prefill chunk (Engine::forward's full-attention branch over many rows,
 * src/core/engine.cpp:1424-1469): h [M][hidden] fp32 in DEVICE memory, the residual rows at positions pos0.. of session `slot`
 * (pages mapped by the caller), += o(gate * attention(prepare(q|k|v(norm(h))))) with the layer's FP8 projections; K and V of the
 * rows go to the session's pages.  The rows go through the step's kernels as 32-row chains, many chains a launch.  The call
 * returns when the work is complete; a staged verify step is replaced (stage again).  _host: h in host memory, in and out. */
int ling_b200_chunk_attention_layer(ling_b200_ctx* ctx, int slot, int layer, int pos0, int M, float* h_device);
int ling_b200_chunk_attention_layer_host(ling_b200_ctx* ctx, int slot, int layer, int pos0, int M, float* h);
/* Measurement aid: the layer over M zero rows with an event pair around every launch.  ms[0] the two FP8 projections, ms[1] the
 * attention kernel, ms[2] the combine, ms[3] the two norms, ms[5] the prepare kernel; *passes = launches of chains. */
int ling_b200_chunk_attention_layer_profile(ling_b200_ctx* ctx, int slot, int layer, int pos0, int M, float ms[8], int* passes);
/* Attaches a verify context to the chunk stack: every `full_every`-th layer (the full-attention layers) then runs
 * ling_b200_chunk_attention_layer on that context ahead of its feed-forward block, the chunk being positions pos0.. of `slot`.
 * No counterpart of its own in the reference: there one engine holds both paths. */
int ling_b200_nvfp4_ffn_attach_context(ling_b200_nvfp4_ffn* ffn, ling_b200_ctx* ctx, int slot, int pos0, int full_every);

/* ------------------------------------------------------------------------------------------------ the prefill path's DeltaNet core */
/* gdn_conv_prefill + gdn_recurrent_prefill (src/core/kernels.cuh:445-456; src/core/prefill_gdn.cu:34-142) over the M rows
 * of one sequence, host buffers: pre [M][C] the raw in-projection rows (q | k | v channels, C = 2 Hk Dk + HV Dv), convw_bf16
 * [C][4] the conv taps as BF16 bit patterns, g / beta [M][HV]; conv [C][3] (the window) and state [HV][Dk][Dv] are read and
 * advanced in place; post [M][C] (optional) = silu(conv(pre)), core [M][HV Dv] the recurrence's output.  The recurrence runs
 * in its chunked (WY) form, 32-token chunks from the first row on, FP16 tensor-core products with fp32 accumulation, so its
 * result differs from the token-by-token fp32 rule by FP16 operand rounding (the reference's prefill kernel likewise).
 * Dk = Dv = 128. */
int ling_b200_gdn_prefill_host(int device, int Hk, int HV, int Dk, int Dv, int M, const float* pre, const uint16_t* convw_bf16,
                               const float* g, const float* beta, float* state, float* conv, float* post, float* core);
/* One DeltaNet layer's mixer on the prefill path, held on the device with synthetic weights (Engine::forward's
 * linear-attention branch over many rows, quantized path: rmsnorm, NVFP4 in projections, gdn_conv_prefill, gdn_gating,
 * gdn_recurrent_prefill, gated_rmsnorm, NVFP4 out projection; src/core/kernels.cuh:190-221,436-456,543-554):
 *   h += out( gated_norm( delta_rule( conv(in_qkv(norm(h))), gating(in_a, in_b) ), in_z(norm(h)) ) )
 * for rows of one sequence; the session's state [HV][128][128] and conv window [C][3] advance.  forward takes and returns
 * host rows; read_stages gives what the last forward left between the stages and read_weights the weights as the device
 * holds them, both for parity checks; bench times passes over the resident residual. */
typedef struct ling_b200_prefill_gdn ling_b200_prefill_gdn;
int ling_b200_prefill_gdn_create(int device, int hidden, int k_heads, int v_heads, int max_rows, uint64_t seed, ling_b200_prefill_gdn** out);
void ling_b200_prefill_gdn_destroy(ling_b200_prefill_gdn* f);
int ling_b200_prefill_gdn_state(ling_b200_prefill_gdn* f, int write, float* state, float* conv);
int ling_b200_prefill_gdn_forward(ling_b200_prefill_gdn* f, const float* h_in, int rows, float* h_out);
int ling_b200_prefill_gdn_bench(ling_b200_prefill_gdn* f, int rows, int repeats, float* ms);
int ling_b200_prefill_gdn_read_stages(ling_b200_prefill_gdn* f, int rows, float* xn, float* pre, float* z, float* g, float* beta, float* core);
int ling_b200_prefill_gdn_read_weights(ling_b200_prefill_gdn* f, uint16_t* norm, uint16_t* convw, uint16_t* wa, uint16_t* wb, uint16_t* A_log,
                                       uint16_t* dt_bias, uint16_t* lin_norm, uint8_t* qkv_q, uint8_t* qkv_s, uint8_t* z_q, uint8_t* z_s,
                                       uint8_t* out_q, uint8_t* out_s, float* scales5);
/* Device time (ms per launch) of the chunked delta rule alone over M rows of synthetic inputs. */
int ling_b200_gdn_chunk_bench(int device, int Hk, int HV, int M, int iters, float* ms);

/* ------------------------------------------------------------------------------------------------ the drafter's last stage */
/* topk_rows (src/core/kernels.cuh:400-410, src/core/topk.cu:83-129) over host rows x [rows][vocab]: per row the k <= 64
 * largest values, descending, ties to the lower index (entry 0 is the argmax); a row with fewer rankable values (NaN never
 * ranks) ends in (-FLT_MAX, 0x7fffffff) pairs. */
int ling_b200_topk_rows_host(int device, const float* x, int rows, int vocab, int k, float* vals, int* ids);
/* The candidate selector (src/core/kernels.cuh:573-579, src/core/draft_kernels.cu:328-351): scores[e][p][c] = unary[e][c] +
 * sum_r P[pred(e, p)][r] hp[e][r] S[cand[e][c]][r] over r < 256, pred(0, p) the anchor and pred(e, p) = cand[e - 1][p];
 * cand / unary [E][16], scores [E][16][16], the predecessor / successor codebooks P, S [vocab][256] as BF16 bit patterns.
 * With x [E][hidden] and proj_bf16 [256][hidden] given, hp [E][256] = x . proj^T is computed first (and returned in hp:
 * linear_bf16_drafter over selector_projection, speculate.cpp:610); with x NULL, hp is the input. */
int ling_b200_selector_lattice_host(int device, const float* x, const uint16_t* proj_bf16, int hidden, float* hp, const int* cand,
                                    const float* unary, const uint16_t* pred_bf16, const uint16_t* succ_bf16, int vocab, int anchor,
                                    int E, float* scores);
/* Engine::draft_launch from its final norm on (src/core/speculate.cpp:598-617) on a context: x [E][hidden] are the drafted
 * positions' rows after the drafter's final norm; they go through the context's LM head, the top 16 of each row are the
 * candidates (cand, and their logits in unary when asked for), the selector gives scores [E][16][16]: what build_tree takes.
 * The selector's weights (BF16 bit patterns: projection [256][hidden], codebooks [vocab][256]) are uploaded at creation; the
 * handle's device memory belongs to the context and goes with it.  The drafter's transformer body, which produces x, is not
 * part of this library. */
typedef struct ling_b200_draft_head ling_b200_draft_head;
int ling_b200_draft_head_create(ling_b200_ctx* ctx, const uint16_t* selector_projection, const uint16_t* predecessor_codebook,
                                const uint16_t* successor_codebook, ling_b200_draft_head** out);
void ling_b200_draft_head_destroy(ling_b200_draft_head* h);
int ling_b200_draft_head_run(ling_b200_draft_head* h, const float* x, int E, int anchor, int* cand, float* unary, float* scores);

/* ---- the drafter's sparse head (src/core/sparse_head.cu; Engine::draft_launch, src/core/speculate.cpp:598-610) ----
 * Instead of the whole vocabulary a draft step scores the rows its session's mask marks (a fixed list of frequent tokens joined
 * with the ids of the session's prompt and output) and the `dynamic` rows a rank-256 factor of the head rates best for the step's
 * rows: approx[n] = max_m p[m] . us[n], p = x . vt^T (BF16 factors, fp32 sums; ties at the threshold all taken; if fewer
 * unmarked rows than `dynamic` exist none of them is taken, as in the reference's radix walk).  The selected rows' logits are the
 * full head's, bit for bit: they are gathered into a compact matrix that the head GEMM multiplies. */
/* sparse_head_select (kernels.cuh:296-306) over host buffers: masks = n_masks arrays of N bytes; rows [cap] ascending ids,
 * *nrows their count; keys (may be NULL) [N] the ranked 32-bit keys, 0 = marked. */
int ling_b200_sparse_select_host(int device, const float* p, int M, const uint16_t* us_bf16, int N, const uint8_t* masks, int n_masks,
                                 int dynamic, int cap, int* rows, int* nrows, uint32_t* keys);
/* Timing aid: the selection on synthetic factors resident in HBM; ms[0] the scores kernel alone (reads N x 512 bytes), ms[1] the
 * whole selection.  No counterpart in the reference. */
int ling_b200_sparse_select_bench(int device, int N, int M, int dynamic, int cap, int iters, float ms[2]);
/* SparseHeadBufs (kernels.cuh:318-334) on a draft head: us [vocab][256], vt [256][hidden] BF16; every session starts with an empty mask. */
int ling_b200_draft_head_enable_sparse(ling_b200_draft_head* h, const uint16_t* us_bf16, const uint16_t* vt_bf16, int dynamic, int cap);
/* sparse_head_mark (kernels.cuh:310): reset clears the session's mask first. */
int ling_b200_draft_head_mask_reset(ling_b200_draft_head* h, int session, const int* ids, int n);
int ling_b200_draft_head_mask_mark(ling_b200_draft_head* h, int session, const int* ids, int n);
/* draft_head_rows' sparse branch (sparse_head.cu:262-276) followed by the selector, as ling_b200_draft_head_run; *n_selected and
 * selected [cap] (both may be NULL): the rows that were scored. */
int ling_b200_draft_head_run_sparse(ling_b200_draft_head* h, int session, const float* x, int E, int anchor, int* cand, float* unary,
                                    float* scores, int* n_selected, int* selected);

/* Device memory helpers for callers without a CUDA binding (tests): device count, and name of device 0. */
int ling_b200_device_count(void);
/* How a step of `rows` packed rows runs: the capacity class its graph is captured for (the token tile up to 128 rows,
 * multiples of 32 beyond) and the token rows per MMA tile the weight GEMMs use for a class of that many rows (32, 64, 96 or
 * 128: the smallest that holds up to 128 rows; beyond, the one with the least padding).  Results do not depend on either.
 * No counterpart in the reference, whose rows path takes at most 32 rows (kernels.cuh:107). */
int ling_b200_row_class(int rows);
int ling_b200_token_tile(int rows);
int ling_b200_device_name(int device, char* buf, int len);

#ifdef __cplusplus
}
#endif
#endif /* LING_B200_H_ */
