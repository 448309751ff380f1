/* ling_oracle.h -- CPU oracle of the ragged speculative verify step.  TEST INFRASTRUCTURE ONLY.
 *
 * A scalar C++ restatement of the reference engine's verify step (dreamference/ling-engine), written from the
 * reference's documented arithmetic; each function in ling_oracle.cpp cites the reference file:line it follows.
 * Nothing in the product links or calls this library: only the tests, the smoke check and the benchmark's
 * CPU-baseline leg do, and only as the checker.
 *
 * Pinning: the integer/host parts (tree description, greedy acceptance, context lookup) are checked against the
 * reference's own sources compiled here (oracle/_ref, see oracle/Makefile) and against the golden vectors under
 * tests/golden.  The floating-point forward pass has no stored golden outputs in the reference (its whole-step
 * checks compare two execution modes on private checkpoints), and the reference has no FP8-KV / 1x128
 * block-scaled path at all; for those numerics this oracle defines the answer: "parity unpinned" for logits and
 * hidden states, pinned for every integer result.
 *
 * The POD structs are layout-compatible with include/ling_b200.h on purpose (the tests pass one ctypes
 * structure to both libraries); the code shares nothing with the product.
 */
#ifndef LING_ORACLE_H_
#define LING_ORACLE_H_
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define LO_MAX_LAYERS 128
#define LO_MAX_TREE_ROWS 32
#define LO_MAX_TREE_VARIANTS 32

typedef struct lo_model_config {
  int hidden, intermediate, layers, vocab;
  int heads, kv_heads, head_dim, rotary_dim;
  float rope_theta, eps;
  int lin_k_heads, lin_v_heads, lin_k_dim, lin_v_dim, conv_kernel;
  unsigned char full_attention[LO_MAX_LAYERS];
} lo_model_config;

typedef struct lo_options {
  int sessions, max_context, page_tokens, pool_pages, max_seqs, max_rows, gemm_impl, use_graph, device;
  int debug_rows, pdl;
  int reserved[5];
} lo_options;

typedef struct lo_seq_step {
  int slot, pos, rope_delta, n_rows, chain;
  const int* tokens;
  const int* parent;
  const int* force_argmax;
} lo_seq_step;

typedef struct lo_seq_result {
  int status, n_path;
  int path[LO_MAX_TREE_ROWS];
  int next_token, n_out;
  int out[LO_MAX_TREE_ROWS + 1];
} lo_seq_result;

typedef struct lo_tree_desc {
  int n;
  int depth[LO_MAX_TREE_ROWS];
  int var[LO_MAX_TREE_ROWS];
  int nvar;
  int path[LO_MAX_TREE_VARIANTS][LO_MAX_TREE_ROWS];
  int ngdn;
  int gdn_len[LO_MAX_TREE_VARIANTS];
  int gdn_step[LO_MAX_TREE_VARIANTS][2 * LO_MAX_TREE_ROWS];
} lo_tree_desc;

typedef struct lo_model lo_model;

void lo_set_threads(int n);
int lo_threads(void);

/* number formats */
uint8_t lo_e4m3_encode(float x);
float lo_e4m3_decode(uint8_t c);
float lo_bf16_round(float x);
void lo_quant_rows(const float* x, int rows, int cols, int bf16_first, uint8_t* codes, float* scales);
/* the generator: n elements of stream (seed, stream) from element `offset`; value = z * std (+ bias), bf16-rounded when asked */
void lo_synth(uint64_t seed, uint64_t stream, size_t offset, size_t n, float std, float bias, int bf16, float* out);
uint64_t lo_weight_stream(int layer, int tensor);

/* host logic */
int lo_describe_tree(const int* parent, int n_rows, int chain, lo_tree_desc* out);
int lo_accept_tree_greedy(const int* parent, const int* token, int n_rows, const int* argmax, int* path, int* next);
int lo_lookup_propose(const int* seq, int len, int max, int ngram, int* out, int* match);

/* kernels */
void lo_gemm_fp8(const float* x, const float* w, float* y, int M, int N, int K);
void lo_gdn_tree(int Hk, int HV, int Dk, int Dv, const lo_tree_desc* td, const float* pre, const float* convw,
                 const float* g, const float* beta, const float* state, const float* conv, float* post, float* core);
void lo_gdn_prefill(int Hk, int HV, int Dk, int Dv, int M, const float* pre, const float* convw, const float* g, const float* beta,
                    float* state, float* conv, float* post, float* core);
void lo_gdn_commit(int Hk, int HV, int Dk, int Dv, const int* path, int n, int rows, const float* pre,
                   const float* post, const float* g, const float* beta, float* state, float* conv);
void lo_argmax(const float* logits, int rows, int vocab, int* ids, float* vals);
void lo_topk_rows(const float* x, int rows, int vocab, int k, float* vals, int* ids);
void lo_selector_lattice(const float* hp, const int* cand, const float* unary, const float* P, const float* S, int anchor, int E,
                         float* scores);
void lo_selector_project(const float* x, const float* W, int E, int H, float* hp);

/* model + sessions */
lo_model* lo_create(const lo_model_config* cfg, const lo_options* opt);
void lo_destroy(lo_model* m);
int lo_set_tensor(lo_model* m, int layer, int tensor, const float* host, int rows, int cols);
int lo_synth_weights(lo_model* m, uint64_t seed);
/* only these layers (and the globals) are materialized by lo_synth_weights; -1 entries ignored. Used by the CPU-baseline sample. */
int lo_synth_weights_layers(lo_model* m, uint64_t seed, const int* layers, int n_layers, int head_rows);
int lo_get_matrix(lo_model* m, int layer, int tensor, uint8_t* codes, float* scales, int rows, int cols);
int lo_kv_table_set(lo_model* m, int slot, const int* idx, const int* page, int n);
int lo_kv_write(lo_model* m, int slot, int attn_layer, int from, int n, const float* k, const float* v);
int lo_kv_read(lo_model* m, int slot, int attn_layer, int from, int n, float* k, float* v, uint8_t* kcodes,
               float* kscales, uint8_t* vcodes, float* vscales);
int lo_synth_kv(lo_model* m, int slot, int n, uint64_t seed);
int lo_state_write(lo_model* m, int slot, int gdn_layer, const float* state, const float* conv);
int lo_state_read(lo_model* m, int slot, int gdn_layer, float* state, float* conv);
int lo_synth_state(lo_model* m, int slot, uint64_t seed);
int lo_state_hash(lo_model* m, int slot, uint64_t* hash);

/* the step (flags as in the product header: 1 commit, 2 keep logits, 4 keep taps) */
int lo_verify_step(lo_model* m, const lo_seq_step* seqs, int n_seqs, int flags, lo_seq_result* results);
/* the same step restricted to a sample: only the listed layers run and only head_rows vocabulary rows are scored */
int lo_verify_step_sample(lo_model* m, const lo_seq_step* seqs, int n_seqs, const int* layers, int n_layers,
                          int head_rows);
int lo_attention(lo_model* m, const lo_seq_step* seqs, int n_seqs, int attn_layer, const float* q, float* out);
/* one layer alone on a given residual stream (teacher forcing); layer == cfg.layers: the final norm and the head */
int lo_layer_forward(lo_model* m, const lo_seq_step* seqs, int n_seqs, int layer, const float* h_in, float* h_out,
                     int head_rows);
/* the layer's mixer alone: h_out = h_in + mixer(norm(h_in)), no feed-forward block */
int lo_mixer_forward(lo_model* m, const lo_seq_step* seqs, int n_seqs, int layer, const float* h_in, float* h_out);
/* attn_prepare alone: q|k|v projection rows in, normed + rotated q (and k before the cache rounding) out, K/V stored */
int lo_attn_prepare(lo_model* m, const lo_seq_step* seqs, int n_seqs, int attn_layer, const float* qkv, float* q_out,
                    float* k_out);
int lo_read_tree_desc(lo_model* m, int seq, lo_tree_desc* out);
int lo_read_packing(lo_model* m, int* row0, int* token, int* seq_of, int* depth, int* rope_pos, int* cache_slot,
                    uint32_t* anc_mask);
int lo_read_argmax(lo_model* m, int* ids, float* vals);
int lo_read_logits(lo_model* m, float* out);
int lo_read_tap(lo_model* m, int layer, float* out);

/* NVFP4 operands of the prefill chunk (E2M1 values two a byte, low nibble first; E4M3 scale per 16; fp32 tensor scale). */
int lo_nvfp4_quantize_weight(const uint16_t* w_bf16, int N, int K, uint8_t* q, uint8_t* sf, float* scale2);
int lo_nvfp4_quant_act(const float* x, const float* up, int M, int K, float input_scale, uint8_t* q, uint8_t* sf);
int lo_nvfp4_dequant(const uint8_t* q, const uint8_t* sf, int rows, int K, float* out);
int lo_nvfp4_gemm(const uint8_t* xq, const uint8_t* xs, int M, const uint8_t* wq, const uint8_t* ws, int N, int K, float alpha,
                  float* y, int ldy, int accumulate);
int lo_rmsnorm_rows(const float* x, const uint16_t* w_bf16, int M, int H, float eps, float* out);

#ifdef __cplusplus
}
#endif
#endif
