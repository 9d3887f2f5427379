// Host API of the sequence-mixing kernels (see seqmix.cu and seqmix_parallel.cu).  Pointers are device pointers; `bf16` selects the activation type
// (__nv_bfloat16, else float).  Functions returning bool report false for sizes no kernel instance covers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200seq {

struct DeltaArgs {
  const void *q, *k, *v;          // [T, KH, d], [T, KH, d], [T, H, dv] with row strides ldq / ldk / ldv (elements)
  int64_t ldq, ldk, ldv;
  const float* log_decay;         // [T, H, d], or [T, H] with decay_per_head
  int decay_per_head;
  const float* beta;              // [T, H]
  const int *cu, *rows;
  float* state;                   // [rows, H, d, dv]
  float* out;                     // [T, H, dv]
  int H, KH, d, dv;
  int max_len;                    // the longest sequence of the step (0: unknown)
  float unit_eps, q_scale;        // unit_eps < 0: q / k are used as given
};

struct MlstmArgs {
  const void *q, *k, *v;          // [T, H, d], [T, H, d], [T, H, dv]
  int64_t ldq, ldk, ldv;
  const float *log_i, *log_f;     // [T, H]
  const int *cu, *rows;
  float *state, *norm_state, *max_state;
  float* out;
  int H, d, dv;
  int max_len;                    // the longest sequence of the step (0: unknown)
  float q_scale, denom_eps;
};

struct LatentAttnArgs {
  const void* q;                  // [T, H, r]
  const void* cache;              // [slots, r]
  const int *block_table, *tok_req, *tok_len;
  float* out;                     // [T, H, r]
  float* ws;                      // [T, H, n_splits, r + 2] when n_splits > 1
  int H, r, block_size, max_blocks, n_splits;
  int vec_ok;                     // rows of the cache may be copied 16 bytes at a time
  float scale;
};

void add_rms_norm(float* x, const void* delta, const void* w, void* y, int rows, int cols, float eps, float w_off, bool bf16, cudaStream_t s);
// w nullptr: no weight; gate [T, H * dv] with row stride ldg (nullptr: none), through a sigmoid or (silu) a SiLU
void gated_head_rms_norm(const float* o, const void* w, const void* gate, int64_t ldg, void* y, int n_tok, int H, int dv,
                         bool w_per_head, float eps, bool silu, bool bf16, cudaStream_t s);
// residual: the input is added to the (activated) convolution
void causal_conv_silu(const void* x, int64_t ldx, const void* w, const void* bias, const int* cu, const int* rows, const int* tok_seq, void* window,
                      void* y, int n_tok, int R, int C, int taps, int max_len, bool silu, bool residual, bool bf16, cudaStream_t s);
bool delta_rule_scan(const DeltaArgs& p, int R, bool bf16, cudaStream_t s);
bool mlstm_scan(const MlstmArgs& p, int R, bool bf16, cudaStream_t s);
bool latent_attention_paged(const LatentAttnArgs& p, int n_tok, bool bf16, cudaStream_t s);
// key splits per query token for a batch of n_tok tokens whose longest context is max_len
int latent_attention_splits(int H, int r, int n_tok, int max_len);
bool group_limited_router(const float* logits, float* probs, bool* rmap, int n_tok, int E, int topk, int G, int keep, bool renorm,
                          cudaStream_t s);

struct NormRopeArgs {
  const void *q, *k;              // [T, q_ch], [T, k_ch] with row strides ldq / ldk (elements)
  int64_t ldq, ldk;
  const void *wq, *wk;            // norm weights, one per channel of all heads
  const int64_t* positions;       // [T]
  const float* inv_freq;          // [rot / 2]
  void *q_out, *k_out;            // contiguous [T, q_ch], [T, k_ch]
  int q_ch, k_ch, head_dim, rot;
  float eps;
};

struct MixAttnArgs {
  const void* q;                  // [T, H, d], row stride ldq
  int64_t ldq;
  const void *kcache, *vcache;    // [slots, G, d], [slots, G, dv]
  const int *block_table, *tok_req, *tok_len;
  const float* talk;              // [H, H] mixing matrix (nullptr: none)
  const void* gate;               // [T, H * dv] pre-activation of the output gate, row stride ldg (nullptr: none)
  int64_t ldg;
  void* out;                      // [T, H * dv]
  float* ws_stats;                // [T, n_splits, H, 2] when n_splits > 1
  float* ws_acc;                  // [T, n_splits, H * dv] when n_splits > 1
  int H, G, d, dv, block_size, max_blocks, n_splits;
  int query_block;                // hint: new tokens per sequence in this step (>= 4: several queries share a key tile)
  int force_generic;              // 1: the scalar kernel whatever the sizes (for tests)
  int key_tile, head_words, ldk_s;  // filled by the launcher
  float scale;
};

struct GenDeltaArgs {
  const void *r, *k, *v;          // [T, H, d], [T, H, d], [T, H, dv] with row strides
  const void *w_pre, *a_pre;      // [T, H * d] pre-activations of decay and removal rate, row strides ldw / lda
  const void* w_bias;             // [H * d] added to w_pre (nullptr: none)
  int64_t ldr, ldk, ldv, ldw, lda;
  const int *cu, *rows;
  float* state;                   // [rows, H, d, dv]
  float* out;                     // [T, H, dv]
  int H, d, dv;
  int max_len;                    // the longest sequence of the step (0: unknown)
  float decay_scale, unit_eps;
};

struct MinGruArgs {
  const void *z_pre, *u_pre, *g_pre;   // [T, C] with row strides
  int64_t ldz, ldu, ldg;
  const int *cu, *rows;
  float* state;                   // [rows, C]
  void* y;                        // [T, C]
  float* ws;                      // [R, max_runs, C, 2] when max_runs > 1
  int C, max_runs;
};

// x += rms_norm(m) * (w_off + w) + extra, m = a or the mean of the two normed branches; w nullptr: m is added as it is;
// y = the new x, or with next_w its RMS norm times next_w
void norm_add(float* x, const void* a, const void* b, const void* wa, const void* wb, const void* w, void* y, int rows, int cols,
              float eps, float w_off, const void* extra, const void* next_w, bool bf16, cudaStream_t s);
void norm_rope(const NormRopeArgs& p, int n_tok, bool bf16, cudaStream_t s);
int mixed_attention_splits(int n_tok, int max_len);
bool mixed_attention_paged(const MixAttnArgs& p, int n_tok, bool bf16, cudaStream_t s);
bool gen_delta_scan(const GenDeltaArgs& p, int R, bool bf16, cudaStream_t s);
int mingru_runs(int max_len);
void mingru_scan(const MinGruArgs& p, int R, bool bf16, cudaStream_t s);
void clamped_glu(const void* x, int64_t ldx, void* y, int64_t n_tok, int F, float limit, float alpha, float shift, bool bf16,
                 cudaStream_t s);

struct StreamNormArgs {
  float* x;                       // [T, S, W] residual streams, updated in place
  const void *a, *b;              // pending sublayer output(s) [T, W] with row strides lda / ldb (a nullptr: no update)
  int64_t lda, ldb;
  const void* bias_a;             // [W] added to a (nullptr: none)
  const void* ls;                 // [W] layer scale (nullptr: none)
  float scale_a, scale_b;
  const float *mix, *outc;        // [S, S] (from, to) and [S]
  const float* inp;               // [S] read weights of the norm's input (nullptr: no norm, only the update)
  const void *w, *beta;           // norm weight and bias (beta nullptr: none)
  void* h;                        // [T, W] normed output
  int S, W, center;               // center 0: RMS norm
  float eps;
};

struct WindowAttnArgs {
  const void* q;                  // [T, H, d], row stride ldq
  int64_t ldq;
  const void *kcache, *vcache;    // [slots, G, d], [slots, G, dv]
  const int *block_table, *tok_req, *tok_len;
  const float* slopes;            // [H] distance penalty per head (nullptr: none)
  const float* dist_bias;         // [n_bias, H] added to the score by distance, the last row for larger distances (nullptr: none)
  int n_bias;
  const void* gate;               // [T, H] pre-activation of the per-head output gate, row stride ldg (nullptr: none)
  int64_t ldg;
  void* out;                      // [T, H * dv]
  int n_tok, H, G, d, dv, block_size, max_blocks;
  int window;                     // 0: every earlier key is visible
  int sink;                       // 1: one is added to the softmax denominator
  int decode;                     // 1: a decoding batch, one token per sequence
  int n_splits;                   // > 1 (decode only): the visible keys are cut over that many CTAs
  float* ws;                      // [T, H, n_splits, dv + 2] when n_splits > 1
  int QB, HC;                     // filled by the launcher
  float scale, out_scale;
};

struct SelScanArgs {
  const void *x, *z, *B, *Cm;     // [T, C], [T, C] (nullptr: no gate), [T, N], [T, N] with row strides
  int64_t ldx, ldz, ldb, ldc, lddt, ldy;
  const float* dt_pre;            // [T, C] step size before bias and softplus
  const void *dt_bias, *A_log, *D;  // [C] (nullptr: none), [C, N], [C]
  const int *cu, *rows;
  float* state;                   // [rows, C, N]
  void* y;                        // [T, C]
  int C, N;
  float out_scale;
};

bool stream_mix_norm(const StreamNormArgs& p, int n_tok, bool bf16, cudaStream_t s);
void add_sinusoid(float* x, const int64_t* positions, const float* freq, int n_tok, int width, cudaStream_t s);
void head_rms_norm(const void* x, int64_t ldx, const void* w, void* y, int n_tok, int heads, int d, float eps, bool bf16,
                   cudaStream_t s);
bool window_attention_paged(const WindowAttnArgs& p, bool bf16, cudaStream_t s);
// key splits for a batch of n_tok single-token sequences whose longest visible context is max_keys
int window_attention_splits(int H, int G, int n_tok, int max_keys);
bool selective_scan(const SelScanArgs& p, int R, bool bf16, cudaStream_t s);

struct RetentionArgs {
  const void *q, *k, *v;          // [T, H, d], [T, H, d], [T, H, dv] with row strides ldq / ldk / ldv (elements)
  int64_t ldq, ldk, ldv;
  const float* decay;             // [H]
  const int64_t* positions;       // [T] (nullptr with n_rot = 0)
  const float* inv_freq;          // [n_rot]: dimension i of a head turns with dimension i + n_rot
  const int *cu, *rows;
  float* state;                   // [rows, H, d, dv]
  float* out;                     // [T, H, dv]
  int H, d, dv, n_rot;
  int max_len;                    // the longest sequence of the step (0: unknown)
  float k_scale;
};
bool retention_scan(const RetentionArgs& p, int R, bool bf16, cudaStream_t s);
// y = a N(z) + b N(z^2) + c N(z^3) + e per row, N = division by the root mean square; coef = (a, b, c, e) fp32 on the device
bool poly_norm(const void* z, int64_t ldz, const float* coef, void* y, int64_t rows, int cols, float eps, bool bf16, cudaStream_t s);
// log_decay [rows, C] = -exp(A_log[c / (C / H)]) * softplus(a + dt_bias), beta [rows, H] = sigmoid(b); a [rows, C], b [rows, H] with row strides
void decay_gates(const void* a, int64_t lda, const void* b, int64_t ldb, const void* A_log, const void* dt_bias, float* log_decay, float* beta,
                 int64_t rows, int C, int H, bool bf16, cudaStream_t s);
// y = gelu_tanh(g) * e
void gelu_mul(const void* g, int64_t ldg, const void* e, int64_t lde, void* y, int64_t rows, int cols, bool bf16, cudaStream_t s);

}  // namespace b200seq
