// C interface of libherbert_b200: every launcher the library exports (the allocation-free entry
// point has its own header, no_alloc.h).  All pointers are device pointers; `stream` is a
// cudaStream_t.  A launcher returns 0 when it has launched; otherwise hb_last_error() holds the
// reason and nothing was launched.  The Python side (ops/__init__.py) keeps a ctypes signature per
// launcher; a test compares those with the declarations below.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// dtype codes used where one entry point serves both paths
#define HB_F32 0
#define HB_BF16 1

// epilogues of the matrix products
#define HB_EPI_STORE 0      // C (activation dtype) = A W^T
#define HB_EPI_STORE_F32 1  // C (float)            = A W^T
#define HB_EPI_RESIDUAL 2   // C (float)           += A W^T
#define HB_EPI_SWIGLU 3     // C (activation dtype) = silu(gate) * up, W rows in groups of 8 gate, 8 up

// activations of the gated and routed feed-forwards
#define HB_ACT_SILU 0       // z / (1 + exp(-z))
#define HB_ACT_GELU_TANH 1  // 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
#define HB_ACT_GELU 2       // 0.5 z (1 + erf(z / sqrt(2)))
#define HB_ACT_RELU 3       // max(z, 0)
// gated experts only, with a limit L: g' = min(gate, L), u' = clamp(up, -L, L); g' sigmoid(1.702 g') (u' + 1)
#define HB_ACT_SWISH_CLAMP 4
#define HB_SWISH_CLAMP_SLOPE 1.702f


// attention_decode.cu: decode attention over the paged cache (one query per sequence, keys cut into splits)
long long hb_attention_decode_scratch_floats(int n_seqs, int nh, int hd, int nsplit);
int hb_attention_decode_bf16(const void* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
    const int* seq_len, const int* seq_pages, int pages_stride, float* scratch, int n_seqs, int nh, int nkv, int hd,
    int page_size, int nsplit, float scale, int window, float softcap, const float* sink, const float* gate_bias, const float* out_gate, int ldg, void* stream);
int hb_attention_decode_fused_bf16(const void* qkv, int ld, void* out, int ldo, void* kcache, void* vcache,
    const float* qw, const float* kw, float eps, const float* cos_tab, const float* sin_tab, int table_rows,
    int write_cache, const int* seq_len, const int* seq_pages, int pages_stride, float* scratch, int*
    counters, int n_seqs, int nh, int nkv, int page_size, int nsplit, float scale, int window, void* stream);

// attention_prefill.cu: prefill attention, mma.sync flash form, head sizes in steps of 16 up to 256
int hb_attention_prefill_bf16(const void* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
    const int* seq_start, const int* seq_pos0, const int* seq_pages, int pages_stride, int n_seqs, int max_q_len, int
    nh, int nkv, int hd, int page_size, float scale, int window, float softcap, const float* sink, const float* gate_bias, const float* out_gate, int ldg, void* stream);

// attention_prefill_tc.cu: prefill attention on tcgen05 tensor cores, head sizes 64 and 128
int hb_attention_prefill_tc_bf16(const void* q, int ldq, int n_tokens, void* out, int ldo, const void* kcache,
    const void* vcache, int n_pages, const int* seq_start, const int* seq_pos0, const int* seq_pages, int
    pages_stride, int n_seqs, int max_q_len, int nh, int nkv, int hd, int page_size, float scale, int window, float
    softcap, const float* sink, const float* gate_bias, const float* out_gate, int ldg, int* error_flag, int* work_counter, void* stream);

// attention_simt.cu: attention of any shape on the CUDA cores (the 32-bit path)
int hb_attention_simt(int dtype, const void* q, int ldq, void* out, int ldo, const void* kcache, const void*
    vcache, const int* tok_seq, const int* tok_pos, const int* seq_pages, int pages_stride, int n_tokens, int nh, int
    nkv, int hd, int page_size, float scale, int window, float softcap, const float* sink, const float* gate_bias, const float* out_gate, int ldg, void* stream);

// elementwise.cu: embedding, RMSNorm, SwiGLU, head norm + rotation + cache write, residual sum, shared-norm finish
int hb_embed(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden, int vocab, float
    scale, const void* pos_table, const int* positions, int n_positions, void* stream);
int hb_rmsnorm(int dtype, const float* x, const float* w, void* out, const int* rows, int n_rows, int dim,
    float eps, void* stream);
int hb_swiglu(int dtype, const void* gu, int ld, void* out, int ldo, int n_tokens, int inter, int interleave,
    int act, void* stream);
int hb_qk_norm_rope_cache(int dtype, void* qkv, int ld, const float* qw, const float* kw, float eps, const
    float* cos_tab, const float* sin_tab, int rot, int table_rows, const int* tok_seq, const int* tok_pos,
    const int* seq_pages, int pages_stride, void* kcache, void* vcache, int n_tokens, int nh, int nkv, int hd,
    int page_size, int write_cache, void* stream);
int hb_add_residual(int dtype, float* res, const void* y, int ld, int n_tokens, int dim, void* stream);
int hb_finish_norm(const void* xw, int ld, const float* sumsq, int parts, int stride, float eps, void* out,
    int ldo, int n_rows, int dim, void* stream);

// errors.cu: error text, ABI version, programmatic dependent launch mode
const char* hb_last_error(void);
int hb_abi_version(void);
void hb_set_pdl(int mode);
int hb_get_pdl(void);

// fill.cu: load-time kernels: counter-based normal fill, constant fill, dtype casts
int hb_rng_normal(int dtype, void* out, long long n, unsigned long long key, float mean, float stdev, void*
    stream);
int hb_fill(int dtype, void* out, long long n, float value, void* stream);
int hb_cast(int src, const void* in, int dst, void* out, long long n, int round_bf16, void* stream);

// gemm_simt.cu: matrix product of any shape on the CUDA cores (the 32-bit path)
int hb_gemm_simt(int dtype, const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, int epi, void* stream);

// gemm_skinny.cu: decode product (at most 64 activation rows), mma.sync, optional shared norm
int hb_gemm_skinny_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
    int epi, void* stream);
int hb_gemm_skinny_norm_parts(int M, int N);
int hb_gemm_skinny_norm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, int epi, const float* in_sumsq, int in_parts, float in_eps, const float* out_w, void* out_xw, int
    out_ld, float* out_sumsq, void* stream);

// gemm_stream.cu: decode product, TMA + tcgen05, K slices (the output head)
long long hb_gemm_stream_scratch_floats(int M, int N, int K);
int hb_gemm_stream_counters(int N);
int hb_gemm_stream_bf16(const void* X, int ldx, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
    int epi, float* scratch, long long scratch_floats, int* counters, int n_counters, int* error_flag, void*
    stream);

// gemm_tcgen05.cu: prefill product, TMA + tcgen05, persistent; optional shared norm
int hb_gemm_tcgen05_set_pairs(int on);
int hb_gemm_tcgen05_set_ksplit(int on);
long long hb_gemm_tcgen05_workspace_floats(int ctas);
int hb_gemm_tcgen05_set_workspace(float* floats, int* counters, int ctas);
int hb_gemm_tcgen05_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int
    K, int epi, int* error_flag, void* stream);
int hb_gemm_tcgen05_grouped_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M_max, int
    N, int K, int E, int epi, float glu_limit, const int* rows_used, const int* tile_expert, int* error_flag, void*
    stream);
int hb_gemm_tcgen05_qkv_ok(int M, int N);
int hb_gemm_tcgen05_qkv_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, const float* in_sumsq, int in_parts, int in_stride, float in_eps, const float* qw, const float* kw,
    float eps, const float* cos_tab, const float* sin_tab, int table_rows, const int* tok_seq, const int*
    tok_pos, const int* seq_pages, int pages_stride, void* kcache, void* vcache, int nh, int nkv, int
    page_size, int write_cache, int* error_flag, void* stream);
int hb_gemm_tcgen05_norm_parts(int M, int N);
int hb_gemm_tcgen05_norm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, int epi, const float* in_sumsq, int in_parts, int in_stride, float in_eps, const float* out_w,
    void* out_xw, int out_ld, float* out_sumsq, int out_stride, int* error_flag, void* stream);

// gla.cu: gated linear attention: decays, the recurrence over a step's tokens, output norm and gate
int hb_gla_decay(int dtype, const float* low, int ld, const void* w2, const float* bias, float inv_tau, float* a,
    int n_tokens, int channels, int low_rank, void* stream);
int hb_gla_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
    const int* seq_slot, const int* seq_start, float* out, int ldo, int n_seqs, int heads, int dk, int dv, float
    qscale, void* stream);
int hb_gla_output(int dtype, const float* o, int ldo, const float* w, float eps, const float* gate, int ldg,
    void* y, int ldy, int n_tokens, int heads, int dv, void* stream);

// latent_attention.cu: attention over a cached latent (one shared key/value vector per token), with a sink
int hb_latent_kv_store(int dtype, const float* kv, int ld, const float* norm_w, float eps, const float* freq,
    float mscale, int rank, int rot, const int* tok_seq, const int* tok_pos, const int* seq_pages, int
    pages_stride, void* cache, int n_tokens, int page_size, void* stream);
int hb_rotate_heads(const float* in, int ld_in, int in_head_stride, int in_offset, float* out, int ld_out, int
    out_head_stride, int out_offset, const float* freq, float mscale, const int* tok_pos, int n_tokens, int
    heads, int rot, float scale, void* stream);
int hb_headwise_gemm(int dtype, int out_dtype, const float* in, int ld_in, int in_head_stride, const void* w,
    void* out, int ld_out, int out_head_stride, const float* gate, int ld_gate, int n_tokens, int heads, int K,
    int N, float scale, void* stream);
int hb_latent_attention(int dtype, const float* q, int ldq, float* out, int ldo, const void* cache, const float*
    sink, const int* tok_seq, const int* tok_pos, const int* seq_pages, int pages_stride, int n_tokens, int
    heads, int rank, int rot, int page_size, int window, void* stream);
int hb_latent_attention_mma_ok(int rank, int rot);
int hb_latent_attention_mma_bf16(const float* q, int ldq, float* out, int ldo, const void* cache, const float*
    sink, const int* seq_start, const int* seq_pos0, const int* seq_pages, int pages_stride, int n_seqs, int
    max_q_len, int heads, int rank, int rot, int page_size, int window, int nsplit, float* scratch, void*
    stream);
long long hb_latent_attention_mma_scratch_floats(int n_seqs, int max_q_len, int heads, int rank, int nsplit);

// layernorm.cu: layer normalisation (weight, no bias), alone and with the scaled residual sum after it
int hb_layernorm(int dtype, const float* x, const float* w, void* out, const int* rows, int n_rows, int dim,
    float eps, void* stream);
int hb_layernorm_residual(int dtype, const float* y, int ldy, const float* w, const float* scale, float* x, void*
    h, int n_rows, int dim, float eps, void* stream);

// moe.cu: routed feed-forward: router (softmax or sigmoid scores, groups of experts) and choice, the chosen experts' products (plain or gated)
int hb_moe_route(int dtype, const void* h, int ld, const void* w_router, int* ids, float* weights, int n_tokens,
    int D, int E, int top, int renorm, int sigmoid, int groups, int keep, int group_top, float wscale, void* stream);
int hb_moe_experts(int dtype, const void* h, int ld, const void* up, const void* down, const int* ids, const
    float* weights, void* mid, float* y, int ldy, int n_tokens, int D, int F, int top, int act, int gated, float
    act_limit, int accumulate, void* stream);
long long hb_moe_grouped_scratch_ints(int n_tokens, int E, int top);
int hb_moe_experts_tc_rows(int n_tokens, int E, int top);
int hb_moe_experts_tc_bf16(const void* h, int ld, const void* up, const void* down, const int* ids, const float*
    weights, int* ints, void* sorted, void* mid, float* part, float* y, int ldy, int n_tokens, int D, int E, int F,
    int top, float act_limit, int accumulate, int* error_flag, void* stream);
int hb_moe_experts_grouped_bf16(const void* h, int ld, const void* up, const void* down, const int* ids, const
    float* weights, int* scratch, void* mid, float* part, float* y, int ldy, int n_tokens, int D, int E, int F, int
    top, int act, int gated, float act_limit, int accumulate, void* stream);

// qk_prepare.cu: biases, query temperature and cache write for a mixer that neither norms nor rotates its heads
int hb_qk_prepare_cache(int dtype, const float* qkv, int ld, const float* bias, void* q_out, int ldq, float
    temp_coef, int temp_every, const int* tok_seq, const int* tok_pos, const int* seq_pages, int pages_stride,
    void* kcache, void* vcache, int n_tokens, int nh, int nkv, int hd, int page_size, int write_cache,
    void* stream);

// residual_norm.cu: x += mult * y, and the next block's RMS norm of the updated row
int hb_scaled_residual_norm(int dtype, const float* y, int ldy, float mult, float* x, const float* w, void* h,
    int n_rows, int dim, float eps, void* stream);

// sampling.cu: argmax and temperature / top-k / top-p sampling
int hb_argmax(const float* logits, int ld, int n_rows, int vocab, int* out, void* scratch, long long
    scratch_words, void* stream);
int hb_sample(const float* logits, int ld, int n_rows, int vocab, float temperature, int top_k, float top_p,
    const float* uniforms, int* out, int* overflow, void* stream);

// group_norm.cu: RMS norm in groups (alone, or of a sublayer's result on its way into the stream), a gated activation with biases, a weighted sum of two arrays, a tanh cap
int hb_group_rmsnorm(int dtype, const float* x, const float* w, void* out, const int* rows, int n_rows, int dim,
    int groups, float eps, void* stream);
int hb_group_rmsnorm_residual(int dtype, const float* y, int ldy, const float* z, int ldz, float a, float b,
    const float* bias, const float* w, float* x, void* h, int n_rows, int dim, int groups, float eps, void* stream);
int hb_axpby(float* y, int ldy, float a, const float* z, int ldz, float b, int rows, int cols, void* stream);
int hb_bias_glu(int dtype, const float* gu, int ld, const float* bias, void* out, int ldo, int n_tokens, int
    inter, int interleave, int act, void* stream);
int hb_tanh_cap(float* x, int ld, float cap, int rows, int cols, void* stream);

// short_conv.cu: a short causal convolution over time whose last inputs are state; an embedding plus a row chosen by (previous token, token)
int hb_short_conv(int out_dtype, const float* in, int ld_in, const float* w, float* state, const int* seq_slot,
    const int* seq_start, const int* seq_pos0, void* out, int ldo, int n_seqs, int max_q_len, int channels, int
    taps, int add_input, int act_silu, void* stream);
int hb_pair_embed(int dtype, const void* table, const void* pair_table, const int* ids, const int* tok_seq,
    const int* tok_pos, const int* seq_slot, const int* seq_start, int* last_id, float* out, int n_tokens, int
    hidden, int vocab, int buckets, long long mul_prev, long long mul_cur, float scale, void* stream);

// linear_scan.cu: recurrent mixers with a matrix of state per head: the decaying form and the gated delta rule
int hb_silu_columns(float* x, int ld, int col0, int cols, int rows, void* stream);
int hb_delta_prepare(float* qk, int ld, int q_off, int k_off, int qk_heads, int dk, float qscale, const float*
    ab, int ldab, int b_off, int a_off, const float* a_log, const float* dt_bias, float* gates, int heads, int
    n_tokens, void* stream);
int hb_linear_scan(int delta, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const
    float* gates, const float* decay, float* state, const int* seq_slot, const int* seq_start, float* out, int ldo,
    int n_seqs, int max_q_len, int heads, int qk_heads, int dk, int dv, void* stream);
int hb_gated_rmsnorm(int dtype, const float* o, int ldo, const float* w, float eps, const float* gate, int ldg,
    void* y, int ldy, int n_tokens, int units, int n, int act, int w_stride, void* stream);

// rotary_pairs.cu: whole-projection q/k norm, rotation of pairs by position (q, k and v), cache write; the turn back of the results
int hb_qkv_rotary_cache(int dtype, const float* rows, int ld, const float* wq, const float* wk, float eps, int
    whole_norm, const float* fqk, int rot, int halves, const float* fv, const int* tok_seq, const int* tok_pos,
    const int* seq_pages, int pages_stride, void* q_out, int ldq, void* kcache, void* vcache, int n_tokens, int nh,
    int nkv, int dk, int dv, int hd, int page_size, int write_cache, void* stream);
int hb_rotate_heads_back(int dtype, const void* att, int ld, int hd, const float* fv, int halves, const int*
    tok_pos, void* y, int ldy, int n_tokens, int nh, int dv, void* stream);
int hb_head_gate(int dtype, const void* att, int ld, int hd, const float* gate, int ldg, void* y, int ldy, int
    n_tokens, int nh, int dv, void* stream);

// general_delta.cu: the generalised delta rule (decay per key channel, removal along the unit key): its vectors, its recurrence
int hb_general_delta_prepare(int dtype, const float* rows, int ld, int r_off, int k_off, int a_off, int low_off,
    const void* w2, const float* w0, const float* a0, float decay_c, float unit_eps, float* prep, int n_tokens, int
    heads, int dk, int rank, void* stream);
int hb_general_delta_scan(const float* prep, const float* v, int ldv, float* state, const int* seq_slot, const int*
    seq_start, float* out, int ldo, int n_seqs, int heads, int dk, int dv, void* stream);

// gated_residual.cu: a sublayer's result through a sigmoid gate and an RMS norm into the stream (+ the next norm); a gate chosen by the token's id
int hb_gated_norm_residual(int dtype, const float* y, int ldy, const float* z, int ldz, const float* zb, const float*
    w, float eps, float* x, const float* w2, float eps2, void* h, int n_rows, int D, void* stream);
int hb_token_gate(int dtype, const float* s, int lds, const void* table, int ldt, int col0, const int* ids, void*
    out, int ldo, int n_tokens, int m, int vocab, void* stream);

#ifdef __cplusplus
}
#endif
