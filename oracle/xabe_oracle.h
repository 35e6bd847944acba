/*
 * CPU oracle for the per-layer MoE FFN path of nixabe/llmxabe.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, operand for operand, the
 * scalar fp32 references of the reference project's `xabe-kernels` crate (and
 * the summation orders its device kernels pin for the quantities that select
 * experts).  It is the checker for the CUDA path and the timed CPU baseline.
 * Nothing in the product package may call it; the product has no CPU path.
 *
 * Parity is PINNED: every function below is checked against the reference's
 * own known-answer tests (transcribed into tests/golden/reference_kats.json
 * with the reference file:line of each) by tests/test_oracle_kats.py.
 *
 * The reference is Rust and cannot be compiled in this environment (no
 * rustc/cargo), so there is no oracle/_ref build.
 *
 * Build: see oracle/Makefile (-O2 -ffp-contract=off -fno-fast-math so that a
 * multiply and the add that follows round separately, as the Rust does).
 */
#ifndef XABE_ORACLE_H
#define XABE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XO_QK_K 256
#define XO_QK8_0 32
#define XO_Q6K_BYTES 210
#define XO_Q8_0_BYTES 34
#define XO_QUANT_Q6K 0
#define XO_QUANT_Q8_0 1
#define XO_INACTIVE_EXPERT (-1)

/* ---- rng.rs ---------------------------------------------------------- */
typedef struct { uint64_t state; } xo_rng;
void xo_rng_seed(xo_rng* r, uint64_t seed);
uint64_t xo_rng_next_u64(xo_rng* r);
float xo_rng_next_f32(xo_rng* r);
float xo_rng_next_f32_range(xo_rng* r, float lo, float hi);
uint32_t xo_rng_next_u32_below(xo_rng* r, uint32_t bound);
void xo_rng_vec_f32(xo_rng* r, float* out, size_t n, float lo, float hi);

/* ---- f16.rs ---------------------------------------------------------- */
uint16_t xo_f32_to_f16_bits(float x);
float xo_f16_bits_to_f32(uint16_t h);

/* ---- quant.rs -------------------------------------------------------- */
void xo_dequantize_q6_k_block(const uint8_t* block210, float* y256);
void xo_dequantize_q8_0_block(const uint8_t* block34, float* y32);
void xo_quantize_q6_k_block(const float* x256, uint8_t* block210);
void xo_quantize_q8_0_block(const float* x32, uint8_t* block34);
/* whole rows; return 0, or -1 when n_bytes is not a whole number of blocks */
int xo_dequantize_row(int quant, const uint8_t* bytes, size_t n_bytes, float* out);
int xo_quantize_row(int quant, const float* x, size_t n, uint8_t* bytes);
size_t xo_block_bytes(int quant);
size_t xo_block_elements(int quant);

/* ---- norm.rs / gemv.rs ----------------------------------------------- */
void xo_rms_norm(const float* x, const float* w, float eps, size_t n, float* out);
float xo_silu(float x);
float xo_sigmoid(float x);
void xo_swiglu(const float* gate, const float* up, size_t n, float* out);
void xo_gemv(const float* w, size_t out_dim, size_t in_dim, const float* x, float* out);
size_t xo_argmax(const float* v, size_t n);
int xo_lm_head(int quant, const uint8_t* bytes, size_t vocab, size_t hidden, const float* x, size_t tokens,
               float* logits, int threads);

/* ---- summation orders pinned by the reference's DEVICE kernels -------- */
void xo_rms_norm_dev(const float* x, const float* w, float eps, size_t n, float* out);
void xo_router_logits_dev(const float* w, const float* x, size_t num_experts,
                          size_t hidden, float* logits);
float xo_shared_gate_dot_dev(const float* w, const float* x, size_t hidden);
float xo_softmax_denominator_dev(const float* exps, size_t n);

/* ---- moe/router.rs --------------------------------------------------- */
void xo_route_token(const float* logits, size_t num_experts, size_t k,
                    int32_t* ids, float* weights);
void xo_route_batch(const float* logits, size_t tokens, size_t num_experts,
                    size_t k, int32_t* ids, float* weights);

/* ---- moe/dispatch.rs ------------------------------------------------- */
/* sorted capacity in: size of sorted_token_ids / expert_ids arrays provided.
 * Returns num_tokens_post_pad, or -1 for a bad argument. Only the first
 * num_tokens_post_pad (resp. /block_size) entries are written. */
long xo_moe_align_block_size(const int32_t* topk_ids, size_t tokens, size_t top_k,
                             size_t block_size, size_t num_experts,
                             int32_t* sorted_token_ids, int32_t* expert_ids);
size_t xo_sorted_capacity(size_t num_experts, size_t top_k, size_t block_size,
                          size_t max_tokens);

/* ---- moe/gemm.rs (dense fp32 expert weights) ------------------------- */
void xo_expert_mlp(const float* gate, const float* up, const float* down,
                   const float* x, size_t hidden, size_t inter, float* out);
void xo_naive_forward(const float* hidden_states, size_t tokens,
                      const int32_t* ids, const float* weights, size_t top_k,
                      const float* gate, const float* up, const float* down,
                      size_t hidden, size_t inter, float* out);
void xo_grouped_forward(const float* hidden_states, size_t tokens,
                        const int32_t* sorted_token_ids, const int32_t* expert_ids,
                        size_t num_blocks, size_t block_size,
                        const float* flat_weights, size_t top_k,
                        const float* gate, const float* up, const float* down,
                        size_t hidden, size_t inter, float* out);

/* ---- compare.rs ------------------------------------------------------ */
typedef struct {
    float max_abs_error; uint64_t max_abs_error_index;
    float max_rel_error; uint64_t max_rel_error_index;
    float cosine_similarity; uint64_t non_finite_count; uint64_t len;
    double rel_l2; /* ||c-r||2 / ||r||2, an addition used by the layer-output gate */
} xo_comparison;
void xo_compare(const float* candidate, const float* reference, size_t n, xo_comparison* out);

/* ---- whole block over quantized weights ------------------------------ */
typedef struct {
    uint32_t num_experts, top_k, hidden, inter;
    const float* post_norm;      /* [hidden] */
    const float* router;         /* [num_experts][hidden] */
    const float* router_bias;    /* [num_experts] added to the logits, or NULL (benchmark Zipf skew) */
    const uint8_t* gate_exps; int gate_quant;   /* [E][inter][hidden] file layout */
    const uint8_t* up_exps;   int up_quant;
    const uint8_t* down_exps; int down_quant;   /* [E][hidden][inter] */
    const float* shared_gate_inp; /* [hidden] */
    const uint8_t* shared_gate; int shared_gate_quant;
    const uint8_t* shared_up;   int shared_up_quant;
    const uint8_t* shared_down; int shared_down_quant;
    float eps;
} xo_moe_layer;

typedef struct {
    float* normed;       /* [T][hidden] */
    float* logits;       /* [T][E] */
    int32_t* topk_ids;   /* [T][K] */
    float* topk_weights; /* [T][K] */
    float* routed;       /* [T][hidden] */
    float* shexp;        /* [T][hidden] ungated */
    float* gate;         /* [T] */
    float* ffn_out;      /* [T][hidden] */
    float* l_out;        /* [T][hidden] */
} xo_moe_outputs;

/* order: 0 = every reduction in the CPU reference's sequential order;
 *        1 = RMSNorm, router logits and shared-gate dot in the order the
 *            reference's device kernels pin (what the CUDA path reproduces
 *            bit for bit, so that the expert selection is identical).
 * threads: OpenMP threads (0 = all). Any pointer of `out` may be NULL. */
int xo_moe_block_forward(const xo_moe_layer* layer, const float* residual,
                         size_t tokens, int order, int threads, xo_moe_outputs* out);

/* Routed experts only, from given routing (the reference's `naive_forward`
 * over dequantized weights, tests/moe_differential.rs:716-782). */
int xo_routed_forward_q(const xo_moe_layer* layer, const float* hidden_states,
                        size_t tokens, const int32_t* ids, const float* weights,
                        int threads, float* out);
/* expert_mlp over quantized matrices for every token (shared expert / dense FFN). */
int xo_mlp_forward_q(const uint8_t* gate, int gate_quant, const uint8_t* up, int up_quant,
                     const uint8_t* down, int down_quant, size_t hidden, size_t inter,
                     const float* x, size_t tokens, int threads, float* out);
/* dense block: l_out = mlp(rms_norm(x)) + x  (block/dense_ffn.rs:9-16) */
int xo_dense_block_forward(const float* post_norm, float eps,
                           const uint8_t* gate, int gate_quant, const uint8_t* up, int up_quant,
                           const uint8_t* down, int down_quant, size_t hidden, size_t inter,
                           const float* residual, size_t tokens, int order, int threads,
                           float* ffn_out, float* l_out);
int xo_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
