/*
 * CPU oracle for the per-layer MoE FFN path of nixabe/llmxabe.
 * TEST INFRASTRUCTURE ONLY -- see xabe_oracle.h.  Parity is pinned by the
 * reference's known-answer tests (tests/test_oracle_kats.py).
 *
 * Every function cites the reference file:line it restates (paths relative to
 * the reference project root).  Sums are sequential left folds in fp32 with
 * the multiply and the add rounded separately (compile with
 * -ffp-contract=off); Rust's `Iterator::sum::<f32>()` starts from -0.0.
 */
#include "xabe_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ===================================================================== */
/* crates/xabe-kernels/src/rng.rs:16-55  (xorshift64*)                   */
/* ===================================================================== */
void xo_rng_seed(xo_rng* r, uint64_t seed) {
    r->state = seed ? seed : 0x9E3779B97F4A7C15ull; /* rng.rs:20-23 */
}
uint64_t xo_rng_next_u64(xo_rng* r) { /* rng.rs:26-33 */
    uint64_t x = r->state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    r->state = x;
    return x * 0x2545F4914F6CDD1Dull;
}
float xo_rng_next_f32(xo_rng* r) { /* rng.rs:36-39 */
    return (float)(xo_rng_next_u64(r) >> 40) / (float)(1ull << 24);
}
float xo_rng_next_f32_range(xo_rng* r, float lo, float hi) { /* rng.rs:42-44 */
    return lo + xo_rng_next_f32(r) * (hi - lo);
}
uint32_t xo_rng_next_u32_below(xo_rng* r, uint32_t bound) { /* rng.rs:47-50 */
    return (uint32_t)(xo_rng_next_u64(r) % (uint64_t)bound);
}
void xo_rng_vec_f32(xo_rng* r, float* out, size_t n, float lo, float hi) { /* rng.rs:53-55 */
    for (size_t i = 0; i < n; ++i) out[i] = xo_rng_next_f32_range(r, lo, hi);
}

/* ===================================================================== */
/* crates/xabe-kernels/src/f16.rs:17-94 -- IEEE binary16 <-> binary32,    */
/* round to nearest even (also what `half` 2.7.1's f16::from_f32/to_f32   */
/* compute, quant.rs:41,63,85,172,565).                                   */
/* ===================================================================== */
static uint32_t f32_bits(float x) { uint32_t b; memcpy(&b, &x, 4); return b; }
static float bits_f32(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }

uint16_t xo_f32_to_f16_bits(float x) {
    uint32_t b = f32_bits(x);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int e = (int)((b >> 23) & 0xffu);
    uint32_t m = b & 0x7fffffu;
    if (e == 0xff) return (uint16_t)(sign | 0x7c00u | (m ? 0x0200u : 0u));
    int he = e - 112; /* rebias 127 -> 15 */
    if (he >= 31) return (uint16_t)(sign | 0x7c00u);
    uint32_t sig;   /* significand with the implicit one */
    unsigned drop;  /* low bits to round away */
    if (he <= 0) {
        if (he < -10) return sign; /* below half the smallest subnormal */
        sig = m | 0x800000u;
        drop = (unsigned)(14 - he);
        he = 0;
    } else {
        sig = m;
        drop = 13;
    }
    uint32_t kept = sig >> drop;
    uint32_t rem = sig & ((1u << drop) - 1u);
    uint32_t halfway = 1u << (drop - 1);
    if (rem > halfway || (rem == halfway && (kept & 1u))) kept += 1;
    /* a carry out of the mantissa walks into the exponent field by itself */
    uint32_t out = ((uint32_t)he << 10) + kept;
    if (out >= 0x7c00u) out = 0x7c00u;
    return (uint16_t)(sign | out);
}

float xo_f16_bits_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    if (e == 0x1f) return bits_f32(sign | 0x7f800000u | (m << 13));
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        /* subnormal: value = m * 2^-24, exact in binary32 */
        float v = (float)m * 5.9604644775390625e-8f;
        return sign ? -v : v;
    }
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* ===================================================================== */
/* crates/xabe-kernels/src/quant.rs                                      */
/* ===================================================================== */
size_t xo_block_bytes(int quant) { return quant == XO_QUANT_Q6K ? XO_Q6K_BYTES : XO_Q8_0_BYTES; }
size_t xo_block_elements(int quant) { return quant == XO_QUANT_Q6K ? XO_QK_K : XO_QK8_0; }

/* quant.rs:171-202 (dequantize_q6_k) over the byte layout of
 * quant.rs:797-820 (from_bytes): ql[128] | qh[64] | scales[16] i8 | d f16. */
void xo_dequantize_q6_k_block(const uint8_t* blk, float* y) {
    const uint8_t* ql_all = blk;
    const uint8_t* qh_all = blk + 128;
    const int8_t* sc_all = (const int8_t*)(blk + 192);
    float d = xo_f16_bits_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
    for (int half = 0; half < 2; ++half) {
        const uint8_t* ql = ql_all + half * 64;
        const uint8_t* qh = qh_all + half * 32;
        const int8_t* sc = sc_all + half * 8;
        float* yo = y + half * 128;
        for (int l = 0; l < 32; ++l) {
            int is = l / 16;
            int raw1 = (ql[l] & 0xF) | ((qh[l] & 3) << 4);
            int raw2 = (ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4);
            int raw3 = (ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4);
            int raw4 = (ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4);
            /* operand order (d * sc) * q, quant.rs:195-198 */
            yo[l]      = d * (float)sc[is]     * (float)(raw1 - 32);
            yo[l + 32] = d * (float)sc[is + 2] * (float)(raw2 - 32);
            yo[l + 64] = d * (float)sc[is + 4] * (float)(raw3 - 32);
            yo[l + 96] = d * (float)sc[is + 6] * (float)(raw4 - 32);
        }
    }
}

/* quant.rs:62-69 over quant.rs:762-776: d f16 | qs[32] i8; y = q * d. */
void xo_dequantize_q8_0_block(const uint8_t* blk, float* y) {
    float d = xo_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    const int8_t* qs = (const int8_t*)(blk + 2);
    for (int j = 0; j < XO_QK8_0; ++j) y[j] = (float)qs[j] * d;
}

/* quant.rs:76-90 (quantize_q8_0): delta = amax/127, round half away. */
void xo_quantize_q8_0_block(const float* x, uint8_t* blk) {
    float amax = 0.0f;
    for (int j = 0; j < XO_QK8_0; ++j) amax = fmaxf(amax, fabsf(x[j]));
    float d = amax / 127.0f;
    float inv_d = d != 0.0f ? 1.0f / d : 0.0f;
    uint16_t h = xo_f32_to_f16_bits(d);
    blk[0] = (uint8_t)(h & 0xff);
    blk[1] = (uint8_t)(h >> 8);
    for (int j = 0; j < XO_QK8_0; ++j) {
        float q = roundf(x[j] * inv_d);
        if (q > 127.0f) q = 127.0f;   /* Rust `as i8` saturates */
        if (q < -128.0f) q = -128.0f;
        blk[2 + j] = (uint8_t)(int8_t)q;
    }
}

/* quant.rs:495-567 (quantize_q6_k) with the group map of quant.rs:205-215:
 * group (half, lane, is) -> scale half*8 + lane*2 + is, positions
 * half*128 + lane*32 + is*16 + 0..15. */
void xo_quantize_q6_k_block(const float* x, uint8_t* blk) {
    memset(blk, 0, XO_Q6K_BYTES);
    uint8_t* ql = blk;
    uint8_t* qh = blk + 128;
    int8_t* scales = (int8_t*)(blk + 192);
    float amax = 0.0f;
    for (int i = 0; i < XO_QK_K; ++i) amax = fmaxf(amax, fabsf(x[i]));
    float d = amax > 0.0f ? amax / (32.0f * 127.0f) : 0.0f;
    for (int half = 0; half < 2; ++half)
        for (int lane = 0; lane < 4; ++lane)
            for (int is = 0; is < 2; ++is) {
                int scale_index = half * 8 + lane * 2 + is;
                int p0 = half * 128 + lane * 32 + is * 16;
                float gmax = 0.0f;
                for (int k = 0; k < 16; ++k) gmax = fmaxf(gmax, fabsf(x[p0 + k]));
                int sc = 0;
                if (d > 0.0f) {
                    float s = roundf(gmax / (d * 32.0f));
                    if (s < 0.0f) s = 0.0f;
                    if (s > 127.0f) s = 127.0f;
                    sc = (int)s;
                }
                scales[scale_index] = (int8_t)sc;
                float denom = d * (float)sc;
                for (int k = 0; k < 16; ++k) {
                    int l = is * 16 + k;
                    int code = 0;
                    if (denom != 0.0f) {
                        float c = roundf(x[p0 + k] / denom);
                        if (c < -32.0f) c = -32.0f;
                        if (c > 31.0f) c = 31.0f;
                        code = (int)c;
                    }
                    unsigned raw = (unsigned)(code + 32);
                    qh[half * 32 + l] |= (uint8_t)((raw >> 4) << (lane * 2));
                    int ql_index = half * 64 + ((lane & 1) ? l + 32 : l);
                    if (lane >= 2) ql[ql_index] |= (uint8_t)((raw & 0xF) << 4);
                    else ql[ql_index] |= (uint8_t)(raw & 0xF);
                }
            }
    uint16_t h = xo_f32_to_f16_bits(d);
    blk[208] = (uint8_t)(h & 0xff);
    blk[209] = (uint8_t)(h >> 8);
}

/* quant.rs:954-983 (dequantize_row_q8_0 / dequantize_row_q6_k) */
int xo_dequantize_row(int quant, const uint8_t* bytes, size_t n_bytes, float* out) {
    size_t bb = xo_block_bytes(quant), be = xo_block_elements(quant);
    if (n_bytes % bb != 0) return -1;
    size_t nb = n_bytes / bb;
    for (size_t b = 0; b < nb; ++b) {
        if (quant == XO_QUANT_Q6K) xo_dequantize_q6_k_block(bytes + b * bb, out + b * be);
        else xo_dequantize_q8_0_block(bytes + b * bb, out + b * be);
    }
    return 0;
}

int xo_quantize_row(int quant, const float* x, size_t n, uint8_t* bytes) {
    size_t bb = xo_block_bytes(quant), be = xo_block_elements(quant);
    if (n % be != 0) return -1;
    for (size_t b = 0; b < n / be; ++b) {
        if (quant == XO_QUANT_Q6K) xo_quantize_q6_k_block(x + b * be, bytes + b * bb);
        else xo_quantize_q8_0_block(x + b * be, bytes + b * bb);
    }
    return 0;
}

/* ===================================================================== */
/* crates/xabe-kernels/src/norm.rs, gemv.rs                              */
/* ===================================================================== */
void xo_rms_norm(const float* x, const float* w, float eps, size_t n, float* out) { /* norm.rs:28-43 */
    float s = -0.0f;
    for (size_t i = 0; i < n; ++i) s = s + x[i] * x[i];
    float mean_sq = s / (float)n;
    float inv_rms = 1.0f / sqrtf(mean_sq + eps);
    for (size_t i = 0; i < n; ++i) out[i] = x[i] * inv_rms * w[i];
}
float xo_silu(float x) { return x / (1.0f + expf(-x)); }     /* norm.rs:46-48 */
float xo_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); } /* norm.rs:58-60 */
void xo_swiglu(const float* gate, const float* up, size_t n, float* out) { /* norm.rs:93-103 */
    for (size_t i = 0; i < n; ++i) out[i] = xo_silu(gate[i]) * up[i];
}

/* Sequential fp32 dot products for up to ROWS rows at once: the rows are
 * independent chains, so interleaving them changes no row's order
 * (gemv.rs:45-58, moe/gemm.rs:25-34). */
#define XO_ROWS 8
static void matvec_rows(const float* w, size_t out_dim, size_t in_dim, const float* x, float* out) {
    size_t o = 0;
    for (; o + XO_ROWS <= out_dim; o += XO_ROWS) {
        float acc[XO_ROWS];
        for (int r = 0; r < XO_ROWS; ++r) acc[r] = -0.0f;
        const float* base = w + o * in_dim;
        for (size_t i = 0; i < in_dim; ++i) {
            float xi = x[i];
            for (int r = 0; r < XO_ROWS; ++r) acc[r] = acc[r] + base[(size_t)r * in_dim + i] * xi;
        }
        for (int r = 0; r < XO_ROWS; ++r) out[o + r] = acc[r];
    }
    for (; o < out_dim; ++o) {
        float acc = -0.0f;
        const float* row = w + o * in_dim;
        for (size_t i = 0; i < in_dim; ++i) acc = acc + row[i] * x[i];
        out[o] = acc;
    }
}
void xo_gemv(const float* w, size_t out_dim, size_t in_dim, const float* x, float* out) {
    matvec_rows(w, out_dim, in_dim, x, out);
}

/* gemv.rs:102-111: index of the largest element, ties to the lower index. */
size_t xo_argmax(const float* v, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; ++i)
        if (v[i] > v[best]) best = i;
    return best;
}

/* The LM head's CPU reference as crates/xabe-engine/tests/lm_head_differential.rs:17-19
 * builds it: `gemv_batch` (gemv.rs:71-88) over rows dequantised from the file
 * bytes (quant.rs:62-69,171-202), logits [tokens][vocab].  Rows are independent,
 * so sharing them over threads changes no sum. */
int xo_lm_head(int quant, const uint8_t* bytes, size_t vocab, size_t hidden, const float* x, size_t tokens,
               float* logits, int threads) {
    size_t be = xo_block_elements(quant), bb = xo_block_bytes(quant);
    if (be == 0 || hidden % be != 0) return -1;
    size_t row_bytes = hidden / be * bb;
    int nt = threads > 0 ? threads : omp_get_num_procs();
    int failed = 0;
#pragma omp parallel num_threads(nt)
    {
        float* row = (float*)malloc(hidden * sizeof(float));
        if (!row) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(static)
        for (long long v = 0; v < (long long)vocab; ++v) {
            if (!row) continue;
            xo_dequantize_row(quant, bytes + (size_t)v * row_bytes, row_bytes, row);
            for (size_t t = 0; t < tokens; ++t) {
                float acc = -0.0f; /* Rust's f32 sum() starts from -0.0 */
                const float* xt = x + t * hidden;
                for (size_t i = 0; i < hidden; ++i) acc = acc + row[i] * xt[i];
                logits[t * vocab + (size_t)v] = acc;
            }
        }
        free(row);
    }
    return failed ? -2 : 0;
}

/* ===================================================================== */
/* Orders pinned by the reference's device kernels.                       */
/* `block_reduce_sum` (crates/xabe-cuda/src/kernels/layer_ops.rs:93-110,   */
/* crates/xabe-engine/src/block/moe.rs:209-226): shuffle-down tree inside  */
/* each warp of 32 consecutive threads, then the warp totals added in      */
/* ascending warp order starting from +0.0.  The per-thread partials use    */
/* fused multiply-add (NVRTC's default contraction of `acc += a * b`).      */
/* ===================================================================== */
static float warp_tree_lane0(float* v /* 32 values, clobbered */) {
    for (int off = 16; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) v[i] = v[i] + v[i + off];
    return v[0];
}
static float block_reduce_dev(const float* partial, size_t threads) {
    float total = 0.0f;
    for (size_t w0 = 0; w0 < threads; w0 += 32) {
        float v[32];
        for (int i = 0; i < 32; ++i) v[i] = (w0 + (size_t)i < threads) ? partial[w0 + i] : 0.0f;
        total = total + warp_tree_lane0(v);
    }
    return total;
}

/* layer_ops.rs:129-150 with the launch shape of layer_ops.rs:1219-1221
 * (block = width rounded up to 32, at most 1024 threads). */
void xo_rms_norm_dev(const float* x, const float* w, float eps, size_t n, float* out) {
    size_t threads = (n + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    float partial[1024];
    for (size_t t = 0; t < threads; ++t) {
        float p = 0.0f;
        for (size_t j = t; j < n; j += threads) p = fmaf(x[j], x[j], p);
        partial[t] = p;
    }
    float sum_sq = block_reduce_dev(partial, threads);
    float inv_rms = 1.0f / sqrtf(sum_sq / (float)n + eps);
    for (size_t i = 0; i < n; ++i) out[i] = x[i] * inv_rms * w[i];
}

/* crates/xabe-engine/src/block/moe.rs:301-382: thread tid of 256 sums
 * j = tid, tid+256, ... ascending; shuffle-down per warp; warps ascending. */
void xo_router_logits_dev(const float* w, const float* x, size_t num_experts,
                          size_t hidden, float* logits) {
    for (size_t e = 0; e < num_experts; ++e) {
        const float* row = w + e * hidden;
        float partial[256];
        for (size_t t = 0; t < 256; ++t) {
            float p = 0.0f;
            for (size_t j = t; j < hidden; j += 256) p = fmaf(row[j], x[j], p);
            partial[t] = p;
        }
        logits[e] = block_reduce_dev(partial, 256);
    }
}

/* crates/xabe-engine/src/block/moe.rs:455-464: 256 gate lanes, stride 256. */
float xo_shared_gate_dot_dev(const float* w, const float* x, size_t hidden) {
    float partial[256];
    for (size_t t = 0; t < 256; ++t) {
        float p = 0.0f;
        for (size_t j = t; j < hidden; j += 256) p = fmaf(w[j], x[j], p);
        partial[t] = p;
    }
    return block_reduce_dev(partial, 256);
}

/* crates/xabe-cuda/src/kernels/moe.rs:1883-1917: thread t of 256 adds
 * exps[t], exps[t+256], ... then a halving tree in shared memory. */
float xo_softmax_denominator_dev(const float* exps, size_t n) {
    float v[256];
    for (size_t t = 0; t < 256; ++t) {
        float s = 0.0f;
        for (size_t e = t; e < n; e += 256) s = s + exps[e];
        v[t] = s;
    }
    for (size_t s = 128; s > 0; s >>= 1)
        for (size_t i = 0; i < s; ++i) v[i] = v[i] + v[i + s];
    return v[0];
}

/* ===================================================================== */
/* crates/xabe-kernels/src/moe/router.rs:32-81                           */
/* ===================================================================== */
void xo_route_token(const float* logits, size_t n, size_t k, int32_t* ids, float* weights) {
    float max_logit = -INFINITY;
    for (size_t i = 0; i < n; ++i) max_logit = fmaxf(max_logit, logits[i]); /* router.rs:42 */
    float* probs = (float*)malloc(n * sizeof(float));
    uint8_t* taken = (uint8_t*)calloc(n, 1);
    float sum_exp = -0.0f;
    for (size_t i = 0; i < n; ++i) { probs[i] = expf(logits[i] - max_logit); }
    for (size_t i = 0; i < n; ++i) sum_exp = sum_exp + probs[i];               /* router.rs:44 */
    for (size_t i = 0; i < n; ++i) probs[i] = probs[i] / sum_exp;              /* router.rs:45 */
    /* router.rs:50-60: stable sort by (prob desc, index asc), truncate to k.
     * k selection passes give the same prefix of that total order. */
    for (size_t j = 0; j < k; ++j) {
        long best = -1;
        for (size_t i = 0; i < n; ++i) {
            if (taken[i]) continue;
            if (best < 0 || probs[i] > probs[best]) best = (long)i;
        }
        taken[best] = 1;
        ids[j] = (int32_t)best;
    }
    float selected_sum = -0.0f;
    for (size_t j = 0; j < k; ++j) selected_sum = selected_sum + probs[ids[j]]; /* router.rs:62 */
    for (size_t j = 0; j < k; ++j)
        weights[j] = selected_sum > 0.0f ? probs[ids[j]] / selected_sum
                                         : 1.0f / (float)k;                    /* router.rs:64-71 */
    free(probs);
    free(taken);
}
void xo_route_batch(const float* logits, size_t tokens, size_t n, size_t k,
                    int32_t* ids, float* weights) { /* router.rs:79-81 */
    for (size_t t = 0; t < tokens; ++t)
        xo_route_token(logits + t * n, n, k, ids + t * k, weights + t * k);
}

/* ===================================================================== */
/* crates/xabe-kernels/src/moe/dispatch.rs:24-131                        */
/* ===================================================================== */
long xo_moe_align_block_size(const int32_t* topk_ids, size_t tokens, size_t top_k,
                             size_t block_size, size_t num_experts,
                             int32_t* sorted_token_ids, int32_t* expert_ids) {
    if (block_size == 0) return -1; /* dispatch.rs:65-68 */
    size_t numel = tokens * top_k;
    for (size_t i = 0; i < numel; ++i)
        if (topk_ids[i] < 0 || (size_t)topk_ids[i] >= num_experts) return -1; /* dispatch.rs:83-88 */
    uint32_t* counts = (uint32_t*)calloc(num_experts + 1, sizeof(uint32_t));
    uint32_t* cumsum = (uint32_t*)calloc(num_experts + 1, sizeof(uint32_t));
    uint32_t* running = (uint32_t*)calloc(num_experts + 1, sizeof(uint32_t));
    for (size_t i = 0; i < numel; ++i) counts[topk_ids[i]] += 1;
    for (size_t e = 0; e < num_experts; ++e) {
        uint32_t padded = (uint32_t)((counts[e] + block_size - 1) / block_size * block_size);
        cumsum[e + 1] = cumsum[e] + padded;                                   /* dispatch.rs:95-105 */
    }
    size_t post_pad = cumsum[num_experts];
    int32_t sentinel = (int32_t)numel;                                        /* dispatch.rs:24-26 */
    for (size_t i = 0; i < post_pad; ++i) sorted_token_ids[i] = sentinel;
    for (size_t i = 0; i < numel; ++i) {                                      /* dispatch.rs:110-115 */
        int32_t e = topk_ids[i];
        sorted_token_ids[cumsum[e] + running[e]] = (int32_t)i;
        running[e] += 1;
    }
    size_t num_blocks = post_pad / block_size;
    for (size_t b = 0; b < num_blocks; ++b) expert_ids[b] = XO_INACTIVE_EXPERT;
    for (size_t e = 0; e < num_experts; ++e)                                  /* dispatch.rs:117-125 */
        for (size_t b = cumsum[e] / block_size; b < cumsum[e + 1] / block_size; ++b)
            expert_ids[b] = (int32_t)e;
    free(counts); free(cumsum); free(running);
    return (long)post_pad;
}

/* crates/xabe-cuda/src/kernels/moe.rs:4575-4589 (sorted_capacity) */
size_t xo_sorted_capacity(size_t num_experts, size_t top_k, size_t block_size, size_t max_tokens) {
    size_t numel = max_tokens * top_k;
    size_t active = num_experts < numel ? num_experts : numel;
    size_t bound = numel + active * (block_size - 1);
    return (bound + block_size - 1) / block_size * block_size;
}

/* ===================================================================== */
/* crates/xabe-kernels/src/moe/gemm.rs:25-125                            */
/* ===================================================================== */
void xo_expert_mlp(const float* gate, const float* up, const float* down,
                   const float* x, size_t hidden, size_t inter, float* out) { /* gemm.rs:37-47 */
    float* g = (float*)malloc(3 * inter * sizeof(float));
    float* u = g + inter;
    float* a = u + inter;
    matvec_rows(gate, inter, hidden, x, g);
    matvec_rows(up, inter, hidden, x, u);
    xo_swiglu(g, u, inter, a);
    matvec_rows(down, hidden, inter, a, out);
    free(g);
}

void xo_naive_forward(const float* hs, size_t tokens, const int32_t* ids, const float* weights,
                      size_t top_k, const float* gate, const float* up, const float* down,
                      size_t hidden, size_t inter, float* out) { /* gemm.rs:102-125 */
    size_t gu = inter * hidden;
    float* c = (float*)malloc(hidden * sizeof(float));
    for (size_t t = 0; t < tokens; ++t) {
        float* acc = out + t * hidden;
        for (size_t j = 0; j < hidden; ++j) acc[j] = 0.0f;
        for (size_t k = 0; k < top_k; ++k) {
            size_t e = (size_t)ids[t * top_k + k];
            float wgt = weights[t * top_k + k];
            xo_expert_mlp(gate + e * gu, up + e * gu, down + e * gu, hs + t * hidden, hidden, inter, c);
            for (size_t j = 0; j < hidden; ++j) acc[j] += wgt * c[j];
        }
    }
    free(c);
}

void xo_grouped_forward(const float* hs, size_t tokens, const int32_t* sorted_token_ids,
                        const int32_t* expert_ids, size_t num_blocks, size_t block_size,
                        const float* flat_weights, size_t top_k, const float* gate,
                        const float* up, const float* down, size_t hidden, size_t inter,
                        float* out) { /* gemm.rs:58-98 */
    size_t gu = inter * hidden;
    int32_t sentinel = (int32_t)(tokens * top_k);
    float* c = (float*)malloc(hidden * sizeof(float));
    for (size_t i = 0; i < tokens * hidden; ++i) out[i] = 0.0f;
    for (size_t b = 0; b < num_blocks; ++b) {
        int32_t e = expert_ids[b];
        if (e == XO_INACTIVE_EXPERT) continue;
        for (size_t slot = b * block_size; slot < (b + 1) * block_size; ++slot) {
            int32_t flat = sorted_token_ids[slot];
            if (flat == sentinel) continue;
            size_t t = (size_t)flat / top_k;
            float wgt = flat_weights[flat];
            xo_expert_mlp(gate + (size_t)e * gu, up + (size_t)e * gu, down + (size_t)e * gu,
                          hs + t * hidden, hidden, inter, c);
            for (size_t j = 0; j < hidden; ++j) out[t * hidden + j] += wgt * c[j];
        }
    }
    free(c);
}

/* ===================================================================== */
/* crates/xabe-kernels/src/compare.rs:67-135                             */
/* ===================================================================== */
void xo_compare(const float* c, const float* r, size_t n, xo_comparison* out) {
    memset(out, 0, sizeof(*out));
    double dot = 0, nc = 0, nr = 0, nd = 0;
    for (size_t i = 0; i < n; ++i) {
        if (!isfinite(c[i])) { out->non_finite_count++; continue; }
        float ae = fabsf(c[i] - r[i]);
        if (ae > out->max_abs_error) { out->max_abs_error = ae; out->max_abs_error_index = i; }
        float re = ae / fmaxf(fabsf(r[i]), 1e-6f);
        if (re > out->max_rel_error) { out->max_rel_error = re; out->max_rel_error_index = i; }
        dot += (double)c[i] * (double)r[i];
        nc += (double)c[i] * (double)c[i];
        nr += (double)r[i] * (double)r[i];
        nd += ((double)c[i] - (double)r[i]) * ((double)c[i] - (double)r[i]);
    }
    double denom = sqrt(nc) * sqrt(nr);
    out->cosine_similarity = denom > 0 ? (float)(dot / denom) : ((nc == 0 && nr == 0) ? 1.0f : 0.0f);
    out->len = n;
    out->rel_l2 = nr > 0 ? sqrt(nd / nr) : sqrt(nd);
}

/* ===================================================================== */
/* Whole block over quantized stacks.  Composition per                    */
/* crates/xabe-engine/src/block/moe.rs:12-25; weights of only the          */
/* selected experts are dequantized, as                                    */
/* crates/xabe-engine/tests/moe_differential.rs:716-782 does.              */
/* ===================================================================== */
/* The processors this process may run on: a launcher that exports OMP_NUM_THREADS=1 for its
 * ranks does not shrink the CPU baseline to one thread. */
int xo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}
static int pick_threads(int threads) {
    int m = xo_max_threads();
    if (threads <= 0 || threads > m) return m;
    return threads;
}

static float* dequant_matrix(const uint8_t* bytes, int quant, size_t elements) {
    size_t nb = elements / xo_block_elements(quant) * xo_block_bytes(quant);
    float* w = (float*)malloc(elements * sizeof(float));
    if (!w) return NULL;
    xo_dequantize_row(quant, bytes, nb, w);
    return w;
}
static size_t stack_stride_bytes(int quant, size_t elements) {
    return elements / xo_block_elements(quant) * xo_block_bytes(quant);
}

int xo_mlp_forward_q(const uint8_t* gate, int gq, const uint8_t* up, int uq,
                     const uint8_t* down, int dq, size_t hidden, size_t inter,
                     const float* x, size_t tokens, int threads, float* out) {
    size_t n = hidden * inter;
    float* g = dequant_matrix(gate, gq, n);
    float* u = dequant_matrix(up, uq, n);
    float* d = dequant_matrix(down, dq, n);
    if (!g || !u || !d) { free(g); free(u); free(d); return -1; }
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
    for (long t = 0; t < (long)tokens; ++t)
        xo_expert_mlp(g, u, d, x + (size_t)t * hidden, hidden, inter, out + (size_t)t * hidden);
    free(g); free(u); free(d);
    return 0;
}

int xo_routed_forward_q(const xo_moe_layer* L, const float* hs, size_t tokens,
                        const int32_t* ids, const float* weights, int threads, float* out) {
    size_t E = L->num_experts, K = L->top_k, H = L->hidden, I = L->inter;
    size_t n = H * I;
    int nt = pick_threads(threads);
    (void)nt;
    float** cache = (float**)calloc(E * 3, sizeof(float*));
    uint8_t* used = (uint8_t*)calloc(E, 1);
    for (size_t i = 0; i < tokens * K; ++i) used[ids[i]] = 1;
    int fail = 0;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
    for (long e = 0; e < (long)E; ++e) {
        if (!used[e]) continue;
        cache[e * 3 + 0] = dequant_matrix(L->gate_exps + (size_t)e * stack_stride_bytes(L->gate_quant, n), L->gate_quant, n);
        cache[e * 3 + 1] = dequant_matrix(L->up_exps + (size_t)e * stack_stride_bytes(L->up_quant, n), L->up_quant, n);
        cache[e * 3 + 2] = dequant_matrix(L->down_exps + (size_t)e * stack_stride_bytes(L->down_quant, n), L->down_quant, n);
        if (!cache[e * 3] || !cache[e * 3 + 1] || !cache[e * 3 + 2]) {
#pragma omp atomic write
            fail = 1;
        }
    }
    if (!fail) {
        float* contrib = (float*)malloc(tokens * K * H * sizeof(float));
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
        for (long p = 0; p < (long)(tokens * K); ++p) {
            size_t e = (size_t)ids[p];
            xo_expert_mlp(cache[e * 3], cache[e * 3 + 1], cache[e * 3 + 2],
                          hs + ((size_t)p / K) * H, H, I, contrib + (size_t)p * H);
        }
        /* gemm.rs:113-121: acc += weight * contribution, k ascending */
        for (size_t t = 0; t < tokens; ++t)
            for (size_t j = 0; j < H; ++j) {
                float acc = 0.0f;
                for (size_t k = 0; k < K; ++k)
                    acc += weights[t * K + k] * contrib[(t * K + k) * H + j];
                out[t * H + j] = acc;
            }
        free(contrib);
    }
    for (size_t i = 0; i < E * 3; ++i) free(cache[i]);
    free(cache); free(used);
    return fail ? -1 : 0;
}

int xo_moe_block_forward(const xo_moe_layer* L, const float* residual, size_t tokens,
                         int order, int threads, xo_moe_outputs* o) {
    size_t E = L->num_experts, K = L->top_k, H = L->hidden;
    float* normed = (float*)malloc(tokens * H * sizeof(float));
    float* logits = (float*)malloc(tokens * E * sizeof(float));
    int32_t* ids = (int32_t*)malloc(tokens * K * sizeof(int32_t));
    float* wts = (float*)malloc(tokens * K * sizeof(float));
    float* routed = (float*)malloc(tokens * H * sizeof(float));
    float* shexp = (float*)malloc(tokens * H * sizeof(float));
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel for schedule(static) num_threads(nt)
    for (long t = 0; t < (long)tokens; ++t) {
        const float* x = residual + (size_t)t * H;
        float* nrm = normed + (size_t)t * H;
        if (order == 1) {
            xo_rms_norm_dev(x, L->post_norm, L->eps, H, nrm);
            xo_router_logits_dev(L->router, nrm, E, H, logits + (size_t)t * E);
        } else {
            xo_rms_norm(x, L->post_norm, L->eps, H, nrm);
            xo_gemv(L->router, E, H, nrm, logits + (size_t)t * E);
        }
        if (L->router_bias)
            for (size_t e = 0; e < E; ++e) logits[(size_t)t * E + e] = logits[(size_t)t * E + e] + L->router_bias[e];
        xo_route_token(logits + (size_t)t * E, E, K, ids + (size_t)t * K, wts + (size_t)t * K);
    }
    int rc = xo_routed_forward_q(L, normed, tokens, ids, wts, threads, routed);
    if (rc == 0)
        rc = xo_mlp_forward_q(L->shared_gate, L->shared_gate_quant, L->shared_up, L->shared_up_quant,
                              L->shared_down, L->shared_down_quant, H, L->inter, normed, tokens,
                              threads, shexp);
    if (rc == 0) {
        for (size_t t = 0; t < tokens; ++t) {
            const float* nrm = normed + t * H;
            float s;
            if (order == 1) s = xo_shared_gate_dot_dev(L->shared_gate_inp, nrm, H);
            else { s = -0.0f; for (size_t j = 0; j < H; ++j) s = s + L->shared_gate_inp[j] * nrm[j]; }
            float g = xo_sigmoid(s);
            if (o->gate) o->gate[t] = g;
            for (size_t j = 0; j < H; ++j) {
                /* block/moe.rs:22-23: ffn_out = routed + shexp * g; l_out = ffn_out + input */
                float v = routed[t * H + j] + shexp[t * H + j] * g;
                if (o->ffn_out) o->ffn_out[t * H + j] = v;
                if (o->l_out) o->l_out[t * H + j] = v + residual[t * H + j];
            }
        }
        if (o->normed) memcpy(o->normed, normed, tokens * H * sizeof(float));
        if (o->logits) memcpy(o->logits, logits, tokens * E * sizeof(float));
        if (o->topk_ids) memcpy(o->topk_ids, ids, tokens * K * sizeof(int32_t));
        if (o->topk_weights) memcpy(o->topk_weights, wts, tokens * K * sizeof(float));
        if (o->routed) memcpy(o->routed, routed, tokens * H * sizeof(float));
        if (o->shexp) memcpy(o->shexp, shexp, tokens * H * sizeof(float));
    }
    free(normed); free(logits); free(ids); free(wts); free(routed); free(shexp);
    return rc;
}

/* crates/xabe-engine/src/block/dense_ffn.rs:9-16; oracle composition as in
 * crates/xabe-engine/tests/dense_ffn_differential.rs:46-49. */
int xo_dense_block_forward(const float* post_norm, float eps, const uint8_t* gate, int gq,
                           const uint8_t* up, int uq, const uint8_t* down, int dq,
                           size_t hidden, size_t inter, const float* residual, size_t tokens,
                           int order, int threads, float* ffn_out, float* l_out) {
    float* normed = (float*)malloc(tokens * hidden * sizeof(float));
    for (size_t t = 0; t < tokens; ++t) {
        if (order == 1) xo_rms_norm_dev(residual + t * hidden, post_norm, eps, hidden, normed + t * hidden);
        else xo_rms_norm(residual + t * hidden, post_norm, eps, hidden, normed + t * hidden);
    }
    float* tmp = ffn_out ? ffn_out : (float*)malloc(tokens * hidden * sizeof(float));
    int rc = xo_mlp_forward_q(gate, gq, up, uq, down, dq, hidden, inter, normed, tokens, threads, tmp);
    if (rc == 0 && l_out)
        for (size_t i = 0; i < tokens * hidden; ++i) l_out[i] = tmp[i] + residual[i];
    if (!ffn_out) free(tmp);
    free(normed);
    return rc;
}
