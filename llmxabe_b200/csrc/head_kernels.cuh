// LM head: logits[t][v] = sum_j W[v][j] * x[t][j], W in file layout (Q8_0 or Q6_K rows of `hidden`
// elements), x fp32 (LmHeadKernels::forward, crates/xabe-cuda/src/kernels/lm_head.rs:1695-1937).
//
// One pass over the weights serves up to eight tokens, as the reference's batch tile does
// (lm_head.rs:125, weight_passes :1380-1383): grid.y walks the passes.  The pass is HBM-bound
// (540 MB at the real geometry), so it is built like k_gateup_rows: one persistent CTA per SM, a
// producer warp that streams 256-element spans of 128 consecutive rows through a ring with 2-D TMA
// boxes over the weight bytes, and sixteen consumer warps that each own sixteen rows for the whole
// contraction (no exchange between warps).  Codes stay exact integers in f16 A fragments and the
// block scales are applied in fp32; the fp32 activations are split into two f16 parts,
// x = hi + lo, and both products are summed inside the tensor core (stream_half<.., SPLIT>), so an
// activation keeps about 22 bits: the logits agree with the fp32 reference to ~1e-6 relative and
// the argmax is the reference's.  A token's logits depend on its own column only.
//
// Unit of work: 256 consecutive vocabulary rows; group gi of the CTA owns rows 128 gi .. 128 gi + 127
// of the unit and takes every other ring stage; warp w of the group owns rows 8 w + g and
// 64 + 8 w + g (g = lane / 4).  Per row the spans are added in ascending order, half 0 then half 1.
#pragma once

#include <cuda.h>

#include "stream_rows_kernels.cuh"

namespace xabe {

constexpr int kHeadUnitRows = 2 * kRowsUnitRows;  // 256
constexpr int kHeadMaxStages = 5;

struct HeadLaunch {
    CUtensorMap tm_w;          // weight bytes [vocab][row_bytes / 4] as 32-bit words, box = box_w bytes x 64 rows
    const __half* x_hi;        // [max_tokens][hidden]
    const __half* x_lo;        // [max_tokens][hidden]
    float* logits;             // [max_tokens][vocab]
    int* status;
    int vocab, hidden, tokens;
    int n_stages;
    uint32_t box_w, stage_bytes, x_stride;
};

struct HeadSmem {
    uint32_t stages, x_hi, x_lo, bars, total;
};

__host__ __device__ inline HeadSmem head_smem_layout(int n_stages, uint32_t stage_bytes, uint32_t x_stride) {
    HeadSmem R;
    R.stages = 0;  // relative to the 128-byte aligned base
    R.x_hi = R.stages + (uint32_t)n_stages * stage_bytes;
    R.x_lo = R.x_hi + 8u * x_stride;
    R.bars = R.x_lo + 8u * x_stride;
    R.total = R.bars + 8u * 2u * kHeadMaxStages + 128u;  // + slack for aligning the base
    return R;
}

// x (fp32) -> hi = f16(x), lo = f16(x - hi).  grid: tokens.
__global__ void k_head_split(const float* __restrict__ x, int tokens, int hidden, __half* __restrict__ hi,
                             __half* __restrict__ lo) {
    const int t = blockIdx.x;
    if (t >= tokens) return;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float v = x[(size_t)t * hidden + j];
        const __half h = __float2half_rn(v);
        hi[(size_t)t * hidden + j] = h;
        lo[(size_t)t * hidden + j] = __float2half_rn(v - __half2float(h));
    }
}

template <int QUANT>
__device__ __forceinline__ void head_half(const uint8_t* pa, const uint8_t* pb, int h, const uint2* bh, const uint2* bl,
                                          int lane, float (&acc)[4]) {
    if ((uintptr_t)pa & 2) stream_half<QUANT, true, true>(pa, pb, h, bh, lane, acc, bl);
    else stream_half<QUANT, false, true>(pa, pb, h, bh, lane, acc, bl);
}

// grid: (number of SMs, passes); block: 32 * 17 (warp 0 streams weights, warps 1-16 consume).
// Every wait is bounded as in k_expert_stream.
template <int QUANT>
__global__ void __launch_bounds__(32 * (1 + kStreamConsumerWarps), 1) k_head_rows(const __grid_constant__ HeadLaunch P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int abort_flag;
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const int S = P.n_stages;
    const HeadSmem lay = head_smem_layout(S, P.stage_bytes, P.x_stride);
    uint64_t* full = (uint64_t*)(smem + lay.bars);
    uint64_t* empty = full + kHeadMaxStages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kStreamGroupWarps);
        }
        fence_mbar_init();
    }
    // this pass's activation rows (up to eight tokens), both parts; rows past the batch are zero
    const int t0 = (int)blockIdx.y * 8;
    const int ncols = min(8, P.tokens - t0);
    {
        const int words_per_row = P.hidden / 2;  // two f16 per word
        for (int i = threadIdx.x; i < 8 * words_per_row; i += blockDim.x) {
            const int c = i / words_per_row, j = i - c * words_per_row;
            uint32_t vh = 0u, vl = 0u;
            if (c < ncols) {
                vh = ((const uint32_t*)(P.x_hi + (size_t)(t0 + c) * P.hidden))[j];
                vl = ((const uint32_t*)(P.x_lo + (size_t)(t0 + c) * P.hidden))[j];
            }
            *(uint32_t*)(smem + lay.x_hi + (uint32_t)c * P.x_stride + 4u * j) = vh;
            *(uint32_t*)(smem + lay.x_lo + (uint32_t)c * P.x_stride + 4u * j) = vl;
        }
    }
    __syncthreads();
    volatile int* abortp = &abort_flag;
    const int n_spans = P.hidden / kSpanElems;
    const int units = (P.vocab + kHeadUnitRows - 1) / kHeadUnitRows;
    const int span_b = span_bytes_of(QUANT);

    if (warp == 0) {
        // ------------------------------ weight producer ------------------------------
        if (lane != 0) return;
        int st = 0;
        uint32_t use = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            const int y0 = u * kHeadUnitRows;
            for (int s = 0; s < n_spans; ++s) {
                const int x = rows_box_start(span_b * s, span_b * n_spans, (int)P.box_w) >> 2;  // in 32-bit words
#pragma unroll
                for (int gi = 0; gi < kStreamGroups; ++gi) {
                    if (use >= 1 && !stream_wait(&empty[st], (use - 1) & 1, abortp, P.status)) return;
                    uint8_t* dst = smem + lay.stages + (uint32_t)st * P.stage_bytes;
                    mbar_expect_tx(&full[st], 2u * kRowsGroupRows * P.box_w);
                    // rows past the end of the matrix read as zero and are never stored
                    tma_load_box_2d(dst, &P.tm_w, x, y0 + gi * kRowsUnitRows, &full[st]);
                    tma_load_box_2d(dst + kRowsGroupRows * P.box_w, &P.tm_w, x, y0 + gi * kRowsUnitRows + kRowsGroupRows,
                                    &full[st]);
                    if (++st == S) {
                        st = 0;
                        ++use;
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------- consumers ----------------------------------
    const int cw = warp - 1;
    const int gi = cw / kStreamGroupWarps;
    const int w = cw % kStreamGroupWarps;
    const int g = lane >> 2, t = lane & 3;
    int st = gi % S;
    uint32_t use = (uint32_t)(gi / S);
    const uint8_t* xh = smem + lay.x_hi + (uint32_t)g * P.x_stride;  // column g of the pass
    const uint8_t* xl = smem + lay.x_lo + (uint32_t)g * P.x_stride;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < n_spans; ++s) {
            if (!stream_wait(&full[st], use & 1, abortp, P.status)) return;
            const uint8_t* pa = smem + lay.stages + (uint32_t)st * P.stage_bytes + (uint32_t)(w * 8 + g) * P.box_w +
                                (uint32_t)(span_b * s - rows_box_start(span_b * s, span_b * n_spans, (int)P.box_w));
            const uint8_t* pb = pa + kRowsGroupRows * P.box_w;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint2 bh[8], bl[8];
                load_bfrags_half<QUANT>(xh, s, h, t, bh);
                load_bfrags_half<QUANT>(xl, s, h, t, bl);
                head_half<QUANT>(pa, pb, h, bh, bl, lane, acc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);  // the ring stage may be refilled
            st += kStreamGroups;
            if (st >= S) {
                st -= S;
                ++use;
            }
        }
        // acc[0..1]: row a, columns 2t and 2t + 1; acc[2..3]: row b
        const int row_a = u * kHeadUnitRows + gi * kRowsUnitRows + w * 8 + g;
        const int row_b = row_a + kRowsGroupRows;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int col = 2 * t + i;
            if (col < ncols) {
                float* dst = P.logits + (size_t)(t0 + col) * P.vocab;
                if (row_a < P.vocab) dst[row_a] = acc[i];
                if (row_b < P.vocab) dst[row_b] = acc[2 + i];
            }
        }
    }
}

// Index of the largest of n values, ties to the lower index (gemv.rs:102-111; the reference's
// device form is LmHeadKernels::argmax, lm_head.rs:1950-2015).  One block per row of `logits`.
__global__ void __launch_bounds__(1024) k_head_argmax(const float* __restrict__ logits, int vocab, int tokens,
                                                      int* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const int tk = blockIdx.x;
    if (tk >= tokens) return;
    const float* v = logits + (size_t)tk * vocab;
    float best = v[0];
    int idx = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = v[i];
        if (x > best || (x == best && i < idx)) {
            best = x;
            idx = i;
        }
    }
    // a thread that saw nothing larger than v[0] holds (v[0], 0), which is a valid candidate
    for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (ob > best || (ob == best && oi < idx)) {
            best = ob;
            idx = oi;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        bv[warp] = best;
        bi[warp] = idx;
    }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? bv[lane] : bv[0];
        idx = lane < nw ? bi[lane] : bi[0];
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
            if (ob > best || (ob == best && oi < idx)) {
                best = ob;
                idx = oi;
            }
        }
        if (lane == 0) out[tk] = idx;
    }
}

}  // namespace xabe
