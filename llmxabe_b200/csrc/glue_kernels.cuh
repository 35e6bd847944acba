// Everything in the MoE block that is not an expert matrix product:
// RMSNorm, router logits, softmax top-k routing, the block-aligned dispatch
// tables, the gate-and-combine epilogue, and standalone dequantisation.
//
// RMSNorm, the router logits and the shared-gate dot product reproduce, sum
// for sum, the reduction order of the reference's device kernels, because
// their results pick experts: a last-bit change in a logit can run a
// different expert (crates/xabe-engine/src/block/moe.rs:250-269).
#pragma once

#include "common.cuh"

namespace xabe {

// ---------------------------------------------------------------------------
// RMSNorm.  Order of crates/xabe-cuda/src/kernels/layer_ops.rs:129-150 with
// the block width of layer_ops.rs:1219-1221 (the launcher passes it): thread
// tid sums x[j]^2 for j = tid, tid+blockDim, ... with fused multiply-add,
// then block_reduce_sum; 1/sqrtf (not rsqrtf); x * inv_rms * w in that order.
// Also writes a half-precision copy, the B operand of the expert kernels.
// With `gate_w` (and `width` floats of dynamic shared memory) it also leaves the shared expert's
// gate of the row in gate[row]: sigmoid(dot(gate_w, normed row)) in the order of
// moe_block_gate_and_combine (256 lanes at stride 256, block_reduce_sum), for a block whose last
// stage is folded into the down projection and so has no kernel of its own to compute it.
// grid: (max_tokens); rows at and beyond *valid_tokens are skipped.
// ---------------------------------------------------------------------------
__global__ void k_rms_norm(const float* __restrict__ x, const float* __restrict__ weight,
                           float* __restrict__ out, __half* __restrict__ out_h,
                           const int* __restrict__ valid_tokens, int width, float eps,
                           const float* __restrict__ gate_w, float* __restrict__ gate) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float norm_row[];
    __shared__ float scratch[32];
    int row = blockIdx.x;
    if (row >= *valid_tokens) return;
    size_t base = (size_t)row * width;
    float partial = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = x[base + j];
        partial = fmaf(v, v, partial);
    }
    float sum_sq = block_reduce_sum_pinned(partial, scratch);
    float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)width), eps)));
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float y = __fmul_rn(__fmul_rn(x[base + j], inv_rms), weight[j]);
        out[base + j] = y;
        if (out_h) out_h[base + j] = __float2half_rn(y);
        if (gate_w) norm_row[j] = y;
    }
    if (gate_w) {
        __syncthreads();
        float s = 0.0f;
        if (threadIdx.x < 256)
            for (int j = threadIdx.x; j < width; j += 256) s = fmaf(gate_w[j], norm_row[j], s);
        // warps past the eighth add +0 after the eight totals: the sum is the eight-warp sum
        s = block_reduce_sum_pinned(s, scratch);
        if (threadIdx.x == 0) gate[row] = __fdiv_rn(1.0f, 1.0f + expf(-s));
    }
}

// k_rms_norm for many rows: the same sums in the same order, but a block walks rows blockIdx.x,
// + gridDim.x, ... with the NEXT row's elements already on their way while it reduces the current one,
// and keeps a row's elements in registers between the sum and the scaling (one read of x instead of
// two).  One block per row spends most of a row's time waiting for its first load: 16384 rows of 2048
// took 160 us where the 335 MB they move need 52 us.
// EPT: elements per thread = ceil(width / blockDim.x), at most 8.  grid: a few blocks per SM.
template <int EPT>
__global__ void __launch_bounds__(1024) k_rms_norm_stream(const float* __restrict__ x, const float* __restrict__ weight,
                                                          float* __restrict__ out, __half* __restrict__ out_h,
                                                          const int* __restrict__ valid_tokens, int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    // block_reduce_sum_pinned's sums on a scratch that alternates by row: a row's total is read before
    // the next row's first barrier and its copy is rewritten only after that row's second, so the third
    // barrier of the one-row form is not needed
    __shared__ float scratch[2][33];
    const int rows = *valid_tokens;
    int parity = 0;
    float wv[EPT], v[EPT], vn[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        const int j = threadIdx.x + i * blockDim.x;
        wv[i] = j < width ? weight[j] : 0.0f;
        vn[i] = 0.0f;
    }
    int row = blockIdx.x;
    if (row < rows) {
#pragma unroll
        for (int i = 0; i < EPT; ++i) {
            const int j = threadIdx.x + i * blockDim.x;
            if (j < width) vn[i] = x[(size_t)row * width + j];
        }
    }
    for (; row < rows; row += gridDim.x) {
#pragma unroll
        for (int i = 0; i < EPT; ++i) v[i] = vn[i];
        const int next = row + gridDim.x;
        if (next < rows) {
#pragma unroll
            for (int i = 0; i < EPT; ++i) {
                const int j = threadIdx.x + i * blockDim.x;
                if (j < width) vn[i] = x[(size_t)next * width + j];
            }
        }
        float partial = 0.0f;
#pragma unroll
        for (int i = 0; i < EPT; ++i)
            if (threadIdx.x + i * blockDim.x < width) partial = fmaf(v[i], v[i], partial);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) partial += __shfl_down_sync(0xffffffffu, partial, off);
        if ((threadIdx.x & 31) == 0) scratch[parity][threadIdx.x >> 5] = partial;
        __syncthreads();
        if (threadIdx.x == 0) {  // the warp totals in ascending order, by one thread
            const int n_warps = (blockDim.x + 31) >> 5;
            float total = 0.0f;
            for (int w = 0; w < n_warps; ++w) total += scratch[parity][w];
            scratch[parity][32] = total;
        }
        __syncthreads();
        const float sum_sq = scratch[parity][32];
        parity ^= 1;
        const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)width), eps)));
        const size_t base = (size_t)row * width;
#pragma unroll
        for (int i = 0; i < EPT; ++i) {
            const int j = threadIdx.x + i * blockDim.x;
            if (j < width) {
                const float y = __fmul_rn(__fmul_rn(v[i], inv_rms), wv[i]);
                out[base + j] = y;
                if (out_h) out_h[base + j] = __float2half_rn(y);
            }
        }
    }
}

__global__ void k_set_scalar(int* dst, int value) { *dst = value; }

// fp32 rows -> half rows (for callers that hand hidden states straight to the
// expert entry points).
__global__ void k_rows_to_half(const float* __restrict__ x, __half* __restrict__ out,
                               const int* __restrict__ valid_tokens, int width) {
    int row = blockIdx.x;
    if (row >= *valid_tokens) return;
    size_t base = (size_t)row * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) out[base + j] = __float2half_rn(x[base + j]);
}

// ---------------------------------------------------------------------------
// Router logits.  The value-level order of moe_block_router_logits
// (crates/xabe-engine/src/block/moe.rs:301-382): 256 lanes; lane v sums
// w[e][j] * x[t][j] for j = v, v+256, ... ascending with fused multiply-add;
// shuffle-down tree inside each group of 32 consecutive lanes; the eight
// group totals added in ascending order starting from +0.  Here one real warp
// carries all 256 lanes of one expert (lane l holds lanes l, l+32, ...), so
// the result is bit-identical for every token-tile width TT.
// The four expert rows of a CTA (contiguous in the router tensor) arrive in
// shared memory through ONE bulk TMA copy, and so do the TT activation rows of
// each token tile (contiguous rows of `x`): every byte is in flight at once
// instead of one dependent L2 round trip per loop iteration and token.
// grid: (ceil(E / 4), ceil(max_tokens / (TT * tiles_per_cta))), block 128.
// dynamic shared memory: (4 + TT) * hidden * 4 bytes.
// ---------------------------------------------------------------------------
template <int TT>
__global__ void __launch_bounds__(128) k_router_logits(const float* __restrict__ w,
                                                        const float* __restrict__ x,
                                                        const int* __restrict__ valid_tokens,
                                                        int hidden, int num_experts,
                                                        const float* __restrict__ bias,
                                                        float* __restrict__ logits, int tiles_per_cta,
                                                        int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) float w_rows[];
    __shared__ __align__(8) uint64_t bar, xbar;
    float* x_rows = w_rows + (size_t)4 * hidden;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int e0 = blockIdx.x * 4;
    int e = e0 + warp;
    int t_first = blockIdx.y * TT * tiles_per_cta;
    int live = *valid_tokens;
    if (t_first >= live) return;
    if (threadIdx.x == 0) {
        int rows = min(4, num_experts - e0);
        uint32_t bytes = (uint32_t)rows * hidden * 4u;
        mbar_init(&bar, 1);
        mbar_init(&xbar, 1);
        fence_mbar_init();
        mbar_expect_tx(&bar, bytes);
        tma_bulk_g2s(w_rows, w + (size_t)e0 * hidden, bytes, &bar);
        uint32_t xbytes = (uint32_t)min(TT, live - t_first) * hidden * 4u;
        mbar_expect_tx(&xbar, xbytes);
        tma_bulk_g2s(x_rows, x + (size_t)t_first * hidden, xbytes, &xbar);
    }
    __syncthreads();
    if (!__syncthreads_and(mbar_wait_bounded(&bar, 0, status))) return;
    const bool active = e < num_experts;
    const float* wrow = w_rows + (size_t)warp * hidden;
    for (int tile = 0; tile < tiles_per_cta; ++tile) {
        int t0 = t_first + tile * TT;
        if (t0 >= live) break;
        if (tile > 0) {
            __syncthreads();  // every warp has left the rows of the tile before
            if (threadIdx.x == 0) {
                uint32_t xbytes = (uint32_t)min(TT, live - t0) * hidden * 4u;
                mbar_expect_tx(&xbar, xbytes);
                tma_bulk_g2s(x_rows, x + (size_t)t0 * hidden, xbytes, &xbar);
            }
        }
        if (!__syncthreads_and(mbar_wait_bounded(&xbar, tile & 1, status))) return;
        if (!active) continue;
        float acc[8][TT];
#pragma unroll
        for (int g = 0; g < 8; ++g)
#pragma unroll
            for (int u = 0; u < TT; ++u) acc[g][u] = 0.0f;
        // hidden is a multiple of 256 (checked when the handle is created).  Rows of the tile
        // past the live tokens were not copied; their sums are formed from whatever the buffer
        // holds and never stored.
        for (int jc = 0; jc < hidden; jc += 256) {
            float wv[8];
#pragma unroll
            for (int g = 0; g < 8; ++g) wv[g] = wrow[jc + g * 32 + lane];
#pragma unroll
            for (int u = 0; u < TT; ++u) {
                const float* xr = x_rows + (size_t)u * hidden;
                float xv[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) xv[g] = xr[jc + g * 32 + lane];
#pragma unroll
                for (int g = 0; g < 8; ++g) acc[g][u] = fmaf(wv[g], xv[g], acc[g][u]);
            }
        }
#pragma unroll
        for (int u = 0; u < TT; ++u) {
            float total = 0.0f;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                float v = acc[g][u];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
                total += v;  // only lane 0's value is the tree's root
            }
            if (lane == 0 && t0 + u < live)
                logits[(size_t)(t0 + u) * num_experts + e] = bias ? __fadd_rn(total, bias[e]) : total;
        }
    }
}

// ---------------------------------------------------------------------------
// Router logits for wide passes (hundreds of tokens and more): same values,
// same order of additions as k_router_logits, arranged for the FMA pipe.
// A CTA of 256 threads IS the 256 lanes of the reference kernel: thread v sums
// j = v, v + 256, ... ascending.  It keeps sixteen expert rows in shared memory
// (one bulk TMA copy) and walks its share of the tokens four at a time, so a
// thread holds 64 accumulators and does 64 multiply-adds per 16 shared-memory
// and 4 (prefetched) global loads.  A warp is one group of 32 lanes of every
// output, so the shuffle-down trees run inside the warp, 32 outputs at a time
// (warp_trees32 below), and the eight group totals are added in ascending order
// starting from +0.
// grid: (E / 16, token shares); block 256;
// dynamic shared memory: 16 * hidden * 4 + 512 * 4 bytes.
// ---------------------------------------------------------------------------
// The shuffle-down trees of 32 outputs over the 32 lanes of a warp, all at once: `a[o]` is this lane's
// addend of output o.  At the level with offset 16 lanes l and l ^ 16 swap halves -- the lower lane keeps
// outputs 0-15 and gets the partner's addends of those, the upper lane keeps 16-31 -- and each adds what
// it received to what it kept; then offset 8 within each half, and so on.  Every sum formed is
// v[l] + v[l + off] of the shuffle-down tree of its output (the left operand is the lower lane's), so
// after five levels lane o holds in a[0] exactly what lane 0 of `for (off = 16; off; off >>= 1)
// v += shfl_down(v, off)` would hold for output o.  31 shuffles per lane instead of 160, and no shared
// memory.
template <int HALF>
__device__ __forceinline__ void warp_trees_level(float (&a)[32], int lane) {
    const bool upper = (lane & HALF) != 0;
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
        const float send = upper ? a[i] : a[HALF + i];
        const float keep = upper ? a[HALF + i] : a[i];
        const float recv = __shfl_xor_sync(0xffffffffu, send, HALF);
        a[i] = upper ? __fadd_rn(recv, keep) : __fadd_rn(keep, recv);
    }
}
__device__ __forceinline__ float warp_trees32(float (&a)[32], int lane) {
    warp_trees_level<16>(a, lane);
    warp_trees_level<8>(a, lane);
    warp_trees_level<4>(a, lane);
    warp_trees_level<2>(a, lane);
    warp_trees_level<1>(a, lane);
    return a[0];
}

constexpr int kRwExperts = 16;
constexpr int kRwTokens = 4;
constexpr int kRwOutputs = kRwExperts * kRwTokens;

__host__ __device__ inline size_t router_wide_smem(int hidden) {
    return (size_t)kRwExperts * hidden * 4 + 512 * 4;
}

template <int NI>
__global__ void __launch_bounds__(256, 1) k_router_logits_wide(const float* __restrict__ w,
                                                               const float* __restrict__ x,
                                                               const int* __restrict__ valid_tokens,
                                                               int num_experts, const float* __restrict__ bias,
                                                               float* __restrict__ logits,
                                                               int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int hidden = NI * 256;
    extern __shared__ __align__(128) float rw_smem[];
    float* w_s = rw_smem;                                 // [16][hidden]
    float* group_tot = rw_smem + kRwExperts * hidden;     // [64][8]
    __shared__ __align__(8) uint64_t bar;
    const int tid = threadIdx.x;
    const int e0 = blockIdx.x * kRwExperts;
    const int live = *valid_tokens;
    const int tiles_total = (live + kRwTokens - 1) / kRwTokens;
    const int tiles_per = (tiles_total + gridDim.y - 1) / gridDim.y;
    const int tile0 = blockIdx.y * tiles_per;
    const int tile1 = min(tiles_total, tile0 + tiles_per);
    if (tile0 >= tile1) return;
    if (tid == 0) {
        const uint32_t bytes = (uint32_t)kRwExperts * hidden * 4u;
        mbar_init(&bar, 1);
        fence_mbar_init();
        mbar_expect_tx(&bar, bytes);
        tma_bulk_g2s(w_s, w + (size_t)e0 * hidden, bytes, &bar);
    }
    float xn[kRwTokens][NI];
    auto load_tile = [&](int tile) {
#pragma unroll
        for (int u = 0; u < kRwTokens; ++u) {
            const int t = min(tile * kRwTokens + u, live - 1);
            const float* xr = x + (size_t)t * hidden + tid;
#pragma unroll
            for (int i = 0; i < NI; ++i) xn[u][i] = __ldg(xr + i * 256);
        }
    };
    load_tile(tile0);
    __syncthreads();
    if (!__syncthreads_and(mbar_wait_bounded(&bar, 0, status))) return;
    for (int tile = tile0; tile < tile1; ++tile) {
        float xc[kRwTokens][NI];
#pragma unroll
        for (int u = 0; u < kRwTokens; ++u)
#pragma unroll
            for (int i = 0; i < NI; ++i) xc[u][i] = xn[u][i];
        if (tile + 1 < tile1) load_tile(tile + 1);  // in flight during this tile's arithmetic
        // outputs o = 4 e + u, in two halves of 32 (experts 0-7 and 8-15 of the CTA)
        float acc[2][32];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int o = 0; o < 32; ++o) acc[h][o] = 0.0f;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
#pragma unroll
            for (int e = 0; e < kRwExperts; ++e) {
                const float wv = w_s[e * hidden + i * 256 + tid];
#pragma unroll
                for (int u = 0; u < kRwTokens; ++u)
                    acc[e >> 3][(e & 7) * kRwTokens + u] = fmaf(wv, xc[u][i], acc[e >> 3][(e & 7) * kRwTokens + u]);
            }
        }
        // this warp is lane group tid / 32 of every output: lane o ends with the totals of outputs o and 32 + o
        __syncthreads();  // the previous tile's totals have been read
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float tot = warp_trees32(acc[h], tid & 31);
            group_tot[(h * 32 + (tid & 31)) * 8 + (tid >> 5)] = tot;
        }
        __syncthreads();
        if (tid < kRwOutputs) {
            float total = 0.0f;
#pragma unroll
            for (int g = 0; g < 8; ++g) total += group_tot[tid * 8 + g];
            const int e = e0 + (tid >> 2), t = tile * kRwTokens + (tid & 3);
            if (t < live && e < num_experts) logits[(size_t)t * num_experts + e] = bias ? __fadd_rn(total, bias[e]) : total;
        }
    }
}

// ---------------------------------------------------------------------------
// Router logits for prefill widths (hundreds of tokens per CTA): the same
// values and order again, with the sixteen expert rows held in REGISTERS.
// Thread v owns w[e][v + 256 i] for its CTA's sixteen experts (16 * NI
// registers, loaded once, coalesced); the CTA's tokens (a contiguous range of
// rows) arrive four at a time through a ring of bulk TMA copies issued several
// stages ahead, so neither the weights nor the L2 latency of the activations
// sit in the inner loop (k_router_logits_wide spends one shared load per four
// multiply-adds and waits for its prefetched global loads once per tile).  A warp
// is one lane group of every output, so the 32 trees of a token pair run inside the
// warp (warp_trees32: no shared memory, no barrier); only the eight group totals
// per output cross warps, through shared memory and one block barrier per ring stage.
// grid: (E / 16, token shares); block 256;
// dynamic shared memory: router_regw_smem(hidden).
// ---------------------------------------------------------------------------
constexpr int kRrOutputs = 32;                      // outputs per accumulator set: NE experts x 32 / NE tokens
constexpr int kRrStageTokens = 4;                   // token rows per ring stage
__host__ __device__ constexpr int rr_stages(int ne) { return ne == 16 ? 4 : 3; }

__host__ __device__ inline size_t router_regw_smem(int hidden, int ne) {
    return (size_t)rr_stages(ne) * kRrStageTokens * hidden * 4 + (size_t)2 * (kRrStageTokens * ne / 32) * kRrOutputs * 8 * 4;
}

// NE: expert rows per CTA held in registers.  16: one CTA per SM, two tokens per accumulator set.
// 8: two CTAs per SM (half the weight registers), four tokens per set, a three-stage ring; twice as
// many CTAs read each token row.
template <int NI, int NE>
__global__ void __launch_bounds__(256, NE == 16 ? 1 : 2) k_router_logits_regw(const float* __restrict__ w,
                                                               const float* __restrict__ x,
                                                               const int* __restrict__ valid_tokens,
                                                               int num_experts, const float* __restrict__ bias,
                                                               float* __restrict__ logits,
                                                               int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int hidden = NI * 256;
    constexpr int kRrTokens = kRrOutputs / NE;  // tokens per accumulator set
    constexpr int kRrStages = rr_stages(NE);
    extern __shared__ __align__(128) float rr_smem[];
    float* xs = rr_smem;                                             // [stages][4][hidden]
    float* group_tot = xs + kRrStages * kRrStageTokens * hidden;     // [2 stages][sets per stage][32][8]
    __shared__ __align__(8) uint64_t full[kRrStages];
    const int tid = threadIdx.x;
    const int e0 = blockIdx.x * NE;
    const int live = *valid_tokens;
    // this CTA's tokens: a contiguous range, a whole number of stages except at the end of the batch
    const int stages_total = (live + kRrStageTokens - 1) / kRrStageTokens;
    const int stages_per = (stages_total + gridDim.y - 1) / gridDim.y;
    const int stage0 = blockIdx.y * stages_per;
    const int stage1 = min(stages_total, stage0 + stages_per);
    if (stage0 >= stage1) return;
    auto issue = [&](int k) {  // thread 0: fetch the rows of stage k (counted from stage0) into ring slot k % stages
        const int t = (stage0 + k) * kRrStageTokens;
        const uint32_t bytes = (uint32_t)min(kRrStageTokens, live - t) * hidden * 4u;
        mbar_expect_tx(&full[k % kRrStages], bytes);
        tma_bulk_g2s(xs + (size_t)(k % kRrStages) * kRrStageTokens * hidden, x + (size_t)t * hidden, bytes,
                     &full[k % kRrStages]);
    };
    const int n_stages = stage1 - stage0;
    if (tid == 0) {
        for (int i = 0; i < kRrStages; ++i) mbar_init(&full[i], 1);
        fence_mbar_init();
        for (int k = 0; k < min(kRrStages, n_stages); ++k) issue(k);
    }
    float wr[NE][NI];
#pragma unroll
    for (int e = 0; e < NE; ++e)
#pragma unroll
        for (int i = 0; i < NI; ++i) wr[e][i] = __ldg(w + (size_t)(e0 + e) * hidden + i * 256 + tid);
    __syncthreads();  // the barriers are initialised
    if (!__syncthreads_and(mbar_wait_bounded(&full[0], 0u, status))) return;
    constexpr int kPairs = kRrStageTokens / kRrTokens;  // token pairs per ring stage
    for (int k = 0; k < n_stages; ++k) {
        const int slot = k % kRrStages;
        const float* xk = xs + (size_t)slot * kRrStageTokens * hidden;
        const int t_stage = (stage0 + k) * kRrStageTokens;
        // `group_tot` holds the totals of two stages (four pairs): a copy is rewritten two stages after it
        // was written, one block barrier after the warp that reads it has done so
        float* tot_stage = group_tot + (k & 1) * kPairs * kRrOutputs * 8;
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            if (t_stage + p * kRrTokens >= live) break;  // uniform: the batch ended inside this stage
            float acc[kRrOutputs];  // output o = e * tokens + u
#pragma unroll
            for (int o = 0; o < kRrOutputs; ++o) acc[o] = 0.0f;
            // a row past the live tokens was not copied: its sums are formed from stale bytes and never stored
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                float xv[kRrTokens];
#pragma unroll
                for (int u = 0; u < kRrTokens; ++u) xv[u] = xk[(p * kRrTokens + u) * hidden + i * 256 + tid];
#pragma unroll
                for (int e = 0; e < NE; ++e)
#pragma unroll
                    for (int u = 0; u < kRrTokens; ++u)
                        acc[e * kRrTokens + u] = fmaf(wr[e][i], xv[u], acc[e * kRrTokens + u]);
            }
            // this warp is lane group tid / 32 of every output: its 32 trees, then lane o's total of output o
            const float tot = warp_trees32(acc, tid & 31);
            tot_stage[p * kRrOutputs * 8 + (tid & 31) * 8 + (tid >> 5)] = tot;
        }
        // One block barrier per stage: it publishes the group totals, tells thread 0 that every thread has
        // read the stage's rows, and agrees on whether the next stage's rows (requested kRrStages stages
        // ago) have landed.
        bool ok = true;
        if (k + 1 < n_stages)
            ok = mbar_wait_bounded(&full[(k + 1) % kRrStages], (uint32_t)((k + 1) / kRrStages) & 1u, status);
        if (!__syncthreads_and(ok)) return;
        if (tid == 0 && k + kRrStages < n_stages) issue(k + kRrStages);
        // the eight group totals of an output, ascending, from +0; the pairs of a stage go to different warps
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            if (t_stage + p * kRrTokens >= live) break;
            if ((tid >> 5) == ((k * kPairs + p) & 7)) {
                const int o = tid & 31;
                const float* totb = tot_stage + p * kRrOutputs * 8;
                float total = 0.0f;
#pragma unroll
                for (int g = 0; g < 8; ++g) total += totb[o * 8 + g];
                const int e = e0 + o / kRrTokens, t = t_stage + p * kRrTokens + o % kRrTokens;
                if (t < live && e < num_experts)
                    logits[(size_t)t * num_experts + e] = bias ? __fadd_rn(total, bias[e]) : total;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Routing: stable softmax over all experts, k selection passes by
// (probability desc, index asc), renormalise over the selected k in selection
// order (crates/xabe-kernels/src/moe/router.rs:32-76).  One warp per token.
// The softmax denominator keeps the reference device kernel's tree
// (crates/xabe-cuda/src/kernels/moe.rs:1883-1917): 256 lanes, lane v adds
// exp[v], exp[v+256], ...; halving steps 128..1.  Lane l of the warp holds
// experts l, l+32, ..., so steps 128/64/32 are in-register and 16..1 are
// shuffle-downs.  num_experts <= 512.
// grid: (ceil(max_tokens / 8)), block 256.
// ---------------------------------------------------------------------------
template <int kRouteLaneExperts>
__device__ __forceinline__ void route_one_token(const float* __restrict__ row, int num_experts, int top_k,
                                                int lane, int* __restrict__ ids_out,
                                                float* __restrict__ w_out) {
    // the row may have been written by other CTAs of the same launch: read it through L2
    float lg[kRouteLaneExperts];
    float mx = __ldcg(row);
#pragma unroll
    for (int i = 0; i < kRouteLaneExperts; ++i) {
        int e = lane + 32 * i;
        lg[i] = e < num_experts ? __ldcg(row + e) : 0.0f;
        if (e < num_experts) mx = fmaxf(mx, lg[i]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float p[kRouteLaneExperts];
#pragma unroll
    for (int i = 0; i < kRouteLaneExperts; ++i) {
        int e = lane + 32 * i;
        p[i] = e < num_experts ? expf(lg[i] - mx) : 0.0f;
    }
    // lane v of 256: v = lane + 32*i (i < 8) holds p[i] + p[i + 8]
    float v8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v8[i] = kRouteLaneExperts > 8 ? p[i] + p[(i + 8) % kRouteLaneExperts] : p[i];
#pragma unroll
    for (int i = 0; i < 4; ++i) v8[i] += v8[i + 4];  // step 128
    v8[0] += v8[2];                                  // step 64
    v8[1] += v8[3];
    float s = v8[0] + v8[1];                         // step 32
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    float sum_exp = __shfl_sync(0xffffffffu, s, 0);
    // Selection keys: a probability is a non-negative float, so its bit pattern orders like the value;
    // key 0 marks "not selectable" (already taken, past the last expert, or not a number).
    unsigned key[kRouteLaneExperts];
#pragma unroll
    for (int i = 0; i < kRouteLaneExperts; ++i) {
        int e = lane + 32 * i;
        float pv = e < num_experts ? __fdiv_rn(p[i], sum_exp) : -1.0f;
        key[i] = pv >= 0.0f ? __float_as_uint(pv) + 1u : 0u;
    }
    float sel_sum = 0.0f;
    float sel[16];
    for (int j = 0; j < top_k; ++j) {
        // this lane's best (largest key, lowest expert on a tie), then two warp reductions: the
        // largest key, and the lowest expert index among the lanes that hold it
        unsigned bk = 0u;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kRouteLaneExperts; ++i)
            if (key[i] > bk) { bk = key[i]; be = lane + 32 * i; }
        const unsigned mk = __reduce_max_sync(0xffffffffu, bk);
        const int cand = (bk == mk && mk != 0u) ? be : 0x7fffffff;
        const int bi_raw = (int)__reduce_min_sync(0xffffffffu, (unsigned)cand);
        const int bi = mk != 0u ? bi_raw : -1;
        const float bv = mk != 0u ? __uint_as_float(mk - 1u) : -1.0f;
#pragma unroll
        for (int i = 0; i < kRouteLaneExperts; ++i)
            if (bi >= 0 && lane + 32 * i == bi) key[i] = 0u;
        if (lane == 0) ids_out[j] = bi;
        if (j < 16) sel[j] = bv;
        sel_sum += bv;  // selection order, as router.rs:62
    }
    if (lane == 0) {
        for (int j = 0; j < top_k; ++j)
            w_out[j] = sel_sum > 0.0f ? __fdiv_rn(sel[j], sel_sum) : __fdiv_rn(1.0f, (float)top_k);
    }
}

__global__ void __launch_bounds__(256) k_route(const float* __restrict__ logits,
                                               const int* __restrict__ valid_tokens, int num_experts,
                                               int top_k, int* __restrict__ topk_ids,
                                               float* __restrict__ topk_weights) {
    pdl_launch_dependents();
    pdl_wait();
    int lane = threadIdx.x & 31;
    int token = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (token >= *valid_tokens) return;
    if (num_experts <= 256)
        route_one_token<8>(logits + (size_t)token * num_experts, num_experts, top_k, lane,
                           topk_ids + (size_t)token * top_k, topk_weights + (size_t)token * top_k);
    else
        route_one_token<16>(logits + (size_t)token * num_experts, num_experts, top_k, lane,
                            topk_ids + (size_t)token * top_k, topk_weights + (size_t)token * top_k);
}

// ---------------------------------------------------------------------------
// Dispatch tables (crates/xabe-kernels/src/moe/dispatch.rs:60-131).  Three
// passes over fixed-size chunks of the flat (token, k) list, no float and no
// order-dependent atomics: (1) per-chunk expert histograms + sentinel fill of
// the whole capacity, (2) one block turns them into padded exclusive offsets,
// expert_ids and num_tokens_post_pad, (3) each chunk places its pairs in
// ascending flat order with warp match ranks.  The sentinel is
// valid_tokens * top_k (dispatch.rs:24-26), inactive blocks are -1.
// ---------------------------------------------------------------------------
// Flat pairs per chunk (one warp each): small chunks put more warps to work, large ones keep the
// one-thread-per-expert scan over the chunks short.
__host__ __device__ inline int align_chunk_pairs(uint64_t pairs) { return pairs <= 65536 ? 256 : 1024; }

__global__ void __launch_bounds__(32) k_align_count(const int* __restrict__ topk_ids,
                                                    const int* __restrict__ valid_tokens, int top_k,
                                                    int num_experts, int n_chunks, int chunk, int sorted_capacity,
                                                    int block_capacity, int* __restrict__ chunk_hist,
                                                    int* __restrict__ sorted_token_ids,
                                                    int* __restrict__ expert_ids) {
    extern __shared__ int hist[];
    int c = blockIdx.x, lane = threadIdx.x;
    int numel = *valid_tokens * top_k;
    for (int e = lane; e < num_experts; e += 32) hist[e] = 0;
    __syncwarp();
    int begin = c * chunk;
    for (int i = begin + lane; i < begin + chunk && i < numel; i += 32) {
        int e = topk_ids[i];
        if (e >= 0) atomicAdd(&hist[e], 1);  // a negative id marks a row that holds nothing (expert-parallel receive slots)
    }
    __syncwarp();
    for (int e = lane; e < num_experts; e += 32) chunk_hist[(size_t)c * num_experts + e] = hist[e];
    // sentinel / inactive fill over this chunk's share of the capacity
    int per = (sorted_capacity + n_chunks - 1) / n_chunks;
    for (int i = c * per + lane; i < (c + 1) * per && i < sorted_capacity; i += 32) sorted_token_ids[i] = numel;
    int perb = (block_capacity + n_chunks - 1) / n_chunks;
    for (int i = c * perb + lane; i < (c + 1) * perb && i < block_capacity; i += 32) expert_ids[i] = -1;
}

// One block, one thread per expert (num_experts <= 1024).  chunk_hist[c][e] becomes the number of expert
// e's pairs in the chunks before c; the scatter adds the expert's padded offset itself.
__global__ void k_align_scan(int num_experts, int n_chunks, int block_size, int* __restrict__ chunk_hist,
                             int* __restrict__ expert_offsets, int* __restrict__ expert_counts,
                             int* __restrict__ expert_ids, int* __restrict__ num_tokens_post_pad) {
    __shared__ int warp_sums[33];
    int e = threadIdx.x;
    int total = 0;
    if (e < num_experts) {
        for (int c0 = 0; c0 < n_chunks; c0 += 8) {  // eight loads in flight, then their exclusive prefixes
            int h[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) h[u] = c0 + u < n_chunks ? chunk_hist[(size_t)(c0 + u) * num_experts + e] : 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (c0 + u < n_chunks) chunk_hist[(size_t)(c0 + u) * num_experts + e] = total;
                total += h[u];
            }
        }
        expert_counts[e] = total;
    }
    const int padded = e < num_experts ? (total + block_size - 1) / block_size * block_size : 0;
    int all = 0;
    const int start = block_exclusive_scan(padded, warp_sums, &all);
    if (e < num_experts) {
        expert_offsets[e] = start;
        if (e == 0) {
            expert_offsets[num_experts] = all;
            *num_tokens_post_pad = all;
        }
        for (int b = start / block_size; b < (start + padded) / block_size; ++b) expert_ids[b] = e;
    }
}

__global__ void __launch_bounds__(32) k_align_scatter(const int* __restrict__ topk_ids,
                                                      const int* __restrict__ valid_tokens, int top_k,
                                                      int num_experts, int chunk,
                                                      const int* __restrict__ chunk_hist,
                                                      const int* __restrict__ expert_offsets,
                                                      int* __restrict__ sorted_token_ids) {
    extern __shared__ int cursor[];
    int c = blockIdx.x, lane = threadIdx.x;
    int numel = *valid_tokens * top_k;
    int begin = c * chunk;
    if (begin >= numel) return;
    for (int e = lane; e < num_experts; e += 32)
        cursor[e] = expert_offsets[e] + chunk_hist[(size_t)c * num_experts + e];
    __syncwarp();
    for (int i0 = begin; i0 < begin + chunk && i0 < numel; i0 += 32) {
        int i = i0 + lane;
        int e = i < numel ? topk_ids[i] : -1;
        bool on = e >= 0;
        unsigned active = __ballot_sync(0xffffffffu, on);
        if (on) {
            unsigned same = __match_any_sync(active, e);
            int rank = __popc(same & ((1u << lane) - 1u));
            int pos = cursor[e] + rank;
            sorted_token_ids[pos] = i;
            __syncwarp(active);
            if (rank == 0) cursor[e] += __popc(same);
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------
// Column groups: the unit of work of the streaming expert kernels.  The live
// slots of an expert are contiguous in sorted_token_ids (from its padded
// offset), so they are cut into groups of up to 8 consecutive slots = the 8
// token columns of one n8 tensor-core tile.  One item is 20 ints (80 bytes,
// 16-byte aligned): expert, first slot, columns, pad, 8 flat (token, k) ids,
// 8 routing weights (float bits).
// ---------------------------------------------------------------------------
constexpr int kWorkItemInts = 20;

__device__ __forceinline__ void emit_expert_groups(int e, int count, int start, int base,
                                                   const int* __restrict__ sorted_token_ids,
                                                   const float* __restrict__ topk_weights,
                                                   int* __restrict__ work_items) {
    int groups = (count + 7) >> 3;
    for (int i = 0; i < groups; ++i) {
        int* it = work_items + (size_t)(base + i) * kWorkItemInts;
        int first = start + 8 * i;
        int ncols = min(8, count - 8 * i);
        it[0] = e;
        it[1] = first;
        it[2] = ncols;
        it[3] = 0;
        for (int c = 0; c < 8; ++c) {
            int flat = c < ncols ? sorted_token_ids[first + c] : 0;
            it[4 + c] = flat;
            it[12 + c] = c < ncols ? __float_as_int(topk_weights[flat]) : 0;
        }
    }
}

// General path, after k_align_scatter.  One block, one thread per expert.
__global__ void k_build_work(int num_experts, const int* __restrict__ expert_offsets,
                             const int* __restrict__ expert_counts, const int* __restrict__ sorted_token_ids,
                             const float* __restrict__ topk_weights, int* __restrict__ work_items,
                             int* __restrict__ n_work) {
    extern __shared__ int base_s[];  // [num_experts + 1]
    int e = threadIdx.x;
    if (e < num_experts) base_s[e] = (expert_counts[e] + 7) >> 3;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < num_experts; ++i) {
            int g = base_s[i];
            base_s[i] = run;
            run += g;
        }
        *n_work = run;
    }
    __syncthreads();
    if (e < num_experts)
        emit_expert_groups(e, expert_counts[e], expert_offsets[e], base_s[e], sorted_token_ids, topk_weights,
                           work_items);
}

// ---------------------------------------------------------------------------
// Decode widths (at most 2048 flat pairs): routing, the dispatch tables and
// the column groups in ONE single-CTA launch instead of five.  Same results
// as the general path: warps route tokens; per-warp chunks of the flat list
// are histogrammed, offset and scattered in ascending flat order.
// block 256 (8 warps); dynamic shared memory: (3 * 2048 + 11 * E + 2) ints.
// `logits` NULL = the routing was done by k_route already.
// ---------------------------------------------------------------------------
constexpr int kSmallPairs = 2048;

// The tables and the column groups from a routing decision that is already in topk_ids /
// topk_weights (global memory, written by this block or made visible to it), by a block of NT
// threads.  `sm` is the block's scratch: (3 * kSmallPairs + (NT / 32 + 3) * E + 2) ints.
template <int NT>
__device__ __forceinline__ void dispatch_small_body(
    int* sm, int live, int num_experts, int top_k, int block_size, int sorted_capacity, int block_capacity,
    const int* __restrict__ topk_ids, const float* __restrict__ topk_weights, int* __restrict__ sorted_token_ids,
    int* __restrict__ expert_ids, int* __restrict__ num_tokens_post_pad, int* __restrict__ expert_offsets,
    int* __restrict__ expert_counts, int* __restrict__ work_items, int* __restrict__ n_work) {
    constexpr int NW = NT / 32;
    int* ids_s = sm;                          // [kSmallPairs]
    int* hist = ids_s + kSmallPairs;          // [NW][E] per-warp chunk histograms -> cursors
    int* start_s = hist + NW * num_experts;   // [E + 1] padded exclusive offsets
    int* count_s = start_s + num_experts + 1; // [E] live counts
    int* cstart_s = count_s + num_experts;    // [E] unpadded exclusive offsets
    int* sorted_s = cstart_s + num_experts;   // [kSmallPairs] live flat ids in dispatch order
    float* wts_s = (float*)(sorted_s + kSmallPairs);  // [kSmallPairs] routing weights by flat id
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int numel = live * top_k;
    for (int i = tid; i < NW * num_experts; i += NT) hist[i] = 0;
    for (int i = tid; i < sorted_capacity; i += NT) sorted_token_ids[i] = numel;
    for (int i = tid; i < block_capacity; i += NT) expert_ids[i] = -1;
    for (int i = tid; i < numel; i += NT) {
        ids_s[i] = __ldcg(topk_ids + i);
        wts_s[i] = __ldcg(topk_weights + i);
    }
    __syncthreads();
    // warp w owns flat pairs [w * chunk, (w + 1) * chunk), chunk a multiple of 32
    int chunk = ((numel + NW - 1) / NW + 31) / 32 * 32;
    int begin = warp * chunk, end = min(numel, begin + chunk);
    for (int i = begin + lane; i < end; i += 32) {
        int e = ids_s[i];
        if (e >= 0) atomicAdd(&hist[warp * num_experts + e], 1);  // negative: a row that holds nothing
    }
    __syncthreads();
    for (int e = tid; e < num_experts; e += NT) {
        int total = 0;
        for (int w = 0; w < NW; ++w) {
            int h = hist[w * num_experts + e];
            hist[w * num_experts + e] = total;
            total += h;
        }
        count_s[e] = total;
        start_s[e] = (total + block_size - 1) / block_size * block_size;
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the padded counts: each lane owns a contiguous run of experts
        int per = (num_experts + 31) / 32;
        int lo = lane * per, hi = min(num_experts, lo + per);
        int sum = 0, csum = 0;
        for (int e = lo; e < hi; ++e) {
            sum += start_s[e];
            csum += count_s[e];
        }
        int incl = sum, cincl = csum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, off);
            int cv = __shfl_up_sync(0xffffffffu, cincl, off);
            if (lane >= off) {
                incl += v;
                cincl += cv;
            }
        }
        int run = incl - sum, crun = cincl - csum;
        for (int e = lo; e < hi; ++e) {
            int p = start_s[e];
            start_s[e] = run;
            run += p;
            cstart_s[e] = crun;
            crun += count_s[e];
        }
        if (lane == 31) {
            start_s[num_experts] = incl;
            *num_tokens_post_pad = incl;
        }
    }
    __syncthreads();
    for (int e = tid; e < num_experts; e += NT) {
        int s0 = start_s[e], s1 = start_s[e + 1];
        expert_offsets[e] = s0;
        expert_counts[e] = count_s[e];
        for (int b = s0 / block_size; b < s1 / block_size; ++b) expert_ids[b] = e;
        for (int w = 0; w < NW; ++w) hist[w * num_experts + e] += s0;
    }
    if (tid == 0) expert_offsets[num_experts] = start_s[num_experts];
    __syncthreads();
    int* cursor = hist + warp * num_experts;
    for (int i0 = begin; i0 < end; i0 += 32) {
        int i = i0 + lane;
        int e = i < end ? ids_s[i] : -1;
        bool on = e >= 0;
        unsigned active = __ballot_sync(0xffffffffu, on);
        if (on) {
            unsigned same = __match_any_sync(active, e);
            int rank = __popc(same & ((1u << lane) - 1u));
            int pos = cursor[e] + rank;
            sorted_token_ids[pos] = i;
            sorted_s[cstart_s[e] + (pos - start_s[e])] = i;
            __syncwarp(active);
            if (rank == 0) cursor[e] += __popc(same);
        }
        __syncwarp();
    }
    __syncthreads();
    // column groups: reuse hist[0..E) as the group base
    for (int e = tid; e < num_experts; e += NT) hist[e] = (count_s[e] + 7) >> 3;
    __syncthreads();
    if (warp == 0) {
        int per = (num_experts + 31) / 32;
        int lo = lane * per, hi = min(num_experts, lo + per);
        int sum = 0;
        for (int e = lo; e < hi; ++e) sum += hist[e];
        int incl = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        int run = incl - sum;
        for (int e = lo; e < hi; ++e) {
            int gcount = hist[e];
            hist[e] = run;
            run += gcount;
        }
        if (lane == 31) *n_work = incl;
    }
    __syncthreads();
    for (int e = tid; e < num_experts; e += NT) {
        int count = count_s[e], groups = (count + 7) >> 3;
        for (int i = 0; i < groups; ++i) {
            int* it = work_items + (size_t)(hist[e] + i) * kWorkItemInts;
            int ncols = min(8, count - 8 * i);
            it[0] = e;
            it[1] = start_s[e] + 8 * i;
            it[2] = ncols;
            it[3] = 0;
            for (int c = 0; c < 8; ++c) {
                int flat = c < ncols ? sorted_s[cstart_s[e] + 8 * i + c] : 0;
                it[4 + c] = flat;
                it[12 + c] = c < ncols ? __float_as_int(wts_s[flat]) : 0;
            }
        }
    }
}

constexpr int kTinyPairs = 128;  // flat pairs dispatch_tiny_warp holds: handles of up to 16 tokens at top-8

// The dispatch tables and column groups for at most 128 flat (token, k) pairs, by ONE warp (lane i
// holds pairs i, i + 32, i + 64, i + 96): no block barrier on the way.  Same tables as dispatch_small_body.  The
// caller has filled sorted_token_ids with the sentinel and expert_ids with -1, zeroed cnt_s, and
// synchronised the block.  cnt_s / start_s / gbase_s: shared scratch of num_experts ints each.
__device__ __forceinline__ void dispatch_tiny_warp(
    int lane, int numel, int num_experts, int block_size, int* cnt_s, int* start_s, int* gbase_s,
    const int* __restrict__ topk_ids, const float* __restrict__ topk_weights, int* __restrict__ sorted_token_ids,
    int* __restrict__ expert_ids, int* __restrict__ num_tokens_post_pad, int* __restrict__ expert_offsets,
    int* __restrict__ expert_counts, int* __restrict__ work_items, int* __restrict__ n_work) {
    const unsigned lt = (1u << lane) - 1u;
    constexpr int NB = kTinyPairs / 32;
    int e[NB], rank[NB];
    float wt[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const int i = lane + 32 * b;
        e[b] = i < numel ? __ldcg(topk_ids + i) : -1;
        wt[b] = i < numel ? __ldcg(topk_weights + i) : 0.0f;
        rank[b] = 0;
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {  // pairs in ascending flat order: batch 0 first, lanes ascending inside a batch
        if (32 * b >= numel) break;  // uniform over the warp
        const bool on = e[b] >= 0;  // a negative id marks a row that holds nothing
        const int base = on ? cnt_s[e[b]] : 0;
        const unsigned active = __ballot_sync(0xffffffffu, on);
        unsigned same = 0u;
        if (on) {
            same = __match_any_sync(active, e[b]);
            rank[b] = base + __popc(same & lt);
        }
        __syncwarp();
        if (on && (same & lt) == 0u) cnt_s[e[b]] = base + __popc(same);
        __syncwarp();
    }
    // padded offsets, live counts and column-group bases: each lane owns a contiguous run of experts
    const int per = (num_experts + 31) / 32;
    const int lo = lane * per, hi = min(num_experts, lo + per);
    int sum_pad = 0, sum_grp = 0;
    for (int x = lo; x < hi; ++x) {
        const int c = cnt_s[x];
        sum_pad += (c + block_size - 1) / block_size * block_size;
        sum_grp += (c + 7) >> 3;
    }
    int incl_pad = sum_pad, incl_grp = sum_grp;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, incl_pad, off);
        const int g = __shfl_up_sync(0xffffffffu, incl_grp, off);
        if (lane >= off) {
            incl_pad += a;
            incl_grp += g;
        }
    }
    int run_pad = incl_pad - sum_pad, run_grp = incl_grp - sum_grp;
    for (int x = lo; x < hi; ++x) {
        const int c = cnt_s[x];
        const int pad = (c + block_size - 1) / block_size * block_size;
        start_s[x] = run_pad;
        gbase_s[x] = run_grp;
        expert_offsets[x] = run_pad;
        expert_counts[x] = c;
        for (int blk = run_pad / block_size; blk < (run_pad + pad) / block_size; ++blk) expert_ids[blk] = x;
        run_pad += pad;
        run_grp += (c + 7) >> 3;
    }
    if (lane == 31) {
        expert_offsets[num_experts] = incl_pad;
        *num_tokens_post_pad = incl_pad;
        *n_work = incl_grp;
    }
    __syncwarp();
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        if (e[b] < 0) continue;
        const int flat = lane + 32 * b;
        const int first = start_s[e[b]], gi = rank[b] >> 3, c = rank[b] & 7;
        sorted_token_ids[first + rank[b]] = flat;
        int* it = work_items + (size_t)(gbase_s[e[b]] + gi) * kWorkItemInts;
        it[4 + c] = flat;
        it[12 + c] = __float_as_int(wt[b]);
        if (c == 0) {  // the group's first column also writes its header and clears the unused columns
            const int ncols = min(8, cnt_s[e[b]] - 8 * gi);
            it[0] = e[b];
            it[1] = first + 8 * gi;
            it[2] = ncols;
            it[3] = 0;
            for (int c2 = ncols; c2 < 8; ++c2) {
                it[4 + c2] = 0;
                it[12 + c2] = 0;
            }
        }
    }
}

__host__ __device__ inline size_t dispatch_small_smem(int num_experts, int threads) {
    return (size_t)(3 * kSmallPairs + (threads / 32 + 3) * num_experts + 2) * sizeof(int);
}

__global__ void __launch_bounds__(256) k_route_dispatch_small(
    const float* __restrict__ logits, const int* __restrict__ valid_tokens, int num_experts, int top_k,
    int block_size, int sorted_capacity, int block_capacity, int* __restrict__ topk_ids,
    float* __restrict__ topk_weights, int* __restrict__ sorted_token_ids, int* __restrict__ expert_ids,
    int* __restrict__ num_tokens_post_pad, int* __restrict__ expert_offsets, int* __restrict__ expert_counts,
    int* __restrict__ work_items, int* __restrict__ n_work) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int sm[];
    int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int live = *valid_tokens;
    if (logits) {  // at most one token per warp is routed here; wider steps route in k_route first
        for (int t = warp; t < live; t += 8) {
            if (num_experts <= 256)
                route_one_token<8>(logits + (size_t)t * num_experts, num_experts, top_k, lane,
                                   topk_ids + (size_t)t * top_k, topk_weights + (size_t)t * top_k);
            else
                route_one_token<16>(logits + (size_t)t * num_experts, num_experts, top_k, lane,
                                    topk_ids + (size_t)t * top_k, topk_weights + (size_t)t * top_k);
        }
    }
    __threadfence();  // the ids were written by this block; the body reads them back through L2
    const int numel = live * top_k;
    if (numel <= kTinyPairs) {
        // A handful of pairs: the block clears the tables, then ONE warp builds them with no further block
        // barrier (the block-wide body spends its time in ten barriers over 256-entry arrays).
        int* cnt_s = sm;
        int* start_s = cnt_s + num_experts;
        int* gbase_s = start_s + num_experts;
        for (int i = tid; i < num_experts; i += 256) cnt_s[i] = 0;
        for (int i = tid; i < sorted_capacity; i += 256) sorted_token_ids[i] = numel;
        for (int i = tid; i < block_capacity; i += 256) expert_ids[i] = -1;
        __syncthreads();
        if (warp == 0)
            dispatch_tiny_warp(lane, numel, num_experts, block_size, cnt_s, start_s, gbase_s, topk_ids, topk_weights,
                               sorted_token_ids, expert_ids, num_tokens_post_pad, expert_offsets, expert_counts,
                               work_items, n_work);
        return;
    }
    __syncthreads();
    dispatch_small_body<256>(sm, live, num_experts, top_k, block_size, sorted_capacity, block_capacity, topk_ids,
                             topk_weights, sorted_token_ids, expert_ids, num_tokens_post_pad, expert_offsets,
                             expert_counts, work_items, n_work);
}

// ---------------------------------------------------------------------------
// moe_reduce (crates/xabe-cuda/src/kernels/moe.rs:4049-4065):
// out[t][h] = sum over ascending k of partial[t*K + k][h].
// grid: (max_tokens, ceil(hidden / 256)), block 256.
// ---------------------------------------------------------------------------
__global__ void k_reduce(const float* __restrict__ partial, const int* __restrict__ valid_tokens, int top_k,
                         int hidden, float* __restrict__ out) {
    int t = blockIdx.x;
    if (t >= *valid_tokens) return;
    int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= hidden) return;
    size_t pbase = (size_t)t * top_k * hidden;
    float r = 0.0f;
    for (int k = 0; k < top_k; ++k) r += partial[pbase + (size_t)k * hidden + j];
    out[(size_t)t * hidden + j] = r;
}

// ---------------------------------------------------------------------------
// moe_block_gate_and_combine (crates/xabe-engine/src/block/moe.rs:424-483):
// g = 1 / (1 + expf(-dot(w_gate, normed[t]))) with the dot product on 256
// lanes at stride 256 and block_reduce_sum; routed = ascending-k sum of
// partial; ffn_out = routed + shexp * g (routed on the left); l_out =
// ffn_out + residual (the pre-norm input).
// grid: (max_tokens, 1 or hidden / 256), block 256.  VEC (grid.y == 1, hidden a multiple of 4, every
// row pointer 16-byte aligned): a thread owns four neighbouring columns and moves them 16 bytes at a
// time; each column's sums are the same operations in the same order.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float4 f4_add(float4 a, float4 b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
template <bool VEC>
__global__ void __launch_bounds__(256) k_gate_and_combine(
    const float* __restrict__ w, const float* __restrict__ normed, const float* __restrict__ partial,
    const float* __restrict__ shexp, const float* __restrict__ residual, const int* __restrict__ valid_tokens,
    int top_k, int hidden, float* __restrict__ gate, float* __restrict__ routed, float* __restrict__ ffn_out,
    float* __restrict__ l_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    int t = blockIdx.x;
    if (t >= *valid_tokens) return;
    size_t base = (size_t)t * hidden;
    const float* xs = normed + base;
    float s = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += 256) s = fmaf(w[j], xs[j], s);
    s = block_reduce_sum_pinned(s, scratch);
    float g = __fdiv_rn(1.0f, 1.0f + expf(-s));
    if (threadIdx.x == 0 && blockIdx.y == 0) gate[t] = g;
    size_t pbase = (size_t)t * top_k * hidden;
    if (VEC && top_k == 8) {
        const float4* p4 = (const float4*)(partial + pbase);
        const float4* sh4 = (const float4*)(shexp + base);
        const float4* res4 = (const float4*)(residual + base);
        const int h4 = hidden >> 2;
        for (int j = threadIdx.x; j < h4; j += 256) {
            float4 pv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) pv[k] = p4[(size_t)k * h4 + j];
            const float4 sh = sh4[j], res = res4[j];
            float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 8; ++k) r = f4_add(r, pv[k]);
            const float4 v = make_float4(fmaf(sh.x, g, r.x), fmaf(sh.y, g, r.y), fmaf(sh.z, g, r.z), fmaf(sh.w, g, r.w));
            ((float4*)(routed + base))[j] = r;
            ((float4*)(ffn_out + base))[j] = v;
            ((float4*)(l_out + base))[j] = f4_add(v, res);
        }
        return;
    }
    // gridDim.y blocks share a token's columns: 1 at prefill widths (the gate, a block-wide reduction,
    // is then computed once per token), hidden / 256 at decode widths (more blocks than SMs)
    for (int j = blockIdx.y * 256 + threadIdx.x; j < hidden; j += 256 * gridDim.y) {
        float r = 0.0f;
        if (top_k == 8) {  // the shipped geometry: all eight loads in flight, then the same ascending-k sum
            float pv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) pv[k] = partial[pbase + (size_t)k * hidden + j];
#pragma unroll
            for (int k = 0; k < 8; ++k) r += pv[k];
        } else {
            for (int k = 0; k < top_k; ++k) r += partial[pbase + (size_t)k * hidden + j];
        }
        float v = fmaf(shexp[base + j], g, r);
        routed[base + j] = r;
        ffn_out[base + j] = v;
        l_out[base + j] = v + residual[base + j];
    }
}

// ---------------------------------------------------------------------------
// Expert parallelism, sender side.  (No counterpart in the reference, whose
// multi-GPU model is one replica per device.)
// k_ep_pack: row i of the send buffer is the f16 activation row of the token of
// flat (token, k) pair order[i]; also the pair's expert id local to its owner
// rank and the inverse map flat -> i.  grid: pairs, block 256.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_ep_pack(const long long* __restrict__ order, const __half* __restrict__ normed_h,
                                                 const int* __restrict__ topk_ids, int top_k, int hidden,
                                                 int experts_per_rank, __half* __restrict__ send_rows,
                                                 int* __restrict__ send_local_expert, int* __restrict__ inverse) {
    const int i = blockIdx.x;
    const int flat = (int)order[i];
    const uint4* src = (const uint4*)(normed_h + (size_t)(flat / top_k) * hidden);
    uint4* dst = (uint4*)(send_rows + (size_t)i * hidden);
    for (int u = threadIdx.x; u < hidden / 8; u += 256) dst[u] = __ldg(src + u);
    if (threadIdx.x == 0) {
        send_local_expert[i] = topk_ids[flat] % experts_per_rank;
        inverse[flat] = i;
    }
}

// k_ep_plan + k_ep_pack_sorted: the same send buffer straight from the dispatch
// tables the handle already holds.  Pairs sorted by expert are also grouped by
// owner rank (a rank owns a contiguous range of experts), so the send order is
// the dispatch order with the padding slots dropped.
// k_ep_plan: one block, one thread per expert: compact[e] = live pairs of the
// experts before e; send_counts[r] = live pairs of rank r's experts.
__global__ void k_ep_plan(int num_experts, int experts_per_rank, const int* __restrict__ expert_counts,
                          int* __restrict__ compact, int* __restrict__ send_counts) {
    extern __shared__ int cnt_s[];  // [num_experts + 1]
    int e = threadIdx.x;
    if (e < num_experts) cnt_s[e] = expert_counts[e];
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < num_experts; ++i) {
            int c = cnt_s[i];
            cnt_s[i] = run;
            run += c;
        }
        cnt_s[num_experts] = run;
    }
    __syncthreads();
    if (e <= num_experts) compact[e] = cnt_s[e];
    int world = num_experts / experts_per_rank;
    if (e < world) send_counts[e] = cnt_s[(e + 1) * experts_per_rank] - cnt_s[e * experts_per_rank];
}
// grid: sorted_capacity slots, block 256.
__global__ void __launch_bounds__(256) k_ep_pack_sorted(
    const int* __restrict__ sorted_token_ids, const int* __restrict__ expert_ids,
    const int* __restrict__ expert_offsets, const int* __restrict__ compact,
    const int* __restrict__ num_tokens_post_pad, const int* __restrict__ valid_tokens,
    const __half* __restrict__ normed_h, int top_k, int hidden, int block_size, int experts_per_rank,
    __half* __restrict__ send_rows, int* __restrict__ send_local_expert, int* __restrict__ inverse) {
    const int s = blockIdx.x;
    if (s >= *num_tokens_post_pad) return;
    const int flat = sorted_token_ids[s];
    if (flat >= *valid_tokens * top_k) return;  // padding slot
    const int e = expert_ids[s / block_size];
    const int i = compact[e] + (s - expert_offsets[e]);
    const uint4* src = (const uint4*)(normed_h + (size_t)(flat / top_k) * hidden);
    uint4* dst = (uint4*)(send_rows + (size_t)i * hidden);
    for (int u = threadIdx.x; u < hidden / 8; u += 256) dst[u] = __ldg(src + u);
    if (threadIdx.x == 0) {
        send_local_expert[i] = e % experts_per_rank;
        inverse[flat] = i;
    }
}

// k_ep_combine: k_gate_and_combine with the routed term read through the
// inverse map from the rows that came back from the owner ranks (unweighted):
// routed = sum over ascending k of weight[t][k] * back[inverse[t*K + k]], each
// product rounded to fp32 before it is added -- the value the one-GPU path
// stores in `partial` and sums, so the result is bit-identical to it.
template <bool VEC>
__global__ void __launch_bounds__(256) k_ep_combine(
    const float* __restrict__ w, const float* __restrict__ normed, const float* __restrict__ back,
    const int* __restrict__ inverse, const float* __restrict__ topk_weights, const float* __restrict__ shexp,
    const float* __restrict__ residual, const int* __restrict__ valid_tokens, int top_k, int hidden,
    float* __restrict__ gate, float* __restrict__ routed, float* __restrict__ ffn_out, float* __restrict__ l_out) {
    __shared__ float scratch[32];
    int t = blockIdx.x;
    if (t >= *valid_tokens) return;
    size_t base = (size_t)t * hidden;
    const float* xs = normed + base;
    float s = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += 256) s = fmaf(w[j], xs[j], s);
    s = block_reduce_sum_pinned(s, scratch);
    float g = __fdiv_rn(1.0f, 1.0f + expf(-s));
    if (threadIdx.x == 0 && blockIdx.y == 0) gate[t] = g;
    if (top_k == 8) {  // the shipped geometry: row addresses and weights once per token, eight rows in flight
        int src[8];
        float pw[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            src[k] = inverse[t * 8 + k];
            pw[k] = topk_weights[t * 8 + k];
        }
        if (VEC) {  // as in k_gate_and_combine: four neighbouring columns per thread
            const float4* sh4 = (const float4*)(shexp + base);
            const float4* res4 = (const float4*)(residual + base);
            const int h4 = hidden >> 2;
            for (int j = threadIdx.x; j < h4; j += 256) {
                float4 pv[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) pv[k] = ((const float4*)(back + (size_t)src[k] * hidden))[j];
                const float4 sh = sh4[j], res = res4[j];
                float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    r = make_float4(__fadd_rn(r.x, __fmul_rn(pw[k], pv[k].x)), __fadd_rn(r.y, __fmul_rn(pw[k], pv[k].y)),
                                    __fadd_rn(r.z, __fmul_rn(pw[k], pv[k].z)), __fadd_rn(r.w, __fmul_rn(pw[k], pv[k].w)));
                const float4 v =
                    make_float4(fmaf(sh.x, g, r.x), fmaf(sh.y, g, r.y), fmaf(sh.z, g, r.z), fmaf(sh.w, g, r.w));
                ((float4*)(routed + base))[j] = r;
                ((float4*)(ffn_out + base))[j] = v;
                ((float4*)(l_out + base))[j] = f4_add(v, res);
            }
            return;
        }
        for (int j = blockIdx.y * 256 + threadIdx.x; j < hidden; j += 256 * gridDim.y) {
            float pv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) pv[k] = back[(size_t)src[k] * hidden + j];
            float r = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) r = __fadd_rn(r, __fmul_rn(pw[k], pv[k]));
            float v = fmaf(shexp[base + j], g, r);
            routed[base + j] = r;
            ffn_out[base + j] = v;
            l_out[base + j] = v + residual[base + j];
        }
        return;
    }
    for (int j = blockIdx.y * 256 + threadIdx.x; j < hidden; j += 256 * gridDim.y) {
        float r = 0.0f;
        for (int k = 0; k < top_k; ++k) {
            const int flat = t * top_k + k;
            r = __fadd_rn(r, __fmul_rn(topk_weights[flat], back[(size_t)inverse[flat] * hidden + j]));
        }
        float v = fmaf(shexp[base + j], g, r);
        routed[base + j] = r;
        ffn_out[base + j] = v;
        l_out[base + j] = v + residual[base + j];
    }
}

// Dense FFN epilogue (crates/xabe-engine/src/block/dense_ffn.rs:234-251):
// l_out = ffn_out + residual for the live rows.
__global__ void k_add_residual(const float* __restrict__ ffn, const float* __restrict__ residual,
                               const int* __restrict__ valid_tokens, int hidden, float* __restrict__ l_out) {
    int t = blockIdx.x;
    if (t >= *valid_tokens) return;
    size_t base = (size_t)t * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) l_out[base + j] = ffn[base + j] + residual[base + j];
}

// bf16 rows -> fp32 rows for the live tokens: the widening is a 16-bit shift,
// exact (crates/xabe-kernels/src/quant.rs:1350-1358 pins the same for tensors).
__global__ void k_rows_bf16_to_f32(const unsigned short* __restrict__ x, float* __restrict__ out,
                                   const int* __restrict__ valid_tokens, int width) {
    int row = blockIdx.x;
    if (row >= *valid_tokens) return;
    size_t base = (size_t)row * width;
    if ((width & 7) == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {  // eight elements per thread and pass
        const uint4* src = (const uint4*)(x + base);
        float4* dst = (float4*)(out + base);
        for (int u = threadIdx.x; u < width / 8; u += blockDim.x) {
            const uint4 v = __ldg(src + u);
            dst[2 * u] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u),
                                     __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
            dst[2 * u + 1] = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xFFFF0000u),
                                         __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xFFFF0000u));
        }
        return;
    }
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        out[base + j] = __uint_as_float((unsigned)x[base + j] << 16);
}

// Calibration for the benchmark: a pure 128-bit coalesced streaming read of a
// byte range, no arithmetic beyond the XOR that keeps the loads alive -- what
// the card streams, as opposed to what a kernel achieves on the same bytes
// (the reference prints the same row, docs/BENCHMARKS.md:448-452).
__global__ void __launch_bounds__(256) k_stream_read(const uint4* __restrict__ src, size_t n_units,
                                                     unsigned* __restrict__ sink) {
    uint4 acc = make_uint4(0, 0, 0, 0);
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_units; i += stride) {
        uint4 v = __ldg(src + i);
        acc.x ^= v.x; acc.y ^= v.y; acc.z ^= v.z; acc.w ^= v.w;
    }
    unsigned r = acc.x ^ acc.y ^ acc.z ^ acc.w;
    if (r == 0x9E3779B9u) *sink = r;  // practically never: the result is not needed
}

// ---------------------------------------------------------------------------
// Standalone dequantisation, bit-identical to the scalar reference because
// reconstruction is multiplications only: Q6_K (d * sc) * q
// (crates/xabe-kernels/src/quant.rs:171-202), Q8_0 q * d (quant.rs:62-69).
// One thread per element.
// ---------------------------------------------------------------------------
__global__ void k_dequant_q6k(const uint8_t* __restrict__ bytes, size_t n_elems, float* __restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    const uint8_t* blk = bytes + (i >> 8) * kQ6KBlockBytes;
    int r = (int)(i & 255);
    int half = r >> 7, grp = (r & 127) >> 5, l = r & 31;
    uint8_t qb = blk[half * 64 + (grp & 1) * 32 + l];
    int nib = grp < 2 ? (qb & 0xF) : (qb >> 4);
    int hi = (blk[128 + half * 32 + l] >> (2 * grp)) & 3;
    int q = (nib | (hi << 4)) - 32;
    int sc = (int)(int8_t)blk[192 + half * 8 + 2 * grp + (l >> 4)];
    float d = __half2float(__ushort_as_half((unsigned short)(blk[208] | (blk[209] << 8))));
    out[i] = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}

__global__ void k_dequant_q8_0(const uint8_t* __restrict__ bytes, size_t n_elems, float* __restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    const uint8_t* blk = bytes + (i >> 5) * kQ8BlockBytes;
    float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
    int q = (int)(int8_t)blk[2 + (i & 31)];
    out[i] = __fmul_rn((float)q, d);
}

}  // namespace xabe
