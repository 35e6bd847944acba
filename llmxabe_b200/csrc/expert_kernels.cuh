// Decode-shaped expert projections: bandwidth-bound streaming of raw GGUF
// Q6_K / Q8_0 rows with in-register dequantisation.
//
// Data movement: each CTA pulls one contiguous tile of weight rows into shared
// memory with 1-D TMA bulk copies (the 16-byte-aligned superset of the tile;
// rows of 210-byte superblocks keep their odd phase in shared memory) and
// several CTAs per SM keep enough bytes in flight to cover HBM latency.
//
// Arithmetic: the quantised CODES are exact small integers, so they are the
// f16 A operand of m16n8k16 tensor-core tiles unchanged; one k16 step covers
// exactly one scale group (16 Q6_K codes, half a Q8_0 block), so the fp32
// scale (d * sc) multiplies the step's fp32 result on its way into the
// accumulator.  Weights therefore enter the sum exactly as the reference's
// (d * sc) * q does; the only rounding beyond fp32 is the activation's
// conversion to f16.  Columns of the tile are tokens: a token's result does
// not depend on which other tokens share the tile, which is what makes a
// sequence's output bit-identical batched or alone.
//
// Work decomposition: blockIdx.y < routed_blocks walks the dispatch table
// (one block_size-wide bucket of one expert); blockIdx.y >= routed_blocks are
// the shared expert's token tiles, riding the same launch.
#pragma once

#include "common.cuh"

namespace xabe {

constexpr int kExpertThreads = 128;  // 4 warps
constexpr int kMaxNB = 8;            // up to 64 token columns per dispatch bucket

struct ExpertLaunch {
    // routed experts (stacks of num_experts matrices); null when absent
    const uint8_t* r_a;  // gate (or down)
    const uint8_t* r_b;  // up
    // shared expert / dense matrices; null when absent
    const uint8_t* s_a;
    const uint8_t* s_b;
    int rows;       // output rows per matrix (intermediate for gate/up, hidden for down)
    int k;          // contraction length
    int routed_blocks;
    int block_size;
    int top_k;
    int max_tokens;
    const int* sorted_token_ids;
    const int* expert_ids;
    const int* valid_tokens;
    const float* topk_weights;
    // B operands (f16 rows of length k)
    const __half* x_routed;  // gate/up: normed_h [token]; down: inter_h [slot]
    const __half* x_shared;  // gate/up: normed_h [token]; down: inter_shared_h [token]
    // outputs
    __half* inter_routed;  // [slot][rows]    (gate/up)
    __half* inter_shared;  // [token][rows]   (gate/up)
    float* partial;        // [flat][rows]    (down, routed) = weight * value
    float* const* partial_rows;  // optional: where row `flat` goes instead (a peer's buffer under expert parallelism; NULL entries are skipped)
    float* shexp;          // [token][rows]   (down, shared)
    int* status;
};

// Unpacks the four 4-code words (groups j = 0..3) that one (ql word A, ql word
// B, qh word) triple holds.  Element map of crates/xabe-kernels/src/quant.rs:175-198:
// group j takes nibbles from ql word (j & 1), low nibble for j < 2, high
// otherwise, and bit pair j of each qh byte.
__device__ __forceinline__ uint32_t q6k_codes(int j, uint32_t ql0, uint32_t ql1, uint32_t qh) {
    uint32_t ql = (j & 1) ? ql1 : ql0;
    uint32_t lo = (j < 2 ? ql : (ql >> 4)) & 0x0F0F0F0Fu;
    uint32_t hi = ((qh >> (2 * j)) & 0x03030303u) << 4;
    return lo | hi;
}

// One warp's share of the contraction for one m16 tile whose fragment rows g
// and g+8 start at `pa` and `pb` in shared memory.  Spans (256 elements) from
// span0 in steps of span_step.  xcol[nb] is the f16 activation row of the
// token in column nb*8 + g.  acc[nb] follows the m16n8 accumulator layout.
template <int QUANT, int NB>
__device__ __forceinline__ void mma_span_loop(const uint8_t* pa, const uint8_t* pb, int span0, int span_step,
                                              int n_spans, const __half* const (&xcol)[NB], int t,
                                              float (&acc)[NB][4]) {
    const uint32_t bias32 = 0x64206420u;    // half2(1056, 1056): 1024 + 32
    const uint32_t bias128 = 0x64806480u;   // half2(1152, 1152): 1024 + 128
    for (int s = span0; s < n_spans; s += span_step) {
        if (QUANT == QUANT_Q6K) {
            const uint8_t* sa = pa + s * kQ6KBlockBytes;
            const uint8_t* sb = pb + s * kQ6KBlockBytes;
            float da = f16_at(sa + 208), db = f16_at(sb + 208);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    int off = half * 64 + 16 * c + 4 * t;
                    uint32_t a_ql0 = ld32_al2(sa + off), a_ql1 = ld32_al2(sa + off + 32);
                    uint32_t a_qh = ld32_al2(sa + 128 + half * 32 + 16 * c + 4 * t);
                    uint32_t b_ql0 = ld32_al2(sb + off), b_ql1 = ld32_al2(sb + off + 32);
                    uint32_t b_qh = ld32_al2(sb + 128 + half * 32 + 16 * c + 4 * t);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // scale index of quant.rs:183,195-198: half*8 + 2*j + (l / 16), l / 16 == c
                        float dsa = da * (float)(int)(int8_t)sa[192 + half * 8 + 2 * j + c];
                        float dsb = db * (float)(int)(int8_t)sb[192 + half * 8 + 2 * j + c];
                        uint32_t ra = q6k_codes(j, a_ql0, a_ql1, a_qh);
                        uint32_t rb = q6k_codes(j, b_ql0, b_ql1, b_qh);
                        uint32_t a[4];
                        a[0] = bytes01_to_h2(ra, bias32);
                        a[1] = bytes01_to_h2(rb, bias32);
                        a[2] = bytes23_to_h2(ra, bias32);
                        a[3] = bytes23_to_h2(rb, bias32);
                        int kk = s * 256 + half * 128 + j * 32 + 16 * c + 4 * t;
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            uint2 b = __ldg((const uint2*)(xcol[nb] + kk));
                            float d[4];
                            mma_f16_16816(d, a, b.x, b.y);
                            acc[nb][0] = fmaf(dsa, d[0], acc[nb][0]);
                            acc[nb][1] = fmaf(dsa, d[1], acc[nb][1]);
                            acc[nb][2] = fmaf(dsb, d[2], acc[nb][2]);
                            acc[nb][3] = fmaf(dsb, d[3], acc[nb][3]);
                        }
                    }
                }
            }
        } else {
            const uint8_t* sa = pa + s * (8 * kQ8BlockBytes);
            const uint8_t* sb = pb + s * (8 * kQ8BlockBytes);
#pragma unroll 2
            for (int blk = 0; blk < 8; ++blk) {
                const uint8_t* ba = sa + blk * kQ8BlockBytes;
                const uint8_t* bb = sb + blk * kQ8BlockBytes;
                float da = f16_at(ba), db = f16_at(bb);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    // int8 -> biased byte (q + 128) -> exact half (q)
                    uint32_t wa = ld32_al2(ba + 2 + 16 * c + 4 * t) ^ 0x80808080u;
                    uint32_t wb = ld32_al2(bb + 2 + 16 * c + 4 * t) ^ 0x80808080u;
                    uint32_t a[4];
                    a[0] = bytes01_to_h2(wa, bias128);
                    a[1] = bytes01_to_h2(wb, bias128);
                    a[2] = bytes23_to_h2(wa, bias128);
                    a[3] = bytes23_to_h2(wb, bias128);
                    int kk = s * 256 + blk * 32 + 16 * c + 4 * t;
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        uint2 b = __ldg((const uint2*)(xcol[nb] + kk));
                        float d[4];
                        mma_f16_16816(d, a, b.x, b.y);
                        acc[nb][0] = fmaf(da, d[0], acc[nb][0]);
                        acc[nb][1] = fmaf(da, d[1], acc[nb][1]);
                        acc[nb][2] = fmaf(db, d[2], acc[nb][2]);
                        acc[nb][3] = fmaf(db, d[3], acc[nb][3]);
                    }
                }
            }
        }
    }
}

// What one CTA works on, resolved from blockIdx.y.
struct Bucket {
    bool shared;
    int expert;   // routed: expert id
    int first;    // routed: first slot of the bucket; shared: first token
    int live;     // live columns (they are contiguous from column 0)
};

// Every thread of the CTA calls this (it contains a block-wide vote).  All
// loads are independent of one another, so the lookup costs one round trip.
// slot_ids[] receives the bucket's flat (token, k) ids (routed) for later use.
__device__ __forceinline__ bool resolve_bucket(const ExpertLaunch& L, Bucket& b, int* slot_ids) {
    int valid = *L.valid_tokens;
    int y = blockIdx.y;
    int tid = threadIdx.x;
    if (y < L.routed_blocks) {
        int e = L.expert_ids[y];
        int numel = valid * L.top_k;
        int sid = numel;
        if (tid < L.block_size) {
            sid = L.sorted_token_ids[(size_t)y * L.block_size + tid];
            slot_ids[tid] = sid;
        }
        // live slots are packed at the front of every bucket (dispatch.rs:107-115)
        int live = __syncthreads_count(sid < numel);
        b.shared = false;
        b.expert = e;
        b.first = y * L.block_size;
        b.live = live;
        return e >= 0 && live > 0;
    }
    int tile = y - L.routed_blocks;
    b.shared = true;
    b.expert = 0;
    b.first = tile * L.block_size;
    b.live = min(L.block_size, valid - b.first);
    return b.first < valid;
}

// Stage [start, start + bytes) of a weight tensor into shared memory through
// its 16-byte-aligned superset.  Returns the superset size; *phase is where
// the tile starts inside the staged bytes.
__device__ __forceinline__ uint32_t stage_tile(uint8_t* dst, const uint8_t* tensor, size_t start, uint32_t bytes,
                                               uint64_t* bar, uint32_t* phase) {
    size_t a0 = start & ~(size_t)15;
    size_t a1 = (start + bytes + 15) & ~(size_t)15;
    *phase = (uint32_t)(start - a0);
    tma_bulk_g2s(dst, tensor + a0, (uint32_t)(a1 - a0), bar);
    return (uint32_t)(a1 - a0);
}

__host__ __device__ inline uint32_t staged_capacity(uint32_t tile_bytes) {
    return ((tile_bytes + 15u) & ~15u) + 32u;  // superset + slack for the 2-byte-aligned word reads
}

// ---------------------------------------------------------------------------
// Gate/up projection + SwiGLU.  CTA tile: 8 gate rows and the same 8 up rows
// of one expert form one m16 tile (gate in fragment rows 0-7, up in 8-15, so
// the pair that SwiGLU joins lives in one thread).  The four warps split the
// contraction span-wise and their partial tiles are added in ascending warp
// order.  inter = silu(gate) * up with silu(g) = g / (1 + expf(-g))
// (crates/xabe-kernels/src/norm.rs:46-48,93-103), stored as f16.
// grid: (rows / 8, routed_blocks + shared_tiles), block 128.
// ---------------------------------------------------------------------------
template <int QUANT, int NB>
__device__ __forceinline__ void gateup_tile(const ExpertLaunch& L, const Bucket& bk, const int* slot_ids,
                                            const uint8_t* ta, const uint8_t* tb, int row_bytes, float* red) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int g = lane >> 2, t = lane & 3;
    const __half* xcol[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        int col = nb * 8 + g;
        if (col >= bk.live) col = 0;  // dead columns recompute column 0 and are never stored
        int token = bk.shared ? bk.first + col : slot_ids[col] / L.top_k;
        xcol[nb] = (bk.shared ? L.x_shared : L.x_routed) + (size_t)token * L.k;
    }
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nb][i] = 0.0f;
    mma_span_loop<QUANT, NB>(ta + g * row_bytes, tb + g * row_bytes, warp, 4, L.k / kSpanElems, xcol, t, acc);
    __syncthreads();  // every warp is done with the weight tile; reuse it
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[((warp * NB + nb) * 4 + i) * 32 + lane] = acc[nb][i];
    __syncthreads();
    // columns are spread over the warps for the epilogue: warp w takes nb = w, w+4
    int r0 = blockIdx.x * 8;
    for (int nb = warp; nb < NB; nb += 4) {
        float tot[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float s = red[((0 * NB + nb) * 4 + i) * 32 + lane];
            s += red[((1 * NB + nb) * 4 + i) * 32 + lane];
            s += red[((2 * NB + nb) * 4 + i) * 32 + lane];
            s += red[((3 * NB + nb) * 4 + i) * 32 + lane];
            tot[i] = s;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            int col = nb * 8 + 2 * t + i;
            if (col < bk.live) {
                float gv = tot[i], uv = tot[2 + i];
                float v = __fdiv_rn(gv, 1.0f + expf(-gv)) * uv;
                __half* dst = bk.shared ? L.inter_shared + (size_t)(bk.first + col) * L.rows
                                        : L.inter_routed + (size_t)(bk.first + col) * L.rows;
                dst[r0 + g] = __float2half_rn(v);
            }
        }
    }
}

template <int QR, int QS>
__global__ void __launch_bounds__(kExpertThreads) k_expert_gateup(ExpertLaunch L) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ int slot_ids[8 * kMaxNB];
    Bucket bk;
    if (!resolve_bucket(L, bk, slot_ids)) return;
    const int quant = bk.shared ? QS : QR;
    const int row_bytes = L.k / kSpanElems * span_bytes_of(quant);
    const uint32_t tile_bytes = 8u * row_bytes;
    const uint32_t cap = staged_capacity(tile_bytes);
    uint8_t* sa = smem;
    uint8_t* sb = smem + cap;
    __shared__ uint32_t phase[2];
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
        const uint8_t* wa = bk.shared ? L.s_a : L.r_a;
        const uint8_t* wb = bk.shared ? L.s_b : L.r_b;
        size_t start = ((size_t)bk.expert * L.rows + (size_t)blockIdx.x * 8) * row_bytes;
        size_t a0 = start & ~(size_t)15, a1 = (start + tile_bytes + 15) & ~(size_t)15;
        mbar_expect_tx(&bar, 2u * (uint32_t)(a1 - a0));
        stage_tile(sa, wa, start, tile_bytes, &bar, &phase[0]);
        stage_tile(sb, wb, start, tile_bytes, &bar, &phase[1]);
    }
    __syncthreads();
    // every thread observes the completion itself; the vote keeps the exit uniform
    if (!__syncthreads_and(mbar_wait_bounded(&bar, 0, L.status))) return;
    const uint8_t* ta = sa + phase[0];
    const uint8_t* tb = sb + phase[1];
    float* red = (float*)smem;
    int nb_needed = (bk.live + 7) >> 3;
    if (quant == QUANT_Q6K) {
        if (nb_needed <= 1) gateup_tile<QUANT_Q6K, 1>(L, bk, slot_ids, ta, tb, row_bytes, red);
        else if (nb_needed <= 2) gateup_tile<QUANT_Q6K, 2>(L, bk, slot_ids, ta, tb, row_bytes, red);
        else if (nb_needed <= 4) gateup_tile<QUANT_Q6K, 4>(L, bk, slot_ids, ta, tb, row_bytes, red);
        else gateup_tile<QUANT_Q6K, 8>(L, bk, slot_ids, ta, tb, row_bytes, red);
    } else {
        if (nb_needed <= 1) gateup_tile<QUANT_Q8_0, 1>(L, bk, slot_ids, ta, tb, row_bytes, red);
        else if (nb_needed <= 2) gateup_tile<QUANT_Q8_0, 2>(L, bk, slot_ids, ta, tb, row_bytes, red);
        else if (nb_needed <= 4) gateup_tile<QUANT_Q8_0, 4>(L, bk, slot_ids, ta, tb, row_bytes, red);
        else gateup_tile<QUANT_Q8_0, 8>(L, bk, slot_ids, ta, tb, row_bytes, red);
    }
}

// ---------------------------------------------------------------------------
// Down projection.  CTA tile: 64 consecutive rows of one expert's down matrix,
// one m16 tile per warp over the whole contraction (the intermediate width is
// short).  Routed buckets store weight * value into partial[flat]
// (store_slot_contribution, crates/xabe-cuda/src/kernels/moe.rs:1215-1221);
// the shared expert stores the value itself.  No atomics: every (flat, row)
// has exactly one writer, and the ascending-k sum happens in the combine.
// grid: (rows / 64, routed_blocks + shared_tiles), block 128.
// ---------------------------------------------------------------------------
template <int QUANT, int NB>
__device__ __forceinline__ void down_tile(const ExpertLaunch& L, const Bucket& bk, const int* slot_ids,
                                          const uint8_t* tile, int row_bytes) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int g = lane >> 2, t = lane & 3;
    const __half* xcol[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        int col = nb * 8 + g;
        int src = bk.first + (col < bk.live ? col : 0);
        xcol[nb] = (bk.shared ? L.x_shared : L.x_routed) + (size_t)src * L.k;
    }
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nb][i] = 0.0f;
    const uint8_t* pa = tile + (size_t)(warp * 16 + g) * row_bytes;
    const uint8_t* pb = pa + 8 * (size_t)row_bytes;
    mma_span_loop<QUANT, NB>(pa, pb, 0, 1, L.k / kSpanElems, xcol, t, acc);
    int row = blockIdx.x * 64 + warp * 16 + g;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            int col = nb * 8 + 2 * t + i;
            if (col < bk.live) {
                if (bk.shared) {
                    float* dst = L.shexp + (size_t)(bk.first + col) * L.rows;
                    dst[row] = acc[nb][i];
                    dst[row + 8] = acc[nb][2 + i];
                } else {
                    int flat = slot_ids[col];
                    float wgt = L.topk_weights[flat];
                    float* dst = result_row(L.partial, L.partial_rows, flat, L.rows);
                    dst[row] = wgt * acc[nb][i];
                    dst[row + 8] = wgt * acc[nb][2 + i];
                }
            }
        }
}

template <int QR, int QS>
__global__ void __launch_bounds__(kExpertThreads) k_expert_down(ExpertLaunch L) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t phase;
    __shared__ int slot_ids[8 * kMaxNB];
    Bucket bk;
    if (!resolve_bucket(L, bk, slot_ids)) return;
    const int quant = bk.shared ? QS : QR;
    const int row_bytes = L.k / kSpanElems * span_bytes_of(quant);
    const uint32_t tile_bytes = 64u * row_bytes;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
        const uint8_t* w = bk.shared ? L.s_a : L.r_a;
        size_t start = ((size_t)bk.expert * L.rows + (size_t)blockIdx.x * 64) * row_bytes;
        size_t a0 = start & ~(size_t)15, a1 = (start + tile_bytes + 15) & ~(size_t)15;
        mbar_expect_tx(&bar, (uint32_t)(a1 - a0));
        stage_tile(smem, w, start, tile_bytes, &bar, &phase);
    }
    __syncthreads();
    // every thread observes the completion itself; the vote keeps the exit uniform
    if (!__syncthreads_and(mbar_wait_bounded(&bar, 0, L.status))) return;
    const uint8_t* tile = smem + phase;
    int nb_needed = (bk.live + 7) >> 3;
    if (quant == QUANT_Q6K) {
        if (nb_needed <= 1) down_tile<QUANT_Q6K, 1>(L, bk, slot_ids, tile, row_bytes);
        else if (nb_needed <= 2) down_tile<QUANT_Q6K, 2>(L, bk, slot_ids, tile, row_bytes);
        else if (nb_needed <= 4) down_tile<QUANT_Q6K, 4>(L, bk, slot_ids, tile, row_bytes);
        else down_tile<QUANT_Q6K, 8>(L, bk, slot_ids, tile, row_bytes);
    } else {
        if (nb_needed <= 1) down_tile<QUANT_Q8_0, 1>(L, bk, slot_ids, tile, row_bytes);
        else if (nb_needed <= 2) down_tile<QUANT_Q8_0, 2>(L, bk, slot_ids, tile, row_bytes);
        else if (nb_needed <= 4) down_tile<QUANT_Q8_0, 4>(L, bk, slot_ids, tile, row_bytes);
        else down_tile<QUANT_Q8_0, 8>(L, bk, slot_ids, tile, row_bytes);
    }
}

}  // namespace xabe
