// Gate/up + SwiGLU for wide decode batches, one warp per eight output rows.
//
// k_expert_stream<MODE_GATEUP> splits the contraction of a row tile over the eight warps of a
// group and adds their partial tiles through shared memory: a handshake per tile that keeps the
// eight warps in lockstep (measured: 13 % of the launch).  Here a consumer warp owns eight gate
// rows and the same eight up rows for the whole contraction, so nothing is exchanged between
// warps.  The ring then carries slices of the contraction instead of whole rows: one stage is
// one 256-element span of 64 gate rows and 64 up rows, fetched as two boxes of a 2-D tensor map
// over the weight bytes ([rows][row_bytes], row pitch a multiple of 16 bytes).  A Q6_K span of
// 210 bytes starts 2 s bytes past a 16-byte boundary, so the box is 240 bytes wide and starts at
// the boundary below (the last span's box starts earlier, so that it ends with the row: see
// rows_box_start); with a 240-byte (272 for Q8_0) row pitch in shared memory the eight rows a
// load touches fall in disjoint banks.
//
// Unit of work: (column group, block of 128 output rows); group gi of the CTA owns rows
// 64 gi .. 64 gi + 63 of the block and takes every other stage.  Arithmetic per row is that of
// stream_half (exact integer codes, fp32 scales, fp32 accumulation), spans in ascending order,
// so a token's value depends on nothing but its own column.
#pragma once

#include <cuda.h>

#include "stream_kernels.cuh"

namespace xabe {

constexpr int kRowsGroupRows = 8 * kStreamGroupWarps;            // 64 rows of each matrix per stage
constexpr int kRowsUnitRows = kStreamGroups * kRowsGroupRows;    // 128 output rows per unit
constexpr int kRowsMaxStages = 6;

struct RowsLaunch {
    StreamLaunch L;
    CUtensorMap tm_r_a, tm_r_b, tm_s_a, tm_s_b;  // gate / up bytes of the routed stack and of the shared expert
    uint32_t box_r, box_s;                       // staged bytes per row
    uint32_t stage_bytes;                        // 2 * 64 * max(box_r, box_s)
};

__host__ __device__ inline uint32_t rows_box_bytes(int quant) { return quant == QUANT_Q6K ? 240u : 272u; }

// Where in its row the box that covers the span at byte `off` starts: the 16-byte boundary below the
// span, but never so far right that the box would reach past the end of the row.  The bytes of a box
// past the row's end are the next row's, and for the last row of a tensor they lie beyond the
// allocation; a copy must not depend on what is mapped there.
__host__ __device__ inline int rows_box_start(int off, int row_bytes, int box) {
    const int lo = off & ~15, hi = row_bytes - box;
    return lo < hi ? lo : hi;
}

struct RowsSmem {
    uint32_t stages, xbuf, items, bars, total;
};

__host__ __device__ inline RowsSmem rows_smem_layout(int n_stages, uint32_t stage_bytes, uint32_t x_stride) {
    RowsSmem R;
    R.stages = 0;  // relative to the 128-byte aligned base
    R.xbuf = R.stages + (uint32_t)n_stages * stage_bytes;
    R.items = R.xbuf + 2u * 8u * x_stride;
    R.bars = R.items + 2u * 96u;
    R.total = R.bars + 8u * (2u * kRowsMaxStages + 4u) + 128u;  // + slack for aligning the base
    return R;
}

__device__ __forceinline__ void tma_load_box_2d(void* dst, const CUtensorMap* tm, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"((uint64_t)tm), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// grid: number of SMs; block: kStreamThreads (warp 0 streams weights, warps 1-16 consume, warp 17
// stages activation rows).  Every wait is bounded as in k_expert_stream.
template <int QR, int QS>
__global__ void __launch_bounds__(kStreamThreads, 1) k_gateup_rows(const __grid_constant__ RowsLaunch P) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int abort_flag;
    const StreamLaunch& L = P.L;
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const int S = L.n_stages;
    const RowsSmem lay = rows_smem_layout(S, P.stage_bytes, L.x_stride);
    uint64_t* full = (uint64_t*)(smem + lay.bars);
    uint64_t* empty = full + kRowsMaxStages;
    uint64_t* xfull = empty + kRowsMaxStages;
    uint64_t* xempty = xfull + 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kStreamGroupWarps);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&xfull[i], 1);
            mbar_init(&xempty[i], kStreamConsumerWarps);
        }
        fence_mbar_init();
    }
    __syncthreads();
    volatile int* abortp = &abort_flag;
    const int n_spans = L.k / kSpanElems;
    const int n_routed = L.has_routed ? *L.n_work : 0;
    const int valid = *L.valid_tokens;
    const int n_groups = n_routed + (L.has_shared ? (valid + 7) >> 3 : 0);
    const int blocks = L.rows / kRowsUnitRows;
    const int units = n_groups * blocks;

    if (warp == 1 + kStreamConsumerWarps) {
        // ---------------------------- activation stager ----------------------------
        if (lane != 0) return;
        int xb = 0;
        uint32_t xuse = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            const int cg = u / blocks;
            const bool shared = cg >= n_routed;
            int* desc = (int*)(smem + lay.items + xb * 96);
            if (xuse >= 1 && !stream_wait(&xempty[xb], (xuse - 1) & 1, abortp, L.status)) return;
            int expert = -1, first, ncols;
            const int* item = nullptr;
            if (!shared) {
                item = L.work_items + (size_t)cg * kWorkItemInts;
                expert = item[0];
                first = item[1];
                ncols = item[2];
            } else {
                first = (cg - n_routed) * 8;
                ncols = min(8, valid - first);
            }
            // self-check: a column group that points outside its buffers is recorded, never dereferenced
            bool sane = ncols >= 1 && ncols <= 8 && first >= 0;
            if (!shared) {
                sane = sane && expert >= 0 && expert < L.num_experts;
                for (int c = 0; sane && c < ncols; ++c) sane = item[4 + c] >= 0 && item[4 + c] / L.top_k < L.max_tokens;
            } else {
                sane = sane && first + ncols <= L.max_tokens;
            }
            if (!sane) {
                *abortp = 1;
                atomicExch(L.status, STATUS_BAD_WORK_ITEM);
                return;
            }
            desc[0] = expert;
            desc[1] = first;
            desc[2] = ncols;
            const uint32_t xrow_bytes = (uint32_t)L.k * 2u;
            mbar_expect_tx(&xfull[xb], ncols * xrow_bytes);
            uint8_t* xdst = smem + lay.xbuf + (uint32_t)xb * 8u * L.x_stride;
            for (int c = 0; c < ncols; ++c) {
                const size_t src_row = shared ? (size_t)(first + c) : (size_t)(item[4 + c] / L.top_k);
                tma_bulk_g2s(xdst + c * L.x_stride, (shared ? L.x_shared : L.x_routed) + src_row * L.k, xrow_bytes,
                             &xfull[xb]);
            }
            if (++xb == 2) {
                xb = 0;
                ++xuse;
            }
        }
        return;
    }

    if (warp == 0) {
        // ------------------------------ weight producer ------------------------------
        if (lane != 0) return;
        int st = 0;
        uint32_t use = 0;
        int expert_next = -1;
        if ((int)blockIdx.x < units) {
            const int cg0 = (int)blockIdx.x / blocks;
            if (cg0 < n_routed) expert_next = L.work_items[(size_t)cg0 * kWorkItemInts];
        }
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            const int cg = u / blocks, blk = u - cg * blocks;
            const bool shared = cg >= n_routed;
            const int expert = expert_next;
            {
                const int un = u + (int)gridDim.x;
                const int cgn = un / blocks;
                if (un < units && cgn < n_routed) expert_next = L.work_items[(size_t)cgn * kWorkItemInts];
            }
            if (!shared && (expert < 0 || expert >= L.num_experts)) return;  // the stager records the bad group
            const CUtensorMap* ta = shared ? &P.tm_s_a : &P.tm_r_a;
            const CUtensorMap* tb = shared ? &P.tm_s_b : &P.tm_r_b;
            const uint32_t box = shared ? P.box_s : P.box_r;
            const int span_b = span_bytes_of(shared ? QS : QR);
            const int y0 = (shared ? 0 : expert * L.rows) + blk * kRowsUnitRows;
            for (int s = 0; s < n_spans; ++s) {
                const int x = rows_box_start(span_b * s, span_b * n_spans, (int)box) >> 2;  // in 32-bit words
#pragma unroll
                for (int gi = 0; gi < kStreamGroups; ++gi) {
                    if (use >= 1 && !stream_wait(&empty[st], (use - 1) & 1, abortp, L.status)) return;
                    uint8_t* dst = smem + lay.stages + (uint32_t)st * P.stage_bytes;
                    mbar_expect_tx(&full[st], 2u * kRowsGroupRows * box);
                    tma_load_box_2d(dst, ta, x, y0 + gi * kRowsGroupRows, &full[st]);
                    tma_load_box_2d(dst + kRowsGroupRows * box, tb, x, y0 + gi * kRowsGroupRows, &full[st]);
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
    const int gi = cw / kStreamGroupWarps;  // group: rows 64 gi .. 64 gi + 63 of the unit's block
    const int w = cw % kStreamGroupWarps;   // warp within the group: rows 8 w .. 8 w + 7 of those
    const int g = lane >> 2, t = lane & 3;
    int st = gi % S;                        // this group's stages are the odd or the even ring positions
    uint32_t use = (uint32_t)(gi / S);
    int xb = 0;
    uint32_t xuse = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int cg = u / blocks, blk = u - cg * blocks;
        const bool shared = cg >= n_routed;
        const int quant = shared ? QS : QR;
        const uint32_t box = shared ? P.box_s : P.box_r;
        const int span_b = span_bytes_of(quant);
        if (!stream_wait(&xfull[xb], xuse & 1, abortp, L.status)) return;
        const int* desc = (const int*)(smem + lay.items + xb * 96);
        const int first = desc[1], ncols = desc[2];
        // column g of the group (dead columns read stale rows and are never stored)
        const uint8_t* xrow = smem + lay.xbuf + (uint32_t)xb * 8u * L.x_stride + g * L.x_stride;
        // The partial sums of k_expert_stream<MODE_GATEUP>, formed and added in its order (see
        // gateup_span_of): slot s = half 0 of span s continued by half 1 of span s + 1, the last
        // slot half 0 of the last span alone, then the idle slots' zeros, then the wrap slot
        // (half 1 of span 0).  `open` is the slot half 1 of the next span completes.
        float open[4] = {0.f, 0.f, 0.f, 0.f}, wrap[4] = {0.f, 0.f, 0.f, 0.f}, tot[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < n_spans; ++s) {
            if (!stream_wait(&full[st], use & 1, abortp, L.status)) return;
            const uint8_t* pa = smem + lay.stages + (uint32_t)st * P.stage_bytes + (uint32_t)(w * 8 + g) * box +
                                (uint32_t)(span_b * s - rows_box_start(span_b * s, span_b * n_spans, (int)box));
            const uint8_t* pb = pa + kRowsGroupRows * box;
            float acc[4];
            uint2 bf[8];
            // half 1: continues the slot opened by the span before (span 0: the wrap slot, from zero)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = s == 0 ? 0.f : open[i];
            if (quant == QUANT_Q6K) {
                load_bfrags_half<QUANT_Q6K>(xrow, s, 1, t, bf);
                half_dispatch<QUANT_Q6K>(pa, pb, 1, bf, lane, acc);
            } else {
                load_bfrags_half<QUANT_Q8_0>(xrow, s, 1, t, bf);
                half_dispatch<QUANT_Q8_0>(pa, pb, 1, bf, lane, acc);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (s == 0) wrap[i] = acc[i];
                else tot[i] = s == 1 ? acc[i] : tot[i] + acc[i];
            }
            // half 0: opens slot s
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = 0.f;
            if (quant == QUANT_Q6K) {
                load_bfrags_half<QUANT_Q6K>(xrow, s, 0, t, bf);
                half_dispatch<QUANT_Q6K>(pa, pb, 0, bf, lane, acc);
            } else {
                load_bfrags_half<QUANT_Q8_0>(xrow, s, 0, t, bf);
                half_dispatch<QUANT_Q8_0>(pa, pb, 0, bf, lane, acc);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) open[i] = acc[i];
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);  // the ring stage may be refilled
            st += kStreamGroups;
            if (st >= S) {
                st -= S;
                ++use;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            tot[i] += open[i];                                  // the last slot
            if (n_spans < kStreamGroupWarps) tot[i] += 0.f;     // the idle slots (-0 + 0 = +0)
            tot[i] += wrap[i];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&xempty[xb]);
        if (++xb == 2) {
            xb = 0;
            ++xuse;
        }
        // SwiGLU of this warp's eight rows: tot[0..1] gate, tot[2..3] up, columns 2t and 2t + 1
        const int row = blk * kRowsUnitRows + gi * kRowsGroupRows + w * 8 + g;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int col = 2 * t + i;
            if (col < ncols) {
                const float gv = tot[i], uv = tot[2 + i];
                const float v = __fdiv_rn(gv, 1.0f + expf(-gv)) * uv;
                __half* dst = (shared ? L.inter_shared : L.inter_routed) + (size_t)(first + col) * L.rows;
                dst[row] = __float2half_rn(v);
            }
        }
    }
}

}  // namespace xabe
