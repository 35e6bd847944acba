// The front of the MoE block for handles of up to 256 tokens in ONE launch: RMSNorm, router
// logits, softmax top-k routing, the block-aligned dispatch tables, the column groups of the
// streaming expert kernels and the shared expert's sigmoid gate.  The reference spends four
// launches on these (crates/xabe-engine/src/block/moe.rs:1117-1230, with route + dispatch fused at
// one token, crates/xabe-cuda/src/kernels/moe.rs:2099-2230); at one token the step is a chain of
// launch latencies, so every launch removed is worth more than any arithmetic in it.
//
// Structure: grid (E / 4, token tiles of TT), block 128.  Every CTA normalises the TT rows of its
// tile itself (the rows are a few KB; recomputing them costs less than a launch boundary) and forms
// the logits of its four experts for them.  The CTAs of a tile take a ticket when their logits are
// stored; the one that draws the last ticket routes the tile's tokens; tiles take a second ticket,
// and the CTA that draws the last of those builds the dispatch tables.  Nothing waits on another
// CTA: a CTA either finds it is the last one or leaves, so the launch cannot hang.
//
// Every value is formed in the order of the kernel it replaces (k_rms_norm, k_router_logits,
// route_one_token, k_route_dispatch_small, the gate of k_gate_and_combine), so the outputs are
// bit-identical to the unfused launches.
#pragma once

#include "common.cuh"
#include "glue_kernels.cuh"

namespace xabe {

constexpr int kFrontThreads = 128;

struct FrontLaunch {
    const float* x;        // residual [max_tokens][hidden]
    const float* norm_w;   // [hidden]
    const float* router;   // [E][hidden]
    const float* bias;     // [E] or null
    const float* gate_w;   // shared-gate vector [hidden], or null (no gate wanted)
    const int* valid_tokens;
    float* normed;
    __half* normed_h;
    float* logits;
    float* gate;
    int* topk_ids;
    float* topk_weights;
    int* sorted_token_ids;
    int* expert_ids;
    int* num_tokens_post_pad;
    int* expert_offsets;
    int* expert_counts;
    int* work_items;
    int* n_work;
    int* tickets;  // [1 + token tiles], zero between launches
    int* zero_buf; // arrival counters of the fused combine (k_expert_stream<DOWN>): cleared here every step,
    int zero_count;//   so a launch that gave up half-way cannot leave counts behind
    int* status;
    int hidden, num_experts, top_k, block_size, sorted_capacity, block_capacity;
    int fused_dispatch;  // 1: at most kTinyPairs flat pairs, the tables are built here; 0: by the launch that follows
    int route;           // 0: the launch ends with the logits (norm fused into the router, nothing else)
    float eps;
};

// dynamic shared memory: four router rows, the tile's TT activation rows and the norm weights (two
// CTAs of the widest tile still share an SM)
__host__ __device__ inline size_t front_smem(int hidden, int tt) {
    return (size_t)(4 + tt + 1) * hidden * sizeof(float);
}

template <int TT>
__global__ void __launch_bounds__(kFrontThreads) k_decode_front(FrontLaunch P) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) float fs[];
    __shared__ __align__(8) uint64_t wbar, xbar;
    __shared__ float warp_tot[TT][32];
    __shared__ float inv_s[TT];
    __shared__ int last_flag;
    __shared__ int cnt_s[512], start_s[512], gbase_s[512];  // dispatch_tiny_warp's scratch (num_experts <= 512)
    const int hidden = P.hidden, num_experts = P.num_experts;
    float* w_rows = fs;
    float* x_rows = fs + (size_t)4 * hidden;
    float* nw_s = x_rows + (size_t)TT * hidden;  // norm weights
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e0 = blockIdx.x * 4;
    const int tile = blockIdx.y, t0 = tile * TT;
    if (tid == 0) {
        // everything that does not depend on the live token count is in flight before it is read
        mbar_init(&wbar, 1);
        mbar_init(&xbar, 1);
        fence_mbar_init();
        const uint32_t wbytes = (uint32_t)min(4, num_experts - e0) * hidden * 4u;
        mbar_expect_tx(&wbar, wbytes);
        tma_bulk_g2s(w_rows, P.router + (size_t)e0 * hidden, wbytes, &wbar);
    }
    const int live = *P.valid_tokens;
    // a tile without live tokens takes no ticket (the counts below are over live tiles); its router
    // rows may still be landing, and a CTA must not exit under a copy into its shared memory
    if (t0 >= live) {
        __syncthreads();
        mbar_wait_bounded(&wbar, 0, P.status);
        return;
    }
    const int nt = min(TT, live - t0);
    const int live_tiles = (live + TT - 1) / TT;
    if (tid == 0) {
        const uint32_t xbytes = (uint32_t)nt * hidden * 4u, vbytes = (uint32_t)hidden * 4u;
        mbar_expect_tx(&xbar, xbytes + vbytes);
        tma_bulk_g2s(x_rows, P.x + (size_t)t0 * hidden, xbytes, &xbar);
        tma_bulk_g2s(nw_s, P.norm_w, vbytes, &xbar);
    }
    __syncthreads();
    // A wait that runs out is recorded in the status word; the CTA goes on with whatever the buffer
    // holds (every index below stays in range whatever the data is), because the tickets must be
    // drawn for the counters to return to zero.
    mbar_wait_bounded(&xbar, 0, P.status);

    __syncthreads();
    // ---- RMSNorm of the tile's rows in k_rms_norm's order: `vl` lanes (its block width), lane v
    // sums x[j]^2 over j = v, v + vl, ...; shuffle-down inside each warp of 32 lanes; the warp totals
    // added in ascending order.  A thread carries lanes tid, tid + 128, ...: they share its lane
    // position, so the shuffles of the real warp are the shuffles of each virtual warp.  The loops
    // are kept rolled: this code runs once per launch, and what it costs is instruction fetch.
    const int vl = hidden < 1024 ? hidden : 1024;
    const int nv = vl / kFrontThreads;  // hidden is a multiple of 256, so 2, 4, 6 or 8
    for (int u = 0; u < nt; ++u) {
        const float* xr = x_rows + (size_t)u * hidden;
#pragma unroll 1
        for (int i0 = 0; i0 < nv; i0 += 2) {  // two virtual lanes per pass: their shuffle chains overlap
            float pa = 0.0f, pb = 0.0f;
            for (int j = tid + kFrontThreads * i0; j < hidden; j += vl) {
                pa = fmaf(xr[j], xr[j], pa);
                pb = fmaf(xr[j + kFrontThreads], xr[j + kFrontThreads], pb);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                pa += __shfl_down_sync(0xffffffffu, pa, off);
                pb += __shfl_down_sync(0xffffffffu, pb, off);
            }
            if (lane == 0) {
                warp_tot[u][warp + 4 * i0] = pa;
                warp_tot[u][warp + 4 * i0 + 4] = pb;
            }
        }
    }
    __syncthreads();
    if (tid < nt) {
        float total = 0.0f;
#pragma unroll 8
        for (int w = 0; w < vl / 32; ++w) total += warp_tot[tid][w];
        inv_s[tid] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)hidden), P.eps)));
    }
    __syncthreads();
    {
        // every CTA holds all normalised rows; CTA b of the tile stores the b-th share of each row,
        // in units of four columns
        const int gx = (int)gridDim.x, b = (int)blockIdx.x, quads = hidden / 4;
        const int q_lo = (b * quads + gx - 1) / gx, q_hi = ((b + 1) * quads + gx - 1) / gx;
        for (int u = 0; u < nt; ++u) {
            float4* xr = (float4*)(x_rows + (size_t)u * hidden);
            const float inv = inv_s[u];
            const size_t o = (size_t)(t0 + u) * hidden;
#pragma unroll 4
            for (int q = tid; q < quads; q += kFrontThreads) {
                const float4 xv = xr[q], nw = ((const float4*)nw_s)[q];
                float4 y;
                y.x = __fmul_rn(__fmul_rn(xv.x, inv), nw.x);
                y.y = __fmul_rn(__fmul_rn(xv.y, inv), nw.y);
                y.z = __fmul_rn(__fmul_rn(xv.z, inv), nw.z);
                y.w = __fmul_rn(__fmul_rn(xv.w, inv), nw.w);
                xr[q] = y;
                if (q >= q_lo && q < q_hi) {
                    *(float4*)(P.normed + o + 4 * (size_t)q) = y;
                    __half2 h01 = __floats2half2_rn(y.x, y.y), h23 = __floats2half2_rn(y.z, y.w);
                    uint2 hv;
                    hv.x = *(uint32_t*)&h01;
                    hv.y = *(uint32_t*)&h23;
                    *(uint2*)(P.normed_h + o + 4 * (size_t)q) = hv;
                }
            }
        }
    }
    mbar_wait_bounded(&wbar, 0, P.status);
    __syncthreads();

    // ---- router logits of this CTA's four experts, one warp per expert, in k_router_logits's
    // order: 256 lanes, lane v sums w[j] x[j] over j = v, v + 256, ...; shuffle-down tree in each
    // group of 32 lanes; the eight group totals added ascending from +0.  A real lane carries four
    // neighbouring lanes of two groups (128-bit shared loads): lane q holds positions 4 (q % 8) ..
    // + 3 of groups q / 8 and q / 8 + 4, so tree levels 16, 8, 4 are shuffles by 4, 2, 1 lanes and
    // levels 2 and 1 are sums inside the lane, the same pairs in the same order.
    {
        const int e = e0 + warp;
        if (e < num_experts) {
            const int sub = lane & 7, gsel = lane >> 3;
            const float* wrow = w_rows + (size_t)warp * hidden + gsel * 32 + 4 * sub;
            float4 acc[2][TT];
#pragma unroll
            for (int gi = 0; gi < 2; ++gi)
#pragma unroll
                for (int u = 0; u < TT; ++u) acc[gi][u] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int jc = 0; jc < hidden; jc += 256) {
                const float4 w0 = *(const float4*)(wrow + jc), w1 = *(const float4*)(wrow + jc + 128);
#pragma unroll
                for (int u = 0; u < TT; ++u) {
                    // rows past nt hold stale bytes; their sums are never stored
                    const float* xr = x_rows + (size_t)u * hidden + gsel * 32 + 4 * sub + jc;
                    const float4 x0 = *(const float4*)xr, x1 = *(const float4*)(xr + 128);
                    acc[0][u].x = fmaf(w0.x, x0.x, acc[0][u].x);
                    acc[0][u].y = fmaf(w0.y, x0.y, acc[0][u].y);
                    acc[0][u].z = fmaf(w0.z, x0.z, acc[0][u].z);
                    acc[0][u].w = fmaf(w0.w, x0.w, acc[0][u].w);
                    acc[1][u].x = fmaf(w1.x, x1.x, acc[1][u].x);
                    acc[1][u].y = fmaf(w1.y, x1.y, acc[1][u].y);
                    acc[1][u].z = fmaf(w1.z, x1.z, acc[1][u].z);
                    acc[1][u].w = fmaf(w1.w, x1.w, acc[1][u].w);
                }
            }
            const float bias = P.bias ? P.bias[e] : 0.0f;
#pragma unroll
            for (int u = 0; u < TT; ++u) {
                float root[2];
#pragma unroll
                for (int gi = 0; gi < 2; ++gi) {
                    float4 v = acc[gi][u];
#pragma unroll
                    for (int off = 4; off > 0; off >>= 1) {  // tree levels 16, 8, 4
                        v.x += __shfl_down_sync(0xffffffffu, v.x, off);
                        v.y += __shfl_down_sync(0xffffffffu, v.y, off);
                        v.z += __shfl_down_sync(0xffffffffu, v.z, off);
                        v.w += __shfl_down_sync(0xffffffffu, v.w, off);
                    }
                    v.x += v.z;  // level 2: positions 0, 1 take 2, 3
                    v.y += v.w;
                    root[gi] = v.x + v.y;  // level 1
                }
                float total = 0.0f;
#pragma unroll
                for (int g = 0; g < 8; ++g) total += __shfl_sync(0xffffffffu, root[g >> 2], (g & 3) * 8);
                if (lane == 0 && u < nt)
                    P.logits[(size_t)(t0 + u) * num_experts + e] = P.bias ? __fadd_rn(total, bias) : total;
            }
        }
    }

    // ---- the shared expert's gate, sigmoid(dot(gate_w, normed[t])): 256 lanes at stride 256,
    // shuffle-down per warp, warps ascending (k_gate_and_combine's order), one real warp carrying the
    // eight virtual warps.  Only the last launch of the block reads it, so a CTA computes it after it
    // has drawn its ticket, off the path to the routing.  Token u of the tile: CTA u modulo the tile's CTAs.
    auto gate_of_this_cta = [&]() {
        if (!P.gate_w || warp != 0) return;
        for (int u = (int)blockIdx.x; u < nt; u += (int)gridDim.x) {
            const float* xr = x_rows + (size_t)u * hidden;
            float sv[8];
#pragma unroll
            for (int vw = 0; vw < 8; ++vw) sv[vw] = 0.0f;
            for (int j0 = 0; j0 < hidden; j0 += 256) {
                float gv[8];
#pragma unroll
                for (int vw = 0; vw < 8; ++vw) gv[vw] = __ldg(P.gate_w + j0 + vw * 32 + lane);
#pragma unroll
                for (int vw = 0; vw < 8; ++vw) sv[vw] = fmaf(gv[vw], xr[j0 + vw * 32 + lane], sv[vw]);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                for (int vw = 0; vw < 8; ++vw) sv[vw] += __shfl_down_sync(0xffffffffu, sv[vw], off);
            float total = 0.0f;
#pragma unroll
            for (int vw = 0; vw < 8; ++vw) total += sv[vw];
            if (lane == 0) P.gate[t0 + u] = __fdiv_rn(1.0f, 1.0f + expf(-total));
        }
    };

    if (!P.route) {  // norm + router only: the routing is the next launch's
        gate_of_this_cta();
        return;
    }
    // ---- ticket 1: the last CTA of the tile routes the tile's tokens
    __syncthreads();
    if (tid == 0) {
        __threadfence();  // this CTA's logits (stored before the barrier) are visible before the ticket is
        const int n = atomicAdd(P.tickets + 1 + tile, 1);
        last_flag = n == (int)gridDim.x - 1;
        if (last_flag) P.tickets[1 + tile] = 0;  // ready for the next launch
        __threadfence();
    }
    __syncthreads();
    if (!last_flag) {
        gate_of_this_cta();
        return;
    }
    const bool tiny = P.fused_dispatch != 0;
    const int numel = live * P.top_k;
    if (tiny) {  // the fills of the tables, by the warps that have no token to route
        for (int i = tid; i < P.sorted_capacity; i += kFrontThreads) P.sorted_token_ids[i] = numel;
        for (int i = tid; i < P.block_capacity; i += kFrontThreads) P.expert_ids[i] = -1;
        for (int i = tid; i < num_experts; i += kFrontThreads) cnt_s[i] = 0;
        for (int i = tid; i < P.zero_count; i += kFrontThreads) P.zero_buf[i] = 0;
    }
    for (int u = warp; u < nt; u += kFrontThreads / 32) {
        const size_t t = (size_t)(t0 + u);
        if (num_experts <= 256)
            route_one_token<8>(P.logits + t * num_experts, num_experts, P.top_k, lane, P.topk_ids + t * P.top_k,
                               P.topk_weights + t * P.top_k);
        else
            route_one_token<16>(P.logits + t * num_experts, num_experts, P.top_k, lane, P.topk_ids + t * P.top_k,
                                P.topk_weights + t * P.top_k);
    }
    if (!tiny) {  // the tables are built by the launch that follows (k_route_dispatch_small)
        gate_of_this_cta();
        return;
    }
    // ---- ticket 2 (only with several live tiles): the last tile builds the tables from every tile's routing
    __syncthreads();
    if (live_tiles > 1) {
        if (tid == 0) {
            __threadfence();
            const int n = atomicAdd(P.tickets, 1);
            last_flag = n == live_tiles - 1;
            if (last_flag) P.tickets[0] = 0;
            __threadfence();
        }
        __syncthreads();
        if (!last_flag) {
            gate_of_this_cta();
            return;
        }
    } else {
        __threadfence();  // the routing stored above is read back through L2 below
        __syncthreads();
    }
    if (warp == 0)
        dispatch_tiny_warp(lane, numel, num_experts, P.block_size, cnt_s, start_s, gbase_s, P.topk_ids, P.topk_weights,
                           P.sorted_token_ids, P.expert_ids, P.num_tokens_post_pad, P.expert_offsets,
                           P.expert_counts, P.work_items, P.n_work);
    gate_of_this_cta();
}

}  // namespace xabe
