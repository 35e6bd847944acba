// The tcgen05 grouped GEMM for experts that meet many tokens: one unpacked pair of weight chunks
// is multiplied against up to FOUR 128-column token tiles (four accumulators fill TMEM's 512
// columns), so the dequantisation work per weight is shared by up to 512 tokens instead of 128.
//
// Same roles and the same arithmetic as k_prefill_gemm (prefill_kernels.cuh); what differs:
//   * an item is one expert x up to 512 token columns; a tile is an item x one 128-row weight tile;
//   * the A ring (two pairs of chunks) and the B ring (units of one pair x one column tile, two
//     16 KB chunk tiles each) are separate.  B tiles come by TMA (2-D tiled, 128-byte swizzle,
//     two copies per unit issued by one thread of a dedicated warp, as far ahead as the ring
//     allows); that needs an item's token columns to be consecutive rows of the source, so the
//     routed gate/up pass reads a copy of the activations permuted into dispatch order
//     (k_permute_rows), the other passes read buffers that are in that order already;
//     a first version whose unpack warps issued 16-byte copies for B between their unpack passes
//     was slower than the one-accumulator kernel: B latency was exposed once per unit;
//   * the four accumulator slots are handed over one by one: the epilogue warps drain a slot and
//     release it, the next tile's MMAs into that slot may start while the others are drained;
//     tiles with fewer column tiles use fewer slots, so small tiles still overlap fully.
// Every wait is bounded; TMEM is freed on every exit path; no multicast, no clusters.
#pragma once

#include "prefill_kernels.cuh"

namespace xabe {

constexpr int kPfWideMaxCt = 4;             // column tiles (accumulators) per item
constexpr int kPfWideItemCols = kPfWideMaxCt * kPfTileN;
constexpr int kPfWideMaxBUnits = 3;
constexpr int kPfWideRaw = 2;

struct PfWideCtl {
    uint64_t a_full[2], a_empty[2];                       // pair slots of the A ring
    uint64_t b_full[kPfWideMaxBUnits], b_empty[kPfWideMaxBUnits];
    uint64_t raw_full[kPfWideRaw], raw_empty[kPfWideRaw];
    uint64_t acc_full[kPfWideMaxCt], acc_empty[kPfWideMaxCt];
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int kPfWideWarpB = kPfWarpEpi0 + 4;        // one more warp: the B loader
constexpr int kPfWideThreads = 32 * (kPfWideWarpB + 1);

// 2-D tiled TMA load: box {64 elements, 128 rows} at (x = first element, y = first row) -> dst
// (1024-byte aligned shared memory); completes `bytes` on the mbarrier.  x * 2 bytes is a multiple
// of 16 for every x this kernel uses (multiples of 64).
__device__ __forceinline__ void tma_load_tile_2d(uint32_t dst, const CUtensorMap* tm, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            dst),
        "l"((uint64_t)tm), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mbar_expect_tx32(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// Activation rows in dispatch order: slot s of the sorted table gets the f16 row of its token
// (the reference permutes the same way before its grouped GEMM, moe.rs:5727-5760); padding slots
// are skipped.  grid: sorted_capacity, block 256.
__global__ void __launch_bounds__(256) k_permute_rows(const int* __restrict__ sorted_token_ids,
                                                      const int* __restrict__ num_tokens_post_pad,
                                                      const int* __restrict__ valid_tokens, int top_k, int hidden,
                                                      const __half* __restrict__ x, __half* __restrict__ x_sorted) {
    const int s = blockIdx.x;
    if (s >= *num_tokens_post_pad) return;
    const int flat = sorted_token_ids[s];
    if (flat >= *valid_tokens * top_k) return;
    const uint4* src = (const uint4*)(x + (size_t)(flat / top_k) * hidden);
    uint4* dst = (uint4*)(x_sorted + (size_t)s * hidden);
    for (int u = threadIdx.x; u < hidden / 8; u += 256) dst[u] = __ldg(src + u);
}

// grid: one CTA per SM (or fewer); block kPfThreads.
template <int MODE, int QR, int QS>
__global__ void __launch_bounds__(kPfWideThreads, 1) k_prefill_gemm_wide(const __grid_constant__ PrefillLaunch L) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) PfWideCtl ctl;
    // MODE_DOWN: the epilogue warps' turn-around buffers and row addresses, as in k_prefill_gemm
    __shared__ __align__(16) float epi_stage[MODE == MODE_DOWN ? 4 : 1][MODE == MODE_DOWN ? 32 * 16 : 4];
    __shared__ float* epi_dst[MODE == MODE_DOWN ? 4 : 1][32];
    constexpr int kTile = kPfTileM * kPfChunkK * 2;  // one 16 KB A or B chunk tile
    constexpr int kUnit = 2 * kTile;                 // a pair of chunk tiles

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int valid = *L.valid_tokens;
    const int n_routed = L.has_routed ? *L.n_items : 0;
    const int n_shared = L.has_shared ? (valid + L.item_cols - 1) / L.item_cols : 0;
    const int n_tiles = (n_routed + n_shared) * L.row_tiles;
    const int R = L.n_raw, NBU = L.n_b_units;
    const int n_spans = L.k / kSpanElems;
    uint8_t* a_ring = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* b_ring = a_ring + 2 * kUnit;
    uint8_t* raw_ring = b_ring + (size_t)NBU * kUnit;
    volatile int* abortp = &ctl.abort_flag;

    if (tid == 0) {
        ctl.abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctl.a_full[i], kPfUnpackWarps);
            mbar_init(&ctl.a_empty[i], 1);
        }
        for (int i = 0; i < NBU; ++i) {
            mbar_init(&ctl.b_full[i], 1);  // the B loader's expect_tx arrival; the two TMA copies complete the bytes
            mbar_init(&ctl.b_empty[i], 1);
        }
        for (int i = 0; i < R; ++i) {
            mbar_init(&ctl.raw_full[i], kPfLoadWarps * 32);
            mbar_init(&ctl.raw_empty[i], kPfUnpackWarps);
        }
        for (int i = 0; i < kPfWideMaxCt; ++i) {
            mbar_init(&ctl.acc_full[i], 1);
            mbar_init(&ctl.acc_empty[i], 4);
        }
        fence_mbar_init();
    }
    if (warp == kPfWarpMma) {
        tmem_alloc(&ctl.tmem_base, kPfWideMaxCt * kPfTileN);  // all 512 columns: four accumulators
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl.tmem_base;
    const int G = gridDim.x;

    if (warp < kPfUnpackWarps) {
        // ------------------------------ unpack warps ------------------------------
        const int rrow = ((lane >> 2) & 1) * 4 + (lane >> 3), j = lane & 3;
        const int trow = 8 * warp + rrow;
        const uint32_t a32 = smem_u32(a_ring), raw32 = smem_u32(raw_ring);
        const uint32_t rowoff = (uint32_t)(warp * 1024 + rrow * 128);
        const uint32_t dst6 = rowoff + (uint32_t)((j ^ rrow) << 4);
        const uint32_t dst8 = rowoff + (uint32_t)((((j & 1) << 2) ^ rrow) << 4) + (uint32_t)(j >> 1) * kTile;
        const uint32_t afull32 = smem_u32(&ctl.a_full[0]);
        uint32_t pc = 0;                 // pairs since the kernel started
        int slot = 0, rphase = 0;        // raw ring position
        bool ok = true;
        PfTile T{}, T1{};
        if ((int)blockIdx.x < n_tiles) T = pf_tile(L, blockIdx.x, n_routed, valid);
        for (int t = blockIdx.x; t < n_tiles && ok; t += G) {
            if (t + G < n_tiles) T1 = pf_tile(L, t + G, n_routed, valid);  // in flight during this tile
            const int quant = T.shared ? QS : QR;
            const int pitch = pf_raw_pitch(quant);
            const int span_bytes = span_bytes_of(quant);
            const uint32_t rowlo =
                (uint32_t)(uintptr_t)pf_row_ptr<MODE>(L, T, trow, (size_t)n_spans * span_bytes);
            for (int s = 0; s < n_spans && ok; ++s) {
                ok = stream_wait_pf(&ctl.raw_full[slot], rphase, abortp, L.status);
                if (!ok) break;
                const uint32_t rawrow =
                    raw32 + (uint32_t)slot * L.slot_bytes + trow * pitch + ((rowlo + s * span_bytes) & 15u);
                const uint32_t aj = (rawrow & ~3u) + 8 * j, sh = (rawrow & 2u) * 8, ps = rawrow + 192 + (j >> 1);
                float d6 = 0.f;
                if (quant == QUANT_Q6K)
                    d6 = __half2float(__ushort_as_half((unsigned short)lds_u16<208>(rawrow))) * kPfWeightScale;
                const uint32_t rj = rawrow + j * kQ8BlockBytes;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t aslot = pc & 1;
                    if (pc >= 2u) {
                        ok = stream_wait_pf(&ctl.a_empty[aslot], ((pc >> 1) & 1) ^ 1, abortp, L.status);
                        if (!ok) break;
                    }
                    const uint32_t a0 = a32 + aslot * kUnit;
                    if (quant == QUANT_Q6K) {
                        if (h == 0) unpack_q6k<0, kTile>(aj, sh, ps, d6, a0 + dst6);
                        else unpack_q6k<1, kTile>(aj, sh, ps, d6, a0 + dst6);
                    } else {
                        if (h == 0) unpack_q8<0>(rj, a0 + dst8);
                        else unpack_q8<1>(rj, a0 + dst8);
                    }
                    fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive32(afull32 + aslot * 8);
                    ++pc;
                }
                __syncwarp();
                if (ok && lane == 0) mbar_arrive_pf(&ctl.raw_empty[slot]);
                if (++slot == R) {
                    slot = 0;
                    rphase ^= 1;
                }
            }
            T = T1;
        }
    } else if (warp == kPfWideWarpB) {
        // -------------------------------- B loader --------------------------------
        // One thread: for every pair of chunks and every column tile of the item, two TMA copies
        // (chunk k0 and k0 + 64, token rows first + 128 ct .. + 127) into the next unit of the B ring.
        // Rows past the item's last column belong to a neighbour or are out of bounds (zero-filled);
        // their sums land in TMEM lanes that are never stored.
        if (lane == 0) {
            const int n_pairs = L.k / (2 * kPfChunkK);
            const uint32_t b32 = smem_u32(b_ring), bfull32 = smem_u32(&ctl.b_full[0]);
            int bslot = 0, bphase = 0;
            bool ok = true, wrapped = false;
            PfTile T{}, T1{};
            if ((int)blockIdx.x < n_tiles) T = pf_tile(L, blockIdx.x, n_routed, valid);
            for (int t = blockIdx.x; t < n_tiles && ok; t += G) {
                if (t + G < n_tiles) T1 = pf_tile(L, t + G, n_routed, valid);  // in flight during this tile
                const CUtensorMap* tm = T.shared ? &L.tm_shared : &L.tm_routed;
                const int nct = (T.ncols + kPfTileN - 1) / kPfTileN;
                for (int p = 0; p < n_pairs && ok; ++p) {
                    for (int ct = 0; ct < nct && ok; ++ct) {
                        if (wrapped) {
                            ok = stream_wait_pf(&ctl.b_empty[bslot], bphase ^ 1, abortp, L.status);
                            if (!ok) break;
                        }
                        const uint32_t bar = bfull32 + bslot * 8;
                        const uint32_t dst = b32 + (uint32_t)bslot * kUnit;
                        mbar_expect_tx32(bar, kUnit);
                        tma_load_tile_2d(dst, tm, p * 2 * kPfChunkK, T.first + ct * kPfTileN, bar);
                        tma_load_tile_2d(dst + kTile, tm, p * 2 * kPfChunkK + kPfChunkK, T.first + ct * kPfTileN, bar);
                        if (++bslot == NBU) {
                            bslot = 0;
                            bphase ^= 1;
                            wrapped = true;
                        }
                    }
                }
                T = T1;
            }
            // an abort elsewhere: give the copies this thread started time to land before the shared
            // memory goes to the next CTA (a TMA copy completes within microseconds)
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == kPfWarpMma) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const int n_pairs = L.k / (2 * kPfChunkK);
            const uint32_t a32 = smem_u32(a_ring), b32 = smem_u32(b_ring);
            uint32_t pc = 0;
            int bslot = 0, bphase = 0;
            uint32_t acc_base = 0, acc_used = 0, acc_par = 0;  // per-slot: used before / parity of the next wait
            bool ok = true;
            int ncols = (int)blockIdx.x < n_tiles ? pf_tile(L, blockIdx.x, n_routed, valid).ncols : 0;
            // D[token][weight row], as in k_prefill_gemm: the token tile is the M operand
            constexpr uint32_t idesc = umma_idesc_f16(kPfTileN, kPfTileM);
            for (int t = blockIdx.x; t < n_tiles && ok; t += G) {
                const int nct = (ncols + kPfTileN - 1) / kPfTileN;
                if (t + G < n_tiles) ncols = pf_tile(L, t + G, n_routed, valid).ncols;  // in flight during this tile
                for (int p = 0; p < n_pairs && ok; ++p, ++pc) {
                    const uint32_t aslot = pc & 1;
                    ok = stream_wait_pf(&ctl.a_full[aslot], (pc >> 1) & 1, abortp, L.status);
                    if (!ok) break;
                    const uint32_t a_addr = a32 + aslot * kUnit;
#pragma unroll
                    for (int ct = 0; ct < kPfWideMaxCt; ++ct) {
                        if (ct >= nct) break;
                        const uint32_t as = (acc_base + ct) & 3u;
                        if (p == 0 && (acc_used >> as & 1u)) {  // the slot's previous tile must have been drained
                            ok = stream_wait_pf(&ctl.acc_empty[as], acc_par >> as & 1u, abortp, L.status);
                            if (!ok) break;
                            acc_par ^= 1u << as;
                        }
                        ok = stream_wait_pf(&ctl.b_full[bslot], bphase, abortp, L.status);
                        if (!ok) break;
                        tc_fence_after();
                        fence_proxy_async_smem();  // the B tiles arrived by cp.async, not through the async proxy
                        const uint32_t b_addr = b32 + (uint32_t)bslot * kUnit;
                        const uint32_t tmem_d = tmem_base + as * kPfTileN;
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const uint64_t wdesc = umma_smem_desc(a_addr + half * kTile);  // weight rows
                            const uint64_t xdesc = umma_smem_desc(b_addr + half * kTile);  // token rows
#pragma unroll
                            for (int k4 = 0; k4 < kPfChunkK / 16; ++k4)
                                umma_f16(tmem_d, xdesc + 2 * k4, wdesc + 2 * k4, idesc,
                                         (p > 0 || half > 0 || k4 > 0) ? 1u : 0u);
                        }
                        umma_commit(&ctl.b_empty[bslot]);  // the unit is free once these MMAs have read it
                        if (++bslot == NBU) {
                            bslot = 0;
                            bphase ^= 1;
                        }
                    }
                    if (!ok) break;
                    umma_commit(&ctl.a_empty[aslot]);
                }
                if (!ok) break;
                for (int ct = 0; ct < nct; ++ct) {
                    const uint32_t as = (acc_base + ct) & 3u;
                    umma_commit(&ctl.acc_full[as]);
                    acc_used |= 1u << as;
                }
                acc_base = (acc_base + nct) & 3u;
            }
        }
    } else if (warp >= kPfWarpLoad && warp < kPfWarpEpi0) {
        // -------------------------------- loaders --------------------------------
        const int lw = warp - kPfWarpLoad, hw = lane >> 4, part = lane & 15;
        const uint32_t raw32 = smem_u32(raw_ring), rawfull32 = smem_u32(&ctl.raw_full[0]);
        int slot = 0, rphase = 0;
        bool ok = true, wrapped = false;
        PfTile T{}, T1{};
        if ((int)blockIdx.x < n_tiles) T = pf_tile(L, blockIdx.x, n_routed, valid);
        for (int t = blockIdx.x; t < n_tiles && ok; t += G) {
            if (t + G < n_tiles) T1 = pf_tile(L, t + G, n_routed, valid);  // in flight during this tile
            const int quant = T.shared ? QS : QR;
            const uint32_t pitch = pf_raw_pitch(quant);
            const uint32_t span_bytes = span_bytes_of(quant);
            const size_t row_bytes = (size_t)n_spans * span_bytes;
            const uint8_t* pg = pf_row_ptr<MODE>(L, T, 2 * lw + hw, row_bytes);
            const uint8_t* pu = MODE == MODE_GATEUP ? pf_row_ptr<MODE>(L, T, 16 + 2 * lw + hw, row_bytes) : pg;
            for (int s = 0; s < n_spans && ok; ++s) {
                if (wrapped) {
                    ok = stream_wait_pf(&ctl.raw_empty[slot], rphase ^ 1, abortp, L.status);
                    if (!ok) break;
                }
                const uint32_t dst0 = raw32 + (uint32_t)slot * L.slot_bytes + (uint32_t)(2 * lw + hw) * pitch + part * 16;
                const uint8_t* sg = pg + (size_t)s * span_bytes;
                const uint8_t* su = pu + (size_t)s * span_bytes;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int wr = MODE == MODE_GATEUP ? (i >> 3) * 16 + 4 * (i & 3) : 4 * i;
                    const uint8_t* p = ((MODE == MODE_GATEUP && (i & 4)) ? su : sg) + (size_t)wr * row_bytes;
                    const uint32_t mis = (uint32_t)(uintptr_t)p & 15u;
                    const uint32_t units = (mis + span_bytes + 15u) >> 4;
                    const uint8_t* src = p - mis + part * 16;
                    const uint32_t dst = dst0 + (uint32_t)(4 * i) * pitch;
                    if ((uint32_t)part < units) cp_async16(dst, src, 16u);
                    if ((uint32_t)part + 16u < units) cp_async16(dst + 256, src + 256, 16u);
                }
                cp_async_arrive_noinc32(rawfull32 + slot * 8);
                if (++slot == R) {
                    slot = 0;
                    rphase ^= 1;
                    wrapped = true;
                }
            }
            T = T1;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else {
        // ------------------------------- epilogue -------------------------------
        // As in k_prefill_gemm: thread (quad, lane) owns token column 32 quad + lane of a column tile;
        // a TMEM read is 32 consecutive tile rows of that token.
        const int quad = warp & 3;
        const int ew = MODE == MODE_DOWN ? warp - kPfWarpEpi0 : 0;
        const float inv = 1.0f / kPfWeightScale;
        uint32_t acc_base = 0, acc_par = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += G) {
            const PfTile T = pf_tile(L, t, n_routed, valid);
            const int nct = (T.ncols + kPfTileN - 1) / kPfTileN;
            for (int ct = 0; ct < nct && ok; ++ct) {
                const uint32_t as = (acc_base + ct) & 3u;
                const int first = T.first + ct * kPfTileN;
                const int ncols = min(kPfTileN, T.ncols - ct * kPfTileN);
                const int tok = quad * 32 + lane;
                const bool live = tok < ncols;
                // down, routed: the three dependent loads of the thread's token are issued before the wait
                float factor = inv;  // the weight scale is a power of two: folded into the routing weight exactly
                float* dst = nullptr;
                __half* hdst = nullptr;
                if (live) {
                    if (MODE == MODE_GATEUP) {
                        hdst = (T.shared ? L.inter_shared : L.inter_routed) + (size_t)(first + tok) * L.rows + T.bx * 64;
                    } else if (T.shared) {
                        dst = L.shexp + (size_t)(first + tok) * L.rows;
                    } else {
                        const int flat = __ldg(L.sorted_token_ids + first + tok);
                        factor = __ldg(L.topk_weights + flat) * inv;
                        dst = result_row(L.partial, L.partial_rows, flat, L.rows);
                    }
                    if (MODE == MODE_DOWN && dst) dst += T.bx * kPfTileM;
                }
                if (MODE == MODE_DOWN) {  // the warp's 32 row addresses (nullptr: nothing to store)
                    epi_dst[ew][lane] = dst;
                    __syncwarp();
                }
                ok = stream_wait_pf<true>(&ctl.acc_full[as], acc_par >> as & 1u, abortp, L.status);
                if (!ok) break;
                acc_par ^= 1u << as;
                tc_fence_after();
                const uint32_t taddr = tmem_base + as * kPfTileN + ((uint32_t)(quad * 32) << 16);
                const bool any_live = quad * 32 < ncols;  // the same for the whole warp
                for (int cb = 0; cb < kPfTileM / 32; ++cb) {
                    uint32_t r[32];
                    if (any_live) {
                        tmem_ld32(taddr + (uint32_t)(cb * 32), r);
                        tmem_ld_wait();
                    }
                    if (cb == kPfTileM / 32 - 1 || !any_live) {  // last read of this accumulator: hand it back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_pf(&ctl.acc_empty[as]);
                        if (!any_live) break;
                    }
                    if (MODE == MODE_GATEUP) {
                        if (hdst) {
                            uint32_t h[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float g0 = __uint_as_float(r[2 * i]) * inv, g1 = __uint_as_float(r[2 * i + 1]) * inv;
                                const float u0 = __uint_as_float(r[16 + 2 * i]) * inv,
                                            u1 = __uint_as_float(r[17 + 2 * i]) * inv;
                                const __half2 v = __floats2half2_rn(__fdiv_rn(g0, 1.0f + expf(-g0)) * u0,
                                                                    __fdiv_rn(g1, 1.0f + expf(-g1)) * u1);
                                h[i] = *(const uint32_t*)&v;
                            }
                            uint4* o = (uint4*)(hdst + cb * 16);
                            o[0] = make_uint4(h[0], h[1], h[2], h[3]);
                            o[1] = make_uint4(h[4], h[5], h[6], h[7]);
                        }
                    } else {
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const int q = half * 16 + 4 * c;
                                *(float4*)(epi_stage[ew] + lane * 16 + ((c ^ ((lane >> 1) & 3)) << 2)) =
                                    make_float4(factor * __uint_as_float(r[q]), factor * __uint_as_float(r[q + 1]),
                                                factor * __uint_as_float(r[q + 2]), factor * __uint_as_float(r[q + 3]));
                            }
                            __syncwarp();
#pragma unroll
                            for (int it = 0; it < 4; ++it) {
                                const int R = it * 8 + (lane >> 2), c = lane & 3;
                                const float4 v = *(const float4*)(epi_stage[ew] + R * 16 + ((c ^ ((R >> 1) & 3)) << 2));
                                float* p = epi_dst[ew][R];
                                if (p) *(float4*)(p + cb * 32 + half * 16 + c * 4) = v;
                            }
                            __syncwarp();
                        }
                    }
                }
            }
            acc_base = (acc_base + nct) & 3u;
        }
    }
    // every thread of the CTA arrives here on every path, so TMEM is always returned
    tc_fence_before();
    __syncthreads();
    if (warp == kPfWarpMma) tmem_dealloc(tmem_base, kPfWideMaxCt * kPfTileN);
}

}  // namespace xabe
