// Decode-width projections of ONE expert whose contraction is too long for k_expert_stream /
// k_gateup_rows to hold a token's activation row in shared memory: the dense SwiGLU block of the 27B
// sibling (hidden 5120, intermediate 17408; crates/xabe-engine/src/block/dense_ffn.rs:440-...), up
// to 64 tokens.  Before this kernel those shapes went through the tensor-core prefill kernel with
// one mostly empty 128-column tile.
//
// The ring carries SLICES of the contraction: a stage is one 256-element span of 128 weight rows
// (raw GGUF bytes, a 16-byte-aligned window per row) together with the same span of every token's
// activation row.  A consumer warp owns an m16 tile of output rows for its whole share of the
// contraction and keeps one fp32 accumulator tile per group of eight tokens, so the Q6_K / Q8_0
// unpack of a weight fragment is paid once for all tokens of the batch (1 shared load + 1 MMA +
// 4 FMA per further group of eight).
//
//   MODE_GATEUP: unit = 128 gate rows + the same 128 up rows; group gi of the CTA's two warp
//                groups takes rows 64 gi .. 64 gi + 63 (a stage holds 64 gate + 64 up rows); a
//                warp's fragment rows 0-7 are gate rows, 8-15 the same up rows; SwiGLU epilogue.
//   MODE_DOWN:   unit = 256 rows x one share of the contraction (`k_splits` shares, so that about
//                as many units as SMs exist although the matrix has few rows); a stage holds 128
//                rows; each share writes its own fp32 partial rows, summed in ascending order by
//                k_sum_k_splits.
//
// Arithmetic: exact integer codes as the f16 A operand, one k16 step per scale group, the fp32
// scale applied to the step's fp32 result, fp32 accumulation, spans in ascending order.  A token's
// value depends only on its own activation row: the accumulator tiles of different groups never mix.
//
// Four loader warps fill the ring with 16-byte asynchronous copies (sixteen lanes per weight row);
// every wait is bounded as in the other streaming kernels.
#pragma once

#include "prefill_kernels.cuh"
#include "stream_kernels.cuh"

namespace xabe {

constexpr int kDrLoadWarps = 4;
constexpr int kDrConsumerWarps = kStreamConsumerWarps;                 // two groups of eight
constexpr int kDrThreads = 32 * (kDrLoadWarps + kDrConsumerWarps);     // 640
constexpr int kDrStageRows = 128;                                      // weight row-spans per stage
constexpr int kDrMaxStages = 6;
constexpr int kDrXPitch = 512 + 32;  // bytes between the activation rows of a slice: a fragment load takes 32 bytes
                                     // of each of eight rows, so rows eight banks apart keep it at two wavefronts
constexpr int kDrMaxTokens = 64;

struct DenseRowsLaunch {
    const uint8_t* w_a;  // gate (or down)
    const uint8_t* w_b;  // up (MODE_GATEUP)
    int rows, k;         // output rows per matrix, contraction length
    const int* valid_tokens;
    const __half* x;     // [tokens][k]
    __half* inter;       // MODE_GATEUP out, [tokens][rows]
    float* out;          // MODE_DOWN out: [k_splits][max_tokens][rows]
    int* status;
    int max_tokens;
    int n_stages;
    int x_rows;          // activation rows a stage holds (8 x groups)
    int raw_pitch;       // bytes between the weight rows of a stage: 240 (Q6_K) or 304 (Q8_0), see dense_rows_pitch
    int k_splits;        // MODE_DOWN: shares of the contraction
};

// A row's span is copied as the 16-byte units that cover it (210 bytes starting up to 14 bytes into
// a unit: 14 units; 272 bytes: 18), and the rows of a stage sit 240 / 304 bytes apart: 60 / 76
// words, so the eight rows a fragment load touches start four banks apart and cover all 32 banks.
__host__ __device__ inline int dense_rows_pitch(int quant) { return quant == QUANT_Q6K ? 240 : 304; }

__host__ __device__ inline uint32_t dense_rows_stage_bytes(int raw_pitch, int x_rows) {
    return (uint32_t)(kDrStageRows * raw_pitch + x_rows * kDrXPitch);
}
__host__ __device__ inline uint32_t dense_rows_smem(int n_stages, int raw_pitch, int x_rows) {
    return (uint32_t)n_stages * dense_rows_stage_bytes(raw_pitch, x_rows) + 8u * 2u * kDrMaxStages + 128u + 64u;
}

// Half a span (8 k16 steps) for fragment rows pa / pb against NG groups of eight token columns.
// `xs`: this lane's column (row g of group 0) in the stage's activation slice.  (A run-time bound
// on the groups that hold live rows was measured: the loop it leaves costs more than the skipped
// groups save, 180 -> 240 us per layer at 64 tokens.)
template <int QUANT, bool MIS, int NG>
__device__ __forceinline__ void dense_half(const uint8_t* pa, const uint8_t* pb, int h, const uint8_t* xs, int lane,
                                           float (&acc)[NG][4]) {
    const uint32_t bias32 = 0x64206420u;   // half2(1056): 1024 + 32
    const uint32_t bias128 = 0x64806480u;  // half2(1152): 1024 + 128
    const int t = lane & 3;
    const int quad = lane & ~3;
    float own_a[2], own_b[2];
    // The B fragments of a step are fetched while the step before it is unpacked and multiplied, so
    // that no MMA waits for its shared-memory load.
    uint2 bnext[NG];
    auto fetch = [&](int st) {
        const uint8_t* xp = xs + 2 * step_k_offset<QUANT>(h, st, t);
#pragma unroll
        for (int q = 0; q < NG; ++q) bnext[q] = *(const uint2*)(xp + q * 8 * kDrXPitch);
    };
    fetch(0);
    auto step = [&](const uint32_t (&a)[4], float dsa, float dsb, int st) {
        uint2 b[NG];
#pragma unroll
        for (int q = 0; q < NG; ++q) b[q] = bnext[q];
        if (st < 7) fetch(st + 1);
#pragma unroll
        for (int q = 0; q < NG; ++q) {
            float d[4];
            mma_f16_16816(d, a, b[q].x, b[q].y);
            acc[q][0] = fmaf(dsa, d[0], acc[q][0]);
            acc[q][1] = fmaf(dsa, d[1], acc[q][1]);
            acc[q][2] = fmaf(dsb, d[2], acc[q][2]);
            acc[q][3] = fmaf(dsb, d[3], acc[q][3]);
        }
    };
    if (QUANT == QUANT_Q6K) {
        const float da = f16_at(pa + 208), db = f16_at(pb + 208);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int si = 192 + h * 8 + 2 * t + c;  // step c*4 + j with j == t (quant.rs:183,195-198)
            own_a[c] = da * (float)(int)(int8_t)pa[si];
            own_b[c] = db * (float)(int)(int8_t)pb[si];
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int off = h * 64 + 16 * c + 4 * t;
            const int offh = 128 + h * 32 + 16 * c + 4 * t;
            uint32_t ra[4], rb[4];
            q6k_codes4(ldw<MIS>(pa + off), ldw<MIS>(pa + off + 32), ldw<MIS>(pa + offh), ra);
            q6k_codes4(ldw<MIS>(pb + off), ldw<MIS>(pb + off + 32), ldw<MIS>(pb + offh), rb);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float dsa = __shfl_sync(0xffffffffu, own_a[c], quad | j);
                const float dsb = __shfl_sync(0xffffffffu, own_b[c], quad | j);
                uint32_t a[4];
                a[0] = bytes01_to_h2(ra[j], bias32);
                a[1] = bytes01_to_h2(rb[j], bias32);
                a[2] = bytes23_to_h2(ra[j], bias32);
                a[3] = bytes23_to_h2(rb[j], bias32);
                step(a, dsa, dsb, c * 4 + j);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // step 4*i + t of this half -> block h*4 + (4*i + t) / 2
            const int blk = h * 4 + ((4 * i + t) >> 1);
            own_a[i] = f16_at(pa + blk * kQ8BlockBytes);
            own_b[i] = f16_at(pb + blk * kQ8BlockBytes);
        }
#pragma unroll
        for (int st = 0; st < 8; ++st) {
            const int blk = h * 4 + (st >> 1), c = st & 1;
            const float dsa = __shfl_sync(0xffffffffu, own_a[st >> 2], quad | (st & 3));
            const float dsb = __shfl_sync(0xffffffffu, own_b[st >> 2], quad | (st & 3));
            const uint8_t* qa = pa + blk * kQ8BlockBytes + 2 + 16 * c + 4 * t;
            const uint8_t* qb = pb + blk * kQ8BlockBytes + 2 + 16 * c + 4 * t;
            const uint32_t wa = ((st >> 1) & 1 ? ldw<MIS>(qa) : ldw<!MIS>(qa)) ^ 0x80808080u;
            const uint32_t wb = ((st >> 1) & 1 ? ldw<MIS>(qb) : ldw<!MIS>(qb)) ^ 0x80808080u;
            uint32_t a[4];
            a[0] = bytes01_to_h2(wa, bias128);
            a[1] = bytes01_to_h2(wb, bias128);
            a[2] = bytes23_to_h2(wa, bias128);
            a[3] = bytes23_to_h2(wb, bias128);
            step(a, dsa, dsb, st);
        }
    }
}

// grid: number of SMs; block: kDrThreads (warps 0-1 load, warps 2-17 consume).
template <int MODE, int QUANT, int NG>
__global__ void __launch_bounds__(kDrThreads, 1) k_dense_rows(DenseRowsLaunch L) {
    extern __shared__ __align__(128) uint8_t dr_raw[];
    __shared__ int abort_flag;
    uint8_t* smem = dr_raw + ((128u - (smem_u32(dr_raw) & 127u)) & 127u);
    const int S = L.n_stages;
    const uint32_t stage_bytes = dense_rows_stage_bytes(L.raw_pitch, L.x_rows);
    uint64_t* full = (uint64_t*)(smem + (uint32_t)S * stage_bytes);
    uint64_t* empty = full + kDrMaxStages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], kDrLoadWarps * 32);  // every loader lane's copies of the stage have landed
            mbar_init(&empty[i], kStreamGroupWarps);
        }
        fence_mbar_init();
    }
    __syncthreads();
    volatile int* abortp = &abort_flag;
    const int valid = min(*L.valid_tokens, L.max_tokens);
    if (valid <= 0) return;
    constexpr int span_b = QUANT == QUANT_Q6K ? 210 : 272;
    const int n_spans = L.k / kSpanElems;
    const size_t row_bytes = (size_t)n_spans * span_b;
    constexpr int UNIT_ROWS = MODE == MODE_GATEUP ? 128 : 256;
    const int row_blocks = L.rows / UNIT_ROWS;
    const int KS = MODE == MODE_GATEUP ? 1 : L.k_splits;
    const int units = row_blocks * KS;
    // spans of contraction share ks: an even split, the first (n_spans % KS) shares one span longer
    auto share = [&](int ks, int& s0, int& s1) {
        const int base = n_spans / KS, extra = n_spans % KS;
        s0 = ks * base + min(ks, extra);
        s1 = s0 + base + (ks < extra ? 1 : 0);
    };

    if (warp < kDrLoadWarps) {
        // -------------------------------- loaders --------------------------------
        const int LL = warp * 32 + lane;                                  // 0 .. 127
        constexpr int ROWS_PER_PASS = kDrLoadWarps * 2;                   // sixteen lanes per weight row
        const int wrow = LL >> 4, wpart = LL & 15;
        const int xrow = LL >> 5, xpart = LL & 31;                        // activations: thirty-two lanes per row
        int st = 0;
        uint32_t use = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            const int rb = u / KS, ks = u - rb * KS;
            int s0, s1;
            share(ks, s0, s1);
            for (int s = s0; s < s1; ++s) {
#pragma unroll 1
                for (int gi = 0; gi < kStreamGroups; ++gi) {
                    if (use >= 1 && !stream_wait(&empty[st], (use - 1) & 1, abortp, L.status)) {
                        asm volatile("cp.async.wait_all;" ::: "memory");
                        return;
                    }
                    uint8_t* slot = smem + (uint32_t)st * stage_bytes;
                    const uint32_t slot32 = smem_u32(slot);
                    const int first_row = rb * UNIT_ROWS + gi * (UNIT_ROWS / 2);
                    // this lane's rows of the stage: wrow, wrow + 8, ...; the source pointer and the
                    // destination advance by a constant per pass
                    constexpr int HALVES = MODE == MODE_GATEUP ? 2 : 1;
                    constexpr int ROWS_EACH = kDrStageRows / HALVES;
#pragma unroll
                    for (int hm = 0; hm < HALVES; ++hm) {
                        const uint8_t* src = (hm == 0 ? L.w_a : L.w_b) + (size_t)(first_row + wrow) * row_bytes +
                                             (size_t)s * span_b;
                        uint32_t dst = slot32 + (uint32_t)(hm * ROWS_EACH + wrow) * L.raw_pitch + (uint32_t)wpart * 16u;
                        const size_t src_step = (size_t)ROWS_PER_PASS * row_bytes;
                        const uint32_t dst_step = (uint32_t)ROWS_PER_PASS * L.raw_pitch;
#pragma unroll 4
                        for (int r = 0; r < ROWS_EACH / ROWS_PER_PASS; ++r) {
                            const uint32_t off = (uint32_t)((uintptr_t)src & 15u);
                            const uint32_t chunks = (off + (uint32_t)span_b + 15u) >> 4;  // never past the span's last unit
                            const uint8_t* win = src - off + wpart * 16;
                            if ((uint32_t)wpart < chunks) cp_async16(dst, win, 16u);
                            if (QUANT != QUANT_Q6K && (uint32_t)wpart + 16u < chunks) cp_async16(dst + 256u, win + 256, 16u);
                            src += src_step;
                            dst += dst_step;
                        }
                    }
                    const uint32_t x32 = slot32 + (uint32_t)(kDrStageRows * L.raw_pitch);
                    for (int tk = xrow; tk < valid; tk += kDrLoadWarps)
                        cp_async16(x32 + (uint32_t)tk * kDrXPitch + (uint32_t)xpart * 16u,
                                   L.x + (size_t)tk * L.k + (size_t)s * kSpanElems + xpart * 8, 16u);
                    cp_async_arrive_noinc(&full[st]);
                    if (++st == S) {
                        st = 0;
                        ++use;
                    }
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        return;
    }

    // ---------------------------------- consumers ----------------------------------
    const int cw = warp - kDrLoadWarps;
    const int gi = cw / kStreamGroupWarps;  // which half of the unit's rows
    const int w = cw % kStreamGroupWarps;   // warp within the group
    const int g = lane >> 2, t = lane & 3;
    int st = gi % S;
    uint32_t use = (uint32_t)(gi / S);
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int rb = u / KS, ks = u - rb * KS;
        int s0, s1;
        share(ks, s0, s1);
        const int first_row = rb * UNIT_ROWS + gi * (UNIT_ROWS / 2);
        // fragment rows g and g + 8 of this warp: where they sit in a stage and in the matrices
        int ra_slot, rb_slot;
        uintptr_t ga, gb;  // global byte addresses of the two rows (only their low bits are used)
        if (MODE == MODE_GATEUP) {
            ra_slot = w * 8 + g;
            rb_slot = 64 + w * 8 + g;
            ga = (uintptr_t)(L.w_a + (size_t)(first_row + w * 8 + g) * row_bytes);
            gb = (uintptr_t)(L.w_b + (size_t)(first_row + w * 8 + g) * row_bytes);
        } else {
            ra_slot = w * 16 + g;
            rb_slot = w * 16 + g + 8;
            ga = (uintptr_t)(L.w_a + (size_t)(first_row + ra_slot) * row_bytes);
            gb = (uintptr_t)(L.w_a + (size_t)(first_row + rb_slot) * row_bytes);
        }
        float acc[NG][4];
#pragma unroll
        for (int q = 0; q < NG; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[q][i] = 0.f;
        for (int s = s0; s < s1; ++s) {
            if (!stream_wait(&full[st], use & 1, abortp, L.status)) return;
            const uint8_t* slot = smem + (uint32_t)st * stage_bytes;
            const uint8_t* pa = slot + (uint32_t)ra_slot * L.raw_pitch + (uint32_t)((ga + (size_t)s * span_b) & 15u);
            const uint8_t* pb = slot + (uint32_t)rb_slot * L.raw_pitch + (uint32_t)((gb + (size_t)s * span_b) & 15u);
            const uint8_t* xs = slot + (uint32_t)(kDrStageRows * L.raw_pitch) + (uint32_t)g * kDrXPitch;
            // every row pitch is a multiple of four bytes (checked by the host), so the two rows and
            // all lanes of the warp share one word alignment
            if ((uintptr_t)pa & 2) {
                dense_half<QUANT, true, NG>(pa, pb, 0, xs, lane, acc);
                dense_half<QUANT, true, NG>(pa, pb, 1, xs, lane, acc);
            } else {
                dense_half<QUANT, false, NG>(pa, pb, 0, xs, lane, acc);
                dense_half<QUANT, false, NG>(pa, pb, 1, xs, lane, acc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);  // the ring stage may be refilled
            st += kStreamGroups;
            if (st >= S) {
                st -= S;
                ++use;
            }
        }
        if (MODE == MODE_GATEUP) {
            // SwiGLU of this warp's eight rows: acc[.][0..1] gate, acc[.][2..3] up, columns 2t and 2t + 1
            const int row = first_row + w * 8 + g;
#pragma unroll
            for (int q = 0; q < NG; ++q)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int tok = q * 8 + 2 * t + i;
                    if (tok < valid) {
                        const float gv = acc[q][i], uv = acc[q][2 + i];
                        L.inter[(size_t)tok * L.rows + row] = __float2half_rn(__fdiv_rn(gv, 1.0f + expf(-gv)) * uv);
                    }
                }
        } else {
            const int row_lo = first_row + ra_slot, row_hi = first_row + rb_slot;
            float* dst = L.out + (size_t)ks * L.max_tokens * L.rows;
#pragma unroll
            for (int q = 0; q < NG; ++q)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int tok = q * 8 + 2 * t + i;
                    if (tok < valid) {
                        dst[(size_t)tok * L.rows + row_lo] = acc[q][i];
                        dst[(size_t)tok * L.rows + row_hi] = acc[q][2 + i];
                    }
                }
        }
    }
}

// out[t][j] = sum over ascending ks of partial[ks][t][j] for the live rows (MODE_DOWN with several
// shares of the contraction).  grid: (max_tokens, ceil(rows / 256)), block 256.
__global__ void __launch_bounds__(256) k_sum_k_splits(const float* __restrict__ partial, int k_splits,
                                                      int max_tokens, int rows,
                                                      const int* __restrict__ valid_tokens,
                                                      float* __restrict__ out) {
    const int tk = blockIdx.x;
    if (tk >= *valid_tokens) return;
    const int j = blockIdx.y * 256 + threadIdx.x;
    if (j >= rows) return;
    float r = 0.0f;
    for (int ks = 0; ks < k_splits; ++ks) r += partial[((size_t)ks * max_tokens + tk) * rows + j];
    out[(size_t)tk * rows + j] = r;
}

}  // namespace xabe
