// Prefill-shaped expert projections: a persistent, warp-specialised grouped
// GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// A tile is D[128 weight rows][128 token columns] of one expert (or of the
// shared expert); every CTA (one per SM) walks tiles blockIdx.x, + gridDim.x,
// ...  The contraction runs in chunks of 64 elements.  Four roles:
//   * two loader warps: asynchronous 16-byte copies (cp.async, sixteen lanes per
//     weight row so that a row's bytes are read as whole cache lines) bring the
//     raw GGUF bytes of a 256-element span of all 128 rows (a 210-byte Q6_K
//     superblock or eight 34-byte Q8_0 blocks per row, widened to 16-byte
//     boundaries) into a ring of raw slots.  One bulk copy (TMA) per row was
//     tried first: at 224 bytes per copy the copy engine, not memory, set the pace;
//   * sixteen unpack warps: read the raw bytes from shared memory, unpack,
//     scale and write f16 values into the A tile of a stage in the
//     128-byte-swizzled K-major layout the tensor core reads, and start the
//     asynchronous 16-byte copies that gather the 128 token rows (B tile);
//   * one thread issues four tcgen05.mma (M128 N128 K16, f16 x f16 -> f32) per
//     stage and commits them to the stage's "empty" barrier; two accumulators
//     in TMEM alternate between tiles.  The token tile is the M operand, the
//     weight tile the N operand: D[token][weight row];
//   * four epilogue warps read a finished accumulator with tcgen05.ld (a thread
//     = one token, 32 consecutive weight rows per read) and apply SwiGLU
//     (gate/up) or the routing weight (down), storing 16 bytes at a time, while
//     the other roles are already on the next tile.
//
// Numerics: weights are rounded to f16 after the fp32-exact code is multiplied
// by the f16-rounded group scale (times 256, undone in the epilogue, which
// keeps small super-scales out of the f16 subnormal range); activations are
// f16; accumulation is fp32 in TMEM.  This differs from the decode kernels
// (exact codes, fp32 scales) by the weight rounding, about 2e-4 relative per
// weight, and stays inside the rel-L2 <= 1e-3 gate.
//
// Every wait is bounded; TMEM is freed on every exit path.
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the encoder is looked up at run time)

#include "common.cuh"
#include "glue_kernels.cuh"

namespace xabe {

constexpr int kPfTileM = 128;       // weight rows per tile (TMEM lanes)
constexpr int kPfTileN = 128;       // token columns per tile
constexpr int kPfChunkK = 64;       // contraction elements per stage (one 128-byte swizzle row of f16)
constexpr int kPfTileBytes = kPfTileM * kPfChunkK * 2;        // one A or B chunk tile: 16 KB
constexpr int kPfStageBytes = 2 * kPfTileBytes;                // A tile + B tile
constexpr int kPfUnpackWarps = 16;
constexpr int kPfWarpMma = 16;
constexpr int kPfWarpLoad = 17;     // two loader warps
constexpr int kPfLoadWarps = 2;
constexpr int kPfWarpEpi0 = 19;     // four epilogue warps; warp % 4 is the TMEM lane quadrant a warp may read
constexpr int kPfThreads = 32 * 23;
constexpr int kPfMaxStages = 4;     // two pairs of chunks
constexpr int kPfMaxRaw = 3;        // raw slots (one span of all 128 rows each)
constexpr int kPfAccums = 2;
constexpr int kPfRawPitchQ6K = 224;   // 210 bytes starting up to 14 bytes into a 16-byte unit
constexpr int kPfRawPitchQ8 = 288;    // 272 bytes likewise
constexpr float kPfWeightScale = 256.0f;
constexpr int kPfItemInts = 4;  // expert, first slot (or first token), columns, pad

__host__ __device__ inline int pf_raw_pitch(int quant) { return quant == QUANT_Q6K ? kPfRawPitchQ6K : kPfRawPitchQ8; }

struct PrefillLaunch {
    const uint8_t* r_a;  // routed gate (or down)
    const uint8_t* r_b;  // routed up
    const uint8_t* s_a;  // shared gate (or down)
    const uint8_t* s_b;  // shared up
    int rows;            // output rows per matrix
    int k;               // contraction length
    int top_k;
    int has_routed, has_shared;
    const int* items;    // token tiles of the routed experts (kPfItemInts each)
    const int* n_items;  // device scalar
    const int* valid_tokens;
    const int* sorted_token_ids;
    const float* topk_weights;
    const __half* x_routed;  // gate/up: normed_h [token]; down: inter [slot]
    const __half* x_shared;  // gate/up: normed_h [token]; down: inter_shared [token]
    __half* inter_routed;
    __half* inter_shared;
    float* partial;
    float* const* partial_rows;  // optional: destination of result row `flat` instead of partial (NULL: use partial)
    float* shexp;
    int* status;
    int n_stages;    // A/B stages (even)
    int n_raw;       // raw slots
    int slot_bytes;  // 128 * the larger raw pitch of the formats in this launch
    int row_tiles;   // tiles along the weight rows: gate/up rows / 64, down rows / 128
    int item_cols;   // token columns per item: 128, or 512 for k_prefill_gemm_wide
    int n_b_units;   // k_prefill_gemm_wide: depth of the B ring
    // k_prefill_gemm_wide: 2-D tiled maps ([rows][k] f16, box 64 x 128, 128-byte swizzle) of the routed
    // and the shared activation rows; a routed item's columns are CONSECUTIVE rows of its source
    CUtensorMap tm_routed, tm_shared;
    int max_tokens;
};

// ---- tcgen05 / TMEM wrappers ------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], one M128 x N128 x K16 step.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle:
// rows are 128 bytes (64 f16), eight rows form a 1024-byte group, groups are
// 1024 bytes apart.  Bits: [0,14) address >> 4, [16,30) leading offset >> 4
// (unused with swizzle, 1), [32,46) stride between row groups >> 4, [46,48)
// descriptor version 1, [61,64) layout 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D f32 (bits 4-5 = 1), A and B f16 (0),
// both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Byte offset of the 16-byte chunk `chunk` (8 f16) of row `row` inside a
// swizzled 128-row tile: chunk index XOR (row mod 8), i.e. Swizzle<3,4,3>.
__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

// Eight exact codes (two words of four bytes) -> four half2 scaled by ds2.
__device__ __forceinline__ uint4 codes8_to_h8(uint32_t c0, uint32_t c1, uint32_t bias, __half2 ds2) {
    uint4 o;
    __half2 v;
    uint32_t t;
    t = bytes01_to_h2(c0, bias); v = __hmul2(*(__half2*)&t, ds2); o.x = *(uint32_t*)&v;
    t = bytes23_to_h2(c0, bias); v = __hmul2(*(__half2*)&t, ds2); o.y = *(uint32_t*)&v;
    t = bytes01_to_h2(c1, bias); v = __hmul2(*(__half2*)&t, ds2); o.z = *(uint32_t*)&v;
    t = bytes23_to_h2(c1, bias); v = __hmul2(*(__half2*)&t, ds2); o.w = *(uint32_t*)&v;
    return o;
}

// 16-byte asynchronous copy global -> shared (zero-filled when src_bytes is 0), and the arrival it
// triggers on an mbarrier once all of this thread's earlier copies have landed.  The arrival does
// not raise the barrier's pending count: the count it was initialised with includes it.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory accesses of the unpack warps, by 32-bit shared address plus a compile-time
// offset, so that the per-lane address arithmetic is done once per span and not per access.
template <int OFF> __device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ int lds_s8(uint32_t a) {
    int v;
    asm volatile("ld.shared.s8 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ void sts_v4(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0+%1], {%2, %3, %4, %5};" ::"r"(a), "n"(OFF), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}
// Eight bytes that start sh / 8 (0 or 2) bytes after the word-aligned shared address al + OFF.
// The third word read lies inside the same raw row for every piece this is used on.
template <int OFF> __device__ __forceinline__ void lds8_shifted(uint32_t al, uint32_t sh, uint32_t (&o)[2]) {
    uint32_t a = lds_u32<OFF>(al), b = lds_u32<OFF + 4>(al), c = lds_u32<OFF + 8>(al);
    o[0] = __funnelshift_r(a, b, sh);
    o[1] = __funnelshift_r(b, c, sh);
}

// One unpack pass: eight weight rows x one PAIR of chunks (128 contraction elements); lane
// (row rrow of the eight, j = lane % 4) produces 32 weights (four 16-byte chunks).
//
// Q6_K, half H of the row's superblock (element map of crates/xabe-kernels/src/quant.rs:175-198):
// positions l = 8j..8j+7 of the four 32-element groups.  aj: word-aligned address of (superblock
// + 8j), sh its distance in bits to the true start; ps: superblock + 192 + j/2; d: the super-scale
// times 256.  Group g goes to chunk (g % 2) * 4 + j of stage g / 2: `dst` is the lane's row and
// chunk j in the first stage's A tile (swizzle applied); chunk 4 + j is dst ^ 64.
template <int H, int OFF2 = kPfStageBytes>
__device__ __forceinline__ void unpack_q6k(uint32_t aj, uint32_t sh, uint32_t ps, float d, uint32_t dst) {
    uint32_t ql0[2], ql1[2], qh[2];
    lds8_shifted<H * 64>(aj, sh, ql0);
    lds8_shifted<H * 64 + 32>(aj, sh, ql1);
    lds8_shifted<128 + H * 32>(aj, sh, qh);
    int sc[4];
    sc[0] = lds_s8<H * 8 + 0>(ps);  // scale index H*8 + 2g + l/16
    sc[1] = lds_s8<H * 8 + 2>(ps);
    sc[2] = lds_s8<H * 8 + 4>(ps);
    sc[3] = lds_s8<H * 8 + 6>(ps);
    const uint32_t dstx = dst ^ 64u;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint32_t* ql = (g & 1) ? ql1 : ql0;
        uint32_t c[2];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            uint32_t nib = (g >> 1) ? (ql[w] >> 4) : ql[w];
            uint32_t two = g == 0 ? (qh[w] << 4) : g == 1 ? (qh[w] << 2) : g == 2 ? qh[w] : (qh[w] >> 2);
            c[w] = (nib & 0x0F0F0F0Fu) | (two & 0x30303030u);
        }
        __half2 ds2 = __float2half2_rn(d * (float)sc[g]);
        uint4 v = codes8_to_h8(c[0], c[1], 0x64206420u, ds2);
        if (g == 0) sts_v4<0>(dst, v);
        else if (g == 1) sts_v4<0>(dstx, v);
        else if (g == 2) sts_v4<OFF2>(dst, v);  // OFF2: distance from the pair's first A tile to its second
        else sts_v4<OFF2>(dstx, v);
    }
}
// Q8_0, pair H of the span: the lane's block is number 4H + j of the row's eight.  rj: the row's
// raw bytes + 34j (2-byte aligned).  `dst`: the lane's row, chunk (j % 2) * 4 of stage j / 2
// (swizzle applied); chunk + t is dst ^ (16 t).
template <int H>
__device__ __forceinline__ void unpack_q8(uint32_t rj, uint32_t dst) {
    const uint32_t p = rj + 2;  // the codes
    const uint32_t al = p & ~3u, sh = (p & 2u) * 8;
    uint32_t a[9];
    a[0] = lds_u32<H * 136 + 0>(al);
    a[1] = lds_u32<H * 136 + 4>(al);
    a[2] = lds_u32<H * 136 + 8>(al);
    a[3] = lds_u32<H * 136 + 12>(al);
    a[4] = lds_u32<H * 136 + 16>(al);
    a[5] = lds_u32<H * 136 + 20>(al);
    a[6] = lds_u32<H * 136 + 24>(al);
    a[7] = lds_u32<H * 136 + 28>(al);
    a[8] = lds_u32<H * 136 + 32>(al);  // may lie past the block: the raw ring ends with padding for it
    const float d = __half2float(__ushort_as_half((unsigned short)lds_u16<H * 136>(rj))) * kPfWeightScale;
    __half2 ds2 = __float2half2_rn(d);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        uint32_t w0 = __funnelshift_r(a[2 * t], a[2 * t + 1], sh) ^ 0x80808080u;
        uint32_t w1 = __funnelshift_r(a[2 * t + 1], a[2 * t + 2], sh) ^ 0x80808080u;
        sts_v4<0>(dst ^ (uint32_t)(t << 4), codes8_to_h8(w0, w1, 0x64806480u, ds2));
    }
}

template <int DST_OFF, int SRC_OFF>
__device__ __forceinline__ void cp_async16_off(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0+%1], [%2+%3], 16;" ::"r"(dst_smem), "n"(DST_OFF), "l"(src),
                 "n"(SRC_OFF)
                 : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc32(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive32(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_pf(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait that also gives up when another warp of the CTA already has.  try_wait itself
// suspends the thread for a hardware-defined slice, so the roles inside the per-pair pipeline poll
// without sleeping (a sleeping waiter adds its sleep to every hand-over); only the epilogue warps,
// which wait for a whole tile, back off.
template <bool BACKOFF = false>
__device__ __forceinline__ bool stream_wait_pf(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* status) {
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u && *abort_flag) return false;
        if (BACKOFF && it >= 16u) __nanosleep(it < 256u ? 32u : 256u);
    }
    *abort_flag = 1;
    if (status) atomicExch(status, STATUS_TMA_TIMEOUT);
    return false;
}

// Token tiles of the routed experts for the prefill kernels: the live slots of
// expert e are contiguous from expert_offsets[e]; they are cut into runs of up
// to `item_cols` (128, or 512 for the kernel that keeps four accumulators).  One block, one thread
// per expert.
__global__ void k_build_prefill_items(int num_experts, const int* __restrict__ expert_offsets,
                                      const int* __restrict__ expert_counts, int* __restrict__ items,
                                      int* __restrict__ n_items, int item_cols) {
    __shared__ int warp_sums[33];
    int e = threadIdx.x;
    const int mine = e < num_experts ? (expert_counts[e] + item_cols - 1) / item_cols : 0;
    int total = 0;
    const int base = block_exclusive_scan(mine, warp_sums, &total);
    if (e == 0) *n_items = total;
    if (e < num_experts) {
        int count = expert_counts[e], start = expert_offsets[e];
        for (int i = 0; i * item_cols < count; ++i) {
            int* it = items + (size_t)(base + i) * kPfItemInts;
            it[0] = e;
            it[1] = start + i * item_cols;
            it[2] = min(item_cols, count - i * item_cols);
            it[3] = 0;
        }
    }
}

// One tile of the walk: which expert (or the shared expert), which token columns, which row tile.
struct PfTile {
    int shared, expert, first, ncols, bx;
};
__device__ __forceinline__ PfTile pf_tile(const PrefillLaunch& L, int t, int n_routed, int valid) {
    PfTile T;
    const int y = t / L.row_tiles;
    T.bx = t - y * L.row_tiles;
    T.shared = y >= n_routed;
    if (!T.shared) {
        const int* it = L.items + (size_t)y * kPfItemInts;
        T.expert = __ldg(it);
        T.first = __ldg(it + 1);
        T.ncols = __ldg(it + 2);
    } else {
        T.expert = 0;
        T.first = (y - n_routed) * L.item_cols;
        T.ncols = min(L.item_cols, valid - T.first);
    }
    return T;
}

// Address of tile row r's weight row.  Gate/up tiles interleave the two matrices in groups of 16
// rows: tile row 32q + i is gate row 64 bx + 16q + i for i < 16, up row 64 bx + 16q + (i - 16) otherwise.
template <int MODE>
__device__ __forceinline__ const uint8_t* pf_row_ptr(const PrefillLaunch& L, const PfTile& T, int r,
                                                     size_t row_bytes) {
    const uint8_t* base;
    size_t wrow;
    if (MODE == MODE_GATEUP) {
        const int i = r & 31;
        base = i < 16 ? (T.shared ? L.s_a : L.r_a) : (T.shared ? L.s_b : L.r_b);
        wrow = (size_t)T.bx * 64 + (r >> 5) * 16 + (i & 15);
    } else {
        base = T.shared ? L.s_a : L.r_a;
        wrow = (size_t)T.bx * kPfTileM + r;
    }
    return base + ((T.shared ? 0 : (size_t)T.expert * L.rows) + wrow) * row_bytes;
}

// Shared-memory control block of the kernel.
struct PfCtl {
    uint64_t full_bar[kPfMaxStages / 2];    // per PAIR of stages: unpack warps + their B-tile copies -> MMA
    uint64_t empty_bar[kPfMaxStages / 2];   // MMA (tcgen05.commit) -> unpack warps
    uint64_t raw_full[kPfMaxRaw];       // bulk copies landed -> unpack warps
    uint64_t raw_empty[kPfMaxRaw];      // unpack warps -> loader
    uint64_t acc_full[kPfAccums];       // MMA (tcgen05.commit) -> epilogue
    uint64_t acc_empty[kPfAccums];      // epilogue -> MMA
    uint32_t tmem_base;
    int abort_flag;
};

// The accumulator is D[token][tile row]: TMEM lane = token column of the tile, TMEM column = tile row.
// MODE_GATEUP (0): tile row m = 32q + i is gate row r0 + 16q + i for i < 16 and up row
// r0 + 16q + (i - 16) otherwise (r0 = 64 * bx), so SwiGLU pairs two columns of one lane.
// MODE_DOWN (1): tile row m is row 128 * bx + m.
// grid: one CTA per SM (or fewer); block kPfThreads.
template <int MODE, int QR, int QS>
__global__ void __launch_bounds__(kPfThreads, 1) k_prefill_gemm(PrefillLaunch L) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) PfCtl ctl;
    // MODE_DOWN: an epilogue warp turns 32 tokens x 16 outputs around in shared memory, so that four
    // lanes store 64 neighbouring bytes of one result row instead of every lane 16 bytes of a row of its
    // own (32 rows per store instruction: slow through L1, and slower still when the rows are in
    // another GPU's memory, as with a caller's table of result rows).
    __shared__ __align__(16) float epi_stage[MODE == MODE_DOWN ? 4 : 1][MODE == MODE_DOWN ? 32 * 16 : 4];
    __shared__ float* epi_dst[MODE == MODE_DOWN ? 4 : 1][32];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int valid = *L.valid_tokens;
    const int n_routed = L.has_routed ? *L.n_items : 0;
    const int n_shared = L.has_shared ? (valid + L.item_cols - 1) / L.item_cols : 0;
    const int n_tiles = (n_routed + n_shared) * L.row_tiles;
    const int R = L.n_raw;
    const int n_spans = L.k / kSpanElems;
    uint8_t* stages = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* raw_ring = stages + (size_t)kPfMaxStages * kPfStageBytes;
    volatile int* abortp = &ctl.abort_flag;

    if (tid == 0) {
        ctl.abort_flag = 0;
        for (int i = 0; i < kPfMaxStages / 2; ++i) {
            // one arrival per unpack warp (A tiles written) + one per unpack thread (its B-tile copies landed)
            mbar_init(&ctl.full_bar[i], kPfUnpackWarps + kPfUnpackWarps * 32);
            mbar_init(&ctl.empty_bar[i], 1);
        }
        for (int i = 0; i < R; ++i) {
            mbar_init(&ctl.raw_full[i], kPfLoadWarps * 32);  // every loader lane's copies landed
            mbar_init(&ctl.raw_empty[i], kPfUnpackWarps);
        }
        for (int i = 0; i < kPfAccums; ++i) {
            mbar_init(&ctl.acc_full[i], 1);
            mbar_init(&ctl.acc_empty[i], 4);
        }
        fence_mbar_init();
    }
    if (warp == kPfWarpMma) {
        tmem_alloc(&ctl.tmem_base, kPfAccums * kPfTileN);  // two accumulators of 128 fp32 columns
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl.tmem_base;

    constexpr int S = kPfMaxStages;
    if (warp < kPfUnpackWarps) {
        // ------------------------------ unpack warps ------------------------------
        // Per pair of chunks: this warp unpacks tile rows 8w..8w+7 (32 weights per lane) and every
        // thread starts up to four 16-byte copies of the B tiles (token columns tid/8 and tid/8 + 64
        // of both stages; columns the tile does not have are skipped: the tensor core reads stale rows
        // there, whose sums land in TMEM lanes nobody stores).
        // Lanes 4q..4q+3 serve one row; eight consecutive lanes (the unit a 128-bit shared store is
        // processed in) serve rows r and r + 4, whose chunks fall into different halves of the
        // swizzled 128-byte line, so the A-tile stores are free of bank conflicts.
        const int rrow = ((lane >> 2) & 1) * 4 + (lane >> 3), j = lane & 3;
        const int trow = 8 * warp + rrow;
        const int r0 = tid >> 3, piece = tid & 7;
        const uint32_t stages32 = smem_u32(stages), raw32 = smem_u32(raw_ring);
        const uint32_t boff = (uint32_t)(kPfTileM * kPfChunkK * 2) + swz_off(r0, piece);
        const uint32_t rowoff = (uint32_t)(warp * 1024 + rrow * 128);
        const uint32_t dst6 = rowoff + (uint32_t)((j ^ rrow) << 4);
        const uint32_t dst8 = rowoff + (uint32_t)((((j & 1) << 2) ^ rrow) << 4) + (uint32_t)(j >> 1) * kPfStageBytes;
        const uint32_t full32 = smem_u32(&ctl.full_bar[0]), empty32 = smem_u32(&ctl.empty_bar[0]);
        uint32_t kc = 0;              // chunks since the kernel started
        int slot = 0, rphase = 0;     // raw ring position
        bool ok = true;
        // Tile metadata runs two tiles ahead of the work (the tile record) and one ahead (the token
        // rows, whose addresses come from the record), so no tile starts by waiting for global loads.
        auto token_rows = [&](const PfTile& T, int (&xo)[2]) {
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int c = r0 + 64 * m;
                int src = -1;
                if (c < T.ncols) {
                    if (T.shared || MODE == MODE_DOWN) src = T.first + c;
                    else src = __ldg(L.sorted_token_ids + T.first + c) / L.top_k;
                }
                xo[m] = src;
            }
        };
        const int G = gridDim.x;
        PfTile T{}, T1{}, T2{};
        int xrow[2] = {-1, -1}, xrow1[2] = {-1, -1};
        if ((int)blockIdx.x < n_tiles) {
            T = pf_tile(L, blockIdx.x, n_routed, valid);
            token_rows(T, xrow);
        }
        if ((int)blockIdx.x + G < n_tiles) T1 = pf_tile(L, blockIdx.x + G, n_routed, valid);
        for (int t = blockIdx.x; t < n_tiles && ok; t += G) {
            if (t + G < n_tiles) token_rows(T1, xrow1);
            if (t + 2 * G < n_tiles) T2 = pf_tile(L, t + 2 * G, n_routed, valid);
            const int quant = T.shared ? QS : QR;
            const int pitch = pf_raw_pitch(quant);
            const int span_bytes = span_bytes_of(quant);
            // where in its 16-byte unit the lane's weight row starts (the loaders copy whole units)
            const uint32_t rowlo =
                (uint32_t)(uintptr_t)pf_row_ptr<MODE>(L, T, trow, (size_t)n_spans * span_bytes);
            const __half* xb = T.shared ? L.x_shared : L.x_routed;
            const __half* xp0 = xb + (size_t)(xrow[0] < 0 ? 0 : xrow[0]) * L.k + piece * 8;
            const __half* xp1 = xb + (size_t)(xrow[1] < 0 ? 0 : xrow[1]) * L.k + piece * 8;
            const bool live0 = xrow[0] >= 0, live1 = xrow[1] >= 0;
            for (int s = 0; s < n_spans && ok; ++s) {
                ok = stream_wait_pf(&ctl.raw_full[slot], rphase, abortp, L.status);
                if (!ok) break;
                const uint32_t rawrow =
                    raw32 + (uint32_t)slot * L.slot_bytes + trow * pitch + ((rowlo + s * span_bytes) & 15u);
                // Q6_K
                const uint32_t aj = (rawrow & ~3u) + 8 * j, sh = (rawrow & 2u) * 8, ps = rawrow + 192 + (j >> 1);
                float d6 = 0.f;
                if (quant == QUANT_Q6K)
                    d6 = __half2float(__ushort_as_half((unsigned short)lds_u16<208>(rawrow))) * kPfWeightScale;
                // Q8_0
                const uint32_t rj = rawrow + j * kQ8BlockBytes;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t st0 = kc & (S - 1);  // even: the pair's stages are st0 and st0 + 1
                    if (kc >= (uint32_t)S) {
                        const uint32_t par = ((kc / S) & 1) ^ 1;
                        ok = stream_wait_pf(&ctl.empty_bar[st0 >> 1], par, abortp, L.status);
                        if (!ok) break;
                    }
                    const uint32_t a0 = stages32 + st0 * kPfStageBytes;
                    const uint32_t fb = full32 + (st0 >> 1) * 8;
                    if (live0) {
                        cp_async16_off<0, 0>(a0 + boff, xp0);
                        cp_async16_off<kPfStageBytes, 128>(a0 + boff, xp0);
                    }
                    if (live1) {
                        cp_async16_off<8192, 0>(a0 + boff, xp1);
                        cp_async16_off<kPfStageBytes + 8192, 128>(a0 + boff, xp1);
                    }
                    cp_async_arrive_noinc32(fb);
                    xp0 += 2 * kPfChunkK;
                    xp1 += 2 * kPfChunkK;
                    if (quant == QUANT_Q6K) {
                        if (h == 0) unpack_q6k<0>(aj, sh, ps, d6, a0 + dst6);
                        else unpack_q6k<1>(aj, sh, ps, d6, a0 + dst6);
                    } else {
                        if (h == 0) unpack_q8<0>(rj, a0 + dst8);
                        else unpack_q8<1>(rj, a0 + dst8);
                    }
                    fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive32(fb);
                    kc += 2;
                }
                __syncwarp();
                if (ok && lane == 0) mbar_arrive_pf(&ctl.raw_empty[slot]);
                if (++slot == R) {
                    slot = 0;
                    rphase ^= 1;
                }
            }
            T = T1;
            T1 = T2;
            xrow[0] = xrow1[0];
            xrow[1] = xrow1[1];
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == kPfWarpMma) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const int n_chunks = L.k / kPfChunkK;
            const int G = gridDim.x;
            uint32_t kc = 0, n = 0;
            bool ok = true;
            // D[token][weight row]: the TOKEN tile is the M operand, so a TMEM lane (= an epilogue thread)
            // holds one token's outputs for consecutive weight rows and stores them 16 bytes at a time.
            // Token rows past the tile's count hold whatever the stage held before; each lane's sums
            // depend on its own row only, and those lanes are never stored.
            constexpr uint32_t idesc = umma_idesc_f16(kPfTileN, kPfTileM);
            for (int t = blockIdx.x; t < n_tiles && ok; t += G, ++n) {
                const uint32_t acc = n % kPfAccums;
                if (n >= (uint32_t)kPfAccums) {
                    ok = stream_wait_pf(&ctl.acc_empty[acc], (n / kPfAccums - 1) & 1, abortp, L.status);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t tmem_d = tmem_base + acc * kPfTileN;
                for (int c = 0; c < n_chunks && ok; c += 2, kc += 2) {
                    const int st = kc & (S - 1);  // the pair's stages are st and st + 1
                    ok = stream_wait_pf(&ctl.full_bar[st >> 1], (kc / S) & 1, abortp, L.status);
                    if (!ok) break;
                    tc_fence_after();
                    fence_proxy_async_smem();  // the B tiles arrived by cp.async, not through the async proxy
                    const uint32_t a_addr = smem_u32(stages + (size_t)st * kPfStageBytes);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const uint64_t wdesc = umma_smem_desc(a_addr + half * kPfStageBytes);  // weight rows
                        const uint64_t xdesc = umma_smem_desc(a_addr + half * kPfStageBytes + kPfTileM * kPfChunkK * 2);
#pragma unroll
                        for (int k4 = 0; k4 < kPfChunkK / 16; ++k4)  // 32 bytes per K16 step inside the swizzle row
                            umma_f16(tmem_d, xdesc + 2 * k4, wdesc + 2 * k4, idesc,
                                     (c > 0 || half > 0 || k4 > 0) ? 1u : 0u);
                    }
                    umma_commit(&ctl.empty_bar[st >> 1]);  // the pair is free once these MMAs have read it
                }
                if (ok) umma_commit(&ctl.acc_full[acc]);
            }
        }
    } else if (warp < kPfWarpEpi0) {
        // -------------------------------- loaders --------------------------------
        // Copy i of a span serves tile rows 4i + 2lw + (lane / 16) (lw: which loader warp): sixteen
        // lanes per row, 16 bytes each, as many as the row's widened bytes need.
        const int lw = warp - kPfWarpLoad, hw = lane >> 4, part = lane & 15;
        const uint32_t raw32 = smem_u32(raw_ring), rawfull32 = smem_u32(&ctl.raw_full[0]);
        int slot = 0, rphase = 0;
        bool ok = true, wrapped = false;
        const int G = gridDim.x;
        PfTile T{}, T1{};
        if ((int)blockIdx.x < n_tiles) T = pf_tile(L, blockIdx.x, n_routed, valid);
        for (int t = blockIdx.x; t < n_tiles && ok; t += G) {
            if (t + G < n_tiles) T1 = pf_tile(L, t + G, n_routed, valid);  // in flight during this tile
            const int quant = T.shared ? QS : QR;
            const uint32_t pitch = pf_raw_pitch(quant);
            const uint32_t span_bytes = span_bytes_of(quant);
            const size_t row_bytes = (size_t)n_spans * span_bytes;
            // rows 2lw + hw of the first gate group and of the first up group (down: the same row twice)
            const uint8_t* pg = pf_row_ptr<MODE>(L, T, 2 * lw + hw, row_bytes);
            const uint8_t* pu = MODE == MODE_GATEUP ? pf_row_ptr<MODE>(L, T, 16 + 2 * lw + hw, row_bytes) : pg;
            for (int s = 0; s < n_spans && ok; ++s) {
                if (wrapped) {  // the slot is free once every unpack warp has left its previous span
                    ok = stream_wait_pf(&ctl.raw_empty[slot], rphase ^ 1, abortp, L.status);
                    if (!ok) break;
                }
                const uint32_t dst0 = raw32 + (uint32_t)slot * L.slot_bytes + (uint32_t)(2 * lw + hw) * pitch + part * 16;
                const uint8_t* sg = pg + (size_t)s * span_bytes;
                const uint8_t* su = pu + (size_t)s * span_bytes;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    // tile row 4i + c (c = 2lw + hw): in the gate/up interleave rows 4i..4i+3 of the tile are
                    // rows (i / 8) * 16 + 4 (i % 4) + c of the gate (i % 8 < 4) or up matrix
                    const int wr = MODE == MODE_GATEUP ? (i >> 3) * 16 + 4 * (i & 3) : 4 * i;
                    const uint8_t* p = ((MODE == MODE_GATEUP && (i & 4)) ? su : sg) + (size_t)wr * row_bytes;
                    const uint32_t mis = (uint32_t)(uintptr_t)p & 15u;
                    const uint32_t units = (mis + span_bytes + 15u) >> 4;  // ends at or before the tensor's end
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
        // Thread (quad, lane) owns token column 32 quad + lane of every tile: TMEM lane = token, TMEM
        // column = tile row.  Gate/up: columns 32 c .. 32 c + 15 are gate rows 16 c .. 16 c + 15 of the tile's
        // 64, columns 32 c + 16 .. 32 c + 31 the same rows of up, so SwiGLU stays inside the thread.
        const int quad = warp & 3;
        const int ew = MODE == MODE_DOWN ? warp - kPfWarpEpi0 : 0;
        const float inv = 1.0f / kPfWeightScale;
        uint32_t n = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++n) {
            const PfTile T = pf_tile(L, t, n_routed, valid);
            const uint32_t acc = n % kPfAccums;
            const int tok = quad * 32 + lane;
            const bool live = tok < T.ncols;
            // Down, routed: the flat (token, k) id, the routing weight and the result row -- three dependent
            // loads -- are fetched before the wait, so they are in flight while the tile is computed.
            float factor = inv;  // the weight scale is a power of two: folded into the routing weight exactly
            float* dst = nullptr;
            __half* hdst = nullptr;
            if (live) {
                if (MODE == MODE_GATEUP) {
                    hdst = (T.shared ? L.inter_shared : L.inter_routed) + (size_t)(T.first + tok) * L.rows + T.bx * 64;
                } else if (T.shared) {
                    dst = L.shexp + (size_t)(T.first + tok) * L.rows;
                } else {
                    const int flat = __ldg(L.sorted_token_ids + T.first + tok);
                    factor = __ldg(L.topk_weights + flat) * inv;
                    dst = result_row(L.partial, L.partial_rows, flat, L.rows);
                }
                if (MODE == MODE_DOWN && dst) dst += T.bx * kPfTileM;
            }
            if (MODE == MODE_DOWN) {  // the warp's 32 row addresses (nullptr: nothing to store), read back by other lanes
                epi_dst[ew][lane] = dst;
                __syncwarp();
            }
            ok = stream_wait_pf<true>(&ctl.acc_full[acc], (n / kPfAccums) & 1, abortp, L.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + acc * kPfTileN + ((uint32_t)(quad * 32) << 16);
            const bool any_live = quad * 32 < T.ncols;  // the same for the whole warp
            for (int cb = 0; cb < kPfTileM / 32; ++cb) {
                uint32_t r[32];
                if (any_live) {
                    tmem_ld32(taddr + (uint32_t)(cb * 32), r);
                    tmem_ld_wait();
                }
                if (cb == kPfTileM / 32 - 1 || !any_live) {  // last read of this accumulator: hand it back before the stores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_pf(&ctl.acc_empty[acc]);
                    if (!any_live) break;
                }
                if (MODE == MODE_GATEUP) {
                    if (hdst) {
                        uint32_t h[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float g0 = __uint_as_float(r[2 * i]) * inv, g1 = __uint_as_float(r[2 * i + 1]) * inv;
                            const float u0 = __uint_as_float(r[16 + 2 * i]) * inv, u1 = __uint_as_float(r[17 + 2 * i]) * inv;
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
                        // lane = token: its 16 outputs as four 16-byte chunks, chunk c at position
                        // c ^ ((lane / 2) % 4) of the 64-byte row, which keeps both the stores here and the
                        // loads below free of bank conflicts
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int q = half * 16 + 4 * c;
                            *(float4*)(epi_stage[ew] + lane * 16 + ((c ^ ((lane >> 1) & 3)) << 2)) =
                                make_float4(factor * __uint_as_float(r[q]), factor * __uint_as_float(r[q + 1]),
                                            factor * __uint_as_float(r[q + 2]), factor * __uint_as_float(r[q + 3]));
                        }
                        __syncwarp();
                        // lanes 4R' .. 4R' + 3 of a pass: the four chunks of token row R, 64 bytes side by side
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
    }
    // every thread of the CTA arrives here on every path, so TMEM is always returned
    tc_fence_before();
    __syncthreads();
    if (warp == kPfWarpMma) tmem_dealloc(tmem_base, kPfAccums * kPfTileN);
}

}  // namespace xabe
