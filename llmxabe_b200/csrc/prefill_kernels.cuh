// Prefill-shaped expert projections: a grouped GEMM on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA computes one output tile D[128 weight rows][128 token columns] of
// one expert (or of the shared expert).  The contraction runs in chunks of 64
// elements through a ring of shared-memory stages:
//   * sixteen producer warps (two groups on alternate stage pairs) read the raw GGUF bytes (Q6_K superblocks or Q8_0
//     blocks) of the tile's 128 weight rows, unpack them, scale them and write
//     f16 values into the stage's A tile in the 128-byte-swizzled K-major
//     layout the tensor core reads; they also gather the 128 token rows of f16
//     activations into the B tile, same layout;
//   * one thread issues four tcgen05.mma (M128 N128 K16, f16 x f16 -> f32)
//     per stage and commits them to the stage's "empty" barrier;
//   * four of the producer warps then read the accumulator from TMEM with
//     tcgen05.ld and apply SwiGLU (gate/up) or the routing weight (down).
//
// Numerics: weights are rounded to f16 after the fp32-exact code is multiplied
// by the f16-rounded group scale (times 256, undone in the epilogue, which
// keeps small super-scales out of the f16 subnormal range); activations are
// f16; accumulation is fp32 in TMEM.  This differs from the decode kernels
// (exact codes, fp32 scales) by the weight rounding, about 2e-4 relative per
// weight, and stays inside the rel-L2 <= 1e-3 gate.
//
// Every wait is bounded; TMEM is freed on every exit path that allocated it.
#pragma once

#include "common.cuh"
#include "glue_kernels.cuh"

namespace xabe {

constexpr int kPfTileM = 128;       // weight rows per tile (TMEM lanes)
constexpr int kPfTileN = 128;       // token columns per tile
constexpr int kPfChunkK = 64;       // contraction elements per stage (one 128-byte swizzle row of f16)
constexpr int kPfStageBytes = 2 * kPfTileM * kPfChunkK * 2;  // A tile + B tile, 16 KB each
constexpr int kPfProducerWarps = 8;   // warps that fill one stage pair
constexpr int kPfProducerGroups = 2;  // groups working on alternate stage pairs
// warp 4 issues the MMAs; every other warp is a producer, and warps 0-3 (one per TMEM lane quadrant)
// also run the epilogue once the contraction is done
constexpr int kPfThreads = 32 * (1 + kPfProducerWarps * kPfProducerGroups);
constexpr int kPfMaxStages = 6;
constexpr float kPfWeightScale = 256.0f;
constexpr int kPfItemInts = 4;  // expert, first slot (or first token), columns, pad

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
    float* shexp;
    int* status;
    int n_stages;
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

// What one lane holds for one producer pass.  A pass is eight weight rows x one PAIR of chunks
// (128 contraction elements); lane (rrow = lane / 4, j = lane % 4) serves row rrow:
//   Q6_K  positions l = 8j..8j+7 of all four 32-element groups of half a superblock
//         (element map of crates/xabe-kernels/src/quant.rs:175-198): 8 bytes of each ql run,
//         8 bytes of bit pairs, the four group scales and d  -> 32 weights
//   Q8_0  block j of the pair's four blocks: 32 codes and d   -> 32 weights
// The four lanes of a row read consecutive bytes, so a load touches few cache lines.
struct RawQ6 {
    uint32_t ql0[2], ql1[2], qh[2];
    int sc[4];
    uint32_t d;
};
struct RawQ8 {
    uint32_t w[8];
    uint32_t d;
};

// Eight bytes that start `sh / 8` (0 or 2) bytes after the 4-byte-aligned address q.  The third
// word read lies inside the same superblock for every piece this is used on.
__device__ __forceinline__ void ldg8_shifted(const uint8_t* q, uint32_t sh, uint32_t (&o)[2]) {
    const uint32_t* w = (const uint32_t*)q;
    uint32_t a = __ldg(w), b = __ldg(w + 1), c = __ldg(w + 2);
    o[0] = __funnelshift_r(a, b, sh);
    o[1] = __funnelshift_r(b, c, sh);
}

// `pa`: 4-byte-aligned address at or 2 bytes below (superblock + h*64 + 8j); `pb` likewise for
// (superblock + 128 + h*32 + 8j); `ps` = superblock + 192 + h*8 + j/2; `pd` = superblock + 208.
__device__ __forceinline__ void load_pass(const uint8_t* pa, const uint8_t* pb, const uint8_t* ps,
                                          const uint8_t* pd, uint32_t sh, RawQ6& r) {
    ldg8_shifted(pa, sh, r.ql0);
    ldg8_shifted(pa + 32, sh, r.ql1);
    ldg8_shifted(pb, sh, r.qh);
#pragma unroll
    for (int g = 0; g < 4; ++g) r.sc[g] = (int)(int8_t)__ldg(ps + 2 * g);  // scale index h*8 + 2g + l/16
    r.d = __ldg((const unsigned short*)pd);
}
// `blk`: the lane's 34-byte block (2-byte aligned).
__device__ __forceinline__ void load_pass(const uint8_t* blk, RawQ8& r) {
    const uint32_t mis = ((uintptr_t)blk & 2) ? 0u : 1u;  // the codes start at blk + 2
    const uint32_t* w = (const uint32_t*)(blk + 2 - 2 * mis);
    uint32_t a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = __ldg(w + i);
    // misaligned codes: a[0] starts with d and the last two codes follow a[7]; aligned: d precedes a[0]
    uint32_t extra = __ldg((const unsigned short*)(blk + 32 * mis));
    r.d = mis ? (a[0] & 0xFFFFu) : extra;
    const uint32_t sh = 16 * mis;
#pragma unroll
    for (int i = 0; i < 8; ++i) r.w[i] = __funnelshift_r(a[i], i < 7 ? a[i + 1] : extra, sh);
}

// Unpack, scale and store the lane's 32 weights: four 16-byte chunks.  `t0`/`t1`: shared-memory
// addresses of the lane's row inside the A tiles of the pair's two stages, with the row's swizzle
// already applied to chunk `c0x` (= chunk index XOR row % 8, times 16).
__device__ __forceinline__ void store_pass(const RawQ6& r, uint8_t* row0, uint8_t* row1, uint32_t cx) {
    const float d = __half2float(__ushort_as_half((unsigned short)r.d)) * kPfWeightScale;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint32_t* ql = (g & 1) ? r.ql1 : r.ql0;
        uint32_t c[2];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            uint32_t nib = (g >> 1) ? (ql[w] >> 4) : ql[w];
            uint32_t two = g == 0 ? (r.qh[w] << 4) : g == 1 ? (r.qh[w] << 2) : g == 2 ? r.qh[w] : (r.qh[w] >> 2);
            c[w] = (nib & 0x0F0F0F0Fu) | (two & 0x30303030u);
        }
        __half2 ds2 = __float2half2_rn(d * (float)r.sc[g]);
        uint4 v = codes8_to_h8(c[0], c[1], 0x64206420u, ds2);
        // group g: elements (g % 2) * 32 + 8j.. of stage g / 2: chunk (g % 2) * 4 + j
        uint8_t* row = (g >> 1) ? row1 : row0;
        *(uint4*)(row + (cx ^ ((g & 1) << 6))) = v;
    }
}
__device__ __forceinline__ void store_pass(const RawQ8& r, uint8_t* row, uint32_t cx) {
    __half2 ds2 = __float2half2_rn(__half2float(__ushort_as_half((unsigned short)r.d)) * kPfWeightScale);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        uint4 v = codes8_to_h8(r.w[2 * t] ^ 0x80808080u, r.w[2 * t + 1] ^ 0x80808080u, 0x64806480u, ds2);
        *(uint4*)(row + (cx ^ (t << 4))) = v;  // chunk (j % 2) * 4 + t
    }
}

__device__ __forceinline__ void mbar_arrive_pf(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait that also gives up when another warp of the CTA already has.
__device__ __forceinline__ bool stream_wait_pf(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* status) {
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u && *abort_flag) return false;
        if (it >= 16u) __nanosleep(it < 256u ? 32u : 256u);  // long waits back off and leave the issue slots to working warps
    }
    *abort_flag = 1;
    if (status) atomicExch(status, STATUS_TMA_TIMEOUT);
    return false;
}

// Token tiles of the routed experts for the prefill kernels: the live slots of
// expert e are contiguous from expert_offsets[e]; they are cut into runs of up
// to 128.  One block, one thread per expert.
__global__ void k_build_prefill_items(int num_experts, const int* __restrict__ expert_offsets,
                                      const int* __restrict__ expert_counts, int* __restrict__ items,
                                      int* __restrict__ n_items) {
    extern __shared__ int base_s[];
    int e = threadIdx.x;
    if (e < num_experts) base_s[e] = (expert_counts[e] + kPfTileN - 1) / kPfTileN;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < num_experts; ++i) {
            int g = base_s[i];
            base_s[i] = run;
            run += g;
        }
        *n_items = run;
    }
    __syncthreads();
    if (e < num_experts) {
        int count = expert_counts[e], start = expert_offsets[e];
        for (int i = 0; i * kPfTileN < count; ++i) {
            int* it = items + (size_t)(base_s[e] + i) * kPfItemInts;
            it[0] = e;
            it[1] = start + i * kPfTileN;
            it[2] = min(kPfTileN, count - i * kPfTileN);
            it[3] = 0;
        }
    }
}

template <int QUANT> struct RawOf;
template <> struct RawOf<QUANT_Q6K> { using T = RawQ6; };
template <> struct RawOf<QUANT_Q8_0> { using T = RawQ8; };

// What a producer warp needs to know; everything here is fixed for the tile.
struct PfProducer {
    uint8_t* stages;
    uint64_t* full_bar;
    uint64_t* empty_bar;
    volatile int* abortp;
    int* status;
    int n_stages, n_pairs, pgroup, gw, lane;
    const uint8_t* row_ptr0;  // the lane's weight row of pass 0; pass 1 is eight rows further
    size_t pass_stride;
    const uint4* x4;          // activations in 16-byte units
    int xoff[4];              // the thread's four token rows: row * (K / 8) + piece, or -1 (zero column)
};

template <int QUANT>
__device__ __forceinline__ void pf_load(const PfProducer& P, int pr, typename RawOf<QUANT>::T (&raw)[2]) {
    const int j = P.lane & 3;
    if constexpr (QUANT == QUANT_Q6K) {
        const int h = pr & 1;
        const uint8_t* blk = P.row_ptr0 + (size_t)(pr >> 1) * kQ6KBlockBytes;
        const uint32_t mis = (uint32_t)((uintptr_t)blk & 2);
        const uint8_t* pa = blk - mis + h * 64 + 8 * j;
        const uint8_t* pb = blk - mis + 128 + h * 32 + 8 * j;
        const uint8_t* ps = blk + 192 + h * 8 + (j >> 1);
        const uint8_t* pd = blk + 208;
#pragma unroll
        for (int q = 0; q < 2; ++q)
            load_pass(pa + q * P.pass_stride, pb + q * P.pass_stride, ps + q * P.pass_stride,
                      pd + q * P.pass_stride, mis * 8, raw[q]);
    } else {
        const uint8_t* blk = P.row_ptr0 + (size_t)(pr * 4 + j) * kQ8BlockBytes;
#pragma unroll
        for (int q = 0; q < 2; ++q) load_pass(blk + q * P.pass_stride, raw[q]);
    }
}

// Fills the stage pair of contraction pair `pr` from `raw`: waits for the two stages to be free,
// starts the asynchronous copies of the token rows (B tiles), writes the unpacked weights (A tiles).
template <int QUANT>
__device__ __forceinline__ bool pf_fill(const PfProducer& P, int pr, const typename RawOf<QUANT>::T (&raw)[2]) {
    const int S = P.n_stages;
    const int kc0 = 2 * pr, kc1 = 2 * pr + 1;
    const int st0 = kc0 % S, st1 = kc1 % S;
    if (kc0 / S >= 1 && !stream_wait_pf(&P.empty_bar[st0], (kc0 / S - 1) & 1, P.abortp, P.status)) return false;
    if (kc1 / S >= 1 && !stream_wait_pf(&P.empty_bar[st1], (kc1 / S - 1) & 1, P.abortp, P.status)) return false;
    uint8_t* a0 = P.stages + (size_t)st0 * kPfStageBytes;
    uint8_t* a1 = P.stages + (size_t)st1 * kPfStageBytes;
    const int lane = P.lane, gw = P.gw;
    {   // B tiles: rows r0 + 32m, 16-byte piece lane % 8
        const int r0 = gw * 4 + (lane >> 3), piece = lane & 7;
        const uint32_t boff = (uint32_t)(kPfTileM * kPfChunkK * 2) + swz_off(r0, piece);
        const uint32_t b0 = smem_u32(a0) + boff, b1 = smem_u32(a1) + boff;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const bool live = P.xoff[m] >= 0;
            const uint4* src = P.x4 + (live ? (size_t)P.xoff[m] + (size_t)pr * 16 : 0);
            cp_async16(b0 + m * 4096, src, live ? 16u : 0u);
            cp_async16(b1 + m * 4096, src + (live ? 8 : 0), live ? 16u : 0u);
        }
        cp_async_arrive_noinc(&P.full_bar[st0]);
        cp_async_arrive_noinc(&P.full_bar[st1]);
    }
    const int rrow = lane >> 2, j = lane & 3;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const uint32_t rowoff = (uint32_t)((2 * gw + q) * 1024 + rrow * 128);
        if constexpr (QUANT == QUANT_Q6K) {
            store_pass(raw[q], a0 + rowoff, a1 + rowoff, (uint32_t)((j ^ rrow) << 4));
        } else {
            store_pass(raw[q], ((j >> 1) ? a1 : a0) + rowoff, (uint32_t)(((((j & 1) << 2)) ^ rrow) << 4));
        }
    }
    fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
    __syncwarp();
    if (lane == 0) {
        mbar_arrive_pf(&P.full_bar[st0]);
        mbar_arrive_pf(&P.full_bar[st1]);
    }
    return true;
}

// The producer loop of one warp: its group takes every second pair; the raw bytes of the group's
// next pair are in flight while the current one is unpacked.
template <int QUANT>
__device__ __forceinline__ void pf_produce(const PfProducer& P) {
    typename RawOf<QUANT>::T ra[2], rb[2];
    const int step = kPfProducerGroups;
    int pr = P.pgroup;
    if (pr < P.n_pairs) pf_load<QUANT>(P, pr, ra);
    while (pr < P.n_pairs) {
        if (pr + step < P.n_pairs) pf_load<QUANT>(P, pr + step, rb);
        if (!pf_fill<QUANT>(P, pr, ra)) break;
        pr += step;
        if (pr >= P.n_pairs) break;
        if (pr + step < P.n_pairs) pf_load<QUANT>(P, pr + step, ra);
        if (!pf_fill<QUANT>(P, pr, rb)) break;
        pr += step;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// MODE_GATEUP (0): TMEM lane m = 32q + i holds gate row r0 + 16q + i for i < 16 and up row
// r0 + 16q + (i - 16) otherwise (r0 = 64 * blockIdx.x), so SwiGLU pairs two lanes of one warp.
// MODE_DOWN (1): lane m holds row 128 * blockIdx.x + m.
// grid: (row tiles, routed item capacity + shared token tiles); block kPfThreads.
template <int MODE, int QR, int QS>
__global__ void __launch_bounds__(kPfThreads, 1) k_prefill_gemm(PrefillLaunch L) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kPfMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kPfMaxStages];
    __shared__ __align__(8) uint64_t accum_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag;
    __shared__ int col_src[kPfTileN];
    __shared__ int col_flat[kPfTileN];
    __shared__ float col_wgt[kPfTileN];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int valid = *L.valid_tokens;
    const int n_routed = L.has_routed ? *L.n_items : 0;
    const int n_shared = L.has_shared ? (valid + kPfTileN - 1) / kPfTileN : 0;
    const int y = blockIdx.y;
    if (y >= n_routed + n_shared) return;  // uniform: nothing allocated yet
    const bool shared = y >= n_routed;
    int expert = 0, first, ncols;
    if (!shared) {
        const int* it = L.items + (size_t)y * kPfItemInts;
        expert = it[0];
        first = it[1];
        ncols = it[2];
    } else {
        first = (y - n_routed) * kPfTileN;
        ncols = min(kPfTileN, valid - first);
    }
    const int quant = shared ? QS : QR;
    const int S = L.n_stages;
    const int n_chunks = L.k / kPfChunkK;
    const int row_bytes = L.k / kSpanElems * span_bytes_of(quant);
    uint8_t* stages = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    volatile int* abortp = &abort_flag;

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            // one arrival per producer warp (A tile written) + one per producer thread (its B-tile copies landed)
            mbar_init(&full_bar[i], kPfProducerWarps + kPfProducerWarps * 32);
            mbar_init(&empty_bar[i], 1);
        }
        mbar_init(&accum_bar, 1);
        fence_mbar_init();
    }
    if (tid < kPfTileN) {
        int c = tid;
        int src = -1, flat = 0;
        float wgt = 0.f;
        if (c < ncols) {
            if (shared) {
                src = first + c;
            } else {
                flat = L.sorted_token_ids[first + c];
                wgt = L.topk_weights[flat];
                src = MODE == MODE_GATEUP ? flat / L.top_k : first + c;
            }
        }
        col_src[c] = src;
        col_flat[c] = flat;
        col_wgt[c] = wgt;
    }
    if (warp == 4) {
        tmem_alloc(&tmem_base_s, kPfTileN);  // 128 fp32 columns
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    const int prod_id = warp < 4 ? warp : warp - 1;        // producer warp index 0..15 (warp 4 is the MMA issuer)
    const int pgroup = prod_id / kPfProducerWarps;        // which stage pairs: pgroup, pgroup + 2, ...
    if (warp != 4) {
        // ------------------------------ producers ------------------------------
        // A producer group (8 warps) fills one PAIR of stages (128 contraction elements) at a time:
        // sixteen passes of eight weight rows, two per warp, 32 weights per lane; and the 2 x 128
        // token rows of the B tiles by asynchronous 16-byte copies, eight per thread.
        PfProducer P;
        P.stages = stages;
        P.full_bar = full_bar;
        P.empty_bar = empty_bar;
        P.abortp = abortp;
        P.status = L.status;
        P.n_stages = S;
        P.n_pairs = n_chunks >> 1;  // the contraction is a multiple of 256
        P.pgroup = pgroup;
        P.gw = prod_id % kPfProducerWarps;
        P.lane = lane;
        {
            // tile rows 16gw..16gw+15 are consecutive weight rows of one matrix (in the gate/up
            // interleave: half of one 32-row group)
            const int gw = P.gw, rrow = lane >> 2;
            const uint8_t* base = shared ? L.s_a : L.r_a;
            size_t wrow;
            if (MODE == MODE_GATEUP) {
                if (gw & 1) base = shared ? L.s_b : L.r_b;
                wrow = (size_t)blockIdx.x * 64 + (gw >> 1) * 16 + rrow;
            } else {
                wrow = (size_t)blockIdx.x * kPfTileM + 16 * gw + rrow;
            }
            const size_t expert_row0 = shared ? 0 : (size_t)expert * L.rows;
            P.row_ptr0 = base + (expert_row0 + wrow) * row_bytes;
            P.pass_stride = (size_t)8 * row_bytes;
            P.x4 = (const uint4*)(shared ? L.x_shared : L.x_routed);
            const int r0 = gw * 4 + (lane >> 3);
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int srow = col_src[r0 + 32 * m];
                P.xoff[m] = srow < 0 ? -1 : srow * (L.k >> 3) + (lane & 7);
            }
        }
        if (quant == QUANT_Q6K) pf_produce<QUANT_Q6K>(P);
        else pf_produce<QUANT_Q8_0>(P);
    } else {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(kPfTileM, kPfTileN);
            bool ok = true;
            for (int kc = 0; kc < n_chunks && ok; ++kc) {
                const int st = kc % S;
                ok = stream_wait_pf(&full_bar[st], (kc / S) & 1, abortp, L.status);
                if (!ok) break;
                tc_fence_after();
                fence_proxy_async_smem();  // the B tile arrived by cp.async, not through the async proxy
                const uint32_t a_addr = smem_u32(stages + (size_t)st * kPfStageBytes);
                const uint64_t adesc = umma_smem_desc(a_addr);
                const uint64_t bdesc = umma_smem_desc(a_addr + kPfTileM * kPfChunkK * 2);
#pragma unroll
                for (int k4 = 0; k4 < kPfChunkK / 16; ++k4)  // 32 bytes per K16 step inside the swizzle row
                    umma_f16(tmem_base, adesc + 2 * k4, bdesc + 2 * k4, idesc, (kc > 0 || k4 > 0) ? 1u : 0u);
                umma_commit(&empty_bar[st]);  // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(&accum_bar);
        }
    }
    if (warp < 4) {
        // ------------------------------- epilogue -------------------------------
        bool ok = stream_wait_pf(&accum_bar, 0, abortp, L.status);
        tc_fence_after();
        const float inv = 1.0f / kPfWeightScale;
        if (ok) {
            for (int cb = 0; cb * 32 < ncols; ++cb) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cb * 32), r);
                tmem_ld_wait();
                if (MODE == MODE_GATEUP) {
                    const int out_row = blockIdx.x * 64 + warp * 16 + (lane & 15);
                    __half* dst_base = shared ? L.inter_shared : L.inter_routed;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float mine = __uint_as_float(r[j]) * inv;
                        float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                        bool do_it = (lane < 16) == (j < 16);  // lanes 0-15 finish columns 0-15, lanes 16-31 the rest
                        int col = cb * 32 + j;
                        if (do_it && col < ncols) {
                            float gv = lane < 16 ? mine : other;
                            float uv = lane < 16 ? other : mine;
                            float v = __fdiv_rn(gv, 1.0f + expf(-gv)) * uv;
                            dst_base[(size_t)(first + col) * L.rows + out_row] = __float2half_rn(v);
                        }
                    }
                } else {
                    const int out_row = blockIdx.x * kPfTileM + warp * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        int col = cb * 32 + j;
                        if (col < ncols) {
                            float v = __uint_as_float(r[j]) * inv;
                            if (shared) L.shexp[(size_t)(first + col) * L.rows + out_row] = v;
                            else L.partial[(size_t)col_flat[col] * L.rows + out_row] = col_wgt[col] * v;
                        }
                    }
                }
            }
        }
    }
    // every thread of the CTA arrives here on every path, so TMEM is always returned
    tc_fence_before();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem_base, kPfTileN);
}

}  // namespace xabe
