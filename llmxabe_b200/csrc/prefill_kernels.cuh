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

// Nine aligned words covering the 32 (+2) bytes at the 2-byte-aligned global
// address p, returned as the eight words that start at p.
__device__ __forceinline__ void ldg_32bytes(const uint8_t* p, uint32_t (&w)[8]) {
    uintptr_t a = (uintptr_t)p;
    const uint32_t* q = (const uint32_t*)(a & ~(uintptr_t)3);
    if (a & 2) {
        uint32_t prev = __ldg(q);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t next = __ldg(q + i + 1);
            w[i] = __funnelshift_r(prev, next, 16);
            prev = next;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = __ldg(q + i);
    }
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

// Five aligned words covering the 16 (+2) bytes at the 2-byte-aligned global
// address p, returned as the four words that start at p.
__device__ __forceinline__ void ldg_16bytes(const uint8_t* p, uint32_t (&w)[4]) {
    uintptr_t a = (uintptr_t)p;
    const uint32_t* q = (const uint32_t*)(a & ~(uintptr_t)3);
    if (a & 2) {
        uint32_t prev = __ldg(q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t next = __ldg(q + i + 1);
            w[i] = __funnelshift_r(prev, next, 16);
            prev = next;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = __ldg(q + i);
    }
}

// One producer thread's share of a PAIR of contraction chunks (128 elements of
// one weight row), fetched one pair ahead of its use.
//   Q6_K: the pair is one half of a superblock.  The thread owns positions
//     l in [16*part, 16*part + 16) of all four 32-element groups: 16 nibble
//     bytes from each of the two ql runs, 16 bit-pair bytes, four scales.
//     Every byte of the half is fetched exactly once per tile.
//   Q8_0: the thread owns elements [64*part, 64*part + 64): two blocks.
struct Raw128 {
    uint32_t a[8];  // Q6_K: ql run 0 (4 words), ql run 1 (4 words); Q8_0: block 0 codes
    uint32_t b[8];  // Q6_K: qh (4 words, rest unused);               Q8_0: block 1 codes
    float s[4];     // Q6_K: scale of group j (for this thread's l range); Q8_0: s[0], s[1] block scales
};

template <int QUANT>
__device__ __forceinline__ void load_raw128(const uint8_t* row_ptr, int pair, int part, Raw128& r) {
    if (QUANT == QUANT_Q6K) {
        // element map of crates/xabe-kernels/src/quant.rs:175-198
        const uint8_t* blk = row_ptr + (size_t)(pair >> 1) * kQ6KBlockBytes;
        const int half = pair & 1;
        uint32_t w[4];
        ldg_16bytes(blk + half * 64 + 16 * part, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) r.a[i] = w[i];
        ldg_16bytes(blk + half * 64 + 32 + 16 * part, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) r.a[4 + i] = w[i];
        ldg_16bytes(blk + 128 + half * 32 + 16 * part, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) r.b[i] = w[i];
        float d = __half2float(__ushort_as_half(__ldg((const unsigned short*)(blk + 208)))) * kPfWeightScale;
#pragma unroll
        for (int j = 0; j < 4; ++j)  // scale index half*8 + 2*j + l/16, l/16 == part
            r.s[j] = d * (float)(int)(int8_t)__ldg(blk + 192 + half * 8 + 2 * j + part);
    } else {
        const uint8_t* blk = row_ptr + (size_t)(pair * 4 + part * 2) * kQ8BlockBytes;
        ldg_32bytes(blk + 2, r.a);
        ldg_32bytes(blk + kQ8BlockBytes + 2, r.b);
        r.s[0] = __half2float(__ushort_as_half(__ldg((const unsigned short*)blk))) * kPfWeightScale;
        r.s[1] = __half2float(__ushort_as_half(__ldg((const unsigned short*)(blk + kQ8BlockBytes)))) * kPfWeightScale;
        r.s[2] = r.s[3] = 0.f;
    }
}

// Unpack, scale and store into the A tiles of the pair's two stages.
template <int QUANT>
__device__ __forceinline__ void store_raw128(const Raw128& r, int part, uint8_t* a_tile0, uint8_t* a_tile1,
                                             int tile_row) {
    if (QUANT == QUANT_Q6K) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // group j: nibbles of ql run (j & 1), low for j < 2 and high otherwise; bit pair j of qh
            __half2 ds2 = __float2half2_rn(r.s[j]);
            uint8_t* tile = (j >> 1) ? a_tile1 : a_tile0;
            uint32_t raw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t q = r.a[(j & 1) * 4 + i];
                uint32_t lo = (j < 2 ? q : (q >> 4)) & 0x0F0F0F0Fu;
                uint32_t hi = ((r.b[i] >> (2 * j)) & 0x03030303u) << 4;
                raw[i] = lo | hi;
            }
            // 16 elements at (j & 1) * 32 + 16 * part of the stage's 64: two 16-byte chunks
            const int chunk = (j & 1) * 4 + 2 * part;
            *(uint4*)(tile + swz_off(tile_row, chunk)) = codes8_to_h8(raw[0], raw[1], 0x64206420u, ds2);
            *(uint4*)(tile + swz_off(tile_row, chunk + 1)) = codes8_to_h8(raw[2], raw[3], 0x64206420u, ds2);
        }
    } else {
        uint8_t* tile = part ? a_tile1 : a_tile0;  // elements [64 * part, 64 * part + 64) are one whole stage row
        __half2 d0 = __float2half2_rn(r.s[0]), d1 = __float2half2_rn(r.s[1]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            *(uint4*)(tile + swz_off(tile_row, c)) =
                codes8_to_h8(r.a[2 * c] ^ 0x80808080u, r.a[2 * c + 1] ^ 0x80808080u, 0x64806480u, d0);
            *(uint4*)(tile + swz_off(tile_row, 4 + c)) =
                codes8_to_h8(r.b[2 * c] ^ 0x80808080u, r.b[2 * c + 1] ^ 0x80808080u, 0x64806480u, d1);
        }
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
            mbar_init(&full_bar[i], kPfProducerWarps);
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
        const int p = (prod_id % kPfProducerWarps) * 32 + lane;  // 0..255
        const int row = p & (kPfTileM - 1);  // tile row = TMEM lane, and B token column
        const int part = p >> 7;             // which 32-element half of the 64-element chunk
        const uint8_t* wbase;
        size_t wrow;
        if (MODE == MODE_GATEUP) {
            int q = row >> 5, i = row & 31;
            wbase = i < 16 ? (shared ? L.s_a : L.r_a) : (shared ? L.s_b : L.r_b);
            wrow = (size_t)blockIdx.x * 64 + q * 16 + (i & 15);
        } else {
            wbase = shared ? L.s_a : L.r_a;
            wrow = (size_t)blockIdx.x * kPfTileM + row;
        }
        const uint8_t* wptr = wbase + ((shared ? 0 : (size_t)expert * L.rows) + wrow) * row_bytes;
        const int src = col_src[row];
        const __half* xptr = (shared ? L.x_shared : L.x_routed) + (size_t)(src < 0 ? 0 : src) * L.k;
        // The contraction is walked in PAIRS of chunks (128 elements, stages 2*pr and 2*pr + 1),
        // so that each byte of a Q6_K half-superblock is fetched once; the bytes of pair pr + 1
        // are in flight while pair pr is unpacked.  The thread fills row `row` of the A tiles and
        // row `row`, elements [64 * part, +64) of the pair, of the B tiles.
        bool ok = true;
        const int n_pairs = n_chunks >> 1;  // the contraction is a multiple of 256
        Raw128 raw;
        uint4 xv[8];
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        for (int pr = pgroup; pr < n_pairs && ok; pr += kPfProducerGroups) {
            // the other producer group and the second CTA-resident warps hide this latency
            if (quant == QUANT_Q6K) load_raw128<QUANT_Q6K>(wptr, pr, part, raw);
            else load_raw128<QUANT_Q8_0>(wptr, pr, part, raw);
#pragma unroll
            for (int c = 0; c < 8; ++c)
                xv[c] = src < 0 ? zero4 : __ldg((const uint4*)(xptr + pr * 128 + 64 * part) + c);
            const Raw128& cur = raw;
            const uint4* xc = xv;
            const int kc0 = 2 * pr, kc1 = 2 * pr + 1;
            const int st0 = kc0 % S, st1 = kc1 % S;
            if (kc0 / S >= 1) ok = stream_wait_pf(&empty_bar[st0], (kc0 / S - 1) & 1, abortp, L.status);
            if (ok && kc1 / S >= 1) ok = stream_wait_pf(&empty_bar[st1], (kc1 / S - 1) & 1, abortp, L.status);
            if (!ok) break;
            uint8_t* a0 = stages + (size_t)st0 * kPfStageBytes;
            uint8_t* a1 = stages + (size_t)st1 * kPfStageBytes;
            if (quant == QUANT_Q6K) store_raw128<QUANT_Q6K>(cur, part, a0, a1, row);
            else store_raw128<QUANT_Q8_0>(cur, part, a0, a1, row);
            uint8_t* b_tile = (part ? a1 : a0) + kPfTileM * kPfChunkK * 2;
#pragma unroll
            for (int c = 0; c < 8; ++c) *(uint4*)(b_tile + swz_off(row, c)) = xc[c];
            fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_pf(&full_bar[st0]);
                mbar_arrive_pf(&full_bar[st1]);
            }
        }
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
