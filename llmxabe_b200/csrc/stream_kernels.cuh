// Streaming expert projections: persistent CTAs, one per SM, that keep a ring
// of TMA-filled weight tiles in flight while sixteen consumer warps unpack and
// multiply.  This is the tuned path for the decode-shaped geometry (a
// contraction of at most 8 superblocks for gate/up and 2 for down); other
// shapes use the one-tile-per-CTA kernels of expert_kernels.cuh.
//
// Unit of work: (column group, run of row tiles).  A column group is up to 8
// token columns of one expert (or of the shared expert): the n8 dimension of
// the tensor-core tile.  For one unit the producer warp copies the group's f16
// activation rows and its descriptor into shared memory once, then streams the
// unit's weight tiles through the ring; each consumer warp loads its B
// fragments from the activation rows into registers once per unit, so the
// inner loop touches nothing but the weight tile.
//
// Arithmetic (same contract as expert_kernels.cuh): exact integer codes as the
// f16 A operand, one k16 step per scale group, fp32 scale applied to the
// step's fp32 result, fp32 accumulation.  gate/up: the eight consumer warps of
// a group split the contraction by superblock and their partial tiles are
// added in ascending warp order.  A token's value never depends on the other
// columns of its group, on the group's position in the list, or on which CTA
// or ring stage carried it.
//
// Every wait is bounded: on a timeout the warp records STATUS_TMA_TIMEOUT,
// raises the CTA's abort flag (which every other wait polls) and returns.
#pragma once

#include "common.cuh"
#include "glue_kernels.cuh"

namespace xabe {

constexpr int kStreamGroups = 2;
constexpr int kStreamGroupWarps = 8;
constexpr int kGateupSlots = kStreamGroupWarps + 1;  // partial sums of a gate/up row, see gateup_span_of
constexpr int kStreamConsumerWarps = kStreamGroups * kStreamGroupWarps;
constexpr int kStreamThreads = 32 * (2 + kStreamConsumerWarps);  // warp 0 streams weights, the last warp stages activations
constexpr int kStreamMaxStages = 4;
constexpr int kXRowPadBytes = 32;  // makes the B-fragment reads bank-conflict free

constexpr int MODE_GATEUP = 0;
constexpr int MODE_DOWN = 1;

struct StreamLaunch {
    const uint8_t* r_a;  // routed gate (or down) stack
    const uint8_t* r_b;  // routed up stack
    const uint8_t* s_a;  // shared gate (or down)
    const uint8_t* s_b;  // shared up
    int rows;            // output rows per matrix
    int k;               // contraction length
    int top_k;
    int has_routed, has_shared;
    const int* work_items;  // column groups (kWorkItemInts each)
    const int* n_work;      // device scalar
    const int* valid_tokens;
    const __half* x_routed;  // gate/up: normed_h [token]; down: inter [slot]
    const __half* x_shared;  // gate/up: normed_h [token]; down: inter_shared [token]
    __half* inter_routed;    // gate/up out, [slot][rows]
    __half* inter_shared;    // gate/up out, [token][rows]
    float* partial;          // down out, [flat][rows]
    float* const* partial_rows;  // optional: destination of result row `flat` instead (NULL: use partial)
    float* shexp;            // down out, [token][rows]
    int* status;
    int n_stages;
    uint32_t tile_cap;    // staged bytes reserved per tensor per stage (multiple of 16)
    uint32_t x_stride;    // bytes between activation rows in shared memory
    int num_experts;      // bounds for the producer's self-check of a column group
    int x_rows_routed;    // rows the routed activation buffer holds
    int max_tokens;
    int down_row_step;    // MODE_DOWN: rows of one fragment half are this far apart (bank-conflict free reads)
    int runs_override;    // tuning aid: > 0 fixes the runs per column group
    // MODE_DOWN, optional: the block's last stage folded into this launch (see combine_tile).  A null
    // tail_done means a separate kernel combines.
    int* tail_done;             // [max_tokens][rows / 128] arrivals per (token, row tile), zero between launches
    int tail_target;            // arrivals that complete a (token, row tile): (top_k + 1) groups x 8 warps
    const float* tail_gate;     // [max_tokens] sigmoid gate of the shared expert
    const float* tail_residual; // [max_tokens][rows]
    float* tail_routed;         // [max_tokens][rows]
    float* tail_ffn;            // [max_tokens][rows]
    float* tail_lout;           // [max_tokens][rows]
};

// The last stage of the block (moe_block_gate_and_combine, crates/xabe-engine/src/block/moe.rs:424-483)
// for 128 output columns of one token, by one warp: routed = ascending-k sum of the weighted expert
// rows, ffn_out = routed + shexp * gate, l_out = ffn_out + residual.  Called by the warp whose
// arrival completed the token's row tile (every expert row and the shared expert's row of these 128
// columns is then in memory; they were written by other CTAs, so they are read through L2).
__device__ __forceinline__ void combine_tile(const StreamLaunch& L, int token, int tile, int lane) {
    const int rows = L.rows;
    const size_t col = (size_t)tile * 128 + (size_t)lane * 4;
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* pbase = L.partial + (size_t)token * L.top_k * rows + col;
    for (int k0 = 0; k0 < L.top_k; k0 += 4) {  // four rows in flight, then the same ascending-k sum
        float4 pv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (k0 + k < L.top_k) pv[k] = __ldcg((const float4*)(pbase + (size_t)(k0 + k) * rows));
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (k0 + k < L.top_k) {
                r.x += pv[k].x;
                r.y += pv[k].y;
                r.z += pv[k].z;
                r.w += pv[k].w;
            }
    }
    const size_t o = (size_t)token * rows + col;
    const float4 sh = __ldcg((const float4*)(L.shexp + o));
    const float4 res = *(const float4*)(L.tail_residual + o);
    const float g = L.tail_gate[token];
    float4 v;
    v.x = fmaf(sh.x, g, r.x);
    v.y = fmaf(sh.y, g, r.y);
    v.z = fmaf(sh.z, g, r.z);
    v.w = fmaf(sh.w, g, r.w);
    *(float4*)(L.tail_routed + o) = r;
    *(float4*)(L.tail_ffn + o) = v;
    *(float4*)(L.tail_lout + o) = make_float4(v.x + res.x, v.y + res.y, v.z + res.z, v.w + res.w);
}

// Buffers for the activation rows of a unit.  The producer stages a unit's rows while the consumers
// still work on the unit before it, into the buffer of the unit before that one.  gate/up gives
// its buffer back as soon as the fragments are in registers (two buffers); down reads the rows
// for every tile and gives it back when the unit ends (three buffers of short rows).
constexpr int kStreamMaxXBuffers = 3;
__host__ __device__ constexpr int stream_x_buffers(int mode) { return mode == 0 ? 2 : 3; }

struct StreamSmem {
    // byte offsets into dynamic shared memory, identical on host and device
    uint32_t stages, xbuf, items, red, bars, total;
};

__host__ __device__ inline StreamSmem stream_smem_layout(int mode, int n_stages, uint32_t tile_cap,
                                                         uint32_t x_stride) {
    StreamSmem L;
    uint32_t stage_bytes = (mode == MODE_GATEUP ? 2u : 1u) * tile_cap;
    L.stages = 0;
    L.xbuf = L.stages + (uint32_t)n_stages * stage_bytes;
    const uint32_t nxb = (uint32_t)stream_x_buffers(mode);
    L.items = L.xbuf + nxb * 8u * x_stride;
    L.red = L.items + nxb * 96u;
    L.bars = L.red + (mode == MODE_GATEUP ? (uint32_t)(kStreamGroups * 2 * kGateupSlots * 4 * 32 * 4) : 0u);
    L.total = L.bars + 8u * (2u * kStreamMaxStages + 2u * kStreamMaxXBuffers + 4u * kStreamGroups) + 64u;
    return L;
}

struct StreamBars {
    uint64_t* full;      // [n_stages]  producer -> consumers (tx bytes)
    uint64_t* empty;     // [n_stages]  8 consumer warps -> producer
    uint64_t* xfull;     // [kStreamMaxXBuffers]
    uint64_t* xempty;    // [kStreamMaxXBuffers]  16 consumer warps -> producer
    uint64_t* redfull;   // [groups][2]  8 warps -> epilogue warp
    uint64_t* redempty;  // [groups][2]  epilogue warp -> 8 warps
};

__device__ __forceinline__ StreamBars stream_bars(uint8_t* smem, const StreamSmem& L) {
    StreamBars b;
    b.full = (uint64_t*)(smem + L.bars);
    b.empty = b.full + kStreamMaxStages;
    b.xfull = b.empty + kStreamMaxStages;
    b.xempty = b.xfull + kStreamMaxXBuffers;
    b.redfull = b.xempty + kStreamMaxXBuffers;
    b.redempty = b.redfull + 2 * kStreamGroups;
    return b;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait that also gives up when another warp of the CTA already has.
__device__ __forceinline__ bool stream_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u && *abort_flag) return false;
        if (it >= 16u) __nanosleep(it < 256u ? 32u : 256u);  // long waits back off and leave the issue slots to working warps
    }
    *abort_flag = 1;
    if (status) atomicExch(status, STATUS_TMA_TIMEOUT);
    return false;
}

// How the units of one launch are laid out; computed identically by every warp.
struct StreamPlan {
    int n_routed, n_groups, row_tiles, tiles_per_unit, runs, units;
};

__device__ __forceinline__ StreamPlan stream_plan(const StreamLaunch& L, int rows_per_tile) {
    StreamPlan p;
    int valid = *L.valid_tokens;
    p.n_routed = L.has_routed ? *L.n_work : 0;
    int n_shared = L.has_shared ? (valid + 7) >> 3 : 0;
    p.n_groups = p.n_routed + n_shared;
    p.row_tiles = L.rows / rows_per_tile;
    // Runs per column group: the smallest power of two that gives every CTA about two units or
    // more.  Measured by sweeping the run count (64-token batch, 264 groups on 148 CTAs: 2 runs
    // 105 us, 4 runs 108, 8 runs 111, 16 runs 115, 1 run 136; one token, 9 groups: 32 runs best):
    // a unit has a fixed cost of about one tile time (staging the activation rows, loading the
    // fragments), so beyond that point shorter runs only add units.
    int best_r = 1;
    if (L.runs_override > 0) {
        best_r = min(L.runs_override, p.row_tiles);
    } else {
        while (best_r * 2 <= p.row_tiles && p.n_groups * best_r < 2 * (int)gridDim.x) best_r *= 2;
    }
    p.tiles_per_unit = (p.row_tiles + best_r - 1) / best_r;
    p.runs = (p.row_tiles + p.tiles_per_unit - 1) / p.tiles_per_unit;
    p.units = p.n_groups * p.runs;
    return p;
}


// it / S and it % S for the ring depths this kernel is launched with (2, 3 or 4) without an
// integer division in the per-tile path.
__device__ __forceinline__ void ring_pos(uint32_t it, int S, uint32_t& use, int& st) {
    if (S == 4) {
        use = it >> 2;
        st = (int)(it & 3u);
    } else if (S == 2) {
        use = it >> 1;
        st = (int)(it & 1u);
    } else if (S == 3) {
        use = __umulhi(it, 0xAAAAAAABu) >> 1;
        st = (int)(it - 3u * use);
    } else {
        use = it / (uint32_t)S;
        st = (int)(it - use * (uint32_t)S);
    }
}

template <bool MIS>
__device__ __forceinline__ uint32_t ldw(const uint8_t* p) {
    if (MIS) {  // p is 2 modulo 4
        const uint32_t* q = (const uint32_t*)(p - 2);
        return __byte_perm(q[0], q[1], 0x5432);
    }
    return *(const uint32_t*)p;
}

// Four 4-code words (groups j = 0..3) of one (ql word 0, ql word 1, qh word)
// triple, five-plus-six operations for all four: the high bit pairs are
// pre-masked so that a bitwise select merges nibble and pair in one LOP3.
__device__ __forceinline__ void q6k_codes4(uint32_t ql0, uint32_t ql1, uint32_t qh, uint32_t (&raw)[4]) {
    const uint32_t m = 0x0F0F0F0Fu;
    uint32_t qa = qh & 0x33333333u;         // pairs of groups 0 (bits 0-1) and 2 (bits 4-5)
    uint32_t qb = (qh >> 2) & 0x33333333u;  // pairs of groups 1 and 3
    raw[0] = (ql0 & m) | ((qa << 4) & ~m);
    raw[1] = (ql1 & m) | ((qb << 4) & ~m);
    raw[2] = ((ql0 >> 4) & m) | (qa & ~m);
    raw[3] = ((ql1 >> 4) & m) | (qb & ~m);
}

// Half a span (128 elements, 8 k16 steps) of the contraction for fragment rows
// pa (g) and pb (g+8); `h` picks the half.  bf[step] is this lane's B fragment
// of step `step` of that half.  Each of the four lanes that share a row pair
// converts the scales of the steps it owns (step % 4 == t); the others fetch
// them with a shuffle.
// With SPLIT the activations come as two f16 parts (value = hi + lo, fragments `bf` and `bl`):
// the step's product is A * lo added to A * hi inside the tensor core, which keeps about 22 bits
// of an fp32 activation (the LM head, whose largest logit is the sampled token).
template <bool SPLIT>
__device__ __forceinline__ void step_mma(float (&d)[4], const uint32_t (&a)[4], const uint2* bf, const uint2* bl,
                                         int i) {
    if (SPLIT) {
        float lo[4];
        mma_f16_16816(lo, a, bl[i].x, bl[i].y);
        mma_f16_16816_acc(d, a, bf[i].x, bf[i].y, lo);
    } else {
        mma_f16_16816(d, a, bf[i].x, bf[i].y);
    }
}

template <int QUANT, bool MIS, bool SPLIT = false>
__device__ __forceinline__ void stream_half(const uint8_t* pa, const uint8_t* pb, int h, const uint2* bf, int lane,
                                            float (&acc)[4], const uint2* bl = nullptr) {
    const uint32_t bias32 = 0x64206420u;   // half2(1056): 1024 + 32
    const uint32_t bias128 = 0x64806480u;  // half2(1152): 1024 + 128
    const int t = lane & 3;
    const int quad = lane & ~3;
    float own_a[2], own_b[2];
    if (QUANT == QUANT_Q6K) {
        float da = f16_at(pa + 208), db = f16_at(pb + 208);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            // step = c*4 + j with j == t: scale index half*8 + 2*j + c  (quant.rs:183,195-198)
            int si = 192 + h * 8 + 2 * t + c;
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
                float dsa = __shfl_sync(0xffffffffu, own_a[c], quad | j);
                float dsb = __shfl_sync(0xffffffffu, own_b[c], quad | j);
                uint32_t a[4];
                a[0] = bytes01_to_h2(ra[j], bias32);
                a[1] = bytes01_to_h2(rb[j], bias32);
                a[2] = bytes23_to_h2(ra[j], bias32);
                a[3] = bytes23_to_h2(rb[j], bias32);
                float d[4];
                step_mma<SPLIT>(d, a, bf, bl, c * 4 + j);
                acc[0] = fmaf(dsa, d[0], acc[0]);
                acc[1] = fmaf(dsa, d[1], acc[1]);
                acc[2] = fmaf(dsb, d[2], acc[2]);
                acc[3] = fmaf(dsb, d[3], acc[3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // step = 4*i + t of this half -> block h*4 + (4*i + t) / 2
            int blk = h * 4 + ((4 * i + t) >> 1);
            own_a[i] = f16_at(pa + blk * kQ8BlockBytes);
            own_b[i] = f16_at(pb + blk * kQ8BlockBytes);
        }
#pragma unroll
        for (int step = 0; step < 8; ++step) {
            const int blk = h * 4 + (step >> 1), c = step & 1;
            float dsa = __shfl_sync(0xffffffffu, own_a[step >> 2], quad | (step & 3));
            float dsb = __shfl_sync(0xffffffffu, own_b[step >> 2], quad | (step & 3));
            // block bases are 34*blk: word alignment alternates with the block index
            const uint8_t* qa = pa + blk * kQ8BlockBytes + 2 + 16 * c + 4 * t;
            const uint8_t* qb = pb + blk * kQ8BlockBytes + 2 + 16 * c + 4 * t;
            uint32_t wa = ((step >> 1) & 1 ? ldw<MIS>(qa) : ldw<!MIS>(qa)) ^ 0x80808080u;
            uint32_t wb = ((step >> 1) & 1 ? ldw<MIS>(qb) : ldw<!MIS>(qb)) ^ 0x80808080u;
            uint32_t a[4];
            a[0] = bytes01_to_h2(wa, bias128);
            a[1] = bytes01_to_h2(wb, bias128);
            a[2] = bytes23_to_h2(wa, bias128);
            a[3] = bytes23_to_h2(wb, bias128);
            float d[4];
            step_mma<SPLIT>(d, a, bf, bl, step);
            acc[0] = fmaf(dsa, d[0], acc[0]);
            acc[1] = fmaf(dsa, d[1], acc[1]);
            acc[2] = fmaf(dsb, d[2], acc[2]);
            acc[3] = fmaf(dsb, d[3], acc[3]);
        }
    }
}

// Element offset (within a span) of this lane's four activations for step
// `step` (0..7) of half `h`.
template <int QUANT>
__device__ __forceinline__ int step_k_offset(int h, int step, int t) {
    if (QUANT == QUANT_Q6K) {
        int c = step >> 2, j = step & 3;
        return h * 128 + j * 32 + 16 * c + 4 * t;
    }
    return (h * 4 + (step >> 1)) * 32 + 16 * (step & 1) + 4 * t;
}

template <int QUANT>
__device__ __forceinline__ void load_bfrags_half(const uint8_t* xrow, int span, int h, int t, uint2* bf) {
#pragma unroll
    for (int step = 0; step < 8; ++step)
        bf[step] = *(const uint2*)(xrow + 2 * (span * 256 + step_k_offset<QUANT>(h, step, t)));
}

// The host only selects these kernels when every row pitch is a multiple of 4
// bytes, so all lanes of a warp (and both fragment rows) share one alignment.
template <int QUANT>
__device__ __forceinline__ void half_dispatch(const uint8_t* pa, const uint8_t* pb, int h, const uint2* bf, int lane,
                                              float (&acc)[4]) {
    if ((uintptr_t)pa & 2) stream_half<QUANT, true>(pa, pb, h, bf, lane, acc);
    else stream_half<QUANT, false>(pa, pb, h, bf, lane, acc);
}

// MODE_DOWN: the tile row (0..127) that fragment row g (half 0) or g+8 (half 1)
// of warp w reads.  With step 1 a warp owns 16 consecutive rows.  With step 4
// the eight rows of a fragment half are four rows apart: a 420-byte row pitch
// (two Q6_K superblocks) is 105 words, so rows four apart start 4 banks apart
// and the eight 16-byte reads of a load cover all 32 banks exactly once.
__device__ __forceinline__ int down_row(int w, int g, int half, int step) {
    if (step == 4) return (w >> 1) * 32 + 4 * g + 2 * (w & 1) + half;
    return w * 16 + g + 8 * half;
}

// Which span feeds half `h` of warp-slot `w`.  Superblocks of 210 bytes
// alternate between word-aligned and not, so a gate/up warp takes its two
// halves from neighbouring spans: every warp then carries one aligned and one
// unaligned half and the eight warps of a group finish together.
__device__ __forceinline__ int gateup_span_of(int w, int h, int n_spans) {
    return h == 0 ? w : (w + 1) % n_spans;
}
// Partial sums of a gate/up row, in the order they are added: slot w < n_spans - 1 is half 0 of
// span w continued by half 1 of span w + 1; slot n_spans - 1 is half 0 of the last span alone;
// the idle slots (n_spans < 8) are zero; and half 1 of span 0 is a sum of its own, the "wrap"
// slot, added last.  Keeping the wrapped-around half out of the last slot lets a kernel that
// walks the spans in ascending order for one set of rows (k_gateup_rows) form the same sums in
// the same order without seeing a span twice.

// ---------------------------------------------------------------------------
// The kernel.  MODE_GATEUP: tile = 8 gate rows + the same 8 up rows (fragment
// rows 0-7 / 8-15), eight warps split the spans, SwiGLU epilogue, f16 out.
// MODE_DOWN: tile = 128 rows, one m16 tile per warp over the whole contraction
// (at most two spans), weight * value (routed) or value (shared) out, fp32.
// TAIL (MODE_DOWN only): the launch also performs the block's last stage, see combine_tile.
// grid: number of SMs; block: kStreamThreads.
// ---------------------------------------------------------------------------
template <int MODE, int QR, int QS, bool TAIL = false>
__global__ void __launch_bounds__(kStreamThreads, 1) k_expert_stream(StreamLaunch L) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int abort_flag;
    __shared__ StreamPlan plan_shared;  // computed once, by thread 0
    constexpr int ROWS_PER_TILE = MODE == MODE_GATEUP ? 8 : 128;
    const StreamSmem lay = stream_smem_layout(MODE, L.n_stages, L.tile_cap, L.x_stride);
    const StreamBars bars = stream_bars(smem, lay);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = L.n_stages;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            mbar_init(&bars.full[i], 1);
            mbar_init(&bars.empty[i], kStreamGroupWarps);
        }
        for (int i = 0; i < kStreamMaxXBuffers; ++i) {
            mbar_init(&bars.xfull[i], 1);
            mbar_init(&bars.xempty[i], kStreamConsumerWarps);
        }
        for (int i = 0; i < 2 * kStreamGroups; ++i) {
            mbar_init(&bars.redfull[i], kStreamGroupWarps);
            mbar_init(&bars.redempty[i], 1);
        }
        fence_mbar_init();
    }
    if (threadIdx.x == 0) plan_shared = stream_plan(L, ROWS_PER_TILE);
    __syncthreads();
    const StreamPlan plan = plan_shared;
    const int n_spans = L.k / kSpanElems;
    const uint32_t stage_bytes = (MODE == MODE_GATEUP ? 2u : 1u) * L.tile_cap;
    volatile int* abortp = &abort_flag;

    if (warp == 0 || warp == 1 + kStreamConsumerWarps) {
        // ------------------------------ producers ------------------------------
        if (lane != 0) return;
        constexpr int NXB = stream_x_buffers(MODE);
        // Stages the activation rows and the descriptor of unit `u` (the CTA's `v`-th) in buffer
        // xb, whose previous user was the CTA's (v - NXB)-th unit.
        auto stage_x = [&](int u, uint32_t v, int xb, uint32_t xuse) -> bool {
            const int cg = u / plan.runs;
            const bool shared = cg >= plan.n_routed;
            int* desc = (int*)(smem + lay.items + xb * 96);  // [0..3] written here, [4..] item copy
            if (v >= (uint32_t)NXB && !stream_wait(&bars.xempty[xb], (xuse - 1) & 1, abortp, L.status)) return false;
            int expert, first, ncols;
            const int* item = nullptr;
            if (!shared) {
                item = L.work_items + (size_t)cg * kWorkItemInts;
                expert = item[0];
                first = item[1];
                ncols = item[2];
            } else {
                expert = -1;
                first = (cg - plan.n_routed) * 8;
                ncols = min(8, *L.valid_tokens - first);
            }
            // self-check: a column group that points outside its buffers is skipped and
            // recorded, never dereferenced
            bool sane = ncols >= 1 && ncols <= 8 && first >= 0;
            if (!shared) {
                sane = sane && expert >= 0 && expert < L.num_experts;
                if (MODE == MODE_GATEUP) {
                    for (int c = 0; sane && c < ncols; ++c) {
                        int tok = item[4 + c] / L.top_k;
                        sane = item[4 + c] >= 0 && tok < L.max_tokens;
                    }
                } else {
                    sane = sane && first + ncols <= L.x_rows_routed;
                }
            } else {
                sane = sane && first + ncols <= L.max_tokens;
            }
            if (!sane) {
                *abortp = 1;
                atomicExch(L.status, STATUS_BAD_WORK_ITEM);
                return false;
            }
            desc[0] = expert;
            desc[1] = first;
            desc[2] = ncols;
            const uint32_t xrow_bytes = (uint32_t)L.k * 2u;
            mbar_expect_tx(&bars.xfull[xb], ncols * xrow_bytes + (shared ? 0u : 64u));
            uint8_t* xdst = smem + lay.xbuf + (uint32_t)xb * 8u * L.x_stride;
            for (int c = 0; c < ncols; ++c) {
                size_t src_row;
                if (MODE == MODE_GATEUP) src_row = shared ? (size_t)(first + c) : (size_t)(item[4 + c] / L.top_k);
                else src_row = (size_t)(first + c);  // slot (routed) or token (shared)
                const __half* src = (shared ? L.x_shared : L.x_routed) + src_row * L.k;
                tma_bulk_g2s(xdst + c * L.x_stride, src, xrow_bytes, &bars.xfull[xb]);
            }
            if (!shared) tma_bulk_g2s(desc + 4, item + 4, 64u, &bars.xfull[xb]);  // flat ids + weights
            return true;
        };
        if (warp != 0) {
            // ---- activation stager: runs up to NXB units ahead of the consumers; its reads of
            // the column-group descriptors never hold up the weight stream
            int xb = 0;
            uint32_t xuse = 0, v = 0;
            for (int u = blockIdx.x; u < plan.units; u += gridDim.x, ++v) {
                if (!stage_x(u, v, xb, xuse)) return;
                if (++xb == NXB) {
                    xb = 0;
                    ++xuse;
                }
            }
            return;
        }
        // ---- weight producer
        uint32_t it = 0;
        int expert_next = -1;
        if ((int)blockIdx.x < plan.units) {
            const int cg0 = (int)blockIdx.x / plan.runs;
            if (cg0 < plan.n_routed) expert_next = L.work_items[(size_t)cg0 * kWorkItemInts];
        }
        for (int u = blockIdx.x; u < plan.units; u += gridDim.x) {
            const int cg = u / plan.runs, run = u % plan.runs;
            const bool shared = cg >= plan.n_routed;
            const int quant = shared ? QS : QR;
            const int row_bytes = n_spans * span_bytes_of(quant);
            const int expert = expert_next;
            {  // the next unit's expert id is fetched while this unit's tiles stream
                const int un = u + (int)gridDim.x;
                const int cgn = un / plan.runs;
                if (un < plan.units && cgn < plan.n_routed) expert_next = L.work_items[(size_t)cgn * kWorkItemInts];
            }
            if (!shared && (expert < 0 || expert >= L.num_experts)) return;  // the stager records the bad group
            const uint8_t* wa = shared ? L.s_a : L.r_a;
            const uint8_t* wb = shared ? L.s_b : L.r_b;
            const size_t row0 = (shared ? 0 : (size_t)expert * L.rows);
            const int t_begin = run * plan.tiles_per_unit;
            const int t_end = min(plan.row_tiles, t_begin + plan.tiles_per_unit);
            for (int tile = t_begin; tile < t_end; ++tile, ++it) {
                int st;
                uint32_t use;
                ring_pos(it, S, use, st);
                if (use >= 1 && !stream_wait(&bars.empty[st], (use - 1) & 1, abortp, L.status)) return;
                const size_t start = (row0 + (size_t)tile * ROWS_PER_TILE) * row_bytes;
                const uint32_t tile_bytes = (uint32_t)ROWS_PER_TILE * row_bytes;
                const size_t a0 = start & ~(size_t)15, a1 = (start + tile_bytes + 15) & ~(size_t)15;
                const uint32_t nbytes = (uint32_t)(a1 - a0);
                uint8_t* dst = smem + lay.stages + (uint32_t)st * stage_bytes;
                mbar_expect_tx(&bars.full[st], (MODE == MODE_GATEUP ? 2u : 1u) * nbytes);
                tma_bulk_g2s(dst, wa + a0, nbytes, &bars.full[st]);
                if (MODE == MODE_GATEUP) tma_bulk_g2s(dst + L.tile_cap, wb + a0, nbytes, &bars.full[st]);
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int cw = warp - 1;
    const int gi = cw / kStreamGroupWarps;  // group
    const int w = cw % kStreamGroupWarps;   // warp within the group
    const int g = lane >> 2, t = lane & 3;
    float* red = (float*)(smem + lay.red);
    constexpr int NXB = stream_x_buffers(MODE);
    uint32_t it = 0, gt = 0;  // ring tile counter, this group's tile counter
    int xb = -1;              // activation buffer of the unit and how often it was used before
    uint32_t xuse = 0;
    for (int u = blockIdx.x; u < plan.units; u += gridDim.x) {
        const int cg = u / plan.runs, run = u % plan.runs;
        const bool shared = cg >= plan.n_routed;
        const int quant = shared ? QS : QR;
        const int row_bytes = n_spans * span_bytes_of(quant);
        if (++xb == NXB) {
            xb = 0;
            ++xuse;
        }
        if (!stream_wait(&bars.xfull[xb], xuse & 1, abortp, L.status)) return;
        const int* desc = (const int*)(smem + lay.items + xb * 96);
        const int expert = desc[0], first = desc[1], ncols = desc[2];
        int flat0 = 0, flat1 = 0;
        float wgt0 = 0.f, wgt1 = 0.f;
        if (MODE == MODE_DOWN && !shared) {
            flat0 = desc[4 + 2 * t];
            flat1 = desc[4 + 2 * t + 1];
            wgt0 = __int_as_float(desc[12 + 2 * t]);
            wgt1 = __int_as_float(desc[12 + 2 * t + 1]);
        }
        // B fragments of this unit: column g of the group (dead columns read stale rows
        // and are never stored)
        const uint8_t* xrow = smem + lay.xbuf + (uint32_t)xb * 8u * L.x_stride + g * L.x_stride;
        // MODE_DOWN re-reads its fragments from the activation rows for every tile (32 steps of
        // fragments in registers spilled), so the rows stay owned until the unit ends.
        uint2 bf[1][16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int span = gateup_span_of(w, h, n_spans);
            if (MODE == MODE_GATEUP && w < n_spans) {
                if (quant == QUANT_Q6K) load_bfrags_half<QUANT_Q6K>(xrow, span, h, t, &bf[0][8 * h]);
                else load_bfrags_half<QUANT_Q8_0>(xrow, span, h, t, &bf[0][8 * h]);
            }
        }
        if (MODE == MODE_GATEUP) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.xempty[xb]);
        }
        const uint32_t phase = (uint32_t)((((shared ? 0 : (size_t)expert * L.rows)) * row_bytes) & 15);
        const int t_begin = run * plan.tiles_per_unit;
        const int t_end = min(plan.row_tiles, t_begin + plan.tiles_per_unit);
        for (int tile = t_begin; tile < t_end; ++tile, ++it) {
            if ((int)(it % kStreamGroups) != gi) continue;
            int st;
            uint32_t use;
            ring_pos(it, S, use, st);
            if (!stream_wait(&bars.full[st], use & 1, abortp, L.status)) return;
            const uint8_t* tb = smem + lay.stages + (uint32_t)st * stage_bytes +
                                (uint32_t)((phase + (size_t)tile * ROWS_PER_TILE * row_bytes) & 15);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            float wrap[4] = {0.f, 0.f, 0.f, 0.f};  // gate/up, last slot only: half 1 of span 0
            const bool wraps = MODE == MODE_GATEUP && n_spans > 1 && w == n_spans - 1;
            if (MODE == MODE_GATEUP) {
                if (w < n_spans) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint8_t* pa = tb + g * row_bytes + gateup_span_of(w, h, n_spans) * span_bytes_of(quant);
                        const uint8_t* pb = pa + L.tile_cap;
                        if (h == 1 && wraps) {  // the wrap slot starts from zero; the last slot is parked in `wrap`
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                wrap[i] = acc[i];
                                acc[i] = 0.f;
                            }
                        }
                        if (quant == QUANT_Q6K) half_dispatch<QUANT_Q6K>(pa, pb, h, &bf[0][8 * h], lane, acc);
                        else half_dispatch<QUANT_Q8_0>(pa, pb, h, &bf[0][8 * h], lane, acc);
                    }
                    if (wraps) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float v = acc[i];
                            acc[i] = wrap[i];
                            wrap[i] = v;
                        }
                    }
                }
            } else {
                const uint8_t* pa = tb + (size_t)down_row(w, g, 0, L.down_row_step) * row_bytes;
                const uint8_t* pb = tb + (size_t)down_row(w, g, 1, L.down_row_step) * row_bytes;
                for (int sp = 0; sp < n_spans; ++sp) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint2 b1[8];
                        if (quant == QUANT_Q6K) {
                            load_bfrags_half<QUANT_Q6K>(xrow, sp, h, t, b1);
                            half_dispatch<QUANT_Q6K>(pa + sp * 210, pb + sp * 210, h, b1, lane, acc);
                        } else {
                            load_bfrags_half<QUANT_Q8_0>(xrow, sp, h, t, b1);
                            half_dispatch<QUANT_Q8_0>(pa + sp * 272, pb + sp * 272, h, b1, lane, acc);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.empty[st]);  // the ring stage may be refilled
            if (MODE == MODE_GATEUP) {
                const int buf = gt & 1;
                float* rb = red + ((size_t)(gi * 2 + buf) * kGateupSlots) * 128;
                if (gt >= 2 && !stream_wait(&bars.redempty[gi * 2 + buf], ((gt >> 1) - 1) & 1, abortp, L.status))
                    return;
#pragma unroll
                for (int i = 0; i < 4; ++i) rb[(w * 4 + i) * 32 + lane] = acc[i];
                if (wraps) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) rb[(kStreamGroupWarps * 4 + i) * 32 + lane] = wrap[i];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.redfull[gi * 2 + buf]);
                if (w == (int)(gt % kStreamGroupWarps)) {  // the epilogue rotates over the group's warps
                    if (!stream_wait(&bars.redfull[gi * 2 + buf], (gt >> 1) & 1, abortp, L.status)) return;
                    float tot[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float s = rb[(0 * 4 + i) * 32 + lane];
#pragma unroll
                        for (int ww = 1; ww < kStreamGroupWarps; ++ww) s += rb[(ww * 4 + i) * 32 + lane];
                        if (n_spans > 1) s += rb[(kStreamGroupWarps * 4 + i) * 32 + lane];
                        tot[i] = s;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.redempty[gi * 2 + buf]);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        int col = 2 * t + i;
                        if (col < ncols) {
                            float gv = tot[i], uv = tot[2 + i];
                            float v = __fdiv_rn(gv, 1.0f + expf(-gv)) * uv;
                            __half* dst = (shared ? L.inter_shared : L.inter_routed) + (size_t)(first + col) * L.rows;
                            dst[tile * 8 + g] = __float2half_rn(v);
                        }
                    }
                }
                ++gt;
            } else {
                const int row_lo = tile * 128 + down_row(w, g, 0, L.down_row_step);
                const int row_hi = tile * 128 + down_row(w, g, 1, L.down_row_step);
                if (shared) {
                    if (2 * t < ncols) {
                        float* dst = L.shexp + (size_t)(first + 2 * t) * L.rows;
                        dst[row_lo] = acc[0];
                        dst[row_hi] = acc[2];
                    }
                    if (2 * t + 1 < ncols) {
                        float* dst = L.shexp + (size_t)(first + 2 * t + 1) * L.rows;
                        dst[row_lo] = acc[1];
                        dst[row_hi] = acc[3];
                    }
                } else {
                    if (2 * t < ncols) {
                        float* dst = result_row(L.partial, L.partial_rows, flat0, L.rows);
                        dst[row_lo] = wgt0 * acc[0];
                        dst[row_hi] = wgt0 * acc[2];
                    }
                    if (2 * t + 1 < ncols) {
                        float* dst = result_row(L.partial, L.partial_rows, flat1, L.rows);
                        dst[row_lo] = wgt1 * acc[1];
                        dst[row_hi] = wgt1 * acc[3];
                    }
                }
                if (TAIL) {
                    // This warp's 16 rows of the tile are stored.  Count the arrival for every token of
                    // the group; the arrival that completes a (token, row tile) combines its 128 columns.
                    __threadfence();
                    __syncwarp();
                    int tok = -1;
                    if (lane < ncols) tok = shared ? first + lane : desc[4 + lane] / L.top_k;
                    bool fin = false;
                    if (tok >= 0) {
                        int* cnt = L.tail_done + (size_t)tok * plan.row_tiles + tile;
                        fin = atomicAdd(cnt, 1) == L.tail_target - 1;
                        if (fin) *cnt = 0;  // the last arrival: ready for the next launch
                    }
                    unsigned todo = __ballot_sync(0xffffffffu, fin);
                    if (todo) __threadfence();
                    while (todo) {
                        const int src = __ffs(todo) - 1;
                        todo &= todo - 1;
                        combine_tile(L, __shfl_sync(0xffffffffu, tok, src), tile, lane);
                    }
                }
            }
        }
        if (MODE == MODE_DOWN) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.xempty[xb]);
        }
    }
}

}  // namespace xabe
