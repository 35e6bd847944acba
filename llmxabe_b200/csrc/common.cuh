// Device helpers shared by the sm_100a MoE kernels: 1-D TMA bulk copies with
// mbarrier completion and BOUNDED waits, the f16 tensor-core tile, and loads
// of 32-bit words that sit on 2-byte boundaries (raw 210-byte Q6_K superblocks
// and 34-byte Q8_0 blocks are only 2-byte aligned).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xabe {

constexpr int kQ6KBlockBytes = 210;  // crates/xabe-kernels/src/quant.rs:735  (ql 128 | qh 64 | sc 16 | d 2)
constexpr int kQ8BlockBytes = 34;    // crates/xabe-kernels/src/quant.rs:732  (d 2 | qs 32)
constexpr int kSpanElems = 256;      // one Q6_K superblock, or eight Q8_0 blocks
constexpr int QUANT_Q6K = 0;
constexpr int QUANT_Q8_0 = 1;

// Device status word values (read by xabe_moe_device_status).
constexpr int STATUS_OK = 0;
constexpr int STATUS_TMA_TIMEOUT = 1;
constexpr int STATUS_BAD_WORK_ITEM = 2;

// Iterations a wait on an mbarrier may spin before the kernel gives up,
// records STATUS_TMA_TIMEOUT and returns.  try_wait itself blocks for a
// hardware-defined slice, so this is several milliseconds at least.
constexpr uint32_t kWaitLimit = 1u << 22;

template <int QUANT> struct QFmt;
template <> struct QFmt<QUANT_Q6K> { static constexpr int span_bytes = 210; };
template <> struct QFmt<QUANT_Q8_0> { static constexpr int span_bytes = 8 * 34; };

__host__ __device__ inline int span_bytes_of(int quant) { return quant == QUANT_Q6K ? 210 : 272; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// 1-D bulk copy global -> this CTA's shared memory.  dst, src and bytes must
// all be multiples of 16.  No multicast.
__device__ __forceinline__ void tma_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after recording the status) when the limit
// ran out; the caller must then skip its work and return.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status) {
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (status) atomicExch(status, STATUS_TMA_TIMEOUT);
    // One more bounded look, so that a copy that was merely slow has landed
    // before this CTA's shared memory is handed to the next one.
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) break;
    }
    return false;
}

// D(16x8,f32) = A(16x16,f16,row) * B(16x8,f16,col) with a zero accumulator.
// Fragment ownership for lane (g = lane/4, t = lane%4):
//   a[0] = A[g][2t,2t+1]   a[1] = A[g+8][2t,2t+1]   a[2] = A[g][2t+8,2t+9]   a[3] = A[g+8][2t+8,2t+9]
//   b0 = B[2t,2t+1][g]     b1 = B[2t+8,2t+9][g]
//   d[0],d[1] = D[g][2t,2t+1]      d[2],d[3] = D[g+8][2t,2t+1]
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f), "f"(0.f), "f"(0.f));
}

// The same product added to `c`.
__device__ __forceinline__ void mma_f16_16816_acc(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                                  const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// 32-bit word at a 2-byte-aligned shared-memory address.
__device__ __forceinline__ uint32_t ld32_al2(const uint8_t* p) {
    uintptr_t a = (uintptr_t)p;
    if (a & 2) {
        const uint32_t* q = (const uint32_t*)(a - 2);
        return __byte_perm(q[0], q[1], 0x5432);
    }
    return *(const uint32_t*)a;
}

__device__ __forceinline__ float f16_at(const uint8_t* p) {
    return __half2float(*(const __half*)p);
}

// Two packed bytes of `w` -> half2 of exact integers (byte - bias) .
// 0x6400 | b is the half 1024 + b, so subtracting 1024 + bias is exact.
__device__ __forceinline__ uint32_t bytes01_to_h2(uint32_t w, uint32_t bias_h2) {
    uint32_t h = __byte_perm(w, 0x64646464u, 0x4140);
    __half2 r = __hsub2(*(__half2*)&h, *(__half2*)&bias_h2);
    return *(uint32_t*)&r;
}
__device__ __forceinline__ uint32_t bytes23_to_h2(uint32_t w, uint32_t bias_h2) {
    uint32_t h = __byte_perm(w, 0x64646464u, 0x4342);
    __half2 r = __hsub2(*(__half2*)&h, *(__half2*)&bias_h2);
    return *(uint32_t*)&r;
}

// Where the down projection stores result row `flat`: the handle's own [flat][rows] buffer, or,
// under expert parallelism, wherever the row's table entry points (the sender's buffer on a peer
// GPU: plain stores over NVLink straight from the epilogue).
__device__ __forceinline__ float* result_row(float* partial, float* const* partial_rows, int flat, int rows) {
    return partial_rows ? partial_rows[flat] : partial + (size_t)flat * rows;
}

// Programmatic dependent launch: a kernel launched with the "programmatic stream serialization"
// attribute may be scheduled while its predecessor in the stream is still running; it must not touch
// anything the predecessor writes before pdl_wait() returns (which is when the predecessor has
// completed and its writes are visible).  pdl_launch_dependents() lets the successor's launch
// begin.  Both are no-ops for a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The reference's block_reduce_sum (crates/xabe-cuda/src/kernels/layer_ops.rs:93-110,
// crates/xabe-engine/src/block/moe.rs:209-226): shuffle-down inside each warp,
// then the warp totals added in ascending order by thread 0.  The order is
// part of the contract: the sums it produces feed the expert selection.
__device__ __forceinline__ float block_reduce_sum_pinned(float v, float* scratch) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int n_warps = (blockDim.x + 31) >> 5;
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < n_warps; ++w) total += scratch[w];
        scratch[0] = total;
    }
    __syncthreads();
    float r = scratch[0];
    __syncthreads();
    return r;
}

// Exclusive prefix sum of one int per thread over the block (blockDim.x a multiple of 32, at most 1024):
// shuffle scans inside the warps, then the warp totals.  `warp_sums` holds 33 ints; *total gets the
// sum over the block.  Integers: any order gives the same result.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += up;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int w = lane < n_warps ? warp_sums[lane] : 0;
        int wi = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += up;
        }
        warp_sums[lane] = wi - w;  // exclusive prefix of the warp totals
        if (lane == 31) warp_sums[32] = wi;
    }
    __syncthreads();
    const int r = warp_sums[warp] + incl - v;
    *total = warp_sums[32];
    __syncthreads();  // warp_sums may be reused
    return r;
}

}  // namespace xabe
