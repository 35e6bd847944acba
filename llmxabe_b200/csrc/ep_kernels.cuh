// Expert-parallel exchange over peer memory (NVLink): rows are written straight into the owner
// rank's receive regions, results straight back into the sender's buffer, counts and "done" flags
// travel the same way -- no library collective and no host read-back on the data path.
// (No counterpart in the reference, whose multi-GPU model is one replica per device.)
//
// Buffers, all of them ordinary device memory of one rank that the other ranks have mapped
// (CUDA IPC), G = ranks, C = the most pairs one rank can send (its tokens x k):
//   recv_rows [G][C][hidden] f16, recv_eid [G][C] int32   region s is written by rank s
//   recv_meta [G][2] int32    {rows rank s sent here, where they start in rank s's send order}
//   flag_in   [G] int32       rank s stores the step number once its rows and meta are written
//   back_rows [C][hidden] f32 the owners write the results of this rank's pairs, in its send order
//   flag_back [G] int32       owner d stores the step number once its results are written
// Step numbers only grow, so nothing is ever reset.  Every wait is bounded: on a timeout the kernel
// records STATUS_PEER_TIMEOUT and returns, and the owner's step that follows is inert: while the
// status word holds STATUS_PEER_TIMEOUT (until the host reads and clears it) k_ep_fill_slots marks
// every receive slot empty, so no expert runs and nothing is stored into a peer.  The step's output
// is then meaningless; the host learns it from the status word.  Plain peer stores and loads only:
// no multimem, no multicast.
#pragma once

#include "common.cuh"

namespace xabe {

constexpr int STATUS_PEER_TIMEOUT = 3;
constexpr int kEpMaxRanks = 8;
constexpr uint32_t kPeerWaitLimit = 1u << 24;  // default iteration limit, x 200 ns of sleep: several seconds

struct EpPeers {
    void* p[kEpMaxRanks];
};
// Entry d of a by-value table: a chain of selects on the kernel parameter, so that the table is
// never copied to local memory (which indexing it with a run-time d would make every thread do).
__device__ __forceinline__ void* peer_at(const EpPeers& e, int d) {
    void* r = e.p[0];
#pragma unroll
    for (int i = 1; i < kEpMaxRanks; ++i) r = d == i ? e.p[i] : r;
    return r;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Sender, one block, one thread per expert: compact[e] = live pairs of the experts before e;
// rank_start[d] / send_counts[d] = where rank d's pairs start in the send order / how many.
__global__ void k_ep_plan_ranks(int num_experts, int experts_per_rank, const int* __restrict__ expert_counts,
                                int* __restrict__ compact, int* __restrict__ rank_start,
                                int* __restrict__ send_counts) {
    extern __shared__ int cnt_s[];  // [num_experts + 1]
    __shared__ int warp_sums[33];
    int e = threadIdx.x;
    int total = 0;
    const int before = block_exclusive_scan(e < num_experts ? expert_counts[e] : 0, warp_sums, &total);
    if (e <= num_experts) {
        cnt_s[e] = before;  // e == num_experts: the total
        compact[e] = before;
    }
    __syncthreads();
    int world = num_experts / experts_per_rank;
    if (e < world) {
        rank_start[e] = cnt_s[e * experts_per_rank];
        send_counts[e] = cnt_s[(e + 1) * experts_per_rank] - cnt_s[e * experts_per_rank];
    }
}

// Sender: every live slot of the dispatch tables -> the owner's receive region of this rank.
// One WARP per slot (eight slots per block): the chain of dependent table reads that tells a slot
// where its row goes is then in flight for 64 slots per SM instead of 8, and a lane keeps eight
// 16-byte loads in flight.  grid: ceil(sorted_capacity / 8), block 256.
constexpr int kEpPushSlotsPerBlock = 8;
__global__ void __launch_bounds__(256) k_ep_push_rows(
    const int* __restrict__ sorted_token_ids, const int* __restrict__ expert_ids,
    const int* __restrict__ expert_offsets, const int* __restrict__ compact, const int* __restrict__ rank_start,
    const int* __restrict__ num_tokens_post_pad, const int* __restrict__ valid_tokens,
    const __half* __restrict__ normed_h, int top_k, int hidden, int block_size, int experts_per_rank, int me,
    int cap, EpPeers peer_rows, EpPeers peer_eid, int* __restrict__ inverse) {
    const int s = blockIdx.x * kEpPushSlotsPerBlock + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= *num_tokens_post_pad) return;
    const int flat = sorted_token_ids[s];
    if (flat >= *valid_tokens * top_k) return;  // padding slot
    const int e = expert_ids[s / block_size];
    const int d = e / experts_per_rank;
    const int i = compact[e] + (s - expert_offsets[e]);  // position in this rank's send order
    const int j = i - rank_start[d];                     // position among the rows bound for rank d
    const uint4* src = (const uint4*)(normed_h + (size_t)(flat / top_k) * hidden);
    uint4* dst = (uint4*)((__half*)peer_at(peer_rows, d) + ((size_t)me * cap + j) * hidden);
    const int units = hidden / 8;
    for (int u0 = 0; u0 < units; u0 += 256) {
        uint4 v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            if (u0 + q * 32 + lane < units) v[q] = __ldg(src + u0 + q * 32 + lane);
#pragma unroll
        for (int q = 0; q < 8; ++q)
            if (u0 + q * 32 + lane < units) dst[u0 + q * 32 + lane] = v[q];
    }
    if (lane == 0) {
        ((int*)peer_at(peer_eid, d))[(size_t)me * cap + j] = e % experts_per_rank;
        inverse[flat] = i;
    }
    // no fence here: the kernel is complete only when its stores are, and the flag is raised by the
    // next kernel on the stream (k_ep_signal_rows), after a system-scope fence of its own
}

// Sender, after k_ep_push_rows on the same stream: thread d tells rank d how many rows it got and
// where they sit in this rank's send order, then raises its flag there.
__global__ void k_ep_signal_rows(int world, int me, const int* __restrict__ send_counts,
                                 const int* __restrict__ rank_start, EpPeers peer_meta, EpPeers peer_flag_in,
                                 int step) {
    int d = threadIdx.x;
    if (d >= world) return;
    int* meta = (int*)peer_at(peer_meta, d) + 2 * me;
    meta[0] = send_counts[d];
    meta[1] = rank_start[d];
    __threadfence_system();
    st_release_sys((int*)peer_at(peer_flag_in, d) + me, step);
}

// One block, `world` threads: wait until every flag has reached `step`, for at most `limit`
// iterations of 200 ns each.
__global__ void k_ep_wait_flags(int world, const int* __restrict__ flags, int step, uint32_t limit,
                                int* __restrict__ status) {
    int s = threadIdx.x;
    if (s >= world) return;
    for (uint32_t it = 0; it < limit; ++it) {
        if (ld_acquire_sys(flags + s) >= step) return;
        __nanosleep(200);
    }
    atomicExch(status, STATUS_PEER_TIMEOUT);
}

// Owner: expert id of every receive slot (-1 where region s holds no row) and where the slot's
// result goes: the sender's back_rows at (its start for this rank + j).  grid: ceil(G*C/256), block 256.
// After a wait that ran out the {count, start} words may be half-written by a late sender, so the
// whole step is made inert (every slot empty); a region whose words do not describe rows inside the
// sender's buffer of `cap` rows is treated as empty as well.
__global__ void k_ep_fill_slots(int world, int cap, int hidden, const int* __restrict__ recv_meta,
                                const int* __restrict__ recv_eid, int experts_per_rank, EpPeers peer_back,
                                const int* __restrict__ status, int* __restrict__ ids,
                                float** __restrict__ result_dst) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)world * cap) return;
    int s = (int)(idx / cap), j = (int)(idx % cap);
    int count = recv_meta[2 * s], start = recv_meta[2 * s + 1];
    const bool sane = count >= 0 && start >= 0 && count <= cap && start <= cap - count;
    bool live = sane && j < count && *status != STATUS_PEER_TIMEOUT;
    int eid = live ? recv_eid[idx] : -1;
    if (eid < 0 || eid >= experts_per_rank) live = false;
    ids[idx] = live ? eid : -1;
    result_dst[idx] = live ? (float*)peer_at(peer_back, s) + (size_t)(start + j) * hidden : nullptr;
}

// Owner: copy each live slot's result row to its sender.  grid: G*C, block 256.
__global__ void __launch_bounds__(256) k_ep_push_results(const float* __restrict__ partial,
                                                         float* const* __restrict__ result_dst, int hidden) {
    float* dst = result_dst[blockIdx.x];
    if (!dst) return;
    const uint4* src = (const uint4*)(partial + (size_t)blockIdx.x * hidden);
    uint4* d4 = (uint4*)dst;
    for (int u = threadIdx.x; u < hidden / 4; u += 256) d4[u] = src[u];
}

// Owner, after k_ep_push_results on the same stream: raise this rank's flag at every sender.
__global__ void k_ep_signal_results(int world, int me, EpPeers peer_flag_back, int step) {
    int s = threadIdx.x;
    if (s >= world) return;
    __threadfence_system();
    st_release_sys((int*)peer_at(peer_flag_back, s) + me, step);
}

}  // namespace xabe
