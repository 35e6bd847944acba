// C ABI of the sm_100a MoE FFN kernel set.  See include/xabe_moe.h for the
// contract and for the reference method each entry point mirrors.
#include "../../include/xabe_moe.h"

#include <atomic>
#include <mutex>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <utility>

#include "common.cuh"
#include "expert_kernels.cuh"
#include "glue_kernels.cuh"
#include "front_kernels.cuh"
#include "stream_kernels.cuh"
#include "stream_rows_kernels.cuh"
#include "head_kernels.cuh"
#include "ep_kernels.cuh"
#include "prefill_wide_kernels.cuh"
#include "dense_rows_kernels.cuh"

using namespace xabe;

namespace {

// Kernels this library has launched in this process (xabe_kernel_launch_count): every launch site
// passes its stream through counted().
std::atomic<uint64_t> g_kernel_launches{0};
inline cudaStream_t counted(cudaStream_t st) {
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    return st;
}

// A kernel's dynamic shared-memory ceiling is an attribute of the FUNCTION (per device), shared by
// every entry point and host thread that launches it.  Every launch site therefore raises it to the
// same value, the most the device allows beside the kernel's static shared memory, once per function
// and device: no site ever lowers it, so concurrent callers cannot invalidate one another's launches.
cudaError_t allow_dynamic_smem(const void* kern, size_t needed) {
    // a fixed table (function -> bit per device already set): no heap allocation on any call
    struct Entry { const void* kern; uint64_t devices; };
    constexpr int kEntries = 128;
    static std::mutex mu;
    static Entry table[kEntries] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < kEntries && table[i].kern; ++i)
            if (table[i].kern == kern && dev < 64 && (table[i].devices >> dev & 1u)) return cudaSuccess;
    }
    cudaFuncAttributes attr{};
    if ((e = cudaFuncGetAttributes(&attr, kern)) != cudaSuccess) return e;
    int optin = 0;
    if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    const int ceiling = optin - (int)attr.sharedSizeBytes;
    if ((long long)needed > (long long)ceiling) return cudaErrorInvalidValue;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ceiling)) != cudaSuccess) return e;
    if (dev < 64) {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < kEntries; ++i) {
            if (!table[i].kern) table[i].kern = kern;
            if (table[i].kern == kern) {
                table[i].devices |= 1ull << dev;
                break;
            }
        }  // a full table only means the attribute is written again next time
    }
    return cudaSuccess;
}

// Launch, optionally with programmatic stream serialization (the kernel may then be scheduled while
// its predecessor on the stream drains; every kernel launched through here waits for the predecessor
// before it touches its output, see pdl_wait()).  Per handle, off unless XABE_TUNE_PDL was set.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(bool pdl, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                       Args&&... args) {
    const bool off = !pdl;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = counted(st);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = off ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

// Handles sized for this many tokens use k_prefill_gemm_wide (set from measurements).
constexpr uint32_t kPrefillWideMinTokens = 1024;

// Wide passes only take the tcgen05 prefill kernels; the launch shape comes from max_tokens.
constexpr uint32_t kPrefillMinTokens = 512;

// Handles narrower than this fold the block's last stage into the down projection's launch.
constexpr uint32_t kTailMaxTokens = 16;

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define CUDA_TRY(expr)                                                                         \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess)                                                                \
            return fail(XABE_ERR_DRIVER, "CUDA driver error: %s (%s)", cudaGetErrorString(e__), #expr); \
    } while (0)

uint64_t sorted_capacity_of(const xabe_moe_geometry& g) {
    // MoeGeometry::sorted_capacity, crates/xabe-cuda/src/kernels/moe.rs:4575-4584
    uint64_t numel = (uint64_t)g.max_tokens * g.experts_per_token;
    uint64_t active = g.num_experts < numel ? g.num_experts : numel;
    uint64_t bound = numel + active * (g.block_size - 1);
    return (bound + g.block_size - 1) / g.block_size * g.block_size;
}

size_t block_bytes_of(int quant) { return quant == XABE_QUANT_Q6_K ? 210 : 34; }
size_t block_elems_of(int quant) { return quant == XABE_QUANT_Q6_K ? 256 : 32; }

int nb_cap_for(int block_size) {
    int nb = (block_size + 7) / 8;
    return nb <= 1 ? 1 : nb <= 2 ? 2 : nb <= 4 ? 4 : 8;
}

}  // namespace

struct xabe_moe {
    xabe_moe_geometry g{};
    int device = 0;
    int scope = XABE_SCOPE_ROUTED;
    float eps = 1e-6f;
    bool exact_decode = false;
    uint64_t sorted_capacity = 0, block_capacity = 0;
    int n_chunks = 0;
    int align_chunk = 1024;
    int published_tokens = -1;
    int* h_status = nullptr;  // pinned
    // device scratch
    int* valid_tokens = nullptr;
    int* status = nullptr;
    int* topk_ids = nullptr;
    float* topk_weights = nullptr;
    int* sorted_token_ids = nullptr;
    int* expert_ids = nullptr;
    int* num_tokens_post_pad = nullptr;
    int* chunk_hist = nullptr;
    int* expert_offsets = nullptr;
    int* expert_counts = nullptr;
    int* work_items = nullptr;  // column groups, kWorkItemInts ints each
    int* n_work = nullptr;      // device scalar: routed column groups this step
    uint64_t work_capacity = 0;
    int sm_count = 0;
    int* pf_items = nullptr;    // token tiles for the tcgen05 prefill kernels
    int* pf_n_items = nullptr;
    uint64_t pf_capacity = 0;
    int pf_item_cols = 128;     // token columns per item: 128 (k_prefill_gemm) or 512 (k_prefill_gemm_wide)
    // per-handle switches (xabe_moe_set_tuning, xabe_moe_disable_tensor_cores, xabe_moe_force_prefill_path)
    bool force_tile_kernels = false;  // use the one-tile-per-CTA kernels even where the streaming ones apply
    bool pdl = false;                 // programmatic dependent launch between the block's kernels
    bool tensor_cores = true;         // false: never the tcgen05 kernels
    bool force_prefill = false;       // the tcgen05 kernels at every width
    int stream_stages = 0;            // 0: as many ring stages as fit
    int stream_runs = 0;              // 0: the kernel's own choice
    int rows_min_tokens = -1;         // -1: the measured default; 0: k_gateup_rows off
    int router_regw = -1;             // -1: by width; 0/1: off/on
    uint32_t peer_wait_limit = 0;     // 0: kPeerWaitLimit
    // Both fusions are off by default.  Measured under CUDA-graph replay at 1 / 3 / 64 tokens (us per
    // layer): one kernel per stage 34.8 / 49.5 / 154.7; last stage folded in 36.9 / 54.4 / -; front
    // fused as well 34.3 / 54.8 / 182.6.  A launch boundary inside a replayed graph costs about 2 us,
    // less than the fences, arrival counts and one-CTA phases that replace it.
    bool fused_tail = false;          // handles under 16 tokens: gate-and-combine folded into the down launch
    bool fused_front = false;         // handles up to 256 tokens: norm .. dispatch in one launch (k_decode_front)
    bool fused_norm = true;           // handles up to 8 tokens: the router normalises its input rows itself
    float* normed = nullptr;
    __half* normed_h = nullptr;
    float* dense_partial = nullptr;  // [dense_k_splits][max_tokens][hidden]: k_dense_rows<DOWN>'s shares of the contraction
    int dense_k_splits = 1;
    bool dense_rows = true;          // decode-width dense block through k_dense_rows (XABE_TUNE_DENSE_ROWS)
    int* tail_done = nullptr;      // [kTailMaxTokens][hidden / 128] arrivals of the fused combine, zero between launches
    int* front_tickets = nullptr;  // [1 + max_tokens] arrival counters of k_decode_front, zero between launches
    int* ep_compact = nullptr;  // [num_experts + 1] live pairs before each expert (expert parallelism)
    int* ep_rank_start = nullptr;   // [kEpMaxRanks] where each rank's pairs start in the send order
    int* ep_send_counts = nullptr;  // [kEpMaxRanks]
    __half* x_sorted = nullptr;  // activations in dispatch order (k_prefill_gemm_wide's routed gate/up source)
    CUtensorMap tm_routed_gu{}, tm_routed_dn{}, tm_shared_gu{}, tm_shared_dn{};
    float* const* partial_rows = nullptr;  // optional per-row destinations of the down projection (expert parallelism)
    const __half* x_routed_override = nullptr;  // caller-provided f16 rows for one grouped pass
    float* logits = nullptr;
    __half* inter_routed = nullptr;
    __half* inter_shared = nullptr;
    float* partial = nullptr;
    float* routed = nullptr;
    float* shexp = nullptr;
    float* gate = nullptr;
    float* stage_in = nullptr;
    float* stage_ffn = nullptr;
    float* stage_out = nullptr;
    // stage profile: CUDA-event spans around each stage of block_forward
    bool prof_on = false;
    int prof_calls = 0;
    cudaEvent_t* prof_events = nullptr;  // [kProfCalls][XABE_STAGE_COUNT + 1]
};

namespace {

constexpr int kProfCalls = 256;

inline void prof_mark(xabe_moe* m, cudaStream_t st, int idx) {
    if (m->prof_on && m->prof_calls < kProfCalls)
        cudaEventRecord(m->prof_events[m->prof_calls * (XABE_STAGE_COUNT + 1) + idx], st);
}

template <typename T>
cudaError_t dev_alloc(T** p, size_t n) {
    cudaError_t e = cudaMalloc((void**)p, (n ? n : 1) * sizeof(T));
    if (e == cudaSuccess) e = cudaMemset(*p, 0, (n ? n : 1) * sizeof(T));
    return e;
}

// check_stack, crates/xabe-cuda/src/kernels/moe.rs:6729-6746
int check_stack(const char* which, const xabe_quant_tensor& t, size_t expected) {
    if (t.quant != XABE_QUANT_Q6_K && t.quant != XABE_QUANT_Q8_0)
        return fail(XABE_ERR_UNSUPPORTED_EXPERT_TYPE,
                    "expert stack `%s` has quant tag %d, which the grouped GEMM cannot unpack (it handles "
                    "Q6_K and Q8_0)", which, t.quant);
    if (!t.dev_bytes) return fail(XABE_ERR_INVALID_ARGUMENT, "%s: null device pointer", which);
    if (((uintptr_t)t.dev_bytes & 15) != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "%s: device pointer must be 16-byte aligned", which);
    size_t bb = block_bytes_of(t.quant);
    if (t.n_bytes % bb != 0)
        return fail(XABE_ERR_RAGGED_WEIGHTS, "%s: %zu bytes is not a whole number of %zu B blocks", which,
                    t.n_bytes, bb);
    size_t found = t.n_bytes / bb * block_elems_of(t.quant);
    if (found != expected)
        return fail(XABE_ERR_WRONG_ELEMENT_COUNT,
                    "%s: expected %zu elements for this geometry, stack holds %zu", which, expected, found);
    return XABE_OK;
}

size_t gateup_smem(int k, int quant, int block_size) {
    uint32_t row_bytes = k / 256 * span_bytes_of(quant);
    size_t tiles = 2 * (size_t)staged_capacity(8u * row_bytes);
    size_t red = (size_t)2048 * nb_cap_for(block_size);
    return tiles > red ? tiles : red;
}
size_t down_smem(int k, int quant) {
    uint32_t row_bytes = k / 256 * span_bytes_of(quant);
    return staged_capacity(64u * row_bytes);
}

template <int QR, int QS>
int launch_gateup(xabe_moe* m, cudaStream_t st, const ExpertLaunch& L, int y_blocks, size_t smem) {
    auto kern = k_expert_gateup<QR, QS>;
    CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
    dim3 grid(L.rows / 8, y_blocks);
    kern<<<grid, kExpertThreads, smem, counted(st)>>>(L);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}
template <int QR, int QS>
int launch_down(xabe_moe* m, cudaStream_t st, const ExpertLaunch& L, int y_blocks, size_t smem) {
    auto kern = k_expert_down<QR, QS>;
    CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
    dim3 grid(L.rows / 64, y_blocks);
    kern<<<grid, kExpertThreads, smem, counted(st)>>>(L);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

#define DISPATCH_QQ(fn, qr, qs, ...)                                                   \
    ((qr) == XABE_QUANT_Q6_K                                                           \
         ? ((qs) == XABE_QUANT_Q6_K ? fn<QUANT_Q6K, QUANT_Q6K>(__VA_ARGS__)           \
                                    : fn<QUANT_Q6K, QUANT_Q8_0>(__VA_ARGS__))         \
         : ((qs) == XABE_QUANT_Q6_K ? fn<QUANT_Q8_0, QUANT_Q6K>(__VA_ARGS__)          \
                                    : fn<QUANT_Q8_0, QUANT_Q8_0>(__VA_ARGS__)))

// ---- streaming (persistent) expert kernels --------------------------------
struct StreamShape {
    bool ok = false;
    int n_stages = 0;
    uint32_t tile_cap = 0, x_stride = 0, smem = 0;
};

// Whether the streaming kernel serves this projection, and with what ring.
StreamShape stream_shape(int mode, int rows, int k, int q_routed, int q_shared, int max_stages = 0) {
    StreamShape sh;
    int n_spans = k / 256;
    int max_spans = mode == MODE_GATEUP ? kStreamGroupWarps : 2;
    if (n_spans > max_spans) return sh;
    if (mode == MODE_DOWN && rows % 128 != 0) return sh;
    if (mode == MODE_GATEUP && rows % 8 != 0) return sh;
    uint32_t rb_max = 0;
    for (int q : {q_routed, q_shared}) {
        uint32_t rb = (uint32_t)n_spans * span_bytes_of(q);
        if (rb % 4 != 0) return sh;  // a warp's rows must share one word alignment
        if (rb > rb_max) rb_max = rb;
    }
    uint32_t rows_per_tile = mode == MODE_GATEUP ? 8 : 128;
    sh.tile_cap = (staged_capacity(rows_per_tile * rb_max) + 15u) & ~15u;
    sh.x_stride = (uint32_t)k * 2u + kXRowPadBytes;
    int s_max = kStreamMaxStages;
    if (max_stages >= 2 && max_stages < s_max) s_max = max_stages;
    for (int S = s_max; S >= 2; --S) {
        StreamSmem L = stream_smem_layout(mode, S, sh.tile_cap, sh.x_stride);
        if (L.total <= 226u * 1024u) {
            sh.ok = true;
            sh.n_stages = S;
            sh.smem = L.total;
            return sh;
        }
    }
    return sh;
}

template <int MODE, int QR, int QS>
int launch_stream_t(xabe_moe* m, cudaStream_t st, const StreamLaunch& L, uint32_t smem) {
    auto kern = (MODE == MODE_DOWN && L.tail_done) ? k_expert_stream<MODE, QR, QS, MODE == MODE_DOWN>
                                                   : k_expert_stream<MODE, QR, QS, false>;
    CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
    CUDA_TRY(launch_pdl(m->pdl, kern, dim3(m->sm_count), dim3(kStreamThreads), smem, st, L));
    return XABE_OK;
}

template <int MODE>
int launch_stream(xabe_moe* m, cudaStream_t st, const StreamLaunch& L, uint32_t smem, int qr, int qs) {
    if (qr == XABE_QUANT_Q6_K)
        return qs == XABE_QUANT_Q6_K ? launch_stream_t<MODE, QUANT_Q6K, QUANT_Q6K>(m, st, L, smem)
                                     : launch_stream_t<MODE, QUANT_Q6K, QUANT_Q8_0>(m, st, L, smem);
    return qs == XABE_QUANT_Q6_K ? launch_stream_t<MODE, QUANT_Q8_0, QUANT_Q6K>(m, st, L, smem)
                                 : launch_stream_t<MODE, QUANT_Q8_0, QUANT_Q8_0>(m, st, L, smem);
}

// ---- prefill (tcgen05) expert kernels ---------------------------------------
// Wide passes only: the launch shape comes from max_tokens, as every other one.

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}
// [rows][k] f16 row-major, box 64 elements x 128 rows, 128-byte swizzle, out-of-bounds rows read as zero.
int make_rows_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(XABE_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
    if (((uintptr_t)base & 15) != 0 || k % 64 != 0 || rows == 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "tensor map source must be 16-byte aligned with k a multiple of 64");
    cuuint64_t dims[2] = {k, rows};
    cuuint64_t strides[1] = {k * 2};
    cuuint32_t box[2] = {(cuuint32_t)kPfChunkK, (cuuint32_t)kPfTileN};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(XABE_ERR_DRIVER, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return XABE_OK;
}

// Weight bytes as a matrix [rows][row_bytes / 4] of 32-bit words (a box side is limited to 256
// elements, and a Q8_0 span is 272 bytes), box `box_w` bytes x 64 rows, no swizzle; the part of a
// box past the end of a row reads as zero.
int make_bytes_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_w) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(XABE_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
    if (((uintptr_t)base & 15) != 0 || row_bytes % 16 != 0 || rows == 0 || box_w % 16 != 0 || box_w > 1024)
        return fail(XABE_ERR_INVALID_ARGUMENT, "weight tensor map needs a 16-byte aligned base and row pitch");
    cuuint64_t dims[2] = {row_bytes / 4, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_w / 4, (cuuint32_t)kRowsGroupRows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(XABE_ERR_DRIVER, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return XABE_OK;
}

// Handles at least this wide run gate/up through k_gateup_rows when the shapes allow.  Measured
// per layer step: 16 tokens 0.120 -> 0.110 ms, 32 tokens 0.143 -> 0.125 ms, 64 tokens
// 0.180 -> 0.161 ms against k_expert_stream.
constexpr uint32_t kRowsKernelMinTokens = 16;

struct RowsShape {
    bool ok = false;
    int n_stages = 0;
    uint32_t stage_bytes = 0, smem = 0;
};

RowsShape rows_shape(const xabe_moe* m, int rows, int k, bool has_routed, int qr, const void* r_a, const void* r_b,
                     bool has_shared, int qs, const void* s_a, const void* s_b, uint32_t x_stride) {
    RowsShape sh;
    uint32_t min_tokens = kRowsKernelMinTokens;
    if (m->rows_min_tokens == 0) return sh;
    if (m->rows_min_tokens > 0) min_tokens = (uint32_t)m->rows_min_tokens;
    if (m->g.max_tokens < min_tokens || m->force_tile_kernels) return sh;
    const int n_spans = k / 256;
    if (n_spans < 2 || rows % kRowsUnitRows != 0) return sh;
    uint32_t box = 0;
    auto fits = [&](bool present, int q, const void* a, const void* b) {
        if (!present) return true;
        const uint32_t rb = (uint32_t)n_spans * span_bytes_of(q);
        if (rb % 16 != 0 || ((uintptr_t)a & 15) || ((uintptr_t)b & 15)) return false;
        if (rows_box_bytes(q) > box) box = rows_box_bytes(q);
        return true;
    };
    if (!fits(has_routed, qr, r_a, r_b) || !fits(has_shared, qs, s_a, s_b)) return sh;
    sh.stage_bytes = 2u * kRowsGroupRows * box;
    for (int S = kRowsMaxStages; S >= 3; --S) {
        RowsSmem R = rows_smem_layout(S, sh.stage_bytes, x_stride);
        if (R.total <= 226u * 1024u) {
            sh.ok = true;
            sh.n_stages = S;
            sh.smem = R.total;
            return sh;
        }
    }
    return sh;
}

template <int QR, int QS>
int launch_rows_t(xabe_moe* m, cudaStream_t st, const RowsLaunch& P, uint32_t smem) {
    auto kern = k_gateup_rows<QR, QS>;
    CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
    CUDA_TRY(launch_pdl(m->pdl, kern, dim3(m->sm_count), dim3(kStreamThreads), smem, st, P));
    return XABE_OK;
}

bool prefill_applies(const xabe_moe* m, int gateup_rows, int down_rows, int hidden, int inter) {
    if (m->force_tile_kernels || !m->tensor_cores) return false;
    if (!(gateup_rows % 64 == 0 && down_rows % kPfTileM == 0 && hidden % kSpanElems == 0 && inter % kSpanElems == 0))
        return false;
    // Contractions too long for the decode kernels (the dense 27B block: 5120 and 17408) go through
    // these kernels at every width; there the exact-decode switch has nothing to select.
    const bool decode_kernels_serve = stream_shape(MODE_GATEUP, gateup_rows, hidden, XABE_QUANT_Q8_0, XABE_QUANT_Q8_0).ok &&
                                      stream_shape(MODE_DOWN, down_rows, inter, XABE_QUANT_Q8_0, XABE_QUANT_Q8_0).ok;
    if (!decode_kernels_serve) return true;
    if (m->exact_decode) return false;
    if (m->force_prefill) return true;
    return m->g.max_tokens >= kPrefillMinTokens;
}

template <int MODE, int QR, int QS>
int launch_prefill_t(cudaStream_t st, const PrefillLaunch& L, dim3 grid, size_t smem, bool wide) {
    auto kern = wide ? k_prefill_gemm_wide<MODE, QR, QS> : k_prefill_gemm<MODE, QR, QS>;
    CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
    kern<<<grid, wide ? kPfWideThreads : kPfThreads, smem, counted(st)>>>(L);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}
template <int MODE>
int launch_prefill(cudaStream_t st, const PrefillLaunch& L, dim3 grid, size_t smem, int qr, int qs, bool wide) {
    if (qr == XABE_QUANT_Q6_K)
        return qs == XABE_QUANT_Q6_K ? launch_prefill_t<MODE, QUANT_Q6K, QUANT_Q6K>(st, L, grid, smem, wide)
                                     : launch_prefill_t<MODE, QUANT_Q6K, QUANT_Q8_0>(st, L, grid, smem, wide);
    return qs == XABE_QUANT_Q6_K ? launch_prefill_t<MODE, QUANT_Q8_0, QUANT_Q6K>(st, L, grid, smem, wide)
                                 : launch_prefill_t<MODE, QUANT_Q8_0, QUANT_Q8_0>(st, L, grid, smem, wide);
}

// ---- decode-width dense block (k_dense_rows) -------------------------------------------
template <int MODE, int QUANT>
int launch_dense_rows_q(xabe_moe* m, cudaStream_t st, const DenseRowsLaunch& P, int ng, uint32_t smem) {
    auto go = [&](auto kern) -> int {
        CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
        kern<<<dim3(m->sm_count), dim3(kDrThreads), smem, counted(st)>>>(P);
        CUDA_TRY(cudaGetLastError());
        return XABE_OK;
    };
    switch (ng) {
        case 1: return go(k_dense_rows<MODE, QUANT, 1>);
        case 2: return go(k_dense_rows<MODE, QUANT, 2>);
        case 4: return go(k_dense_rows<MODE, QUANT, 4>);
        default: return go(k_dense_rows<MODE, QUANT, 8>);
    }
}
template <int MODE>
int launch_dense_rows(xabe_moe* m, cudaStream_t st, const DenseRowsLaunch& P, int quant, int ng, uint32_t smem) {
    return quant == XABE_QUANT_Q6_K ? launch_dense_rows_q<MODE, QUANT_Q6K>(m, st, P, ng, smem)
                                    : launch_dense_rows_q<MODE, QUANT_Q8_0>(m, st, P, ng, smem);
}

struct MlpWeights {
    bool present = false;
    xabe_quant_tensor gate{}, up{}, down{};
};

// The block's last stage, when the down projection is to perform it itself (k_expert_stream<DOWN>'s
// combine_tile) instead of a launch of k_gate_and_combine.
struct TailFusion {
    const float* gate;      // [max_tokens], already computed (k_decode_front)
    const float* residual;
    float* routed;
    float* ffn_out;
    float* l_out;
};

bool tail_applies(const xabe_moe* m, const xabe_moe_layer_weights* w) {
    const auto& g = m->g;
    // Handles of fewer than 16 tokens: the routed and the shared experts always share one launch there
    // (see run_experts), and the per-tile fence the arrival count needs costs less than a launch.
    if (!m->fused_tail || g.max_tokens >= kTailMaxTokens || m->force_tile_kernels || m->partial_rows) return false;
    if (g.hidden > 8192) return false;  // k_rms_norm keeps the row in shared memory for the gate
    if (g.hidden % 128 != 0) return false;
    return stream_shape(MODE_DOWN, (int)g.hidden, (int)g.intermediate, w->down_exps.quant, w->shared_down.quant,
                        m->stream_stages).ok;
}

// Both projections of the routed experts and/or the shared expert, each in one
// launch.  `routed`/`shared` say which halves ride the launch.
int run_experts(xabe_moe* m, cudaStream_t st, const MlpWeights& routed, const MlpWeights& shared,
                float* shexp_out, int mark_between = -1, const TailFusion* tail = nullptr) {
    const auto& g = m->g;
    if (!routed.present && !shared.present) return XABE_OK;
    // Different formats for the routed experts and the shared expert (the shipped file: Q6_K and Q8_0):
    // two launches per projection instead of one mixed one.  A mixed launch sizes its rings for the
    // longer Q8_0 rows and branches on the format per tile; measured, it slowed every tile (64 tokens:
    // gate/up 0.107 -> 0.131 ms; 2048 tokens: 0.279 -> 0.334 ms), far more than the shared expert's own work.
    // Below 16 tokens the two extra launches cost more than they save (1 token: 44.5 -> 56.2 us), so the
    // narrowest handles keep the mixed launch.
    if (routed.present && shared.present && g.max_tokens >= 16 &&
        (routed.gate.quant != shared.gate.quant || routed.down.quant != shared.down.quant)) {
        int rc2 = run_experts(m, st, routed, MlpWeights{}, nullptr, mark_between);
        if (rc2) return rc2;
        return run_experts(m, st, MlpWeights{}, shared, shexp_out, -1);
    }
    if (routed.present && routed.gate.quant != routed.up.quant)
        return fail(XABE_ERR_UNSUPPORTED_EXPERT_TYPE,
                    "routed gate and up stacks must share one format (found tags %d and %d)",
                    routed.gate.quant, routed.up.quant);
    if (shared.present && shared.gate.quant != shared.up.quant)
        return fail(XABE_ERR_UNSUPPORTED_EXPERT_TYPE,
                    "shared gate and up matrices must share one format (found tags %d and %d)",
                    shared.gate.quant, shared.up.quant);
    int shared_tiles = shared.present ? (int)((g.max_tokens + g.block_size - 1) / g.block_size) : 0;
    int routed_blocks = routed.present ? (int)m->block_capacity : 0;
    ExpertLaunch L{};
    L.routed_blocks = routed_blocks;
    L.block_size = (int)g.block_size;
    L.top_k = (int)g.experts_per_token;
    L.max_tokens = (int)g.max_tokens;
    L.sorted_token_ids = m->sorted_token_ids;
    L.expert_ids = m->expert_ids;
    L.valid_tokens = m->valid_tokens;
    L.topk_weights = m->topk_weights;
    L.status = m->status;
    int qr = routed.present ? routed.gate.quant : shared.gate.quant;
    int qs = shared.present ? shared.gate.quant : qr;
    // gate/up + SwiGLU
    L.r_a = routed.present ? (const uint8_t*)routed.gate.dev_bytes : nullptr;
    L.r_b = routed.present ? (const uint8_t*)routed.up.dev_bytes : nullptr;
    L.s_a = shared.present ? (const uint8_t*)shared.gate.dev_bytes : nullptr;
    L.s_b = shared.present ? (const uint8_t*)shared.up.dev_bytes : nullptr;
    L.rows = (int)g.intermediate;
    L.k = (int)g.hidden;
    const __half* x_routed = m->x_routed_override ? m->x_routed_override : m->normed_h;
    L.x_routed = x_routed;
    L.x_shared = m->normed_h;
    L.inter_routed = m->inter_routed;
    L.inter_shared = m->inter_shared;
    // One expert, decode width, contraction too long for the streaming kernels to hold a token's row
    // (the dense 27B block): k_dense_rows streams slices of the contraction.
    if (!routed.present && shared.present && m->dense_rows && !m->force_tile_kernels && !m->force_prefill &&
        g.max_tokens <= (uint32_t)kDrMaxTokens && g.intermediate % 128 == 0 && g.hidden % 256 == 0 &&
        !(stream_shape(MODE_GATEUP, (int)g.intermediate, (int)g.hidden, qs, qs).ok &&
          stream_shape(MODE_DOWN, (int)g.hidden, (int)g.intermediate, shared.down.quant, shared.down.quant).ok)) {
        const int qd = shared.down.quant;
        const size_t rb_gu = (size_t)(g.hidden / 256) * span_bytes_of(qs), rb_dn = (size_t)(g.intermediate / 256) * span_bytes_of(qd);
        const bool ok = rb_gu % 4 == 0 && rb_dn % 4 == 0 && shared.gate.n_bytes % 16 == 0 && shared.up.n_bytes % 16 == 0 &&
                        shared.down.n_bytes % 16 == 0 && (m->dense_k_splits == 1 || m->dense_partial);
        if (ok) {
            int ng = 1;
            while (ng * 8 < (int)g.max_tokens) ng *= 2;
            DenseRowsLaunch P{};
            P.valid_tokens = m->valid_tokens;
            P.status = m->status;
            P.max_tokens = (int)g.max_tokens;
            P.x_rows = 8 * ng;
            auto shape = [&](int quant) {
                P.raw_pitch = dense_rows_pitch(quant == XABE_QUANT_Q6_K ? QUANT_Q6K : QUANT_Q8_0);
                P.n_stages = 2;
                for (int S = kDrMaxStages; S >= 2; --S)
                    if (dense_rows_smem(S, P.raw_pitch, P.x_rows) <= 200u * 1024u) {
                        P.n_stages = S;
                        break;
                    }
                return dense_rows_smem(P.n_stages, P.raw_pitch, P.x_rows);
            };
            P.w_a = (const uint8_t*)shared.gate.dev_bytes;
            P.w_b = (const uint8_t*)shared.up.dev_bytes;
            P.rows = (int)g.intermediate;
            P.k = (int)g.hidden;
            P.x = m->normed_h;
            P.inter = m->inter_shared;
            P.k_splits = 1;
            uint32_t smem = shape(qs);
            int rc = launch_dense_rows<MODE_GATEUP>(m, st, P, qs, ng, smem);
            if (rc) return rc;
            if (mark_between >= 0) prof_mark(m, st, mark_between);
            P.w_a = (const uint8_t*)shared.down.dev_bytes;
            P.w_b = nullptr;
            P.rows = (int)g.hidden;
            P.k = (int)g.intermediate;
            P.x = m->inter_shared;
            P.inter = nullptr;
            P.k_splits = m->dense_k_splits;
            P.out = P.k_splits > 1 ? m->dense_partial : shexp_out;
            smem = shape(qd);
            if ((rc = launch_dense_rows<MODE_DOWN>(m, st, P, qd, ng, smem))) return rc;
            if (P.k_splits > 1) {
                k_sum_k_splits<<<dim3(g.max_tokens, (g.hidden + 255) / 256), 256, 0, counted(st)>>>(
                    m->dense_partial, P.k_splits, (int)g.max_tokens, (int)g.hidden, m->valid_tokens, shexp_out);
                CUDA_TRY(cudaGetLastError());
            }
            return XABE_OK;
        }
    }
    if (prefill_applies(m, (int)g.intermediate, (int)g.hidden, (int)g.hidden, (int)g.intermediate)) {
        PrefillLaunch P{};
        P.top_k = L.top_k;
        P.has_routed = routed.present;
        P.has_shared = shared.present;
        P.items = m->pf_items;
        P.n_items = m->pf_n_items;
        P.valid_tokens = m->valid_tokens;
        P.sorted_token_ids = m->sorted_token_ids;
        P.topk_weights = m->topk_weights;
        P.inter_routed = m->inter_routed;
        P.inter_shared = m->inter_shared;
        P.partial = m->partial;
        P.partial_rows = m->partial_rows;
        P.shexp = shexp_out;
        P.status = m->status;
        P.max_tokens = (int)g.max_tokens;
        P.n_stages = kPfMaxStages;
        P.item_cols = m->pf_item_cols;
        const bool wide = m->pf_item_cols > kPfTileN;
        // one CTA per SM walks the tiles; the rings take what fits beside each other
        dim3 pf_grid((unsigned)m->sm_count);
        auto pf_smem = [&](int q_routed, int q_shared) {
            int pitch = 0;
            if (routed.present) pitch = pf_raw_pitch(q_routed == XABE_QUANT_Q6_K ? QUANT_Q6K : QUANT_Q8_0);
            if (shared.present) {
                int ps = pf_raw_pitch(q_shared == XABE_QUANT_Q6_K ? QUANT_Q6K : QUANT_Q8_0);
                if (ps > pitch) pitch = ps;
            }
            P.slot_bytes = kPfTileM * pitch;
            if (wide) {  // A ring 64 KB, two raw slots, B ring three units (two beside the longer Q8_0 rows)
                P.n_raw = kPfWideRaw;
                P.n_b_units = pitch == kPfRawPitchQ6K ? kPfWideMaxBUnits : 2;
                return (size_t)1024 + (size_t)(2 + P.n_b_units) * 2 * kPfTileBytes + (size_t)P.n_raw * P.slot_bytes + 16;
            }
            P.n_raw = pitch == kPfRawPitchQ6K ? kPfMaxRaw : 2;
            return (size_t)1024 + (size_t)P.n_stages * kPfStageBytes + (size_t)P.n_raw * P.slot_bytes + 16;
        };
        P.r_a = L.r_a; P.r_b = L.r_b; P.s_a = L.s_a; P.s_b = L.s_b;
        P.rows = (int)g.intermediate; P.k = (int)g.hidden;
        P.x_routed = x_routed; P.x_shared = m->normed_h;
        P.row_tiles = (int)g.intermediate / 64;
        const size_t smem_gu = pf_smem(qr, qs);
        if (wide) {
            P.tm_routed = m->tm_routed_gu;
            P.tm_shared = m->tm_shared_gu;
            if (routed.present) {  // activation rows in dispatch order, so that an item's columns are consecutive rows
                k_permute_rows<<<(unsigned)m->sorted_capacity, 256, 0, counted(st)>>>(
                    m->sorted_token_ids, m->num_tokens_post_pad, m->valid_tokens, (int)g.experts_per_token,
                    (int)g.hidden, x_routed, m->x_sorted);
                CUDA_TRY(cudaGetLastError());
            }
        }
        int rcp = launch_prefill<MODE_GATEUP>(st, P, pf_grid, smem_gu, qr, qs, wide);
        if (rcp) return rcp;
        if (mark_between >= 0) prof_mark(m, st, mark_between);
        int qrd = routed.present ? routed.down.quant : shared.down.quant;
        int qsd = shared.present ? shared.down.quant : qrd;
        P.r_a = routed.present ? (const uint8_t*)routed.down.dev_bytes : nullptr;
        P.r_b = nullptr;
        P.s_a = shared.present ? (const uint8_t*)shared.down.dev_bytes : nullptr;
        P.s_b = nullptr;
        P.rows = (int)g.hidden; P.k = (int)g.intermediate;
        P.x_routed = m->inter_routed; P.x_shared = m->inter_shared;
        P.row_tiles = (int)g.hidden / kPfTileM;
        const size_t smem_dn = pf_smem(qrd, qsd);
        if (wide) {
            P.tm_routed = m->tm_routed_dn;
            P.tm_shared = m->tm_shared_dn;
        }
        return launch_prefill<MODE_DOWN>(st, P, pf_grid, smem_dn, qrd, qsd, wide);
    }
    StreamLaunch SL{};
    SL.top_k = L.top_k;
    SL.has_routed = routed.present;
    SL.has_shared = shared.present;
    SL.work_items = m->work_items;
    SL.n_work = m->n_work;
    SL.valid_tokens = m->valid_tokens;
    SL.status = m->status;
    SL.inter_routed = m->inter_routed;
    SL.inter_shared = m->inter_shared;
    SL.partial = m->partial;
    SL.partial_rows = m->partial_rows;
    SL.shexp = shexp_out;
    SL.num_experts = (int)g.num_experts;
    SL.max_tokens = (int)g.max_tokens;
    SL.x_rows_routed = (int)m->sorted_capacity;
    SL.runs_override = m->stream_runs;
    StreamShape gu = stream_shape(MODE_GATEUP, (int)g.intermediate, (int)g.hidden, qr, qs, m->stream_stages);
    if (gu.ok && !m->force_tile_kernels) {
        SL.r_a = L.r_a; SL.r_b = L.r_b; SL.s_a = L.s_a; SL.s_b = L.s_b;
        SL.rows = L.rows; SL.k = L.k;
        SL.x_routed = x_routed; SL.x_shared = m->normed_h;
        SL.n_stages = gu.n_stages; SL.tile_cap = gu.tile_cap; SL.x_stride = gu.x_stride;
        RowsShape rs = rows_shape(m, SL.rows, SL.k, routed.present, qr, SL.r_a, SL.r_b, shared.present, qs, SL.s_a,
                                  SL.s_b, gu.x_stride);
        int rcs;
        if (rs.ok) {
            RowsLaunch RP{};
            RP.L = SL;
            RP.L.n_stages = rs.n_stages;
            RP.box_r = rows_box_bytes(qr);
            RP.box_s = rows_box_bytes(qs);
            RP.stage_bytes = rs.stage_bytes;
            const uint64_t rb_r = (uint64_t)(SL.k / 256) * span_bytes_of(qr), rb_s = (uint64_t)(SL.k / 256) * span_bytes_of(qs);
            rcs = XABE_OK;
            if (routed.present) {
                const uint64_t all_rows = (uint64_t)g.num_experts * (uint64_t)SL.rows;
                rcs = make_bytes_map(&RP.tm_r_a, SL.r_a, all_rows, rb_r, RP.box_r);
                if (!rcs) rcs = make_bytes_map(&RP.tm_r_b, SL.r_b, all_rows, rb_r, RP.box_r);
            }
            if (!rcs && shared.present) {
                rcs = make_bytes_map(&RP.tm_s_a, SL.s_a, (uint64_t)SL.rows, rb_s, RP.box_s);
                if (!rcs) rcs = make_bytes_map(&RP.tm_s_b, SL.s_b, (uint64_t)SL.rows, rb_s, RP.box_s);
            }
            if (!rcs) rcs = DISPATCH_QQ(launch_rows_t, qr, qs, m, st, RP, rs.smem);
        } else {
            rcs = launch_stream<MODE_GATEUP>(m, st, SL, gu.smem, qr, qs);
        }
        if (rcs) return rcs;
        if (mark_between >= 0) prof_mark(m, st, mark_between);
    } else {
    size_t smem = gateup_smem(L.k, qr, L.block_size);
    size_t smem_s = gateup_smem(L.k, qs, L.block_size);
    if (smem_s > smem) smem = smem_s;
    if (smem > 220 * 1024)
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY, "gate/up row tile of %zu bytes does not fit shared memory", smem);
    int rc = DISPATCH_QQ(launch_gateup, qr, qs, m, st, L, routed_blocks + shared_tiles, smem);
    if (rc) return rc;
    if (mark_between >= 0) prof_mark(m, st, mark_between);
    }
    // down
    qr = routed.present ? routed.down.quant : shared.down.quant;
    qs = shared.present ? shared.down.quant : qr;
    L.r_a = routed.present ? (const uint8_t*)routed.down.dev_bytes : nullptr;
    L.r_b = nullptr;
    L.s_a = shared.present ? (const uint8_t*)shared.down.dev_bytes : nullptr;
    L.s_b = nullptr;
    L.rows = (int)g.hidden;
    L.k = (int)g.intermediate;
    L.x_routed = m->inter_routed;
    L.x_shared = m->inter_shared;
    L.partial = m->partial;
    L.partial_rows = m->partial_rows;
    L.shexp = shexp_out;
    StreamShape dn = stream_shape(MODE_DOWN, (int)g.hidden, (int)g.intermediate, qr, qs, m->stream_stages);
    if (dn.ok && !m->force_tile_kernels) {
        SL.r_a = L.r_a; SL.r_b = nullptr; SL.s_a = L.s_a; SL.s_b = nullptr;
        SL.rows = L.rows; SL.k = L.k;
        SL.x_routed = m->inter_routed; SL.x_shared = m->inter_shared;
        SL.n_stages = dn.n_stages; SL.tile_cap = dn.tile_cap; SL.x_stride = dn.x_stride;
        {
            // rows four apart land 4 banks apart when the row pitch in words is 4 * odd + 1 ... see down_row
            uint32_t words = (uint32_t)(L.k / 256) * span_bytes_of(qr) / 4u;
            uint32_t words_s = (uint32_t)(L.k / 256) * span_bytes_of(qs) / 4u;
            bool four = ((words * 4u) % 32u) % 8u == 4u && ((words_s * 4u) % 32u) % 8u == 4u;
            SL.down_row_step = four ? 4 : 1;
        }
        if (tail && routed.present && shared.present) {
            SL.tail_done = m->tail_done;
            SL.tail_target = ((int)g.experts_per_token + 1) * kStreamGroupWarps;
            SL.tail_gate = tail->gate;
            SL.tail_residual = tail->residual;
            SL.tail_routed = tail->routed;
            SL.tail_ffn = tail->ffn_out;
            SL.tail_lout = tail->l_out;
        }
        return launch_stream<MODE_DOWN>(m, st, SL, dn.smem, qr, qs);
    }
    size_t smem = down_smem(L.k, qr);
    size_t smem_s = down_smem(L.k, qs);
    if (smem_s > smem) smem = smem_s;
    if (smem > 220 * 1024)
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY, "down row tile of %zu bytes does not fit shared memory", smem);
    return DISPATCH_QQ(launch_down, qr, qs, m, st, L, routed_blocks + shared_tiles, smem);
}

// What k_prefill_gemm_wide needs beyond the other kernels: the activations in dispatch order and the
// tensor maps of its four activation sources, all handle-owned, made once.  Set-up time only (allocates).
int setup_wide_prefill(xabe_moe* m) {
    const size_t T = m->g.max_tokens, H = m->g.hidden, I = m->g.intermediate;
    if (H % kSpanElems != 0 || I % kSpanElems != 0) {
        m->pf_item_cols = kPfTileN;
        return XABE_OK;
    }
    if (m->scope == XABE_SCOPE_ROUTED && !m->x_sorted) {
        cudaError_t e = dev_alloc(&m->x_sorted, (size_t)m->sorted_capacity * H);
        if (e != cudaSuccess)
            return fail(XABE_ERR_DRIVER, "CUDA driver error: %s (allocating the permuted activations)",
                        cudaGetErrorString(e));
    }
    int rc = make_rows_map(&m->tm_shared_gu, m->normed_h, T, H);
    if (!rc) rc = make_rows_map(&m->tm_shared_dn, m->inter_shared, T, I);
    if (!rc && m->scope == XABE_SCOPE_ROUTED) {
        rc = make_rows_map(&m->tm_routed_gu, m->x_sorted, m->sorted_capacity, H);
        if (!rc) rc = make_rows_map(&m->tm_routed_dn, m->inter_routed, m->sorted_capacity, I);
    }
    if (!rc) m->pf_item_cols = kPfWideItemCols;
    return rc;
}

int check_routed(xabe_moe* m, const char* entry) {
    if (m->scope != XABE_SCOPE_ROUTED)
        return fail(XABE_ERR_SHARED_ONLY_BUFFERS,
                    "`%s` needs the routed dispatch tables, but these buffers were allocated for the "
                    "shared-expert path only", entry);
    return XABE_OK;
}

int rows_to_half(xabe_moe* m, cudaStream_t st, const float* hidden_states) {
    k_rows_to_half<<<m->g.max_tokens, 256, 0, counted(st)>>>(hidden_states, m->normed_h, m->valid_tokens, (int)m->g.hidden);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int launch_rms_norm(xabe_moe* m, cudaStream_t st, const float* x, const float* weight,
                    const float* gate_w = nullptr) {
    // block_for_width, crates/xabe-cuda/src/kernels/layer_ops.rs:1219-1221
    int block = ((int)m->g.hidden + 31) / 32 * 32;
    if (block > 1024) block = 1024;
    if (block < 32) block = 32;
    if (gate_w && block < 256) gate_w = nullptr;  // (hidden is a multiple of 256, so this does not happen)
    const size_t smem = gate_w ? (size_t)m->g.hidden * sizeof(float) : 0;
    // many rows: blocks that walk rows with the next row's loads in flight (same sums, same order)
    const int ept = ((int)m->g.hidden + block - 1) / block;
    if (!gate_w && m->g.max_tokens >= 256 && ept <= 8) {
        const dim3 grid((unsigned)std::min<uint32_t>(m->g.max_tokens, 2u * (uint32_t)m->sm_count));
        auto go = [&](auto kern) -> int {
            CUDA_TRY(launch_pdl(m->pdl, kern, grid, dim3(block), 0, st, x, weight, m->normed, m->normed_h,
                                (const int*)m->valid_tokens, (int)m->g.hidden, m->eps));
            return XABE_OK;
        };
        switch (ept) {
            case 1: return go(k_rms_norm_stream<1>);
            case 2: return go(k_rms_norm_stream<2>);
            case 3: return go(k_rms_norm_stream<3>);
            case 4: return go(k_rms_norm_stream<4>);
            case 5: return go(k_rms_norm_stream<5>);
            case 6: return go(k_rms_norm_stream<6>);
            case 7: return go(k_rms_norm_stream<7>);
            default: return go(k_rms_norm_stream<8>);
        }
    }
    CUDA_TRY(launch_pdl(m->pdl, k_rms_norm, dim3(m->g.max_tokens), dim3(block), smem, st, x, weight, m->normed,
                        m->normed_h, m->valid_tokens, (int)m->g.hidden, m->eps, gate_w, m->gate));
    return XABE_OK;
}

int launch_router(xabe_moe* m, cudaStream_t st, const float* router, const float* bias) {
    const auto& g = m->g;
    if (((uintptr_t)router & 15) != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "router weights must be 16-byte aligned");
    // prefill widths: the expert rows in registers, the tokens streamed two at a time
    bool regw = g.max_tokens >= 256;
    if (m->router_regw >= 0) regw = m->router_regw != 0;
    if (regw && g.max_tokens >= 2 && g.num_experts % kRwExperts == 0 && (g.hidden == 2048 || g.hidden == 1024)) {
        // eight expert rows per CTA and two CTAs per SM (measured 0.085 against 0.091 ms at 2048 tokens);
        // router_regw 1 selects sixteen rows and one CTA per SM
        const int ne = m->router_regw == 1 ? 16 : 8;
        const size_t smem_r = router_regw_smem((int)g.hidden, ne);
        unsigned gx = g.num_experts / ne;
        unsigned gy = (unsigned)m->sm_count * (ne == 16 ? 1u : 2u) / gx;
        unsigned pairs = (g.max_tokens + kRrStageTokens - 1) / kRrStageTokens;
        if (gy < 1) gy = 1;
        if (gy > pairs) gy = pairs;
        auto go_regw = [&](auto kern) -> int {
            CUDA_TRY(allow_dynamic_smem((const void*)kern, smem_r));
            CUDA_TRY(launch_pdl(m->pdl, kern, dim3(gx, gy), dim3(256), smem_r, st, router, (const float*)m->normed,
                                (const int*)m->valid_tokens, (int)g.num_experts, bias, m->logits, m->status));
            return XABE_OK;
        };
        if (ne == 8) return g.hidden == 2048 ? go_regw(k_router_logits_regw<8, 8>) : go_regw(k_router_logits_regw<4, 8>);
        return g.hidden == 2048 ? go_regw(k_router_logits_regw<8, 16>) : go_regw(k_router_logits_regw<4, 16>);
    }
    // wide passes: sixteen expert rows per CTA, the tokens shared out over the SMs
    if (g.max_tokens >= 32 && g.num_experts % kRwExperts == 0 && (g.hidden == 2048 || g.hidden == 1024)) {
        const size_t smem_w = router_wide_smem((int)g.hidden);
        unsigned gx = g.num_experts / kRwExperts;
        unsigned gy = (unsigned)m->sm_count / gx;
        unsigned tiles = (g.max_tokens + kRwTokens - 1) / kRwTokens;
        if (gy < 1) gy = 1;
        if (gy > tiles) gy = tiles;
        auto go_wide = [&](auto kern) -> int {
            CUDA_TRY(allow_dynamic_smem((const void*)kern, smem_w));
            CUDA_TRY(launch_pdl(m->pdl, kern, dim3(gx, gy), dim3(256), smem_w, st, router, (const float*)m->normed,
                                (const int*)m->valid_tokens, (int)g.num_experts, bias, m->logits, m->status));
            return XABE_OK;
        };
        return g.hidden == 2048 ? go_wide(k_router_logits_wide<8>) : go_wide(k_router_logits_wide<4>);
    }
    dim3 block(128);
    if (((uintptr_t)m->normed & 15) != 0 || (g.hidden * sizeof(float)) % 16 != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "normed rows must be 16-byte aligned");
    unsigned ex = (g.num_experts + 3) / 4;
    auto go = [&](auto kern, int tt) -> int {
        const size_t smem = (size_t)(4 + tt) * g.hidden * sizeof(float);  // expert rows + one token tile
        if (smem > 200 * 1024) return fail(XABE_ERR_UNSUPPORTED_GEOMETRY, "router rows do not fit shared memory");
        // wide passes share one staged copy of the rows between eight token tiles
        int tiles_per_cta = g.max_tokens > 128 ? 8 : 1;
        unsigned ty = (g.max_tokens + tt * tiles_per_cta - 1) / (tt * tiles_per_cta);
        CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
        CUDA_TRY(launch_pdl(m->pdl, kern, dim3(ex, ty), block, smem, st, router, (const float*)m->normed,
                            (const int*)m->valid_tokens, (int)g.hidden, (int)g.num_experts, bias, m->logits,
                            tiles_per_cta, m->status));
        return XABE_OK;
    };
    // the widest token tile that the handle can use and that fits beside the four expert rows
    const size_t row_bytes = (size_t)g.hidden * sizeof(float);
    if (g.max_tokens > 4 && 12 * row_bytes <= 200 * 1024) return go(k_router_logits<8>, 8);
    if (g.max_tokens > 1 && 8 * row_bytes <= 200 * 1024) return go(k_router_logits<4>, 4);
    return go(k_router_logits<1>, 1);
}

// `logits` NULL: the routing decision is already in the handle's topk buffers; only the tables are built.
int launch_route_and_dispatch(xabe_moe* m, cudaStream_t st, const float* logits) {
    const auto& g = m->g;
    size_t hist_bytes = (size_t)(g.num_experts + 1) * sizeof(int);
    if ((uint64_t)g.max_tokens * g.experts_per_token <= (uint64_t)kSmallPairs) {
        // decode widths: one single-CTA launch
        size_t smem = dispatch_small_smem((int)g.num_experts, 256);
        const float* fused_logits = logits;
        if (logits && g.max_tokens > 8) {  // more than one token per warp: route on many SMs first
            CUDA_TRY(launch_pdl(m->pdl, k_route, dim3((g.max_tokens + 7) / 8), dim3(256), 0, st, logits,
                                (const int*)m->valid_tokens, (int)g.num_experts, (int)g.experts_per_token,
                                m->topk_ids, m->topk_weights));
            fused_logits = nullptr;
        }
        CUDA_TRY(launch_pdl(m->pdl, k_route_dispatch_small, dim3(1), dim3(256), smem, st, fused_logits,
                            (const int*)m->valid_tokens, (int)g.num_experts, (int)g.experts_per_token,
                            (int)g.block_size, (int)m->sorted_capacity, (int)m->block_capacity, m->topk_ids,
                            m->topk_weights, m->sorted_token_ids, m->expert_ids, m->num_tokens_post_pad,
                            m->expert_offsets, m->expert_counts, m->work_items, m->n_work));
        if (prefill_applies(m, (int)g.intermediate, (int)g.hidden, (int)g.hidden, (int)g.intermediate)) {  // few experts, many tokens
            int threads = ((int)g.num_experts + 31) / 32 * 32;
            k_build_prefill_items<<<1, threads, hist_bytes, counted(st)>>>((int)g.num_experts, m->expert_offsets,
                                                                  m->expert_counts, m->pf_items, m->pf_n_items, m->pf_item_cols);
            CUDA_TRY(cudaGetLastError());
        }
        return XABE_OK;
    }
    if (logits) {
        k_route<<<(g.max_tokens + 7) / 8, 256, 0, counted(st)>>>(logits, m->valid_tokens, (int)g.num_experts,
                                                       (int)g.experts_per_token, m->topk_ids, m->topk_weights);
        CUDA_TRY(cudaGetLastError());
    }
    k_align_count<<<m->n_chunks, 32, hist_bytes, counted(st)>>>(m->topk_ids, m->valid_tokens, (int)g.experts_per_token,
                                                      (int)g.num_experts, m->n_chunks, m->align_chunk, (int)m->sorted_capacity,
                                                      (int)m->block_capacity, m->chunk_hist,
                                                      m->sorted_token_ids, m->expert_ids);
    CUDA_TRY(cudaGetLastError());
    int threads = ((int)g.num_experts + 31) / 32 * 32;
    k_align_scan<<<1, threads, 0, counted(st)>>>((int)g.num_experts, m->n_chunks, (int)g.block_size,
                                                 m->chunk_hist, m->expert_offsets, m->expert_counts,
                                                 m->expert_ids, m->num_tokens_post_pad);
    CUDA_TRY(cudaGetLastError());
    k_align_scatter<<<m->n_chunks, 32, hist_bytes, counted(st)>>>(m->topk_ids, m->valid_tokens,
                                                        (int)g.experts_per_token, (int)g.num_experts,
                                                        m->align_chunk, m->chunk_hist, m->expert_offsets,
                                                        m->sorted_token_ids);
    CUDA_TRY(cudaGetLastError());
    // Only the work list of the kernels that will run: the regime must be chosen before this call.
    if (prefill_applies(m, (int)g.intermediate, (int)g.hidden, (int)g.hidden, (int)g.intermediate)) {
        k_build_prefill_items<<<1, threads, hist_bytes, counted(st)>>>((int)g.num_experts, m->expert_offsets,
                                                              m->expert_counts, m->pf_items, m->pf_n_items, m->pf_item_cols);
    } else {
        k_build_work<<<1, threads, hist_bytes, counted(st)>>>((int)g.num_experts, m->expert_offsets, m->expert_counts,
                                                     m->sorted_token_ids, m->topk_weights, m->work_items,
                                                     m->n_work);
    }
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

// Whether k_decode_front serves this handle and these pointers: decode widths (the single-block
// dispatch holds every flat pair), rows that a bulk copy can fetch, and the streaming expert kernels
// downstream (it builds their column groups, not the tensor-core kernels' items).
int front_tile_tokens(const xabe_moe* m) { return m->g.max_tokens > 4 ? 8 : m->g.max_tokens > 1 ? 4 : 1; }
// Handles of one or two tokens: the router's CTAs normalise the rows themselves (the consumer-side
// fold of the norm; crates/xabe-engine/src/forward.rs:3534-3585 is the seam), which removes the
// RMSNorm launch.  Wider handles keep k_rms_norm: every CTA repeats its tile's normalisation row by
// row, and measured under graph replay that already costs what the launch saves at three tokens
// (1 token 33.7 -> 32.8 us per layer, 3 tokens 49.5 -> 50.3).
constexpr uint32_t kNormInRouterMaxTokens = 2;

bool front_applies(const xabe_moe* m, const float* x, const float* router, bool* with_routing) {
    const auto& g = m->g;
    *with_routing = m->fused_front;
    if (m->scope != XABE_SCOPE_ROUTED) return false;
    if (!m->fused_front && !(m->fused_norm && g.max_tokens <= kNormInRouterMaxTokens)) return false;
    if ((uint64_t)g.max_tokens * g.experts_per_token > (uint64_t)kSmallPairs) return false;
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)router & 15) != 0) return false;
    if (front_smem((int)g.hidden, front_tile_tokens(m)) > 200 * 1024) return false;
    return !prefill_applies(m, (int)g.intermediate, (int)g.hidden, (int)g.hidden, (int)g.intermediate);
}

int launch_front(xabe_moe* m, cudaStream_t st, const float* x, const xabe_moe_layer_weights* w, bool with_routing) {
    const auto& g = m->g;
    FrontLaunch P{};
    P.x = x;
    P.norm_w = w->post_norm;
    P.router = w->router;
    P.bias = w->router_bias;
    P.gate_w = w->shared_gate_inp;
    P.valid_tokens = m->valid_tokens;
    P.normed = m->normed;
    P.normed_h = m->normed_h;
    P.logits = m->logits;
    P.gate = m->gate;
    P.topk_ids = m->topk_ids;
    P.topk_weights = m->topk_weights;
    P.sorted_token_ids = m->sorted_token_ids;
    P.expert_ids = m->expert_ids;
    P.num_tokens_post_pad = m->num_tokens_post_pad;
    P.expert_offsets = m->expert_offsets;
    P.expert_counts = m->expert_counts;
    P.work_items = m->work_items;
    P.n_work = m->n_work;
    P.tickets = m->front_tickets;
    P.zero_buf = m->tail_done;
    P.zero_count = (int)(kTailMaxTokens * (g.hidden / 128 + 1));
    P.status = m->status;
    P.hidden = (int)g.hidden;
    P.num_experts = (int)g.num_experts;
    P.top_k = (int)g.experts_per_token;
    P.block_size = (int)g.block_size;
    P.sorted_capacity = (int)m->sorted_capacity;
    P.block_capacity = (int)m->block_capacity;
    P.eps = m->eps;
    const int tt = front_tile_tokens(m);
    const size_t smem = front_smem((int)g.hidden, tt);
    P.fused_dispatch = (uint64_t)g.max_tokens * g.experts_per_token <= (uint64_t)kTinyPairs ? 1 : 0;
    P.route = with_routing ? 1 : 0;
    const dim3 grid((g.num_experts + 3) / 4, (g.max_tokens + tt - 1) / tt);
    auto go = [&](auto kern) -> int {
        CUDA_TRY(allow_dynamic_smem((const void*)kern, smem));
        CUDA_TRY(launch_pdl(m->pdl, kern, grid, dim3(kFrontThreads), smem, st, P));
        return XABE_OK;
    };
    int rc = tt == 8 ? go(k_decode_front<8>) : tt == 4 ? go(k_decode_front<4>) : go(k_decode_front<1>);
    if (rc) return rc;
    if (!with_routing) return launch_route_and_dispatch(m, st, m->logits);
    if (P.fused_dispatch) return rc;
    // wider handles: the tables from the routing the launch above stored (256 threads, one CTA)
    CUDA_TRY(launch_pdl(m->pdl, k_route_dispatch_small, dim3(1), dim3(256), dispatch_small_smem((int)g.num_experts, 256),
                        st, (const float*)nullptr, (const int*)m->valid_tokens, (int)g.num_experts,
                        (int)g.experts_per_token, (int)g.block_size, (int)m->sorted_capacity, (int)m->block_capacity,
                        m->topk_ids, m->topk_weights, m->sorted_token_ids, m->expert_ids, m->num_tokens_post_pad,
                        m->expert_offsets, m->expert_counts, m->work_items, m->n_work));
    return XABE_OK;
}

int check_mlp(xabe_moe* m, const char* prefix, const xabe_quant_tensor& gate, const xabe_quant_tensor& up,
              const xabe_quant_tensor& down, size_t matrices) {
    size_t n = matrices * (size_t)m->g.intermediate * m->g.hidden;
    char name[64];
    int rc;
    snprintf(name, sizeof(name), "%s gate", prefix);
    if ((rc = check_stack(name, gate, n))) return rc;
    snprintf(name, sizeof(name), "%s up", prefix);
    if ((rc = check_stack(name, up, n))) return rc;
    snprintf(name, sizeof(name), "%s down", prefix);
    if ((rc = check_stack(name, down, n))) return rc;
    return XABE_OK;
}

}  // namespace

extern "C" {

const char* xabe_moe_last_error(void) { return g_last_error.c_str(); }
int xabe_moe_abi_version(void) { return 2; }
uint64_t xabe_kernel_launch_count(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

uint64_t xabe_moe_sorted_capacity(const xabe_moe_geometry* g) { return g ? sorted_capacity_of(*g) : 0; }
uint64_t xabe_moe_expert_block_capacity(const xabe_moe_geometry* g) {
    return g && g->block_size ? sorted_capacity_of(*g) / g->block_size : 0;
}

int xabe_moe_create(const xabe_moe_geometry* geometry, int device, int scope, float eps, xabe_moe** out) {
    if (!geometry || !out) return fail(XABE_ERR_INVALID_ARGUMENT, "null geometry or output pointer");
    *out = nullptr;
    const xabe_moe_geometry g = *geometry;
    auto bad = [&](const char* reason) {
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY,
                    "unsupported MoE geometry {experts %u, top_k %u, hidden %u, intermediate %u, block %u, "
                    "max_tokens %u}: %s",
                    g.num_experts, g.experts_per_token, g.hidden, g.intermediate, g.block_size, g.max_tokens,
                    reason);
    };
    // MoeKernels::new, crates/xabe-cuda/src/kernels/moe.rs:5043-5111
    if (g.block_size == 0) return bad("block_size must be non-zero");
    if (scope == XABE_SCOPE_ROUTED) {
        if (g.experts_per_token == 0) return bad("experts_per_token must be non-zero");
        if (g.experts_per_token > g.num_experts) return bad("experts_per_token must not exceed num_experts");
        if (g.num_experts > 512) return bad("num_experts exceeds the 512 the routing warp holds");
        if (g.experts_per_token > 16) return bad("experts_per_token exceeds 16");
    } else if (scope != XABE_SCOPE_SHARED_ONLY) {
        return fail(XABE_ERR_INVALID_ARGUMENT, "unknown buffer scope %d", scope);
    }
    if (g.max_tokens == 0) return bad("max_tokens must be non-zero");
    if (g.hidden == 0 || g.intermediate == 0) return bad("hidden and intermediate must be non-zero");
    if (g.hidden % 256 != 0) return bad("hidden must be a multiple of the 256-element superblock");
    if (g.intermediate % 256 != 0) return bad("intermediate must be a multiple of the 256-element superblock");
    if (g.block_size > 8 * kMaxNB) return bad("block_size exceeds the slots the tensor-core tile stages");
    // The reference caps this at 65535 because it puts max_tokens on grid.y; here it only ever rides
    // grid.x, so the cap is a sanity bound on the scratch size.
    if (g.max_tokens > (1u << 20)) return bad("max_tokens exceeds the 1048576 sanity limit");
    uint64_t cap = scope == XABE_SCOPE_ROUTED ? sorted_capacity_of(g) : 0;
    uint64_t shared_tiles = (g.max_tokens + g.block_size - 1) / g.block_size;
    if (cap / g.block_size + shared_tiles > 65535)
        return bad("dispatch-block capacity exceeds the 65535 grid.y limit");

    int n_dev = 0;
    CUDA_TRY(cudaGetDeviceCount(&n_dev));
    if (device < 0 || device >= n_dev) return fail(XABE_ERR_DRIVER, "CUDA driver error: no device %d", device);
    CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop{};
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(XABE_ERR_DRIVER, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);

    xabe_moe* m = new (std::nothrow) xabe_moe();
    if (!m) return fail(XABE_ERR_DRIVER, "out of host memory");
    m->sm_count = prop.multiProcessorCount;
    // Items of up to 512 token columns (four accumulators per unpacked weight pair, B tiles by TMA):
    // measured faster only where every item is full and the contraction is long -- the dense block at
    // prefill width (3.40 vs 3.77 ms per layer at 4096 tokens); with the routed experts the extra
    // pass that permutes the activations costs more than the shared unpack work returns.
    // XABE_TUNE_PREFILL_WIDE overrides the choice after creation.
    m->pf_item_cols = (scope == XABE_SCOPE_SHARED_ONLY && g.max_tokens >= kPrefillWideMinTokens) ? kPfWideItemCols
                                                                                                 : kPfTileN;
    m->g = g;
    m->device = device;
    m->scope = scope;
    m->eps = eps;
    m->sorted_capacity = cap;
    m->block_capacity = cap / g.block_size;
    uint64_t pairs = (uint64_t)g.max_tokens * (scope == XABE_SCOPE_ROUTED ? g.experts_per_token : 0);
    m->align_chunk = align_chunk_pairs(pairs);
    m->n_chunks = (int)((pairs + m->align_chunk - 1) / m->align_chunk);
    if (m->n_chunks < 1) m->n_chunks = 1;
    size_t T = g.max_tokens, H = g.hidden, I = g.intermediate, E = g.num_experts, K = g.experts_per_token;
    cudaError_t e = cudaSuccess;
    auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    A(cudaHostAlloc((void**)&m->h_status, sizeof(int), cudaHostAllocDefault));
    A(dev_alloc(&m->valid_tokens, 1));
    A(dev_alloc(&m->status, 1));
    A(dev_alloc(&m->normed, T * H));
    A(dev_alloc(&m->normed_h, T * H));
    A(dev_alloc(&m->inter_shared, T * I));
    A(dev_alloc(&m->shexp, T * H));
    A(dev_alloc(&m->stage_in, T * H));
    A(dev_alloc(&m->stage_ffn, T * H));
    A(dev_alloc(&m->stage_out, T * H));
    if (scope == XABE_SCOPE_ROUTED) {
        A(dev_alloc(&m->topk_ids, T * K));
        A(dev_alloc(&m->topk_weights, T * K));
        A(dev_alloc(&m->sorted_token_ids, (size_t)cap));
        A(dev_alloc(&m->expert_ids, (size_t)m->block_capacity));
        A(dev_alloc(&m->num_tokens_post_pad, 1));
        A(dev_alloc(&m->chunk_hist, (size_t)m->n_chunks * E));
        A(dev_alloc(&m->expert_offsets, E + 1));
        A(dev_alloc(&m->expert_counts, E + 1));
        A(dev_alloc(&m->front_tickets, T + 1));
        A(dev_alloc(&m->tail_done, (size_t)kTailMaxTokens * (H / 128 + 1)));
        A(dev_alloc(&m->ep_compact, E + 1));
        A(dev_alloc(&m->ep_rank_start, kEpMaxRanks));
        A(dev_alloc(&m->ep_send_counts, kEpMaxRanks));
        m->work_capacity = (T * K + 7) / 8 + (E < T * K ? E : T * K) + 1;
        A(dev_alloc(&m->work_items, (size_t)m->work_capacity * kWorkItemInts));
        A(dev_alloc(&m->n_work, 1));
        m->pf_capacity = (T * K + kPfTileN - 1) / kPfTileN + (E < T * K ? E : T * K) + 1;
        A(dev_alloc(&m->pf_items, (size_t)m->pf_capacity * kPfItemInts));
        A(dev_alloc(&m->pf_n_items, 1));
        A(dev_alloc(&m->logits, T * E));
        A(dev_alloc(&m->inter_routed, (size_t)cap * I));
        A(dev_alloc(&m->partial, T * K * H));
        A(dev_alloc(&m->routed, T * H));
        A(dev_alloc(&m->gate, T));
    }
    if (g.max_tokens <= (uint32_t)kDrMaxTokens && H % 256 == 0) {
        // k_dense_rows<DOWN>: about as many units as SMs, by splitting the contraction as well
        const int row_blocks = (int)(H / 256), n_spans = (int)(I / 256);
        int ks = row_blocks > 0 ? m->sm_count / row_blocks : 1;
        if (ks < 1) ks = 1;
        if (ks > n_spans) ks = n_spans;
        if (ks > 16) ks = 16;
        m->dense_k_splits = ks;
        if (ks > 1) A(dev_alloc(&m->dense_partial, (size_t)ks * T * H));
    }
    if (e != cudaSuccess) {
        xabe_moe_destroy(m);
        return fail(XABE_ERR_DRIVER, "CUDA driver error: %s (allocating MoE buffers)", cudaGetErrorString(e));
    }
    if (m->pf_item_cols > kPfTileN) {
        int rc = setup_wide_prefill(m);
        if (rc) {
            xabe_moe_destroy(m);
            return rc;
        }
    }
    *out = m;
    return XABE_OK;
}

void xabe_moe_destroy(xabe_moe* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    void* dev[] = {m->valid_tokens, m->status, m->topk_ids, m->topk_weights, m->sorted_token_ids, m->expert_ids,
                   m->num_tokens_post_pad, m->chunk_hist, m->expert_offsets, m->expert_counts, m->front_tickets, m->tail_done, m->ep_compact, m->ep_rank_start, m->ep_send_counts, m->work_items, m->n_work, m->pf_items,
                   m->pf_n_items, m->normed, m->normed_h, m->logits,
                   m->inter_routed, m->inter_shared, m->x_sorted, m->dense_partial, m->partial, m->routed, m->shexp, m->gate, m->stage_in,
                   m->stage_ffn, m->stage_out};
    for (void* p : dev)
        if (p) cudaFree(p);
    if (m->h_status) cudaFreeHost(m->h_status);
    if (m->prof_events) {
        for (int i = 0; i < kProfCalls * (XABE_STAGE_COUNT + 1); ++i) cudaEventDestroy(m->prof_events[i]);
        delete[] m->prof_events;
    }
    delete m;
}

int xabe_moe_set_valid_tokens(xabe_moe* m, void* stream, int tokens) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    if (tokens < 0 || (uint32_t)tokens > m->g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u the buffers were sized for", tokens,
                    m->g.max_tokens);
    if (tokens == m->published_tokens) return XABE_OK;  // moe.rs:5480-5483
    // The value travels as a kernel argument, so no host memory is read later
    // and nothing has to be synchronised.
    k_set_scalar<<<1, 1, 0, counted((cudaStream_t)stream)>>>(m->valid_tokens, tokens);
    CUDA_TRY(cudaGetLastError());
    m->published_tokens = tokens;
    return XABE_OK;
}

int xabe_moe_rms_norm(xabe_moe* m, void* stream, const float* x, const float* weight) {
    if (!m || !x || !weight) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to rms_norm");
    return launch_rms_norm(m, (cudaStream_t)stream, x, weight);
}

int xabe_moe_router_logits(xabe_moe* m, void* stream, const float* router, const float* bias) {
    if (!m || !router) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to router_logits");
    int rc = check_routed(m, "router_logits");
    if (rc) return rc;
    return launch_router(m, (cudaStream_t)stream, router, bias);
}

int xabe_moe_route_and_dispatch(xabe_moe* m, void* stream, const float* logits) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    int rc = check_routed(m, "route_and_dispatch");
    if (rc) return rc;
    return launch_route_and_dispatch(m, (cudaStream_t)stream, logits ? logits : m->logits);
}

int xabe_moe_build_dispatch(xabe_moe* m, void* stream, const int32_t* topk_ids, const float* topk_weights) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    int rc = check_routed(m, "build_dispatch");
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    size_t n = (size_t)m->g.max_tokens * m->g.experts_per_token;
    if (topk_ids)
        CUDA_TRY(cudaMemcpyAsync(m->topk_ids, topk_ids, n * sizeof(int), cudaMemcpyDeviceToDevice, st));
    if (topk_weights)
        CUDA_TRY(cudaMemcpyAsync(m->topk_weights, topk_weights, n * sizeof(float), cudaMemcpyDeviceToDevice, st));
    return launch_route_and_dispatch(m, st, nullptr);
}

// The combine kernels move 16 bytes per thread when one block owns a token's whole row and every row
// they touch starts on a 16-byte boundary.
static bool combine_vec(const xabe_moe* m, dim3 grid, const void* a, const void* b, const void* c,
                        const void* d = nullptr) {
    auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    return grid.y == 1 && m->g.hidden % 4 == 0 && m->g.experts_per_token == 8 && al(a) && al(b) && al(c) && al(d);
}

int xabe_moe_gate_and_combine(xabe_moe* m, void* stream, const float* shared_gate_inp, const float* residual,
                              size_t residual_len, float* ffn_out, size_t ffn_out_len, float* l_out,
                              size_t l_out_len) {
    if (!m || !shared_gate_inp || !residual || !ffn_out || !l_out)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to gate_and_combine");
    int rc = check_routed(m, "gate_and_combine");
    if (rc) return rc;
    const auto& g = m->g;
    size_t n = (size_t)g.max_tokens * g.hidden;
    if (residual_len != n || ffn_out_len != n || l_out_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "gate_and_combine buffers must hold %zu floats", n);
    dim3 grid(g.max_tokens, g.max_tokens >= 512 ? 1u : (g.hidden + 255) / 256);
    CUDA_TRY(launch_pdl(m->pdl,
                        combine_vec(m, grid, residual, ffn_out, l_out) ? k_gate_and_combine<true> : k_gate_and_combine<false>,
                        grid, dim3(256), 0, (cudaStream_t)stream, shared_gate_inp,
                        (const float*)m->normed, (const float*)m->partial, (const float*)m->shexp, residual,
                        (const int*)m->valid_tokens, (int)g.experts_per_token, (int)g.hidden, m->gate, m->routed,
                        ffn_out, l_out));
    return XABE_OK;
}

int xabe_moe_grouped_forward_partial(xabe_moe* m, void* stream, xabe_quant_tensor gate, xabe_quant_tensor up,
                                     xabe_quant_tensor down, const float* hidden_states) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    int rc = check_routed(m, "grouped_forward");
    if (rc) return rc;
    if ((rc = check_mlp(m, "routed", gate, up, down, m->g.num_experts))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (hidden_states && (rc = rows_to_half(m, st, hidden_states))) return rc;
    MlpWeights r;
    r.present = true;
    r.gate = gate;
    r.up = up;
    r.down = down;
    return run_experts(m, st, r, MlpWeights{}, nullptr);
}

int xabe_moe_grouped_forward_partial_f16(xabe_moe* m, void* stream, xabe_quant_tensor gate, xabe_quant_tensor up,
                                         xabe_quant_tensor down, const void* rows_f16, size_t n_rows) {
    if (!m || !rows_f16) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to grouped_forward_partial_f16");
    int rc = check_routed(m, "grouped_forward");
    if (rc) return rc;
    if ((rc = check_mlp(m, "routed", gate, up, down, m->g.num_experts))) return rc;
    if (((uintptr_t)rows_f16 & 15) != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "f16 rows must be 16-byte aligned");
    if (n_rows > m->g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%zu rows exceed max_tokens %u", n_rows, m->g.max_tokens);
    MlpWeights r;
    r.present = true;
    r.gate = gate;
    r.up = up;
    r.down = down;
    m->x_routed_override = (const __half*)rows_f16;
    rc = run_experts(m, (cudaStream_t)stream, r, MlpWeights{}, nullptr);
    m->x_routed_override = nullptr;
    return rc;
}

int xabe_moe_ep_pack(xabe_moe* m, void* stream, const int64_t* order, size_t n_pairs, int experts_per_rank,
                     void* send_rows_f16, int32_t* send_local_expert, int32_t* inverse) {
    if (!m || !order || !send_rows_f16 || !send_local_expert || !inverse)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to ep_pack");
    int rc = check_routed(m, "ep_pack");
    if (rc) return rc;
    const auto& g = m->g;
    if (n_pairs > (size_t)g.max_tokens * g.experts_per_token)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%zu pairs exceed max_tokens * k", n_pairs);
    if (experts_per_rank <= 0 || g.hidden % 8 != 0 || ((uintptr_t)send_rows_f16 & 15) != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "ep_pack: bad experts_per_rank, hidden or alignment");
    if (n_pairs == 0) return XABE_OK;
    k_ep_pack<<<(unsigned)n_pairs, 256, 0, counted((cudaStream_t)stream)>>>(
        (const long long*)order, m->normed_h, m->topk_ids, (int)g.experts_per_token, (int)g.hidden,
        experts_per_rank, (__half*)send_rows_f16, send_local_expert, inverse);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_ep_plan_pack(xabe_moe* m, void* stream, int experts_per_rank, void* send_rows_f16,
                          int32_t* send_local_expert, int32_t* inverse, int32_t* send_counts) {
    if (!m || !send_rows_f16 || !send_local_expert || !inverse || !send_counts)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to ep_plan_pack");
    int rc = check_routed(m, "ep_plan_pack");
    if (rc) return rc;
    const auto& g = m->g;
    if (experts_per_rank <= 0 || g.num_experts % experts_per_rank != 0 || g.hidden % 8 != 0 ||
        ((uintptr_t)send_rows_f16 & 15) != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "ep_plan_pack: bad experts_per_rank, hidden or alignment");
    cudaStream_t st = (cudaStream_t)stream;
    int threads = ((int)g.num_experts + 1 + 31) / 32 * 32;
    k_ep_plan<<<1, threads, (g.num_experts + 1) * sizeof(int), counted(st)>>>((int)g.num_experts, experts_per_rank,
                                                                     m->expert_counts, m->ep_compact, send_counts);
    CUDA_TRY(cudaGetLastError());
    k_ep_pack_sorted<<<(unsigned)m->sorted_capacity, 256, 0, counted(st)>>>(
        m->sorted_token_ids, m->expert_ids, m->expert_offsets, m->ep_compact, m->num_tokens_post_pad,
        m->valid_tokens, m->normed_h, (int)g.experts_per_token, (int)g.hidden, (int)g.block_size, experts_per_rank,
        (__half*)send_rows_f16, send_local_expert, inverse);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

namespace {
EpPeers peers_of(void* const* p, int world) {
    EpPeers e{};
    for (int i = 0; i < world && i < kEpMaxRanks; ++i) e.p[i] = p[i];
    return e;
}
int check_p2p(const xabe_moe* m, const xabe_ep_peers* peers, int world, int rank, int cap, const char* what) {
    if (!m || !peers) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to %s", what);
    if (world < 1 || world > kEpMaxRanks || rank < 0 || rank >= world || cap < 1)
        return fail(XABE_ERR_INVALID_ARGUMENT, "%s: world %d (at most %d), rank %d, cap %d", what, world,
                    kEpMaxRanks, rank, cap);
    for (int i = 0; i < world; ++i)
        if (!peers->rows[i] || !peers->eid[i] || !peers->meta[i] || !peers->flag_in[i] || !peers->back[i] ||
            !peers->flag_back[i])
            return fail(XABE_ERR_INVALID_ARGUMENT, "%s: rank %d's buffers are not mapped", what, i);
    return XABE_OK;
}
}  // namespace

int xabe_moe_ep_p2p_send(xabe_moe* m, void* stream, int experts_per_rank, int world, int rank, int cap,
                         const xabe_ep_peers* peers, int step, int32_t* inverse) {
    int rc = check_p2p(m, peers, world, rank, cap, "ep_p2p_send");
    if (rc) return rc;
    if ((rc = check_routed(m, "ep_p2p_send"))) return rc;
    const auto& g = m->g;
    if (!inverse || experts_per_rank <= 0 || (int)g.num_experts != experts_per_rank * world || g.hidden % 8 != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "ep_p2p_send: experts do not split as %d x %d", world, experts_per_rank);
    if ((uint64_t)g.max_tokens * g.experts_per_token > (uint64_t)cap)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "ep_p2p_send: %u x %u pairs exceed the receive regions of %d rows",
                    g.max_tokens, g.experts_per_token, cap);
    cudaStream_t st = (cudaStream_t)stream;
    int threads = ((int)g.num_experts + 1 + 31) / 32 * 32;
    k_ep_plan_ranks<<<1, threads, (g.num_experts + 1) * sizeof(int), counted(st)>>>(
        (int)g.num_experts, experts_per_rank, m->expert_counts, m->ep_compact, m->ep_rank_start, m->ep_send_counts);
    CUDA_TRY(cudaGetLastError());
    k_ep_push_rows<<<(unsigned)((m->sorted_capacity + kEpPushSlotsPerBlock - 1) / kEpPushSlotsPerBlock), 256, 0,
                     counted(st)>>>(
        m->sorted_token_ids, m->expert_ids, m->expert_offsets, m->ep_compact, m->ep_rank_start,
        m->num_tokens_post_pad, m->valid_tokens, m->normed_h, (int)g.experts_per_token, (int)g.hidden,
        (int)g.block_size, experts_per_rank, rank, cap, peers_of(peers->rows, world), peers_of(peers->eid, world),
        inverse);
    CUDA_TRY(cudaGetLastError());
    k_ep_signal_rows<<<1, 32, 0, counted(st)>>>(world, rank, m->ep_send_counts, m->ep_rank_start,
                                       peers_of(peers->meta, world), peers_of(peers->flag_in, world), step);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_ep_p2p_receive(xabe_moe* m, void* stream, int world, int rank, int cap, const xabe_ep_peers* peers,
                            int step, int32_t* ids_out, void* result_dst) {
    int rc = check_p2p(m, peers, world, rank, cap, "ep_p2p_receive");
    if (rc) return rc;
    if (!ids_out || !result_dst) return fail(XABE_ERR_INVALID_ARGUMENT, "null output of ep_p2p_receive");
    if ((uint64_t)world * cap > m->g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "ep_p2p_receive: %d x %d slots exceed max_tokens %u", world, cap,
                    m->g.max_tokens);
    cudaStream_t st = (cudaStream_t)stream;
    k_ep_wait_flags<<<1, 32, 0, counted(st)>>>(world, (const int*)peers->flag_in[rank], step,
                                      m->peer_wait_limit ? m->peer_wait_limit : kPeerWaitLimit, m->status);
    CUDA_TRY(cudaGetLastError());
    size_t slots = (size_t)world * cap;
    k_ep_fill_slots<<<(unsigned)((slots + 255) / 256), 256, 0, counted(st)>>>(
        world, cap, (int)m->g.hidden, (const int*)peers->meta[rank], (const int*)peers->eid[rank],
        (int)m->g.num_experts, peers_of(peers->back, world), (const int*)m->status, ids_out, (float**)result_dst);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_ipc_alloc(size_t bytes, void** dev_ptr, unsigned char* handle64) {
    if (!dev_ptr || !handle64 || bytes == 0) return fail(XABE_ERR_INVALID_ARGUMENT, "bad argument to ipc_alloc");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(XABE_ERR_DRIVER, "CUDA driver error: %s (ipc_alloc)", cudaGetErrorString(e));
    }
    memcpy(handle64, &h, 64);
    *dev_ptr = p;
    return XABE_OK;
}

int xabe_ipc_open(const unsigned char* handle64, void** dev_ptr) {
    if (!dev_ptr || !handle64) return fail(XABE_ERR_INVALID_ARGUMENT, "bad argument to ipc_open");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    CUDA_TRY(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return XABE_OK;
}

int xabe_ipc_close(void* dev_ptr) {
    if (dev_ptr) CUDA_TRY(cudaIpcCloseMemHandle(dev_ptr));
    return XABE_OK;
}

int xabe_ipc_free(void* dev_ptr) {
    if (dev_ptr) CUDA_TRY(cudaFree(dev_ptr));
    return XABE_OK;
}

int xabe_moe_set_result_destinations(xabe_moe* m, const void* table) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    m->partial_rows = (float* const*)table;
    return XABE_OK;
}

int xabe_moe_ep_p2p_return(xabe_moe* m, void* stream, int world, int rank, int cap, const xabe_ep_peers* peers,
                           int step, const void* result_dst) {
    int rc = check_p2p(m, peers, world, rank, cap, "ep_p2p_return");
    if (rc) return rc;
    if ((rc = check_routed(m, "ep_p2p_return"))) return rc;
    if (!result_dst || (uint64_t)world * cap > m->g.max_tokens || m->g.experts_per_token != 1 || m->g.hidden % 4 != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "ep_p2p_return: needs the owner-side handle (k = 1) and its slot table");
    cudaStream_t st = (cudaStream_t)stream;
    if (m->partial_rows != (float* const*)result_dst) {  // the down projection did not store through this table itself
        k_ep_push_results<<<(unsigned)((size_t)world * cap), 256, 0, counted(st)>>>(m->partial, (float* const*)result_dst,
                                                                           (int)m->g.hidden);
        CUDA_TRY(cudaGetLastError());
    }
    k_ep_signal_results<<<1, 32, 0, counted(st)>>>(world, rank, peers_of(peers->flag_back, world), step);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_ep_p2p_wait_results(xabe_moe* m, void* stream, int world, int rank, const xabe_ep_peers* peers,
                                 int step) {
    int rc = check_p2p(m, peers, world, rank, 1, "ep_p2p_wait_results");
    if (rc) return rc;
    k_ep_wait_flags<<<1, 32, 0, counted((cudaStream_t)stream)>>>(world, (const int*)peers->flag_back[rank], step,
                                                        m->peer_wait_limit ? m->peer_wait_limit : kPeerWaitLimit,
                                                        m->status);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_ep_combine(xabe_moe* m, void* stream, const float* back_rows, size_t n_rows, const int32_t* inverse,
                        const float* shared_gate_inp, const float* residual, size_t residual_len, float* ffn_out,
                        size_t ffn_out_len, float* l_out, size_t l_out_len) {
    if (!m || !back_rows || !inverse || !shared_gate_inp || !residual || !ffn_out || !l_out)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to ep_combine");
    int rc = check_routed(m, "ep_combine");
    if (rc) return rc;
    const auto& g = m->g;
    size_t n = (size_t)g.max_tokens * g.hidden;
    if (residual_len != n || ffn_out_len != n || l_out_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "ep_combine buffers must hold %zu floats", n);
    if (n_rows > (size_t)g.max_tokens * g.experts_per_token)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%zu rows exceed max_tokens * k", n_rows);
    dim3 grid(g.max_tokens, g.max_tokens >= 512 ? 1u : (g.hidden + 255) / 256);
    auto kern = combine_vec(m, grid, residual, ffn_out, l_out, back_rows) ? k_ep_combine<true> : k_ep_combine<false>;
    kern<<<grid, 256, 0, counted((cudaStream_t)stream)>>>(
        shared_gate_inp, m->normed, back_rows, inverse, m->topk_weights, m->shexp, residual, m->valid_tokens,
        (int)g.experts_per_token, (int)g.hidden, m->gate, m->routed, ffn_out, l_out);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_grouped_forward(xabe_moe* m, void* stream, xabe_quant_tensor gate, xabe_quant_tensor up,
                             xabe_quant_tensor down, const float* hidden_states, float* out) {
    if (!out) return fail(XABE_ERR_INVALID_ARGUMENT, "null output");
    int rc = xabe_moe_grouped_forward_partial(m, stream, gate, up, down, hidden_states);
    if (rc) return rc;
    dim3 grid(m->g.max_tokens, (m->g.hidden + 255) / 256);
    k_reduce<<<grid, 256, 0, counted((cudaStream_t)stream)>>>(m->partial, m->valid_tokens, (int)m->g.experts_per_token,
                                                     (int)m->g.hidden, out);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_shared_expert(xabe_moe* m, void* stream, xabe_quant_tensor gate, xabe_quant_tensor up,
                           xabe_quant_tensor down, const float* hidden_states, float* out) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    int rc;
    if ((rc = check_mlp(m, "shared", gate, up, down, 1))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (hidden_states && (rc = rows_to_half(m, st, hidden_states))) return rc;
    MlpWeights s;
    s.present = true;
    s.gate = gate;
    s.up = up;
    s.down = down;
    return run_experts(m, st, MlpWeights{}, s, out ? out : m->shexp);
}

int xabe_moe_block_forward(xabe_moe* m, void* stream, const xabe_moe_layer_weights* w, const float* residual,
                           size_t residual_len, int tokens, float* ffn_out, size_t ffn_out_len, float* l_out,
                           size_t l_out_len) {
    if (!m || !w || !residual || !ffn_out || !l_out)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to block_forward");
    int rc = check_routed(m, "block_forward");
    if (rc) return rc;
    const auto& g = m->g;
    // block/moe.rs:1100-1110
    if (tokens < 0 || (uint32_t)tokens > g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u this block was sized for", tokens,
                    g.max_tokens);
    size_t n = (size_t)g.max_tokens * g.hidden;
    if (residual_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "residual must hold %zu floats, holds %zu", n, residual_len);
    if (ffn_out_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "ffn_out must hold %zu floats, holds %zu", n, ffn_out_len);
    if (l_out_len != n) return fail(XABE_ERR_BUFFER_LENGTH, "l_out must hold %zu floats, holds %zu", n, l_out_len);
    if (!w->post_norm || !w->router || !w->shared_gate_inp)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null dense weight in layer weights");
    if ((rc = check_mlp(m, "routed", w->gate_exps, w->up_exps, w->down_exps, g.num_experts))) return rc;
    if ((rc = check_mlp(m, "shared", w->shared_gate, w->shared_up, w->shared_down, 1))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if ((rc = xabe_moe_set_valid_tokens(m, stream, tokens))) return rc;
    prof_mark(m, st, 0);
    bool front_routes = false;
    const bool fused_front = front_applies(m, residual, w->router, &front_routes);
    const bool fused_tail = tail_applies(m, w) && ((uintptr_t)residual & 15) == 0 && ((uintptr_t)ffn_out & 15) == 0 &&
                            ((uintptr_t)l_out & 15) == 0;
    if (fused_front) {
        // one launch for norm, router, routing and dispatch: the stage profile books it under stage 0
        if ((rc = launch_front(m, st, residual, w, front_routes))) return rc;
        prof_mark(m, st, 1);
        prof_mark(m, st, 2);
    } else {
        // with the last stage folded into the down launch, the gate it needs is formed here
        if ((rc = launch_rms_norm(m, st, residual, w->post_norm, fused_tail ? w->shared_gate_inp : nullptr))) return rc;
        prof_mark(m, st, 1);
        if ((rc = launch_router(m, st, w->router, w->router_bias))) return rc;
        prof_mark(m, st, 2);
        if ((rc = launch_route_and_dispatch(m, st, m->logits))) return rc;
    }
    prof_mark(m, st, 3);
    MlpWeights r, s;
    r.present = s.present = true;
    r.gate = w->gate_exps;
    r.up = w->up_exps;
    r.down = w->down_exps;
    s.gate = w->shared_gate;
    s.up = w->shared_up;
    s.down = w->shared_down;
    if (fused_tail) {
        // the down launch combines: routed, ffn_out and l_out are complete when it is
        const TailFusion tail{m->gate, residual, m->routed, ffn_out, l_out};
        if ((rc = run_experts(m, st, r, s, m->shexp, 4, &tail))) return rc;
        prof_mark(m, st, 5);
    } else {
        if ((rc = run_experts(m, st, r, s, m->shexp, 4))) return rc;
        prof_mark(m, st, 5);
        dim3 grid(g.max_tokens, g.max_tokens >= 512 ? 1u : (g.hidden + 255) / 256);
        CUDA_TRY(launch_pdl(m->pdl,
                            combine_vec(m, grid, residual, ffn_out, l_out) ? k_gate_and_combine<true>
                                                                           : k_gate_and_combine<false>,
                            grid, dim3(256), 0, st, w->shared_gate_inp,
                            (const float*)m->normed, (const float*)m->partial, (const float*)m->shexp, residual,
                            (const int*)m->valid_tokens, (int)g.experts_per_token, (int)g.hidden, m->gate, m->routed,
                            ffn_out, l_out));
    }
    prof_mark(m, st, 6);
    if (m->prof_on && m->prof_calls < kProfCalls) m->prof_calls++;
    return XABE_OK;
}

int xabe_moe_stack_forward(xabe_moe* m, void* stream, const xabe_moe_layer_weights* layers, int n_layers,
                           float* hidden_a, float* hidden_b, size_t hidden_len, int tokens, float* ffn_out,
                           size_t ffn_out_len, float** final_hidden) {
    if (!m || !layers || !hidden_a || !hidden_b || !ffn_out || n_layers < 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to stack_forward");
    if (hidden_a == hidden_b) return fail(XABE_ERR_INVALID_ARGUMENT, "stack_forward needs two distinct hidden-state buffers");
    int rc = check_routed(m, "stack_forward");
    if (rc) return rc;
    const auto& g = m->g;
    if (tokens < 0 || (uint32_t)tokens > g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u this block was sized for", tokens,
                    g.max_tokens);
    const size_t n = (size_t)g.max_tokens * g.hidden;
    if (hidden_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "hidden state must hold %zu floats, holds %zu", n, hidden_len);
    if (ffn_out_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "ffn_out must hold %zu floats, holds %zu", n, ffn_out_len);
    // every layer is checked before the first launch (check_stack, moe.rs:6729-6746)
    for (int i = 0; i < n_layers; ++i) {
        const xabe_moe_layer_weights* w = layers + i;
        if (!w->post_norm || !w->router || !w->shared_gate_inp)
            return fail(XABE_ERR_INVALID_ARGUMENT, "null dense weight in the weights of layer %d", i);
        if ((rc = check_mlp(m, "routed", w->gate_exps, w->up_exps, w->down_exps, g.num_experts))) return rc;
        if ((rc = check_mlp(m, "shared", w->shared_gate, w->shared_up, w->shared_down, 1))) return rc;
    }
    float* src = hidden_a;
    float* dst = hidden_b;
    for (int i = 0; i < n_layers; ++i) {
        if ((rc = xabe_moe_block_forward(m, stream, layers + i, src, n, tokens, ffn_out, n, dst, n))) return rc;
        float* t = src;
        src = dst;
        dst = t;
    }
    if (final_hidden) *final_hidden = src;
    return XABE_OK;
}

int xabe_moe_block_forward_host(xabe_moe* m, void* stream, const xabe_moe_layer_weights* w,
                                const float* host_residual, int tokens, float* host_ffn_out, float* host_l_out) {
    if (!m || !host_residual) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to block_forward_host");
    if (tokens < 0 || (uint32_t)tokens > m->g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u this block was sized for", tokens,
                    m->g.max_tokens);
    cudaStream_t st = (cudaStream_t)stream;
    size_t bytes = (size_t)tokens * m->g.hidden * sizeof(float);
    size_t n = (size_t)m->g.max_tokens * m->g.hidden;
    if (bytes) CUDA_TRY(cudaMemcpyAsync(m->stage_in, host_residual, bytes, cudaMemcpyHostToDevice, st));
    int rc = xabe_moe_block_forward(m, stream, w, m->stage_in, n, tokens, m->stage_ffn, n, m->stage_out, n);
    if (rc) return rc;
    if (bytes && host_ffn_out)
        CUDA_TRY(cudaMemcpyAsync(host_ffn_out, m->stage_ffn, bytes, cudaMemcpyDeviceToHost, st));
    if (bytes && host_l_out)
        CUDA_TRY(cudaMemcpyAsync(host_l_out, m->stage_out, bytes, cudaMemcpyDeviceToHost, st));
    return XABE_OK;
}

int xabe_moe_block_forward_typed(xabe_moe* m, void* stream, const xabe_moe_layer_weights* w, const void* residual,
                                 int residual_dtype, size_t residual_len, int tokens, float* ffn_out,
                                 size_t ffn_out_len, float* l_out, size_t l_out_len) {
    if (residual_dtype == XABE_DTYPE_F32)
        return xabe_moe_block_forward(m, stream, w, (const float*)residual, residual_len, tokens, ffn_out,
                                      ffn_out_len, l_out, l_out_len);
    if (residual_dtype != XABE_DTYPE_BF16)
        return fail(XABE_ERR_INVALID_ARGUMENT, "unknown activation dtype tag %d", residual_dtype);
    if (!m || !residual) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to block_forward_typed");
    const auto& g = m->g;
    size_t n = (size_t)g.max_tokens * g.hidden;
    if (residual_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "residual must hold %zu elements, holds %zu", n, residual_len);
    if (tokens < 0 || (uint32_t)tokens > g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u this block was sized for", tokens,
                    g.max_tokens);
    int rc = xabe_moe_set_valid_tokens(m, stream, tokens);
    if (rc) return rc;
    k_rows_bf16_to_f32<<<g.max_tokens, 256, 0, counted((cudaStream_t)stream)>>>((const unsigned short*)residual, m->stage_in,
                                                                      m->valid_tokens, (int)g.hidden);
    CUDA_TRY(cudaGetLastError());
    return xabe_moe_block_forward(m, stream, w, m->stage_in, n, tokens, ffn_out, ffn_out_len, l_out, l_out_len);
}

int xabe_dense_ffn_block_forward(xabe_moe* m, void* stream, const float* post_norm, xabe_quant_tensor gate,
                                 xabe_quant_tensor up, xabe_quant_tensor down, const float* residual,
                                 size_t residual_len, int tokens, float* ffn_out, size_t ffn_out_len,
                                 float* l_out, size_t l_out_len) {
    if (!m || !post_norm || !residual || !ffn_out || !l_out)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to dense_ffn_block_forward");
    const auto& g = m->g;
    if (tokens < 0 || (uint32_t)tokens > g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u this block was sized for", tokens,
                    g.max_tokens);
    size_t n = (size_t)g.max_tokens * g.hidden;
    if (residual_len != n || ffn_out_len != n || l_out_len != n)
        return fail(XABE_ERR_BUFFER_LENGTH, "dense block buffers must hold %zu floats", n);
    int rc;
    if ((rc = check_mlp(m, "dense", gate, up, down, 1))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if ((rc = xabe_moe_set_valid_tokens(m, stream, tokens))) return rc;
    if ((rc = launch_rms_norm(m, st, residual, post_norm))) return rc;
    MlpWeights s;
    s.present = true;
    s.gate = gate;
    s.up = up;
    s.down = down;
    if ((rc = run_experts(m, st, MlpWeights{}, s, ffn_out))) return rc;
    k_add_residual<<<g.max_tokens, 256, 0, counted(st)>>>(ffn_out, residual, m->valid_tokens, (int)g.hidden, l_out);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_buffers(xabe_moe* m, xabe_moe_buffer_view* out) {
    if (!m || !out) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to buffers");
    out->valid_tokens = m->valid_tokens;
    out->topk_ids = m->topk_ids;
    out->topk_weights = m->topk_weights;
    out->sorted_token_ids = m->sorted_token_ids;
    out->expert_ids = m->expert_ids;
    out->num_tokens_post_pad = m->num_tokens_post_pad;
    out->partial = m->partial;
    out->normed = m->normed;
    out->logits = m->logits;
    out->routed = m->routed;
    out->shexp = m->shexp;
    out->gate = m->gate;
    out->sorted_capacity = m->sorted_capacity;
    out->expert_block_capacity = m->block_capacity;
    return XABE_OK;
}

int xabe_moe_set_exact_decode_regime(xabe_moe* m, int on) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    m->exact_decode = on != 0;
    return XABE_OK;
}

int xabe_moe_disable_tensor_cores(xabe_moe* m) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    m->tensor_cores = false;
    return XABE_OK;
}

int xabe_moe_tensor_cores_enabled(const xabe_moe* m) { return m && m->tensor_cores ? 1 : 0; }

int xabe_moe_force_prefill_path(xabe_moe* m, int on) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    m->force_prefill = on != 0;
    return XABE_OK;
}

int xabe_moe_set_peer_wait_limit(xabe_moe* m, uint32_t iterations) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    m->peer_wait_limit = iterations;
    return XABE_OK;
}

int xabe_moe_set_tuning(xabe_moe* m, int key, int value) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    switch (key) {
        case XABE_TUNE_PDL: m->pdl = value != 0; return XABE_OK;
        case XABE_TUNE_STREAM_STAGES: m->stream_stages = value; return XABE_OK;
        case XABE_TUNE_STREAM_RUNS: m->stream_runs = value; return XABE_OK;
        case XABE_TUNE_ROWS_MIN_TOKENS: m->rows_min_tokens = value; return XABE_OK;
        case XABE_TUNE_ROUTER_REGW: m->router_regw = value; return XABE_OK;
        case XABE_TUNE_FORCE_TILE_KERNELS: m->force_tile_kernels = value != 0; return XABE_OK;
        case XABE_TUNE_DENSE_ROWS: m->dense_rows = value != 0; return XABE_OK;
        case XABE_TUNE_FUSED_DECODE:
            m->fused_tail = (value & 1) != 0;
            m->fused_front = (value & 2) != 0;
            m->fused_norm = (value & 4) != 0;
            return XABE_OK;
        case XABE_TUNE_PREFILL_WIDE:
            if (value == 0) {
                m->pf_item_cols = kPfTileN;
                return XABE_OK;
            }
            {
                const int rc = setup_wide_prefill(m);
                // 2, 3: items of two or three 128-column tiles (the B ring then runs further ahead of the MMAs)
                if (!rc && m->pf_item_cols > kPfTileN && value >= 2 && value < kPfWideMaxCt)
                    m->pf_item_cols = value * kPfTileN;
                return rc;
            }
        default: return fail(XABE_ERR_INVALID_ARGUMENT, "unknown tuning key %d", key);
    }
}

int xabe_moe_device_status(xabe_moe* m, void* stream, int* status_out) {
    if (!m || !status_out) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to device_status");
    cudaStream_t st = (cudaStream_t)stream;
    CUDA_TRY(cudaMemcpyAsync(m->h_status, m->status, sizeof(int), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaMemsetAsync(m->status, 0, sizeof(int), st));
    CUDA_TRY(cudaStreamSynchronize(st));
    *status_out = *m->h_status;
    if (*status_out != 0)
        return fail(XABE_ERR_DEVICE_STATUS, "a kernel's bounded wait ran out (device status %d)", *status_out);
    return XABE_OK;
}

int xabe_stream_read(void* stream, const void* dev_bytes, size_t n_bytes, void* sink) {
    if (!dev_bytes || !sink || ((uintptr_t)dev_bytes & 15) != 0)
        return fail(XABE_ERR_INVALID_ARGUMENT, "stream_read: null or misaligned argument");
    int dev = 0, sms = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    k_stream_read<<<sms * 8, 256, 0, counted((cudaStream_t)stream)>>>((const uint4*)dev_bytes, n_bytes / 16, (unsigned*)sink);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_moe_stage_profile(xabe_moe* m, int on) {
    if (!m) return fail(XABE_ERR_INVALID_ARGUMENT, "null handle");
    if (on && !m->prof_events) {
        int n = kProfCalls * (XABE_STAGE_COUNT + 1);
        m->prof_events = new (std::nothrow) cudaEvent_t[n];
        if (!m->prof_events) return fail(XABE_ERR_DRIVER, "out of host memory");
        for (int i = 0; i < n; ++i) CUDA_TRY(cudaEventCreate(&m->prof_events[i]));
    }
    m->prof_on = on != 0;
    m->prof_calls = 0;
    return XABE_OK;
}

int xabe_moe_stage_times(xabe_moe* m, void* stream, float* ms_sum, int* calls) {
    if (!m || !ms_sum || !calls) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to stage_times");
    CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    for (int s = 0; s < XABE_STAGE_COUNT; ++s) ms_sum[s] = 0.0f;
    for (int c = 0; c < m->prof_calls; ++c)
        for (int s = 0; s < XABE_STAGE_COUNT; ++s) {
            float ms = 0.0f;
            cudaEvent_t* e = m->prof_events + c * (XABE_STAGE_COUNT + 1);
            CUDA_TRY(cudaEventElapsedTime(&ms, e[s], e[s + 1]));
            ms_sum[s] += ms;
        }
    *calls = m->prof_calls;
    m->prof_calls = 0;
    return XABE_OK;
}

int xabe_dequantize(void* stream, xabe_quant_tensor t, float* out) {
    if (!out) return fail(XABE_ERR_INVALID_ARGUMENT, "null output");
    if (t.quant != XABE_QUANT_Q6_K && t.quant != XABE_QUANT_Q8_0)
        return fail(XABE_ERR_UNSUPPORTED_EXPERT_TYPE, "quant tag %d is neither Q6_K nor Q8_0", t.quant);
    if (!t.dev_bytes) return fail(XABE_ERR_INVALID_ARGUMENT, "null device pointer");
    size_t bb = block_bytes_of(t.quant);
    if (t.n_bytes % bb != 0)
        return fail(XABE_ERR_RAGGED_WEIGHTS, "dequantize: %zu bytes is not a whole number of %zu B blocks",
                    t.n_bytes, bb);
    size_t n = t.n_bytes / bb * block_elems_of(t.quant);
    if (n == 0) return XABE_OK;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (t.quant == XABE_QUANT_Q6_K)
        k_dequant_q6k<<<blocks, 256, 0, counted((cudaStream_t)stream)>>>((const uint8_t*)t.dev_bytes, n, out);
    else
        k_dequant_q8_0<<<blocks, 256, 0, counted((cudaStream_t)stream)>>>((const uint8_t*)t.dev_bytes, n, out);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Shared-expert MLP for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off the table: a
// serving worker whose memory budget was handed out at start-up and is guarded
// by its own arena, or a caller inside a region where the CUDA allocator may
// not be entered (a latency-critical callback, code running under a foreign
// allocator's lock).  xabe_moe_create allocates, so such a caller cannot hold a
// handle.  This entry point needs none: its scratch (the f16 copy of the
// activations, the f16 SwiGLU intermediate, the live-token scalar and the
// status word) lives in one file-scope device array that every GPU loading the
// library carries until the process exits.
// ---------------------------------------------------------------------------
namespace {

constexpr int kNoAllocMaxTokens = 64;
constexpr int kNoAllocMaxHidden = 2048;
constexpr int kNoAllocMaxInter = 512;
constexpr size_t kNoAllocHeader = 256;  // [0] live tokens, [1] status word
constexpr size_t kNoAllocXBytes = (size_t)kNoAllocMaxTokens * kNoAllocMaxHidden * sizeof(__half);
constexpr size_t kNoAllocInterBytes = (size_t)kNoAllocMaxTokens * kNoAllocMaxInter * sizeof(__half);
constexpr size_t kNoAllocBytes = kNoAllocHeader + kNoAllocXBytes + kNoAllocInterBytes;  // 327,936 B

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kNoAllocMaxDevices = 64;
// Device address of the array, per device.  Host threads may race to fill an entry; every one of them
// stores the same value, and the atomic makes the store and the later loads well defined.
std::atomic<unsigned char*> g_noalloc_ptr[kNoAllocMaxDevices] = {};

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an
// address a kernel may use: the device address comes from the runtime, once
// per device, with that device current.
int noalloc_scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kNoAllocMaxDevices)
        return fail(XABE_ERR_DRIVER, "device index %d is outside the %d this entry point tracks", dev,
                    kNoAllocMaxDevices);
    unsigned char* p = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        CUDA_TRY(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
        if (!p) return fail(XABE_ERR_DRIVER, "the runtime returned a null address for the static scratch");
        g_noalloc_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return XABE_OK;
}

}  // namespace

extern "C" int xabe_shared_expert_noalloc(void* stream, xabe_quant_tensor gate, xabe_quant_tensor up,
                                          xabe_quant_tensor down, int hidden, int intermediate,
                                          const float* hidden_states, int tokens, float* out) {
    if (!hidden_states || !out) return fail(XABE_ERR_INVALID_ARGUMENT, "null activation or output pointer");
    if (tokens < 0 || tokens > kNoAllocMaxTokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %d the static scratch holds", tokens,
                    kNoAllocMaxTokens);
    if (hidden <= 0 || intermediate <= 0 || hidden % 256 != 0 || intermediate % 256 != 0 || hidden % 64 != 0)
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY,
                    "hidden %d / intermediate %d: both must be positive multiples of 256", hidden, intermediate);
    if (hidden > kNoAllocMaxHidden || intermediate > kNoAllocMaxInter)
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY,
                    "hidden %d / intermediate %d exceed the %d / %d the static scratch holds", hidden, intermediate,
                    kNoAllocMaxHidden, kNoAllocMaxInter);
    size_t n = (size_t)hidden * intermediate;
    int rc;
    if ((rc = check_stack("shared gate", gate, n))) return rc;
    if ((rc = check_stack("shared up", up, n))) return rc;
    if ((rc = check_stack("shared down", down, n))) return rc;
    if (gate.quant != up.quant)
        return fail(XABE_ERR_UNSUPPORTED_EXPERT_TYPE, "gate and up must share one format (found tags %d and %d)",
                    gate.quant, up.quant);
    const int bucket = 16;
    size_t smem_gu = gateup_smem(hidden, gate.quant, bucket);
    size_t smem_dn = down_smem(intermediate, down.quant);
    if (smem_gu > 48 * 1024 || smem_dn > 48 * 1024)
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY, "row tiles of %zu / %zu bytes exceed the 48 KB this entry point uses",
                    smem_gu, smem_dn);
    if (tokens == 0) return XABE_OK;
    unsigned char* base = nullptr;
    if ((rc = noalloc_scratch_for_current_device(&base))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int* live = (int*)base;
    int* status = live + 1;
    __half* x_h = (__half*)(base + kNoAllocHeader);
    __half* inter = (__half*)(base + kNoAllocHeader + kNoAllocXBytes);
    // the array keeps the previous call's contents: the two words that must start clean are rewritten,
    // the activation and intermediate rows this call reads are all rewritten by it
    k_set_scalar<<<1, 1, 0, counted(st)>>>(live, tokens);
    k_set_scalar<<<1, 1, 0, counted(st)>>>(status, 0);
    k_rows_to_half<<<tokens, 256, 0, counted(st)>>>(hidden_states, x_h, live, hidden);
    CUDA_TRY(cudaGetLastError());
    ExpertLaunch L{};
    L.routed_blocks = 0;
    L.block_size = bucket;
    L.top_k = 1;
    L.max_tokens = kNoAllocMaxTokens;
    L.valid_tokens = live;
    L.status = status;
    L.s_a = (const uint8_t*)gate.dev_bytes;
    L.s_b = (const uint8_t*)up.dev_bytes;
    L.rows = intermediate;
    L.k = hidden;
    L.x_shared = x_h;
    L.inter_shared = inter;
    unsigned tiles = (unsigned)((tokens + bucket - 1) / bucket);
    // (the kernels' shared-memory ceiling: an attribute write through the runtime, not an allocation)
    if (gate.quant == XABE_QUANT_Q6_K) CUDA_TRY(allow_dynamic_smem((const void*)k_expert_gateup<QUANT_Q6K, QUANT_Q6K>, smem_gu));
    else CUDA_TRY(allow_dynamic_smem((const void*)k_expert_gateup<QUANT_Q8_0, QUANT_Q8_0>, smem_gu));
    if (down.quant == XABE_QUANT_Q6_K) CUDA_TRY(allow_dynamic_smem((const void*)k_expert_down<QUANT_Q6K, QUANT_Q6K>, smem_dn));
    else CUDA_TRY(allow_dynamic_smem((const void*)k_expert_down<QUANT_Q8_0, QUANT_Q8_0>, smem_dn));
    if (gate.quant == XABE_QUANT_Q6_K)
        k_expert_gateup<QUANT_Q6K, QUANT_Q6K><<<dim3(intermediate / 8, tiles), kExpertThreads, smem_gu, counted(st)>>>(L);
    else
        k_expert_gateup<QUANT_Q8_0, QUANT_Q8_0><<<dim3(intermediate / 8, tiles), kExpertThreads, smem_gu, counted(st)>>>(L);
    CUDA_TRY(cudaGetLastError());
    L.s_a = (const uint8_t*)down.dev_bytes;
    L.s_b = nullptr;
    L.rows = hidden;
    L.k = intermediate;
    L.x_shared = inter;
    L.shexp = out;
    if (down.quant == XABE_QUANT_Q6_K)
        k_expert_down<QUANT_Q6K, QUANT_Q6K><<<dim3(hidden / 64, tiles), kExpertThreads, smem_dn, counted(st)>>>(L);
    else
        k_expert_down<QUANT_Q8_0, QUANT_Q8_0><<<dim3(hidden / 64, tiles), kExpertThreads, smem_dn, counted(st)>>>(L);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

// The status word of the static array as the last xabe_shared_expert_noalloc call on `stream` left it:
// 0 when every bounded wait of its kernels completed.  Copies four bytes to `status_out` (host memory)
// and synchronises `stream`; allocates nothing.
extern "C" int xabe_shared_expert_noalloc_status(void* stream, int* status_out) {
    if (!status_out) return fail(XABE_ERR_INVALID_ARGUMENT, "null status pointer");
    unsigned char* base = nullptr;
    int rc = noalloc_scratch_for_current_device(&base);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int v = -1;
    CUDA_TRY(cudaMemcpyAsync(&v, base + sizeof(int), sizeof(int), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    *status_out = v;
    if (v != 0) return fail(XABE_ERR_DEVICE_STATUS, "a kernel's bounded wait ran out (device status %d)", v);
    return XABE_OK;
}


// ---------------------------------------------------------------------------
// LM head (LmHeadKernels, crates/xabe-cuda/src/kernels/lm_head.rs:1493-2015)
// ---------------------------------------------------------------------------
struct xabe_lm_head {
    xabe_lm_head_geometry g{};
    int device = 0;
    int sm_count = 0;
    __half* x_hi = nullptr;  // [max_tokens][hidden]
    __half* x_lo = nullptr;
    int* status = nullptr;   // device word the bounded waits write
    int* h_status = nullptr; // pinned
};

extern "C" {

int xabe_lm_head_create(const xabe_lm_head_geometry* geometry, int device, xabe_lm_head** out) {
    if (!geometry || !out) return fail(XABE_ERR_INVALID_ARGUMENT, "null geometry or output pointer");
    *out = nullptr;
    const xabe_lm_head_geometry g = *geometry;
    // LmHeadKernels::new validates rather than assumes (lm_head.rs:1542-1680, test :2359)
    if (g.hidden == 0 || g.vocab == 0 || g.max_tokens == 0)
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY, "unsupported LM head geometry {hidden %u, vocab %u, max_tokens %u}: zero dimension",
                    g.hidden, g.vocab, g.max_tokens);
    if (g.hidden % 256 != 0 || g.hidden > 4096)
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY,
                    "unsupported LM head geometry: hidden %u must be a multiple of 256 and at most 4096 (the pass keeps "
                    "eight activation rows in shared memory)", g.hidden);
    if ((uint64_t)g.vocab * g.hidden > (1ull << 40) || g.max_tokens > (1u << 20))
        return fail(XABE_ERR_UNSUPPORTED_GEOMETRY, "unsupported LM head geometry: sanity limit exceeded");
    int n_dev = 0;
    CUDA_TRY(cudaGetDeviceCount(&n_dev));
    if (device < 0 || device >= n_dev) return fail(XABE_ERR_DRIVER, "CUDA driver error: no device %d", device);
    CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop{};
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(XABE_ERR_DRIVER, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    xabe_lm_head* m = new (std::nothrow) xabe_lm_head();
    if (!m) return fail(XABE_ERR_DRIVER, "out of host memory");
    m->g = g;
    m->device = device;
    m->sm_count = prop.multiProcessorCount;
    const size_t n = (size_t)g.max_tokens * g.hidden;
    cudaError_t e = cudaMalloc(&m->x_hi, n * sizeof(__half));
    if (e == cudaSuccess) e = cudaMalloc(&m->x_lo, n * sizeof(__half));
    if (e == cudaSuccess) e = cudaMalloc(&m->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(m->status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost(&m->h_status, sizeof(int));
    if (e != cudaSuccess) {
        xabe_lm_head_destroy(m);
        return fail(XABE_ERR_DRIVER, "CUDA driver error: %s", cudaGetErrorString(e));
    }
    *out = m;
    return XABE_OK;
}

void xabe_lm_head_destroy(xabe_lm_head* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    cudaFree(m->x_hi);
    cudaFree(m->x_lo);
    cudaFree(m->status);
    if (m->h_status) cudaFreeHost(m->h_status);
    delete m;
}

int xabe_lm_head_forward(xabe_lm_head* m, void* stream, xabe_quant_tensor weight, const float* hidden_states,
                         size_t hidden_states_len, int tokens, float* logits, size_t logits_len) {
    if (!m || !weight.dev_bytes || !hidden_states || !logits)
        return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to lm_head_forward");
    const auto& g = m->g;
    if (weight.quant != XABE_QUANT_Q6_K && weight.quant != XABE_QUANT_Q8_0)
        return fail(XABE_ERR_UNSUPPORTED_DENSE_TYPE, "LM head format %d is not one this kernel reads (Q8_0, Q6_K)",
                    (int)weight.quant);
    // lm_head.rs:1703-1800: whole blocks, then exactly vocab x hidden elements
    const size_t bb = weight.quant == XABE_QUANT_Q6_K ? 210 : 34, be = weight.quant == XABE_QUANT_Q6_K ? 256 : 32;
    if (weight.n_bytes % bb != 0)
        return fail(XABE_ERR_RAGGED_WEIGHTS, "LM head weights: %zu bytes is not a whole number of %zu-byte blocks",
                    weight.n_bytes, bb);
    const size_t found = weight.n_bytes / bb * be, want = (size_t)g.vocab * g.hidden;
    if (found != want)
        return fail(XABE_ERR_WRONG_ELEMENT_COUNT, "LM head weights hold %zu elements, the geometry needs %zu", found,
                    want);
    if (tokens < 0 || (uint32_t)tokens > g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u this head was sized for", tokens, g.max_tokens);
    if (hidden_states_len != (size_t)g.max_tokens * g.hidden)
        return fail(XABE_ERR_BUFFER_LENGTH, "hidden_states must hold %zu floats, holds %zu",
                    (size_t)g.max_tokens * g.hidden, hidden_states_len);
    if (logits_len != (size_t)g.max_tokens * g.vocab)
        return fail(XABE_ERR_BUFFER_LENGTH, "logits must hold %zu floats, holds %zu", (size_t)g.max_tokens * g.vocab,
                    logits_len);
    if (tokens == 0) return XABE_OK;
    const int q = weight.quant == XABE_QUANT_Q6_K ? QUANT_Q6K : QUANT_Q8_0;
    const int n_spans = (int)g.hidden / 256;
    const uint64_t row_bytes = (uint64_t)n_spans * span_bytes_of(q);
    HeadLaunch P{};
    P.box_w = rows_box_bytes(q);
    int rc = make_bytes_map(&P.tm_w, weight.dev_bytes, g.vocab, row_bytes, P.box_w);
    if (rc) return rc;
    P.x_hi = m->x_hi;
    P.x_lo = m->x_lo;
    P.logits = logits;
    P.status = m->status;
    P.vocab = (int)g.vocab;
    P.hidden = (int)g.hidden;
    P.tokens = tokens;
    P.stage_bytes = 2u * kRowsGroupRows * P.box_w;
    P.x_stride = g.hidden * 2u + kXRowPadBytes;
    uint32_t smem = 0;
    for (int S = kHeadMaxStages; S >= 2 && !smem; --S) {
        HeadSmem R = head_smem_layout(S, P.stage_bytes, P.x_stride);
        if (R.total <= 226u * 1024u) {
            P.n_stages = S;
            smem = R.total;
        }
    }
    if (!smem) return fail(XABE_ERR_UNSUPPORTED_GEOMETRY, "LM head pass does not fit shared memory");
    cudaStream_t st = (cudaStream_t)stream;
    k_head_split<<<tokens, 256, 0, counted(st)>>>(hidden_states, tokens, (int)g.hidden, m->x_hi, m->x_lo);
    CUDA_TRY(cudaGetLastError());
    const dim3 grid(m->sm_count, (tokens + 7) / 8), block(32 * (1 + kStreamConsumerWarps));
    if (q == QUANT_Q6K) {
        CUDA_TRY(allow_dynamic_smem((const void*)k_head_rows<QUANT_Q6K>, smem));
        k_head_rows<QUANT_Q6K><<<grid, block, smem, counted(st)>>>(P);
    } else {
        CUDA_TRY(allow_dynamic_smem((const void*)k_head_rows<QUANT_Q8_0>, smem));
        k_head_rows<QUANT_Q8_0><<<grid, block, smem, counted(st)>>>(P);
    }
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_lm_head_argmax(xabe_lm_head* m, void* stream, const float* logits, size_t logits_len, int tokens,
                        int32_t* out) {
    if (!m || !logits || !out) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to lm_head_argmax");
    if (tokens < 0 || (uint32_t)tokens > m->g.max_tokens)
        return fail(XABE_ERR_TOO_MANY_TOKENS, "%d tokens exceeds the %u this head was sized for", tokens,
                    m->g.max_tokens);
    if (logits_len != (size_t)m->g.max_tokens * m->g.vocab)
        return fail(XABE_ERR_BUFFER_LENGTH, "logits must hold %zu floats, holds %zu",
                    (size_t)m->g.max_tokens * m->g.vocab, logits_len);
    if (tokens == 0) return XABE_OK;
    k_head_argmax<<<tokens, 1024, 0, counted((cudaStream_t)stream)>>>(logits, (int)m->g.vocab, tokens, out);
    CUDA_TRY(cudaGetLastError());
    return XABE_OK;
}

int xabe_lm_head_device_status(xabe_lm_head* m, void* stream, int* status_out) {
    if (!m || !status_out) return fail(XABE_ERR_INVALID_ARGUMENT, "null argument to lm_head_device_status");
    cudaStream_t st = (cudaStream_t)stream;
    CUDA_TRY(cudaMemcpyAsync(m->h_status, m->status, sizeof(int), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaMemsetAsync(m->status, 0, sizeof(int), st));
    CUDA_TRY(cudaStreamSynchronize(st));
    *status_out = *m->h_status;
    if (*status_out != 0)
        return fail(XABE_ERR_DEVICE_STATUS, "a kernel's bounded wait ran out (device status %d)", *status_out);
    return XABE_OK;
}

}  // extern "C"
