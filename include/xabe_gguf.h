/*
 * xabe_gguf.h -- C ABI of the GGUF v3 container reader (libxabe_gguf.so, host code only).
 *
 * Mirrors `xabe_gguf::GgufFile` (crates/xabe-gguf/src/file.rs) and the MoE part of
 * the weight schema of `xabe-model` (crates/xabe-model/src/weights.rs:173-212,
 * 403-420): it hands the kernel library tensors as the bytes of the file, in
 * file layout, which is the layout libxabe_moe_sm100.so reads.  Paths cited are
 * relative to the reference project root.
 *
 * Every call returns an `xabe_gguf_status`; the thread-local text of the last
 * failure is available from xabe_gguf_last_error().  Nothing throws.
 */
#ifndef XABE_GGUF_H
#define XABE_GGUF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GgufError variants (crates/xabe-gguf/src/error.rs:14-107) */
typedef enum xabe_gguf_status {
    XABE_GGUF_OK = 0,
    XABE_GGUF_BAD_MAGIC = 1,
    XABE_GGUF_UNSUPPORTED_VERSION = 2,
    XABE_GGUF_UNEXPECTED_EOF = 3,
    XABE_GGUF_NEGATIVE_COUNT = 4,
    XABE_GGUF_DUPLICATE_KEY = 5,
    XABE_GGUF_UNKNOWN_VALUE_TYPE = 6,
    XABE_GGUF_NESTED_ARRAY = 7,
    XABE_GGUF_BAD_ALIGNMENT_TYPE = 8,
    XABE_GGUF_BAD_ALIGNMENT = 9,
    XABE_GGUF_TOO_MANY_DIMENSIONS = 10,
    XABE_GGUF_ZERO_DIMENSION = 11,
    XABE_GGUF_DUPLICATE_TENSOR = 12,
    XABE_GGUF_UNSUPPORTED_GGML_TYPE = 13,
    XABE_GGUF_UNALIGNED_ELEMENT_COUNT = 14,
    XABE_GGUF_OFFSET_OVERFLOW = 15,
    XABE_GGUF_TENSOR_OUT_OF_BOUNDS = 16,
    XABE_GGUF_IO = 17,
    XABE_GGUF_INVALID_UTF8 = 18,
    /* lookups: the reference returns None for these */
    XABE_GGUF_NOT_FOUND = 19,
    XABE_GGUF_TYPE_MISMATCH = 20,
    XABE_GGUF_INVALID_ARGUMENT = 21,
    /* schema (crates/xabe-model/src/weights.rs): a tensor of the layer is missing or has the wrong shape */
    XABE_GGUF_SCHEMA = 22
} xabe_gguf_status;

/* GgmlType (crates/xabe-gguf/src/types.rs:36-60): the ids of `enum ggml_type`. */
#define XABE_GGML_F32 0
#define XABE_GGML_F16 1
#define XABE_GGML_Q4_0 2
#define XABE_GGML_Q8_0 8
#define XABE_GGML_Q4_K 12
#define XABE_GGML_Q5_K 13
#define XABE_GGML_Q6_K 14
#define XABE_GGML_BF16 30

/* GgufValue type tags (file.rs:387-408) */
#define XABE_GGUF_T_U8 0
#define XABE_GGUF_T_I8 1
#define XABE_GGUF_T_U16 2
#define XABE_GGUF_T_I16 3
#define XABE_GGUF_T_U32 4
#define XABE_GGUF_T_I32 5
#define XABE_GGUF_T_F32 6
#define XABE_GGUF_T_BOOL 7
#define XABE_GGUF_T_STRING 8
#define XABE_GGUF_T_ARRAY 9
#define XABE_GGUF_T_U64 10
#define XABE_GGUF_T_I64 11
#define XABE_GGUF_T_F64 12

/* TensorInfo (crates/xabe-gguf/src/tensor.rs) plus where its bytes are. */
typedef struct xabe_gguf_tensor {
    const char* name;     /* owned by the handle */
    uint32_t n_dims;      /* <= 4 */
    uint64_t dims[4];     /* ggml order: dims[0] is the contiguous one */
    int32_t ggml_type;
    uint64_t offset;      /* relative to the data section */
    uint64_t n_elements;
    uint64_t n_bytes;
    const void* data;     /* host pointer into the mapping (or the copied buffer) */
} xabe_gguf_tensor;

typedef struct xabe_gguf xabe_gguf;

const char* xabe_gguf_last_error(void);

/* GgmlType::{block_size, type_size, name, bytes_for_elements} (types.rs:62-117).  0 / NULL for an
 * id that is not in the table; bytes_for_elements fails on a partial block. */
uint64_t xabe_ggml_block_size(int32_t ggml_type);
uint64_t xabe_ggml_type_size(int32_t ggml_type);
const char* xabe_ggml_type_name(int32_t ggml_type);
int xabe_ggml_bytes_for_elements(int32_t ggml_type, uint64_t n, uint64_t* out);

/* GgufFile::open (file.rs:74-78, memory-mapped) and ::from_bytes (:80-82, the bytes are copied). */
int xabe_gguf_open(const char* path, xabe_gguf** out);
int xabe_gguf_from_bytes(const void* bytes, size_t n, xabe_gguf** out);
void xabe_gguf_close(xabe_gguf* f);

/* version / alignment / n_kv / n_tensors (file.rs:126-140); data_offset = start of the data section */
uint32_t xabe_gguf_version(const xabe_gguf* f);
uint32_t xabe_gguf_alignment(const xabe_gguf* f);
uint64_t xabe_gguf_n_kv(const xabe_gguf* f);
uint64_t xabe_gguf_n_tensors(const xabe_gguf* f);
uint64_t xabe_gguf_data_offset(const xabe_gguf* f);

/* tensors()[index], tensor(name) and tensor_bytes(name) (file.rs:142-155) */
int xabe_gguf_tensor_at(const xabe_gguf* f, uint64_t index, xabe_gguf_tensor* out);
int xabe_gguf_find_tensor(const xabe_gguf* f, const char* name, xabe_gguf_tensor* out);

/* Metadata (file.rs:157-260).  A key of another type is TYPE_MISMATCH, never coerced. */
int xabe_gguf_key_at(const xabe_gguf* f, uint64_t index, const char** key, int32_t* type_tag);
int xabe_gguf_get_u32(const xabe_gguf* f, const char* key, uint32_t* out);
int xabe_gguf_get_u64(const xabe_gguf* f, const char* key, uint64_t* out);
int xabe_gguf_get_f32(const xabe_gguf* f, const char* key, float* out);
int xabe_gguf_get_bool(const xabe_gguf* f, const char* key, int* out);
int xabe_gguf_get_str(const xabe_gguf* f, const char* key, const char** out, uint64_t* len);
/* Arrays: element tag and count; numeric and bool elements as a packed host array (bool = 1 byte),
 * strings one at a time. */
int xabe_gguf_get_array(const xabe_gguf* f, const char* key, int32_t* elem_tag, uint64_t* count, const void** data);
int xabe_gguf_get_array_str(const xabe_gguf* f, const char* key, uint64_t index, const char** out, uint64_t* len);

/* The tensors of one MoE layer by role (Role::suffix, weights.rs:173-212; shapes :403-413),
 * `blk.<layer>.<suffix>`, checked against the geometry: router [hidden, experts]; gate/up
 * [hidden, ff, experts]; down [ff, hidden, experts]; shared gate input [hidden]; shared gate/up
 * [hidden, ff]; shared down [ff, hidden]; post-mixer norm [hidden]. */
typedef struct xabe_gguf_moe_layer {
    xabe_gguf_tensor post_norm;        /* post_attention_norm.weight */
    xabe_gguf_tensor router;           /* ffn_gate_inp.weight */
    xabe_gguf_tensor gate_exps;        /* ffn_gate_exps.weight */
    xabe_gguf_tensor up_exps;          /* ffn_up_exps.weight */
    xabe_gguf_tensor down_exps;        /* ffn_down_exps.weight */
    xabe_gguf_tensor shared_gate_inp;  /* ffn_gate_inp_shexp.weight */
    xabe_gguf_tensor shared_gate;      /* ffn_gate_shexp.weight */
    xabe_gguf_tensor shared_up;        /* ffn_up_shexp.weight */
    xabe_gguf_tensor shared_down;      /* ffn_down_shexp.weight */
} xabe_gguf_moe_layer;

int xabe_gguf_moe_layer_tensors(const xabe_gguf* f, uint32_t layer, uint64_t hidden, uint64_t ff, uint64_t experts,
                                xabe_gguf_moe_layer* out);

#ifdef __cplusplus
}
#endif
#endif /* XABE_GGUF_H */
