// GGUF v3 container reader behind include/xabe_gguf.h (host code, no CUDA).
//
// Layout, as crates/xabe-gguf/src/file.rs:1-24 states it: magic "GGUF"; u32 version (3 only);
// i64 tensor count; i64 key-value count; the key-value pairs (string key, i32 type tag, value or
// array); the tensor records (string name, u32 dimension count <= 4, i64 dimensions, i32 ggml type,
// u64 offset relative to the data section); the data section at the end of the metadata rounded up
// to `general.alignment` (u32, default 32).  All integers little-endian.
#include "../../include/xabe_gguf.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

struct TypeRow {
    int32_t id;
    uint64_t block, size;
    const char* name;
};
// GgmlType (types.rs:36-95)
const TypeRow kTypes[] = {{0, 1, 4, "f32"},    {1, 1, 2, "f16"},     {2, 32, 18, "q4_0"},   {8, 32, 34, "q8_0"},
                          {12, 256, 144, "q4_K"}, {13, 256, 176, "q5_K"}, {14, 256, 210, "q6_K"}, {30, 1, 2, "bf16"}};
const TypeRow* type_row(int32_t id) {
    for (const TypeRow& r : kTypes)
        if (r.id == id) return &r;
    return nullptr;
}

struct Value {
    int32_t tag = -1;        // scalar tag, or XABE_GGUF_T_ARRAY
    int32_t elem_tag = -1;   // arrays
    uint64_t count = 0;      // arrays
    uint64_t scalar = 0;     // the scalar's bits, widened (f32/f64 by bit pattern)
    std::string str;         // strings
    std::vector<uint8_t> packed;        // numeric / bool array elements, native width
    std::vector<std::string> strings;   // string arrays
};

struct Tensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {0, 0, 0, 0};
    int32_t type = 0;
    uint64_t offset = 0, n_elements = 0, n_bytes = 0;
};

// reader.rs: a bounds-checked little-endian cursor
struct Cursor {
    const uint8_t* data;
    size_t len, pos = 0;
    const char* eof_context = nullptr;
    bool take(size_t n, const char* context, const uint8_t** out) {
        if (n > len - pos) {
            eof_context = context;
            return false;
        }
        *out = data + pos;
        pos += n;
        return true;
    }
    template <typename T>
    bool num(T* v, const char* context) {
        const uint8_t* p;
        if (!take(sizeof(T), context, &p)) return false;
        memcpy(v, p, sizeof(T));  // the hosts this library builds for are little-endian
        return true;
    }
    // 0 ok, 1 eof, 2 invalid utf-8
    int string(std::string* s) {
        uint64_t n;
        if (!num(&n, "string length")) return 1;
        if (n > len - pos) {
            eof_context = "string bytes";
            return 1;
        }
        s->assign((const char*)data + pos, (size_t)n);
        pos += (size_t)n;
        // String::from_utf8 (reader.rs:108): reject malformed sequences
        const unsigned char* b = (const unsigned char*)s->data();
        const size_t m = s->size();
        size_t i = 0;
        while (i < m) {
            const unsigned char c0 = b[i];
            size_t extra;
            uint32_t cp;
            if (c0 < 0x80) { extra = 0; cp = c0; }
            else if ((c0 >> 5) == 0x6) { extra = 1; cp = c0 & 0x1F; }
            else if ((c0 >> 4) == 0xE) { extra = 2; cp = c0 & 0x0F; }
            else if ((c0 >> 3) == 0x1E) { extra = 3; cp = c0 & 0x07; }
            else return 2;
            if (extra > m - i - 1) return 2;
            for (size_t k = 1; k <= extra; ++k) {
                if ((b[i + k] >> 6) != 2) return 2;
                cp = (cp << 6) | (b[i + k] & 0x3F);
            }
            // overlong forms, surrogates and code points past U+10FFFF are not UTF-8
            if ((extra == 1 && cp < 0x80) || (extra == 2 && cp < 0x800) || (extra == 3 && cp < 0x10000) ||
                cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF))
                return 2;
            i += extra + 1;
        }
        return 0;
    }
};

size_t scalar_width(int32_t tag) {
    switch (tag) {
        case XABE_GGUF_T_U8: case XABE_GGUF_T_I8: case XABE_GGUF_T_BOOL: return 1;
        case XABE_GGUF_T_U16: case XABE_GGUF_T_I16: return 2;
        case XABE_GGUF_T_U32: case XABE_GGUF_T_I32: case XABE_GGUF_T_F32: return 4;
        case XABE_GGUF_T_U64: case XABE_GGUF_T_I64: case XABE_GGUF_T_F64: return 8;
        default: return 0;
    }
}

}  // namespace

struct xabe_gguf {
    const uint8_t* bytes = nullptr;
    size_t len = 0;
    bool mapped = false;
    std::vector<uint8_t> owned;
    uint32_t version = 0, alignment = 32;
    uint64_t data_offset = 0;
    std::vector<std::string> keys;  // file order
    std::unordered_map<std::string, Value> metadata;
    std::vector<Tensor> tensors;
    std::unordered_map<std::string, size_t> tensor_index;
};

namespace {

int eof(const Cursor& c) {
    return fail(XABE_GGUF_UNEXPECTED_EOF, "unexpected end of file reading %s at offset %zu", c.eof_context ? c.eof_context : "?", c.pos);
}

// read_typed_value / read_array (file.rs:387-437)
int read_value(Cursor& c, Value* v) {
    int32_t tag;
    if (!c.num(&tag, "i32")) return eof(c);
    v->tag = tag;
    if (tag == XABE_GGUF_T_STRING) {
        int r = c.string(&v->str);
        return r == 1 ? eof(c) : r == 2 ? fail(XABE_GGUF_INVALID_UTF8, "a metadata string is not valid UTF-8") : 0;
    }
    if (tag == XABE_GGUF_T_ARRAY) {
        if (!c.num(&v->elem_tag, "i32")) return eof(c);
        if (!c.num(&v->count, "u64")) return eof(c);
        if (v->elem_tag == XABE_GGUF_T_ARRAY) return fail(XABE_GGUF_NESTED_ARRAY, "nested arrays are not supported");
        if (v->elem_tag == XABE_GGUF_T_STRING) {
            for (uint64_t i = 0; i < v->count; ++i) {
                std::string s;
                int r = c.string(&s);
                if (r == 1) return eof(c);
                if (r == 2) return fail(XABE_GGUF_INVALID_UTF8, "a metadata string is not valid UTF-8");
                v->strings.push_back(std::move(s));
            }
            return 0;
        }
        const size_t w = scalar_width(v->elem_tag);
        if (!w) return fail(XABE_GGUF_UNKNOWN_VALUE_TYPE, "unknown metadata value type %d", (int)v->elem_tag);
        if (v->count > (c.len - c.pos) / w) {  // an element count the file cannot hold
            c.eof_context = "array elements";
            c.pos = c.len;
            return eof(c);
        }
        const uint8_t* p;
        if (!c.take((size_t)v->count * w, "array elements", &p)) return eof(c);
        v->packed.assign(p, p + (size_t)v->count * w);
        if (v->elem_tag == XABE_GGUF_T_BOOL)
            for (uint8_t& b : v->packed) b = b != 0;  // bool_ (reader.rs:94-96): any non-zero byte is true
        return 0;
    }
    const size_t w = scalar_width(tag);
    if (!w) return fail(XABE_GGUF_UNKNOWN_VALUE_TYPE, "unknown metadata value type %d", (int)tag);
    const uint8_t* p;
    static const char* const names[] = {"u8", "i8", "u16", "i16", "u32", "i32", "f32", "i8", "", "", "u64", "i64", "f64"};
    if (!c.take(w, names[tag], &p)) return eof(c);
    memcpy(&v->scalar, p, w);
    return 0;
}

// parse + from_backing (file.rs:84-124, 273-375)
int parse(xabe_gguf* f) {
    Cursor c{f->bytes, f->len};
    const uint8_t* magic;
    if (!c.take(4, "magic", &magic)) return eof(c);
    if (memcmp(magic, "GGUF", 4) != 0)
        return fail(XABE_GGUF_BAD_MAGIC, "bad magic %02x %02x %02x %02x", magic[0], magic[1], magic[2], magic[3]);
    if (!c.num(&f->version, "u32")) return eof(c);
    if (f->version != 3) return fail(XABE_GGUF_UNSUPPORTED_VERSION, "unsupported GGUF version %u", f->version);
    int64_t n_tensors, n_kv;
    if (!c.num(&n_tensors, "i64")) return eof(c);
    if (n_tensors < 0) return fail(XABE_GGUF_NEGATIVE_COUNT, "negative tensor count %lld", (long long)n_tensors);
    if (!c.num(&n_kv, "i64")) return eof(c);
    if (n_kv < 0) return fail(XABE_GGUF_NEGATIVE_COUNT, "negative kv count %lld", (long long)n_kv);
    for (int64_t i = 0; i < n_kv; ++i) {
        std::string key;
        int r = c.string(&key);
        if (r == 1) return eof(c);
        if (r == 2) return fail(XABE_GGUF_INVALID_UTF8, "a metadata key is not valid UTF-8");
        Value v;
        if (int rc = read_value(c, &v)) return rc;
        if (!f->metadata.emplace(key, std::move(v)).second)
            return fail(XABE_GGUF_DUPLICATE_KEY, "duplicate metadata key %s", key.c_str());
        f->keys.push_back(key);
    }
    auto al = f->metadata.find("general.alignment");
    if (al != f->metadata.end()) {
        if (al->second.tag != XABE_GGUF_T_U32) return fail(XABE_GGUF_BAD_ALIGNMENT_TYPE, "general.alignment is not a u32");
        f->alignment = (uint32_t)al->second.scalar;
    }
    if (f->alignment == 0 || (f->alignment & (f->alignment - 1)) != 0)
        return fail(XABE_GGUF_BAD_ALIGNMENT, "general.alignment %u is not a power of two", f->alignment);
    for (int64_t i = 0; i < n_tensors; ++i) {
        Tensor t;
        int r = c.string(&t.name);
        if (r == 1) return eof(c);
        if (r == 2) return fail(XABE_GGUF_INVALID_UTF8, "a tensor name is not valid UTF-8");
        if (f->tensor_index.count(t.name)) return fail(XABE_GGUF_DUPLICATE_TENSOR, "duplicate tensor %s", t.name.c_str());
        if (!c.num(&t.n_dims, "u32")) return eof(c);
        if (t.n_dims > 4)
            return fail(XABE_GGUF_TOO_MANY_DIMENSIONS, "tensor %s has %u dimensions", t.name.c_str(), t.n_dims);
        t.n_elements = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            int64_t v;
            if (!c.num(&v, "i64")) return eof(c);
            if (v <= 0) return fail(XABE_GGUF_ZERO_DIMENSION, "tensor %s has a zero or negative dimension", t.name.c_str());
            t.dims[d] = (uint64_t)v;
            t.n_elements *= (uint64_t)v;
        }
        if (!c.num(&t.type, "i32")) return eof(c);
        const TypeRow* row = type_row(t.type);
        if (!row) return fail(XABE_GGUF_UNSUPPORTED_GGML_TYPE, "unsupported ggml type %d", (int)t.type);
        if (!c.num(&t.offset, "u64")) return eof(c);
        if (t.n_elements % row->block != 0)
            return fail(XABE_GGUF_UNALIGNED_ELEMENT_COUNT, "tensor %s: %llu elements of %s is not a whole number of %llu-element blocks",
                        t.name.c_str(), (unsigned long long)t.n_elements, row->name, (unsigned long long)row->block);
        t.n_bytes = t.n_elements / row->block * row->size;
        f->tensor_index.emplace(t.name, f->tensors.size());
        f->tensors.push_back(std::move(t));
    }
    const uint64_t a = f->alignment;
    f->data_offset = ((uint64_t)c.pos + a - 1) & ~(a - 1);
    for (const Tensor& t : f->tensors) {
        uint64_t start, end;
        if (__builtin_add_overflow(f->data_offset, t.offset, &start) || __builtin_add_overflow(start, t.n_bytes, &end))
            return fail(XABE_GGUF_OFFSET_OVERFLOW, "tensor %s: offset overflows", t.name.c_str());
        if (end > (uint64_t)f->len)
            return fail(XABE_GGUF_TENSOR_OUT_OF_BOUNDS, "tensor %s spans [%llu, %llu) but the file holds %zu bytes", t.name.c_str(),
                        (unsigned long long)start, (unsigned long long)end, f->len);
    }
    return 0;
}

void fill(const xabe_gguf* f, const Tensor& t, xabe_gguf_tensor* out) {
    out->name = t.name.c_str();
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = t.dims[d];
    out->ggml_type = t.type;
    out->offset = t.offset;
    out->n_elements = t.n_elements;
    out->n_bytes = t.n_bytes;
    out->data = f->bytes + f->data_offset + t.offset;
}

const Value* find(const xabe_gguf* f, const char* key, int* rc) {
    if (!f || !key) {
        *rc = fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
        return nullptr;
    }
    auto it = f->metadata.find(key);
    if (it == f->metadata.end()) {
        *rc = fail(XABE_GGUF_NOT_FOUND, "no metadata key %s", key);
        return nullptr;
    }
    return &it->second;
}

int scalar_of(const xabe_gguf* f, const char* key, int32_t tag, void* out, size_t w) {
    int rc = 0;
    const Value* v = find(f, key, &rc);
    if (!v) return rc;
    if (v->tag != tag) return fail(XABE_GGUF_TYPE_MISMATCH, "metadata key %s has type %d, not %d", key, (int)v->tag, (int)tag);
    memcpy(out, &v->scalar, w);
    return 0;
}

}  // namespace

extern "C" {

const char* xabe_gguf_last_error(void) { return g_error; }

uint64_t xabe_ggml_block_size(int32_t t) {
    const TypeRow* r = type_row(t);
    return r ? r->block : 0;
}
uint64_t xabe_ggml_type_size(int32_t t) {
    const TypeRow* r = type_row(t);
    return r ? r->size : 0;
}
const char* xabe_ggml_type_name(int32_t t) {
    const TypeRow* r = type_row(t);
    return r ? r->name : nullptr;
}
int xabe_ggml_bytes_for_elements(int32_t t, uint64_t n, uint64_t* out) {
    const TypeRow* r = type_row(t);
    if (!r) return fail(XABE_GGUF_UNSUPPORTED_GGML_TYPE, "unsupported ggml type %d", (int)t);
    if (!out) return fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
    if (n % r->block != 0)
        return fail(XABE_GGUF_UNALIGNED_ELEMENT_COUNT, "%llu elements of %s is not a whole number of %llu-element blocks",
                    (unsigned long long)n, r->name, (unsigned long long)r->block);
    *out = n / r->block * r->size;
    return 0;
}

void xabe_gguf_close(xabe_gguf* f) {
    if (!f) return;
    if (f->mapped && f->bytes) munmap((void*)f->bytes, f->len);
    delete f;
}

int xabe_gguf_from_bytes(const void* bytes, size_t n, xabe_gguf** out) {
    if (!out || (!bytes && n)) return fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    xabe_gguf* f = new (std::nothrow) xabe_gguf();
    if (!f) return fail(XABE_GGUF_IO, "out of memory");
    f->owned.assign((const uint8_t*)bytes, (const uint8_t*)bytes + n);
    f->bytes = f->owned.data();
    f->len = n;
    if (int rc = parse(f)) {
        xabe_gguf_close(f);
        return rc;
    }
    *out = f;
    return 0;
}

int xabe_gguf_open(const char* path, xabe_gguf** out) {
    if (!out || !path) return fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail(XABE_GGUF_IO, "%s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0) {
        int e = errno;
        close(fd);
        return fail(XABE_GGUF_IO, "%s: %s", path, strerror(e));
    }
    xabe_gguf* f = new (std::nothrow) xabe_gguf();
    if (!f) {
        close(fd);
        return fail(XABE_GGUF_IO, "out of memory");
    }
    f->len = (size_t)st.st_size;
    if (f->len) {
        void* p = mmap(nullptr, f->len, PROT_READ, MAP_PRIVATE, fd, 0);
        if (p == MAP_FAILED) {
            int e = errno;
            close(fd);
            delete f;
            return fail(XABE_GGUF_IO, "%s: mmap: %s", path, strerror(e));
        }
        f->bytes = (const uint8_t*)p;
        f->mapped = true;
    }
    close(fd);
    if (int rc = parse(f)) {
        xabe_gguf_close(f);
        return rc;
    }
    *out = f;
    return 0;
}

uint32_t xabe_gguf_version(const xabe_gguf* f) { return f ? f->version : 0; }
uint32_t xabe_gguf_alignment(const xabe_gguf* f) { return f ? f->alignment : 0; }
uint64_t xabe_gguf_n_kv(const xabe_gguf* f) { return f ? f->metadata.size() : 0; }
uint64_t xabe_gguf_n_tensors(const xabe_gguf* f) { return f ? f->tensors.size() : 0; }
uint64_t xabe_gguf_data_offset(const xabe_gguf* f) { return f ? f->data_offset : 0; }

int xabe_gguf_tensor_at(const xabe_gguf* f, uint64_t index, xabe_gguf_tensor* out) {
    if (!f || !out) return fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
    if (index >= f->tensors.size()) return fail(XABE_GGUF_NOT_FOUND, "no tensor %llu", (unsigned long long)index);
    fill(f, f->tensors[(size_t)index], out);
    return 0;
}

int xabe_gguf_find_tensor(const xabe_gguf* f, const char* name, xabe_gguf_tensor* out) {
    if (!f || !name || !out) return fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
    auto it = f->tensor_index.find(name);
    if (it == f->tensor_index.end()) return fail(XABE_GGUF_NOT_FOUND, "no tensor %s", name);
    fill(f, f->tensors[it->second], out);
    return 0;
}

int xabe_gguf_key_at(const xabe_gguf* f, uint64_t index, const char** key, int32_t* type_tag) {
    if (!f || !key) return fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
    if (index >= f->keys.size()) return fail(XABE_GGUF_NOT_FOUND, "no key %llu", (unsigned long long)index);
    *key = f->keys[(size_t)index].c_str();
    if (type_tag) *type_tag = f->metadata.at(f->keys[(size_t)index]).tag;
    return 0;
}

int xabe_gguf_get_u32(const xabe_gguf* f, const char* key, uint32_t* out) { return scalar_of(f, key, XABE_GGUF_T_U32, out, 4); }
int xabe_gguf_get_u64(const xabe_gguf* f, const char* key, uint64_t* out) { return scalar_of(f, key, XABE_GGUF_T_U64, out, 8); }
int xabe_gguf_get_f32(const xabe_gguf* f, const char* key, float* out) { return scalar_of(f, key, XABE_GGUF_T_F32, out, 4); }
int xabe_gguf_get_bool(const xabe_gguf* f, const char* key, int* out) {
    uint8_t b = 0;
    int rc = scalar_of(f, key, XABE_GGUF_T_BOOL, &b, 1);
    if (!rc) *out = b != 0;
    return rc;
}

int xabe_gguf_get_str(const xabe_gguf* f, const char* key, const char** out, uint64_t* len) {
    int rc = 0;
    const Value* v = find(f, key, &rc);
    if (!v) return rc;
    if (v->tag != XABE_GGUF_T_STRING) return fail(XABE_GGUF_TYPE_MISMATCH, "metadata key %s is not a string", key);
    *out = v->str.c_str();
    if (len) *len = v->str.size();
    return 0;
}

int xabe_gguf_get_array(const xabe_gguf* f, const char* key, int32_t* elem_tag, uint64_t* count, const void** data) {
    int rc = 0;
    const Value* v = find(f, key, &rc);
    if (!v) return rc;
    if (v->tag != XABE_GGUF_T_ARRAY) return fail(XABE_GGUF_TYPE_MISMATCH, "metadata key %s is not an array", key);
    if (elem_tag) *elem_tag = v->elem_tag;
    if (count) *count = v->count;
    if (data) *data = v->elem_tag == XABE_GGUF_T_STRING ? nullptr : (const void*)v->packed.data();
    return 0;
}

int xabe_gguf_get_array_str(const xabe_gguf* f, const char* key, uint64_t index, const char** out, uint64_t* len) {
    int rc = 0;
    const Value* v = find(f, key, &rc);
    if (!v) return rc;
    if (v->tag != XABE_GGUF_T_ARRAY || v->elem_tag != XABE_GGUF_T_STRING)
        return fail(XABE_GGUF_TYPE_MISMATCH, "metadata key %s is not a string array", key);
    if (index >= v->strings.size()) return fail(XABE_GGUF_NOT_FOUND, "%s has no element %llu", key, (unsigned long long)index);
    *out = v->strings[(size_t)index].c_str();
    if (len) *len = v->strings[(size_t)index].size();
    return 0;
}

int xabe_gguf_moe_layer_tensors(const xabe_gguf* f, uint32_t layer, uint64_t hidden, uint64_t ff, uint64_t experts,
                                xabe_gguf_moe_layer* out) {
    if (!f || !out) return fail(XABE_GGUF_INVALID_ARGUMENT, "null argument");
    struct Want {
        const char* suffix;
        xabe_gguf_tensor* dst;
        uint32_t n_dims;
        uint64_t dims[3];
    };
    // Role::suffix (weights.rs:173-212); shapes in ggml order (weights.rs:403-413)
    const Want wants[] = {
        {"post_attention_norm.weight", &out->post_norm, 1, {hidden, 0, 0}},
        {"ffn_gate_inp.weight", &out->router, 2, {hidden, experts, 0}},
        {"ffn_gate_exps.weight", &out->gate_exps, 3, {hidden, ff, experts}},
        {"ffn_up_exps.weight", &out->up_exps, 3, {hidden, ff, experts}},
        {"ffn_down_exps.weight", &out->down_exps, 3, {ff, hidden, experts}},
        {"ffn_gate_inp_shexp.weight", &out->shared_gate_inp, 1, {hidden, 0, 0}},
        {"ffn_gate_shexp.weight", &out->shared_gate, 2, {hidden, ff, 0}},
        {"ffn_up_shexp.weight", &out->shared_up, 2, {hidden, ff, 0}},
        {"ffn_down_shexp.weight", &out->shared_down, 2, {ff, hidden, 0}},
    };
    for (const Want& w : wants) {
        char name[96];
        snprintf(name, sizeof name, "blk.%u.%s", layer, w.suffix);
        auto it = f->tensor_index.find(name);
        if (it == f->tensor_index.end()) return fail(XABE_GGUF_SCHEMA, "missing tensor %s", name);
        const Tensor& t = f->tensors[it->second];
        bool ok = t.n_dims == w.n_dims;
        for (uint32_t d = 0; ok && d < w.n_dims; ++d) ok = t.dims[d] == w.dims[d];
        if (!ok)
            return fail(XABE_GGUF_SCHEMA, "tensor %s has shape [%llu, %llu, %llu] (%u dims), expected [%llu, %llu, %llu] (%u dims)", name,
                        (unsigned long long)t.dims[0], (unsigned long long)t.dims[1], (unsigned long long)t.dims[2], t.n_dims,
                        (unsigned long long)w.dims[0], (unsigned long long)w.dims[1], (unsigned long long)w.dims[2], w.n_dims);
        fill(f, t, w.dst);
    }
    return 0;
}

}  // extern "C"
