// GGUF container reader and the decoder's file loader.
//
// Mirrors the reference's parser (crates/rnb-loader/src/gguf/parser.rs:244-404: magic, versions 2
// and 3, little-endian only, u64 counts, KV metadata, tensor infos with innermost-first dims,
// `general.alignment`, data section at the next aligned offset; gguf/types.rs for the type ids)
// and its Llama-family metadata extraction (crates/rnb-loader/src/arch/mod.rs:304-560) and tensor
// names (crates/rnb-loader/src/arch/llama.rs:33-155).  The file is mapped read-only; tensor data
// is never copied on the host: the decoder uploads straight from the mapped pages, optionally
// pinned for DMA first (rnb_b200_register_host_range).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <set>
#include <string>
#include <vector>

#include "state.hpp"

using namespace rnb;

namespace {

constexpr size_t MAX_STRING_LENGTH = 64u * 1024 * 1024;
constexpr size_t MAX_ARRAY_ELEMENTS = 4u * 1024 * 1024;
constexpr size_t MAX_ARRAY_NESTING = 64;
constexpr size_t MAX_METADATA_KEY_LENGTH = 65535;
constexpr size_t MAX_TENSOR_NAME_LENGTH = 64;
constexpr size_t MIN_METADATA_RECORD_BYTES = 13;
constexpr size_t MIN_TENSOR_INFO_BYTES = 24;

struct Value {
    uint32_t type = 0;          // GGUF value type 0..12
    uint64_t u = 0;             // integers and bool (sign-extended for signed types)
    double f = 0.0;             // f32 / f64
    std::string s;              // string
    uint32_t elem_type = 0;     // arrays: element type, and the scalar elements
    std::vector<Value> items;
};

struct Tensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};   // row-major (outermost first), as the reference normalises them
    uint32_t type = 0;
    uint64_t offset = 0;
};

struct ParseError {
    int code;
    std::string msg;
};

struct Reader {
    const uint8_t *data;
    size_t len, pos = 0;
    size_t remaining() const { return len - pos; }
    const uint8_t *bytes(size_t n) {
        if (remaining() < n) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(pos) + ": need " + std::to_string(n) + " bytes, only " + std::to_string(remaining()) + " remain"};
        const uint8_t *p = data + pos;
        pos += n;
        return p;
    }
    template <class T>
    T le() {
        const uint8_t *p = bytes(sizeof(T));
        T v;
        memcpy(&v, p, sizeof(T));   // the hosts this library runs on are little-endian
        return v;
    }
    std::string str() {
        const uint64_t n = le<uint64_t>();
        if (n > MAX_STRING_LENGTH) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(pos - 8) + ": string length " + std::to_string(n) + " exceeds maximum supported length " + std::to_string(MAX_STRING_LENGTH)};
        const uint8_t *p = bytes((size_t)n);
        return std::string(reinterpret_cast<const char *>(p), (size_t)n);
    }
};

Value read_value(Reader &r, uint32_t type, size_t depth) {
    if (type > 12) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos) + ": unknown GGUF value type: " + std::to_string(type)};
    if (depth > MAX_ARRAY_NESTING) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos) + ": GGUF array nesting exceeds 64 levels"};
    Value v;
    v.type = type;
    switch (type) {
    case 0: v.u = r.le<uint8_t>(); break;
    case 1: v.u = (uint64_t)(int64_t)r.le<int8_t>(); break;
    case 2: v.u = r.le<uint16_t>(); break;
    case 3: v.u = (uint64_t)(int64_t)r.le<int16_t>(); break;
    case 4: v.u = r.le<uint32_t>(); break;
    case 5: v.u = (uint64_t)(int64_t)r.le<int32_t>(); break;
    case 6: v.f = r.le<float>(); break;
    case 7: {
        const size_t at = r.pos;
        const uint8_t b = r.le<uint8_t>();
        if (b > 1) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(at) + ": invalid GGUF boolean value " + std::to_string(b) + "; expected 0 or 1"};
        v.u = b;
        break;
    }
    case 8: v.s = r.str(); break;
    case 9: {
        v.elem_type = r.le<uint32_t>();
        if (v.elem_type > 12) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - 4) + ": unknown GGUF value type: " + std::to_string(v.elem_type)};
        const uint64_t count = r.le<uint64_t>();
        if (count > MAX_ARRAY_ELEMENTS) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - 8) + ": array element count " + std::to_string(count) + " exceeds maximum " + std::to_string(MAX_ARRAY_ELEMENTS)};
        if (count > r.remaining()) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos) + ": array element count " + std::to_string(count) + " exceeds " + std::to_string(r.remaining()) + " remaining bytes"};
        v.items.reserve((size_t)count);
        for (uint64_t i = 0; i < count; i++) v.items.push_back(read_value(r, v.elem_type, depth + 1));
        break;
    }
    case 10: v.u = r.le<uint64_t>(); break;
    case 11: v.u = (uint64_t)r.le<int64_t>(); break;
    case 12: v.f = r.le<double>(); break;
    }
    return v;
}

// bytes per block and elements per block of the GGML types whose layout is fixed and public
// (gguf/types.rs lists the ids; sizes are GGML's block structs)
bool type_layout(uint32_t t, size_t *block_bytes, size_t *block_elems) {
    struct L {
        uint32_t id;
        size_t bytes, elems;
    };
    static const L table[] = {{0, 4, 1},    {1, 2, 1},     {30, 2, 1},    {2, 18, 32},   {3, 20, 32},   {6, 22, 32},   {7, 24, 32},
                              {8, 34, 32},  {9, 36, 32},   {10, 84, 256}, {11, 110, 256}, {12, 144, 256}, {13, 176, 256}, {14, 210, 256},
                              {15, 292, 256}, {24, 1, 1},  {25, 2, 1},    {26, 4, 1},    {27, 8, 1},    {28, 8, 1}};
    for (const L &l : table)
        if (l.id == t) {
            *block_bytes = l.bytes;
            *block_elems = l.elems;
            return true;
        }
    return false;
}
bool known_type_id(uint32_t t) {
    static const uint32_t ids[] = {0, 1, 30, 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 29, 34, 35, 39, 40, 41, 42, 26, 24, 25, 27, 28};
    for (uint32_t id : ids)
        if (id == t) return true;
    return false;
}

}  // namespace

struct rnb_b200_gguf {
    const uint8_t *data = nullptr;
    size_t len = 0;
    void *map = nullptr;    // non-null when this object owns an mmap
    size_t map_len = 0;
    uint32_t version = 0;
    uint64_t alignment = 32, data_start = 0;
    std::vector<std::pair<std::string, Value>> metadata;
    std::vector<Tensor> tensors;
    const Value *find(const std::string &key) const {
        for (const auto &kv : metadata)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    const Tensor *tensor(const std::string &name) const {
        for (const Tensor &t : tensors)
            if (t.name == name) return &t;
        return nullptr;
    }
};

static void parse_into(rnb_b200_gguf *g) {
    Reader r{g->data, g->len};
    const uint8_t *magic = r.bytes(4);
    if (memcmp(magic, "GGUF", 4) != 0) throw ParseError{RNB_B200_VALIDATION_FAILED, "invalid GGUF magic"};
    const size_t version_offset = r.pos;
    const uint8_t *vb = r.bytes(4);
    const uint32_t version = (uint32_t)vb[0] | ((uint32_t)vb[1] << 8) | ((uint32_t)vb[2] << 16) | ((uint32_t)vb[3] << 24);
    if (version != 2 && version != 3) {
        const uint32_t be = (uint32_t)vb[3] | ((uint32_t)vb[2] << 8) | ((uint32_t)vb[1] << 16) | ((uint32_t)vb[0] << 24);
        if (be == 2 || be == 3)
            throw ParseError{RNB_B200_UNSUPPORTED, "parse error at offset " + std::to_string(version_offset) + ": big-endian GGUF is not supported by the mmap tensor runtime"};
        throw ParseError{RNB_B200_UNSUPPORTED, "unsupported GGUF version " + std::to_string(version)};
    }
    g->version = version;
    const uint64_t tensor_count = r.le<uint64_t>(), kv_count = r.le<uint64_t>();
    // both counts must at least fit as minimal records in what is left of the file
    const unsigned __int128 need = (unsigned __int128)kv_count * MIN_METADATA_RECORD_BYTES + (unsigned __int128)tensor_count * MIN_TENSOR_INFO_BYTES;
    if (need > (unsigned __int128)r.remaining())
        throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos) + ": tensor count " + std::to_string(tensor_count) + " and metadata count " + std::to_string(kv_count) + " cannot fit in " + std::to_string(r.remaining()) + " remaining bytes"};
    std::set<std::string> keys;
    g->metadata.reserve((size_t)kv_count);
    for (uint64_t i = 0; i < kv_count; i++) {
        std::string key = r.str();
        bool ascii = !key.empty() && key.size() <= MAX_METADATA_KEY_LENGTH;
        for (unsigned char c : key) ascii = ascii && c < 0x80;
        if (!ascii) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - key.size()) + ": metadata key must be non-empty ASCII and at most 65535 bytes"};
        if (!keys.insert(key).second) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - key.size()) + ": duplicate metadata key '" + key + "'"};
        const uint32_t vt = r.le<uint32_t>();
        g->metadata.emplace_back(std::move(key), read_value(r, vt, 0));
    }
    // general.alignment: a non-negative integer that is a power of two; 32 when absent
    if (const Value *a = g->find("general.alignment")) {
        const bool is_int = a->type <= 5 || a->type == 10 || a->type == 11;
        const bool negative = (a->type == 1 || a->type == 3 || a->type == 5 || a->type == 11) && (int64_t)a->u < 0;
        if (!is_int || negative) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset 0: general.alignment must be a non-negative integer fitting usize"};
        if (a->u == 0 || (a->u & (a->u - 1)) != 0) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset 0: general.alignment " + std::to_string(a->u) + " must be a positive power of two"};
        g->alignment = a->u;
    }
    std::set<std::string> names;
    g->tensors.reserve((size_t)tensor_count);
    for (uint64_t i = 0; i < tensor_count; i++) {
        Tensor t;
        t.name = r.str();
        if (t.name.size() >= MAX_TENSOR_NAME_LENGTH)
            throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - t.name.size()) + ": tensor name is " + std::to_string(t.name.size()) + " bytes; GGML requires fewer than 64"};
        if (!names.insert(t.name).second) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - t.name.size()) + ": duplicate tensor name '" + t.name + "'"};
        t.n_dims = r.le<uint32_t>();
        if (t.n_dims > 4) throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - 4) + ": tensor '" + t.name + "' has " + std::to_string(t.n_dims) + " dimensions; GGUF supports at most 4"};
        uint64_t inner_first[4] = {1, 1, 1, 1};
        for (uint32_t d = 0; d < t.n_dims; d++) inner_first[d] = r.le<uint64_t>();
        for (uint32_t d = 0; d < t.n_dims; d++) t.dims[d] = inner_first[t.n_dims - 1 - d];   // stored innermost first
        t.type = r.le<uint32_t>();
        if (!known_type_id(t.type)) throw ParseError{RNB_B200_UNSUPPORTED, "unsupported GGML type " + std::to_string(t.type)};
        t.offset = r.le<uint64_t>();
        if (t.offset % g->alignment != 0)
            throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos - 8) + ": tensor '" + t.name + "' offset " + std::to_string(t.offset) + " is not aligned to " + std::to_string(g->alignment) + " bytes"};
        g->tensors.push_back(std::move(t));
    }
    const uint64_t rem = r.pos % g->alignment;
    g->data_start = r.pos + (g->alignment - rem) % g->alignment;
    if (tensor_count > 0 && g->data_start > g->len)
        throw ParseError{RNB_B200_VALIDATION_FAILED, "parse error at offset " + std::to_string(r.pos) + ": tensor data starts at " + std::to_string(g->data_start) + ", beyond file length " + std::to_string(g->len)};
}

static int parse_or_fail(rnb_b200_gguf *g, rnb_b200_gguf **out) {
    try {
        parse_into(g);
    } catch (const ParseError &e) {
        if (g->map) munmap(g->map, g->map_len);
        delete g;
        return fail(e.code, "%s", e.msg.c_str());
    } catch (const std::exception &e) {
        if (g->map) munmap(g->map, g->map_len);
        delete g;
        return fail(RNB_B200_VALIDATION_FAILED, "GGUF parse failed: %s", e.what());
    }
    *out = g;
    return RNB_B200_OK;
}

// element count and byte size of a tensor; bytes = 0 when the type's block layout is not tabulated
static bool tensor_bytes(const Tensor &t, uint64_t *n_elems, uint64_t *bytes) {
    uint64_t n = 1;
    for (uint32_t d = 0; d < t.n_dims; d++) n *= t.dims[d];
    *n_elems = n;
    size_t bb = 0, be = 0;
    if (!type_layout(t.type, &bb, &be)) {
        *bytes = 0;
        return false;
    }
    const uint64_t inner = t.n_dims ? t.dims[t.n_dims - 1] : 1;
    if (inner % be != 0) {
        *bytes = 0;
        return false;
    }
    *bytes = n / be * bb;
    return true;
}

extern "C" {

int rnb_b200_gguf_parse(const void *data, size_t len, rnb_b200_gguf **out) {
    if (!data || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    rnb_b200_gguf *g = new rnb_b200_gguf();
    g->data = static_cast<const uint8_t *>(data);
    g->len = len;
    return parse_or_fail(g, out);
}

int rnb_b200_gguf_open(const char *path, rnb_b200_gguf **out) {
    if (!path || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(RNB_B200_VALIDATION_FAILED, "cannot open GGUF file %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        ::close(fd);
        return fail(RNB_B200_VALIDATION_FAILED, "cannot stat GGUF file %s (or it is empty)", path);
    }
    void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) return fail(RNB_B200_OUT_OF_MEMORY, "mmap of %s failed: %s", path, strerror(errno));
    rnb_b200_gguf *g = new rnb_b200_gguf();
    g->data = static_cast<const uint8_t *>(m);
    g->len = (size_t)st.st_size;
    g->map = m;
    g->map_len = (size_t)st.st_size;
    return parse_or_fail(g, out);
}

void rnb_b200_gguf_close(rnb_b200_gguf *g) {
    if (!g) return;
    if (g->map) munmap(g->map, g->map_len);
    delete g;
}

int rnb_b200_gguf_info(const rnb_b200_gguf *g, uint32_t *version, uint64_t *alignment, uint64_t *data_start, uint64_t *n_tensors, uint64_t *n_metadata) {
    if (!g) return fail(RNB_B200_VALIDATION_FAILED, "null GGUF handle");
    if (version) *version = g->version;
    if (alignment) *alignment = g->alignment;
    if (data_start) *data_start = g->data_start;
    if (n_tensors) *n_tensors = g->tensors.size();
    if (n_metadata) *n_metadata = g->metadata.size();
    return RNB_B200_OK;
}

// Integer metadata of any width (and bool) as u64; RNB_B200_UNSUPPORTED for a missing key,
// RNB_B200_VALIDATION_FAILED for a value of another kind (the reference's MissingKey / TypeMismatch).
int rnb_b200_gguf_get_u64(const rnb_b200_gguf *g, const char *key, uint64_t *out) {
    if (!g || !key || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    const Value *v = g->find(key);
    if (!v) return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s'", key);
    const bool is_int = v->type <= 5 || v->type == 7 || v->type == 10 || v->type == 11;
    if (!is_int) return fail(RNB_B200_VALIDATION_FAILED, "GGUF metadata key '%s' is not an integer", key);
    *out = v->u;
    return RNB_B200_OK;
}
int rnb_b200_gguf_get_f64(const rnb_b200_gguf *g, const char *key, double *out) {
    if (!g || !key || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    const Value *v = g->find(key);
    if (!v) return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s'", key);
    if (v->type != 6 && v->type != 12) return fail(RNB_B200_VALIDATION_FAILED, "GGUF metadata key '%s' is not a float", key);
    *out = v->f;
    return RNB_B200_OK;
}
// Copies the string (NUL-terminated, truncated to cap - 1) and reports its full length.
int rnb_b200_gguf_get_str(const rnb_b200_gguf *g, const char *key, char *buf, size_t cap, size_t *len_out) {
    if (!g || !key) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    const Value *v = g->find(key);
    if (!v) return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s'", key);
    if (v->type != 8) return fail(RNB_B200_VALIDATION_FAILED, "GGUF metadata key '%s' is not a string", key);
    if (len_out) *len_out = v->s.size();
    if (buf && cap) {
        const size_t n = std::min(cap - 1, v->s.size());
        memcpy(buf, v->s.data(), n);
        buf[n] = 0;
    }
    return RNB_B200_OK;
}
// Length of an array value; with `out` the first min(cap, len) integer elements as u64.
int rnb_b200_gguf_get_array_u64(const rnb_b200_gguf *g, const char *key, uint64_t *out, size_t cap, size_t *len_out) {
    if (!g || !key) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    const Value *v = g->find(key);
    if (!v) return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s'", key);
    if (v->type != 9) return fail(RNB_B200_VALIDATION_FAILED, "GGUF metadata key '%s' is not an array", key);
    if (len_out) *len_out = v->items.size();
    if (out) {
        const bool is_int = v->elem_type <= 5 || v->elem_type == 7 || v->elem_type == 10 || v->elem_type == 11;
        if (!is_int) return fail(RNB_B200_VALIDATION_FAILED, "GGUF metadata key '%s' is not an integer array", key);
        for (size_t i = 0; i < cap && i < v->items.size(); i++) out[i] = v->items[i].u;
    }
    return RNB_B200_OK;
}

static int fill_tensor_info(const rnb_b200_gguf *g, const Tensor &t, rnb_b200_gguf_tensor_info *out) {
    memset(out, 0, sizeof(*out));
    snprintf(out->name, sizeof(out->name), "%s", t.name.c_str());
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) out->dims[d] = d < (int)t.n_dims ? t.dims[d] : 1;
    out->ggml_type = t.type;
    out->offset = t.offset;
    uint64_t n = 0, bytes = 0;
    tensor_bytes(t, &n, &bytes);
    out->n_elements = n;
    out->n_bytes = bytes;
    const unsigned __int128 end = (unsigned __int128)g->data_start + t.offset + bytes;
    if (end > (unsigned __int128)g->len)
        return fail(RNB_B200_VALIDATION_FAILED, "tensor '%s' (%llu bytes at data offset %llu) extends beyond the file", t.name.c_str(), (unsigned long long)bytes,
                    (unsigned long long)t.offset);
    out->data = g->data + g->data_start + t.offset;
    return RNB_B200_OK;
}
int rnb_b200_gguf_tensor_at(const rnb_b200_gguf *g, size_t index, rnb_b200_gguf_tensor_info *out) {
    if (!g || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    if (index >= g->tensors.size()) return fail(RNB_B200_VALIDATION_FAILED, "tensor index %zu out of range (%zu tensors)", index, g->tensors.size());
    return fill_tensor_info(g, g->tensors[index], out);
}
int rnb_b200_gguf_tensor(const rnb_b200_gguf *g, const char *name, rnb_b200_gguf_tensor_info *out) {
    if (!g || !name || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    const Tensor *t = g->tensor(name);
    if (!t) return fail(RNB_B200_UNSUPPORTED, "missing GGUF tensor '%s'", name);
    return fill_tensor_info(g, *t, out);
}

// ModelMetadata of the Llama-style families this decoder runs (arch/mod.rs:304-560): keys live
// under the `general.architecture` prefix ("llama" when absent); defaults as the reference's.
int rnb_b200_gguf_model_config(const rnb_b200_gguf *g, int max_ctx, rnb_b200_model_cfg *cfg) {
    if (!g || !cfg) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    std::string arch = "llama";
    if (const Value *a = g->find("general.architecture"))
        if (a->type == 8) arch = a->s;
    auto u32 = [&](const std::string &suffix, uint64_t *out) -> int {
        const Value *v = g->find(arch + "." + suffix);
        if (!v) return 1;
        const bool is_int = v->type <= 5 || v->type == 10 || v->type == 11;
        if (!is_int) return 2;
        *out = v->u;
        return 0;
    };
    auto f32 = [&](const std::string &suffix, double *out) -> int {
        const Value *v = g->find(arch + "." + suffix);
        if (!v) return 1;
        if (v->type != 6 && v->type != 12) return 2;
        *out = v->f;
        return 0;
    };
    memset(cfg, 0, sizeof(*cfg));
    uint64_t hidden = 0, layers = 0, heads = 0, kv_heads = 0, ff = 0, vocab = 32000, ctx = 4096, n_expert = 0, n_used = 0, ff_exp = 0, key_len = 0;
    if (u32("embedding_length", &hidden)) return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s.embedding_length'", arch.c_str());
    if (u32("block_count", &layers)) return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s.block_count'", arch.c_str());
    if (u32("attention.head_count", &heads)) return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s.attention.head_count'", arch.c_str());
    if (heads == 0) return fail(RNB_B200_VALIDATION_FAILED, "%s.attention.head_count must be positive", arch.c_str());
    kv_heads = heads;
    {   // scalar, or a per-layer array of which the largest entry counts
        const Value *v = g->find(arch + ".attention.head_count_kv");
        if (v && v->type == 9) {
            uint64_t mx = 0;
            for (const Value &e : v->items) mx = std::max(mx, e.u);
            kv_heads = v->items.empty() ? heads : mx;
        } else if (v) {
            u32("attention.head_count_kv", &kv_heads);
        }
    }
    u32("expert_count", &n_expert);
    u32("expert_used_count", &n_used);
    u32("expert_feed_forward_length", &ff_exp);
    const int ffrc = u32("feed_forward_length", &ff);
    if (ffrc == 2) {
        const Value *v = g->find(arch + ".feed_forward_length");
        if (v && v->type == 9)
            for (const Value &e : v->items) ff = std::max(ff, e.u);
    } else if (ffrc == 1 && ff_exp == 0) {
        return fail(RNB_B200_UNSUPPORTED, "missing GGUF metadata key '%s.feed_forward_length'", arch.c_str());
    }
    u32("vocab_size", &vocab);
    if (const Value *tok = g->find("tokenizer.ggml.tokens"))
        if (tok->type == 9 && !g->find(arch + ".vocab_size")) vocab = tok->items.size();
    if (const Tensor *emb = g->tensor("token_embd.weight"))
        if (emb->n_dims == 2) vocab = emb->dims[0];       // the table itself is authoritative for the row count
    u32("context_length", &ctx);
    double theta = 10000.0, eps = 1e-5;
    f32("rope.freq_base", &theta);
    f32("attention.layer_norm_rms_epsilon", &eps);
    const uint64_t head_dim = u32("attention.key_length", &key_len) == 0 ? key_len : hidden / heads;
    cfg->n_layer = (int)layers;
    cfg->hidden = (int)hidden;
    cfg->n_head = (int)heads;
    cfg->n_kv_head = (int)kv_heads;
    cfg->head_dim = (int)head_dim;
    cfg->n_ff = n_expert ? 0 : (int)ff;
    cfg->vocab = (int)vocab;
    cfg->max_ctx = max_ctx > 0 ? max_ctx : (int)ctx;
    // adjacent-pair rotation for Llama; the half-split form for the Qwen families (gemma/attention.rs:86-92)
    cfg->rope_neox = arch.rfind("qwen", 0) == 0 ? 1 : 0;
    cfg->rms_eps = (float)eps;
    cfg->rope_theta = (float)theta;
    cfg->n_expert = (int)n_expert;
    cfg->n_expert_used = (int)n_used;
    cfg->n_ff_expert = n_expert ? (int)(ff_exp ? ff_exp : ff) : 0;
    cfg->world_size = 1;
    cfg->rank = 0;
    return RNB_B200_OK;
}

// Points the decoder at the file's tensors (names of arch/llama.rs:33-155; the expert stacks of the
// MoE families are `ffn_gate_inp`, `ffn_{gate,up,down}_exps`).  With register_pages the mapped
// tensor-data section is pinned first, where the mapping allows it, so the uploads run as
// asynchronous DMA from the page cache.
int rnb_b200_decoder_load_gguf(rnb_b200_decoder *d, const rnb_b200_gguf *g, int register_pages) {
    if (!d || !g) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    rnb_b200_model_cfg c;
    RNB_TRY(rnb_b200_decoder_config(d, &c));
    if (register_pages && g->data_start < g->len) {
        // best effort: some file systems' read-only mappings cannot be pinned (the driver answers
        // "invalid argument"); the uploads then run as staged pageable copies, same bytes
        if (rnb_b200_register_host_range(g->data + g->data_start, g->len - g->data_start) != RNB_B200_OK) cudaGetLastError();
    }
    auto quant = [&](const std::string &name, rnb_b200_qweight *out, bool required) -> int {
        const Tensor *t = g->tensor(name);
        if (!t) {
            if (!required) {
                out->type = 0;
                out->data = nullptr;
                out->len = 0;
                return RNB_B200_OK;
            }
            return fail(RNB_B200_UNSUPPORTED, "missing GGUF tensor '%s'", name.c_str());
        }
        rnb_b200_gguf_tensor_info ti;
        RNB_TRY(fill_tensor_info(g, *t, &ti));
        if (ti.n_bytes == 0) return fail(RNB_B200_UNSUPPORTED, "tensor '%s' has GGML type %u, which this decoder cannot size", name.c_str(), ti.ggml_type);
        out->type = ti.ggml_type;
        out->data = ti.data;
        out->len = (size_t)ti.n_bytes;
        return RNB_B200_OK;
    };
    auto f32v = [&](const std::string &name, size_t n, const float **out) -> int {
        const Tensor *t = g->tensor(name);
        if (!t) return fail(RNB_B200_UNSUPPORTED, "missing GGUF tensor '%s'", name.c_str());
        rnb_b200_gguf_tensor_info ti;
        RNB_TRY(fill_tensor_info(g, *t, &ti));
        if (ti.ggml_type != 0 || ti.n_elements != n) return fail(RNB_B200_VALIDATION_FAILED, "tensor '%s' must be %zu f32 values (type %u, %llu elements found)", name.c_str(), n, ti.ggml_type, (unsigned long long)ti.n_elements);
        if ((uintptr_t)ti.data & 3u) return fail(RNB_B200_VALIDATION_FAILED, "tensor '%s' is not 4-byte aligned in the file", name.c_str());
        *out = reinterpret_cast<const float *>(ti.data);
        return RNB_B200_OK;
    };
    for (int l = 0; l < c.n_layer; l++) {
        const std::string p = "blk." + std::to_string(l) + ".";
        rnb_b200_layer_weights w;
        memset(&w, 0, sizeof(w));
        RNB_TRY(f32v(p + "attn_norm.weight", (size_t)c.hidden, &w.attn_norm));
        RNB_TRY(f32v(p + "ffn_norm.weight", (size_t)c.hidden, &w.ffn_norm));
        RNB_TRY(quant(p + "attn_q.weight", &w.wq, true));
        RNB_TRY(quant(p + "attn_k.weight", &w.wk, true));
        RNB_TRY(quant(p + "attn_v.weight", &w.wv, true));
        RNB_TRY(quant(p + "attn_output.weight", &w.wo, true));
        if (c.n_expert > 0) {
            RNB_TRY(f32v(p + "ffn_gate_inp.weight", (size_t)c.n_expert * c.hidden, &w.router));
            RNB_TRY(quant(p + "ffn_gate_exps.weight", &w.gate_exps, true));
            RNB_TRY(quant(p + "ffn_up_exps.weight", &w.up_exps, true));
            RNB_TRY(quant(p + "ffn_down_exps.weight", &w.down_exps, true));
        } else {
            RNB_TRY(quant(p + "ffn_gate.weight", &w.gate, true));
            RNB_TRY(quant(p + "ffn_up.weight", &w.up, true));
            RNB_TRY(quant(p + "ffn_down.weight", &w.down, true));
        }
        RNB_TRY(rnb_b200_decoder_set_layer(d, l, &w));
    }
    rnb_b200_qweight embd, output;
    const float *out_norm = nullptr;
    RNB_TRY(quant("token_embd.weight", &embd, true));
    RNB_TRY(f32v("output_norm.weight", (size_t)c.hidden, &out_norm));
    RNB_TRY(quant("output.weight", &output, false));
    if (!output.data) output = embd;   // tied embeddings: no separate LM head in the file
    return rnb_b200_decoder_set_globals(d, embd, out_norm, output);
}

}  // extern "C"
