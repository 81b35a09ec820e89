// GGUF v2/v3 container reader at model scale: the file is memory-mapped, every offset is 64-bit,
// nothing is copied or boxed; tensor data is handed out as pointers into the mapping and
// quantized tensors go straight to skn_tensor_upload_quant.
//
// Replaces, for this path, gguf/src/commonMain/kotlin/sk/ai/net/gguf/GGUFReader.kt, which reads
// the whole file into one ByteArray (GGUFReader.kt:83), computes byte counts in Int
// (GGUFReader.kt:359), throws on F16 (GGUFReader.kt:363) and boxes every byte
// (utils/BytePresentationUtils.kt:117-153).  The fields / tensors shape of its API
// (GGUFReader.kt:35-61) is kept.  Host code only.
#include "skn_internal.cuh"

#include <fcntl.h>
#include <new>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

#define SKN_MAGIC_GGUF 0x736b6e67u   // 'skng'

struct skn_gguf_kv_rec {
    const char *key; uint64_t key_len;
    uint32_t type, elem_type;      // elem_type only for arrays
    const uint8_t *value;          // scalars: the value; string: its bytes; array: first element
    uint64_t count;                // string: byte length; array: element count; scalars: 1
};

struct skn_gguf_tensor_rec {
    const char *name; uint64_t name_len;
    uint32_t n_dims; uint64_t dims[4];
    uint32_t type; uint64_t offset, n_bytes;
};

struct skn_gguf {
    uint32_t magic;
    int fd;
    const uint8_t *base; uint64_t size;
    uint32_t version; uint64_t alignment, data_start;
    std::vector<skn_gguf_kv_rec> kvs;
    std::vector<skn_gguf_tensor_rec> tensors;
    std::vector<std::string> names;    // NUL-terminated copies of keys and tensor names
};

// (block elements, block bytes) of every GGML type id: Constants.kt:58-90
static bool ggml_type_size(uint32_t t, uint64_t *elems, uint64_t *bytes) {
    static const struct { uint32_t id; uint32_t e, b; } T[] = {
        {0, 1, 4}, {1, 1, 2}, {2, 32, 18}, {3, 32, 20}, {6, 32, 22}, {7, 32, 24}, {8, 32, 34}, {9, 32, 40},
        {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292},
        {16, 256, 66}, {17, 256, 74}, {18, 256, 98}, {19, 256, 50}, {20, 32, 18}, {21, 256, 110}, {22, 256, 82},
        {23, 256, 136}, {24, 1, 1}, {25, 1, 2}, {26, 1, 4}, {27, 1, 8}, {28, 1, 8}, {29, 256, 56}, {30, 1, 2},
        {34, 256, 54}, {35, 256, 66}};
    for (const auto &r : T)
        if (r.id == t) { *elems = r.e; *bytes = r.b; return true; }
    return false;
}

static const uint64_t SCALAR_SIZE[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};   // GGUFValueType 0..12

struct Cursor {
    const uint8_t *p, *end;
    bool ok;
    bool need(uint64_t n) { if (!ok || (uint64_t)(end - p) < n) { ok = false; return false; } return true; }
    uint32_t u32() { uint32_t v = 0; if (need(4)) { memcpy(&v, p, 4); p += 4; } return v; }
    uint64_t u64() { uint64_t v = 0; if (need(8)) { memcpy(&v, p, 8); p += 8; } return v; }
    const uint8_t *bytes(uint64_t n) { if (!need(n)) return nullptr; const uint8_t *r = p; p += n; return r; }
};

static bool gguf_ok(const skn_gguf *g) { return g && g->magic == SKN_MAGIC_GGUF; }

static bool skip_value(Cursor &c, uint32_t type, skn_gguf_kv_rec *rec) {
    if (type <= 12 && SCALAR_SIZE[type]) {
        const uint8_t *v = c.bytes(SCALAR_SIZE[type]);
        if (rec) { rec->value = v; rec->count = 1; }
        return c.ok;
    }
    if (type == 8) {
        const uint64_t n = c.u64();
        const uint8_t *v = c.bytes(n);
        if (rec) { rec->value = v; rec->count = n; }
        return c.ok;
    }
    if (type == 9) {
        const uint32_t et = c.u32();
        const uint64_t n = c.u64();
        if (!c.ok || et == 9 || et > 12) { c.ok = false; return false; }
        if (rec) { rec->elem_type = et; rec->count = n; rec->value = c.p; }
        if (et == 8) {
            for (uint64_t i = 0; i < n && c.ok; ++i) { const uint64_t l = c.u64(); c.bytes(l); }
        } else {
            if (n > (uint64_t)(c.end - c.p) / SCALAR_SIZE[et]) { c.ok = false; return false; }
            c.bytes(n * SCALAR_SIZE[et]);
        }
        return c.ok;
    }
    c.ok = false;
    return false;
}

extern "C" {

int32_t skn_gguf_close(skn_gguf *g);

int32_t skn_gguf_open(const char *path, skn_gguf **out) {
    if (!out || !path) return skn_fail(nullptr, SKN_ERR_ARG, "skn_gguf_open: NULL argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return skn_fail(nullptr, SKN_ERR_ARG, "cannot open %s", path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return skn_fail(nullptr, SKN_ERR_ARG, "%s is too short to be a GGUF file", path);
    }
    void *map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return skn_fail(nullptr, SKN_ERR_OOM, "mmap of %s failed", path);
    }
    skn_gguf *g = new (std::nothrow) skn_gguf();
    if (!g) {
        munmap(map, (size_t)st.st_size);
        close(fd);
        return skn_fail(nullptr, SKN_ERR_OOM, "host allocation failed");
    }
    g->magic = SKN_MAGIC_GGUF;
    g->fd = fd;
    g->base = (const uint8_t *)map;
    g->size = (uint64_t)st.st_size;
    g->alignment = 32;                                  // GGUF_DEFAULT_ALIGNMENT, Constants.kt:12
    Cursor c{g->base, g->base + g->size, true};
    int32_t rc = SKN_OK;
    const uint32_t magic = c.u32();
    g->version = c.u32();
    const uint64_t n_tensors = c.u64(), n_kv = c.u64();
    if (magic != 0x46554747u) rc = skn_fail(nullptr, SKN_ERR_ARG, "GGUF magic invalid");               // Constants.kt:10
    else if (g->version != 2 && g->version != 3) rc = skn_fail(nullptr, SKN_ERR_ARG, "Sorry, file appears to be version %u that we cannot handle", g->version);
    // a metadata entry is at least 13 bytes (key length, type, one value byte), a tensor record at least 24
    // (name length, rank, type, offset): counts the rest of the file cannot hold are corrupt, and nothing
    // is reserved for them
    else if (n_kv > (g->size - 24) / 13 || n_tensors > (g->size - 24) / 24 || n_kv * 13 + n_tensors * 24 > g->size - 24)
        rc = skn_fail(nullptr, SKN_ERR_ARG, "corrupt header counts (%llu tensors, %llu metadata entries in %llu bytes)",
                      (unsigned long long)n_tensors, (unsigned long long)n_kv, (unsigned long long)g->size);
    try {
        if (rc == SKN_OK) {
            g->kvs.reserve((size_t)n_kv);
            g->tensors.reserve((size_t)n_tensors);
            for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
                skn_gguf_kv_rec r{};
                r.key_len = c.u64();
                r.key = (const char *)c.bytes(r.key_len);
                r.type = c.u32();
                if (!c.ok || !skip_value(c, r.type, &r)) break;
                g->names.emplace_back(r.key, (size_t)r.key_len);
                g->kvs.push_back(r);
                if (r.type == 4 && g->names.back() == "general.alignment") {
                    uint32_t a; memcpy(&a, r.value, 4);
                    if (a == 0 || (a & (a - 1))) { rc = skn_fail(nullptr, SKN_ERR_ARG, "bad general.alignment %u", a); break; }
                    g->alignment = a;
                }
            }
            for (uint64_t i = 0; i < n_tensors && c.ok && rc == SKN_OK; ++i) {
                skn_gguf_tensor_rec t{};
                t.name_len = c.u64();
                t.name = (const char *)c.bytes(t.name_len);
                t.n_dims = c.u32();
                if (!c.ok || t.n_dims > 4) { c.ok = false; break; }
                uint64_t n_elems = 1;
                for (uint32_t d = 0; d < 4; ++d) t.dims[d] = 1;
                for (uint32_t d = 0; d < t.n_dims; ++d) {
                    t.dims[d] = c.u64();
                    if (t.dims[d] != 0 && n_elems > UINT64_MAX / t.dims[d]) c.ok = false; else n_elems *= t.dims[d];
                }
                t.type = c.u32();
                t.offset = c.u64();
                if (!c.ok) break;
                uint64_t be, bb;
                if (!ggml_type_size(t.type, &be, &bb)) { rc = skn_fail(nullptr, SKN_ERR_TYPE, "tensor %llu has unknown GGML type %u", (unsigned long long)i, t.type); break; }
                if (t.dims[0] % be) { rc = skn_fail(nullptr, SKN_ERR_SHAPE, "Quantized tensor row size (%llu) is not a multiple of block size (%llu)", (unsigned long long)t.dims[0], (unsigned long long)be); break; }
                t.n_bytes = n_elems / be * bb;          // 64-bit: no overflow at model scale
                g->names.emplace_back(t.name, (size_t)t.name_len);
                g->tensors.push_back(t);
            }
            if (rc == SKN_OK && !c.ok) rc = skn_fail(nullptr, SKN_ERR_ARG, "%s is truncated or corrupt (metadata)", path);
        }
    } catch (...) {
        rc = skn_fail(nullptr, SKN_ERR_OOM, "host allocation failed while indexing %s", path);
    }
    if (rc == SKN_OK) {
        const uint64_t pos = (uint64_t)(c.p - g->base);
        g->data_start = (pos + g->alignment - 1) / g->alignment * g->alignment;
        for (const auto &t : g->tensors) {
            if (t.offset % g->alignment) {
                rc = skn_fail(nullptr, SKN_ERR_ARG, "%s: a tensor's data offset %llu is not a multiple of the alignment %llu", path,
                              (unsigned long long)t.offset, (unsigned long long)g->alignment);
                break;
            }
            if (t.offset > g->size || g->data_start > g->size - t.offset || t.n_bytes > g->size - g->data_start - t.offset) {
                rc = skn_fail(nullptr, SKN_ERR_ARG, "%s is truncated: a tensor's data lies outside the file", path);
                break;
            }
        }
    }
    if (rc != SKN_OK) {
        skn_gguf_close(g);
        return rc;
    }
    *out = g;
    return SKN_OK;
}

int32_t skn_gguf_close(skn_gguf *g) {
    if (!gguf_ok(g)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad GGUF handle");
    munmap((void *)g->base, (size_t)g->size);
    close(g->fd);
    g->magic = 0;
    delete g;
    return SKN_OK;
}

int32_t skn_gguf_counts(const skn_gguf *g, int32_t *version, int64_t *n_tensors, int64_t *n_kv, int64_t *alignment,
                        int64_t *data_offset) {
    if (!gguf_ok(g)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad GGUF handle");
    if (version) *version = (int32_t)g->version;
    if (n_tensors) *n_tensors = (int64_t)g->tensors.size();
    if (n_kv) *n_kv = (int64_t)g->kvs.size();
    if (alignment) *alignment = (int64_t)g->alignment;
    if (data_offset) *data_offset = (int64_t)g->data_start;
    return SKN_OK;
}

// Metadata entry i.  key: NUL-terminated.  value_type / elem_type: GGUFValueType ids
// (Constants.kt GGUFValueType).  value points into the mapping: a little-endian scalar; a
// string's bytes (count = length, not terminated); an array's first element (count elements;
// string elements are u64 length + bytes each).
int32_t skn_gguf_kv(const skn_gguf *g, int64_t i, const char **key, int32_t *value_type, int32_t *elem_type,
                    const void **value, int64_t *count) {
    if (!gguf_ok(g)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad GGUF handle");
    if (i < 0 || (size_t)i >= g->kvs.size()) return skn_fail(nullptr, SKN_ERR_ARG, "metadata index out of range");
    const auto &r = g->kvs[(size_t)i];
    if (key) *key = g->names[(size_t)i].c_str();
    if (value_type) *value_type = (int32_t)r.type;
    if (elem_type) *elem_type = r.type == 9 ? (int32_t)r.elem_type : -1;
    if (value) *value = r.value;
    if (count) *count = (int64_t)r.count;
    return SKN_OK;
}

// Tensor i.  dims are in file order (dims[0] is the contiguous one, i.e. K of a [N, K] weight).
int32_t skn_gguf_tensor(const skn_gguf *g, int64_t i, const char **name, int32_t *n_dims, int64_t *dims4,
                        int32_t *ggml_type, int64_t *data_offset, int64_t *n_bytes, const void **data) {
    if (!gguf_ok(g)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad GGUF handle");
    if (i < 0 || (size_t)i >= g->tensors.size()) return skn_fail(nullptr, SKN_ERR_ARG, "tensor index out of range");
    const auto &t = g->tensors[(size_t)i];
    if (name) *name = g->names[g->kvs.size() + (size_t)i].c_str();
    if (n_dims) *n_dims = (int32_t)t.n_dims;
    if (dims4) for (int d = 0; d < 4; ++d) dims4[d] = (int64_t)t.dims[d];
    if (ggml_type) *ggml_type = (int32_t)t.type;
    if (data_offset) *data_offset = (int64_t)(g->data_start + t.offset);
    if (n_bytes) *n_bytes = (int64_t)t.n_bytes;
    if (data) *data = g->base + g->data_start + t.offset;
    return SKN_OK;
}

int32_t skn_gguf_find_tensor(const skn_gguf *g, const char *name, int64_t *index) {
    if (!gguf_ok(g)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad GGUF handle");
    if (!name || !index) return skn_fail(nullptr, SKN_ERR_ARG, "NULL argument");
    for (size_t i = 0; i < g->tensors.size(); ++i)
        if (g->names[g->kvs.size() + i] == name) { *index = (int64_t)i; return SKN_OK; }
    *index = -1;
    return skn_fail(nullptr, SKN_ERR_ARG, "no tensor named %s", name);
}

// Upload quantized tensor i (1-D or 2-D, one of the four supported block types) to the device:
// rows = dims[1], cols = dims[0]; the raw blocks go from the mapping to HBM unchanged.
int32_t skn_gguf_upload(skn_ctx *ctx, const skn_gguf *g, int64_t i, skn_tensor **out) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    if (!gguf_ok(g)) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad GGUF handle");
    if (i < 0 || (size_t)i >= g->tensors.size()) return skn_fail(ctx, SKN_ERR_ARG, "tensor index out of range");
    const auto &t = g->tensors[(size_t)i];
    if (t.n_dims > 2 && (t.dims[2] != 1 || t.dims[3] != 1)) return skn_fail(ctx, SKN_ERR_SHAPE, "only 1-D and 2-D tensors can be uploaded as weights");
    return skn_tensor_upload_quant(ctx, (int32_t)t.type, (int64_t)t.dims[1], (int64_t)t.dims[0],
                                   g->base + g->data_start + t.offset, (int64_t)t.n_bytes, out);
}

}  // extern "C"
