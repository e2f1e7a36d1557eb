// GGUF ingest: header / metadata / tensor-table parser and the loader contract that turns named tensors into device
// matrices.  Host code only (compiled with the rest of the library so that one shared object carries the whole path).
//
// Follows ferric_gguf::parse (crates/ferric-gguf/src/lib.rs:105-132) with its bounds-safe cursor (:59-103): any read
// past the end marks the parse as failed instead of faulting, so arbitrary bytes are rejected, never trusted; the stride
// guard check_declared_strides (:387-431); Gguf::tensor / raw (:444-453); GgufFile::open (:533-554, here a read-only
// memory mapping instead of prefix probing: the kernel pages the header in on demand, and tensor bytes are handed out
// as pointers into the mapping rather than copied); and the model loaders' qm / qm_cat
// (crates/ferric-llama/src/qwen35.rs:366-402): GGUF lists dims fastest-varying first, so a listed [in, out] is a
// row-major [out, in] weight, and same-format tensors sharing `in` stack along `out` by concatenating their bytes.
// Not taken over: the reference's resolution of vendor type ids that collide with mainline ggml (:216-385) -- none of
// the three formats served here is affected.
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "../../include/ferric_cuda.h"
#include "common.cuh"
#include "handles.h"

using namespace ferric;

namespace {

struct Meta {
    int kind = 0;   // FERRIC_GGUF_META_*
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0.0;
    bool b = false;
    std::string s;
    std::vector<Meta> arr;
};

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t ggml_type = 0;
    uint64_t offset = 0;
    // The element count, or false when the product of the (untrusted) dims does not fit 63 bits.
    bool n_elements_checked(uint64_t* out) const
    {
        uint64_t n = 1;
        for (uint64_t d : dims)
            if (__builtin_mul_overflow(n, d, &n)) return false;
        if (n >> 63) return false;
        *out = n;
        return true;
    }
    uint64_t n_elements() const   // after parse_into has vetted the dims
    {
        uint64_t n = 0;
        return n_elements_checked(&n) ? n : 0;
    }
};

// Bounds-safe cursor (lib.rs:59-103).
struct Cur {
    const uint8_t* b;
    size_t len, p = 0;
    bool ok = true;
    const uint8_t* take(size_t k)
    {
        if (!ok || k > len - p) {
            ok = false;
            return nullptr;
        }
        const uint8_t* s = b + p;
        p += k;
        return s;
    }
    template <typename T>
    T le()
    {
        const uint8_t* s = take(sizeof(T));
        T v = 0;
        if (s) memcpy(&v, s, sizeof(T));   // little-endian host
        return v;
    }
    std::string str()
    {
        const uint64_t n = le<uint64_t>();
        if (!ok || n > len - p) {   // a garbage length must not turn into a huge reservation
            ok = false;
            return std::string();
        }
        const uint8_t* s = take((size_t)n);
        return s ? std::string(reinterpret_cast<const char*>(s), (size_t)n) : std::string();
    }
    Meta val(uint32_t ty, int depth = 0)
    {
        Meta m;
        switch (ty) {
        case 0: m.kind = FERRIC_GGUF_META_U; m.u = le<uint8_t>(); break;
        case 1: m.kind = FERRIC_GGUF_META_I; m.i = (int8_t)le<uint8_t>(); break;
        case 2: m.kind = FERRIC_GGUF_META_U; m.u = le<uint16_t>(); break;
        case 3: m.kind = FERRIC_GGUF_META_I; m.i = (int16_t)le<uint16_t>(); break;
        case 4: m.kind = FERRIC_GGUF_META_U; m.u = le<uint32_t>(); break;
        case 5: m.kind = FERRIC_GGUF_META_I; m.i = (int32_t)le<uint32_t>(); break;
        case 6: {
            const uint32_t bits = le<uint32_t>();
            float f;
            memcpy(&f, &bits, 4);
            m.kind = FERRIC_GGUF_META_F;
            m.f = f;
            break;
        }
        case 7: m.kind = FERRIC_GGUF_META_BOOL; m.b = le<uint8_t>() != 0; break;
        case 8: m.kind = FERRIC_GGUF_META_STR; m.s = str(); break;
        case 9: {
            m.kind = FERRIC_GGUF_META_ARR;
            const uint32_t et = le<uint32_t>();
            const uint64_t n = le<uint64_t>();
            // each element costs at least one byte on disk, so a count beyond the remaining bytes is garbage
            if (!ok || n > len - p || depth > 8) {
                ok = false;
                break;
            }
            m.arr.reserve((size_t)std::min<uint64_t>(n, 1u << 20));
            for (uint64_t k = 0; k < n && ok; k++) m.arr.push_back(val(et, depth + 1));
            break;
        }
        case 10: m.kind = FERRIC_GGUF_META_U; m.u = le<uint64_t>(); break;
        case 11: m.kind = FERRIC_GGUF_META_I; m.i = (int64_t)le<uint64_t>(); break;
        case 12: {
            const uint64_t bits = le<uint64_t>();
            memcpy(&m.f, &bits, 8);
            m.kind = FERRIC_GGUF_META_F;
            break;
        }
        default: ok = false; break;
        }
        return m;
    }
};

bool type_bytes(uint32_t ty, uint64_t n, uint64_t* out)
{
    size_t b = 0;
    if (ferric_gguf_type_size(ty, (size_t)n, &b) != kOk) return false;
    *out = b;
    return true;
}

}  // namespace

struct ferric_gguf {
    std::map<std::string, Meta> metadata;
    std::vector<TensorInfo> tensors;
    const uint8_t* data = nullptr;   // the whole file
    size_t len = 0, data_start = 0;
    void* mapping = nullptr;         // non-null when this object owns a memory mapping of `len` bytes
    std::vector<std::string> keys;   // metadata keys in file order
};

namespace {

// check_declared_strides (lib.rs:387-431): the bytes this reader's block layout needs for a tensor must fit before the
// next tensor starts, and must not be less than half of what the file reserves (a stride that is too small).
int32_t check_strides(const std::vector<TensorInfo>& tensors, size_t data_len, size_t align)
{
    std::vector<const TensorInfo*> by(tensors.size());
    for (size_t i = 0; i < tensors.size(); i++) by[i] = &tensors[i];
    std::stable_sort(by.begin(), by.end(), [](const TensorInfo* a, const TensorInfo* b) { return a->offset < b->offset; });
    for (size_t i = 0; i < by.size(); i++) {
        const TensorInfo& t = *by[i];
        uint64_t sz = 0;
        if (!type_bytes(t.ggml_type, t.n_elements(), &sz)) continue;   // an unknown type fails loudly when it is read
        const uint64_t limit = i + 1 < by.size() ? by[i + 1]->offset : (uint64_t)data_len;
        const uint64_t avail = limit > t.offset ? limit - t.offset : 0;
        if (sz > avail) {
            set_last_error("tensor '%s' (ggml type %u, %llu elements) needs %llu bytes by this reader's block layout, but the "
                           "file leaves only %llu before the next tensor; refusing to load",
                           t.name.c_str(), t.ggml_type, (unsigned long long)t.n_elements(), (unsigned long long)sz,
                           (unsigned long long)avail);
            return kErrShape;
        }
        const uint64_t pad = (uint64_t)std::max<size_t>(align, 64) * 4;
        if (i + 1 < by.size() && avail > sz + pad && avail > sz * 2) {
            set_last_error("tensor '%s' (ggml type %u, %llu elements) is %llu bytes by this reader's block layout, but the file "
                           "reserves %llu for it -- more than twice as much; refusing to load",
                           t.name.c_str(), t.ggml_type, (unsigned long long)t.n_elements(), (unsigned long long)sz,
                           (unsigned long long)avail);
            return kErrShape;
        }
    }
    return kOk;
}

int32_t parse_into(ferric_gguf* g, const uint8_t* bytes, size_t len)
{
    Cur c{bytes, len};
    if (c.le<uint32_t>() != 0x46554747u || !c.ok) {   // "GGUF"
        set_last_error("not a GGUF file");
        return kErrInvalidArg;
    }
    (void)c.le<uint32_t>();   // version
    const uint64_t n_tensors = c.le<uint64_t>(), n_meta = c.le<uint64_t>();
    for (uint64_t i = 0; i < n_meta && c.ok; i++) {
        std::string key = c.str();
        const uint32_t ty = c.le<uint32_t>();
        Meta m = c.val(ty);
        if (!c.ok) break;
        if (!g->metadata.count(key)) g->keys.push_back(key);
        g->metadata[key] = std::move(m);
    }
    for (uint64_t i = 0; i < n_tensors && c.ok; i++) {
        TensorInfo t;
        t.name = c.str();
        const uint32_t nd = c.le<uint32_t>();
        if (nd > 8) c.ok = false;
        for (uint32_t k = 0; k < nd && c.ok; k++) t.dims.push_back(c.le<uint64_t>());
        t.ggml_type = c.le<uint32_t>();
        t.offset = c.le<uint64_t>();
        uint64_t n = 0;
        if (c.ok && !t.n_elements_checked(&n)) {
            // dims whose product wraps would pass every later size check with a small, wrong byte count
            set_last_error("tensor '%s': the product of its dims overflows; refusing to load", t.name.c_str());
            return kErrShape;
        }
        if (c.ok) g->tensors.push_back(std::move(t));
    }
    if (!c.ok) {
        set_last_error("GGUF header truncated or malformed");
        return kErrShape;
    }
    size_t align = 32;
    auto it = g->metadata.find("general.alignment");
    if (it != g->metadata.end() && it->second.kind == FERRIC_GGUF_META_U && it->second.u > 0) align = (size_t)it->second.u;
    g->data_start = (c.p + align - 1) / align * align;
    g->data = bytes;
    g->len = len;
    return check_strides(g->tensors, len > g->data_start ? len - g->data_start : 0, align);
}

const TensorInfo* find_tensor(const ferric_gguf* g, const char* name)
{
    for (const TensorInfo& t : g->tensors)
        if (t.name == name) return &t;
    return nullptr;
}

int32_t tensor_bytes(const ferric_gguf* g, const TensorInfo& t, const uint8_t** data, size_t* nbytes)
{
    uint64_t sz = 0;
    if (!type_bytes(t.ggml_type, t.n_elements(), &sz)) return kErrUnsupportedType;   // message set by type_size
    const uint64_t start = (uint64_t)g->data_start + t.offset;
    if (start > g->len || sz > g->len - start) {
        set_last_error("tensor '%s' lies outside the file (%llu bytes at %llu of %zu)", t.name.c_str(), (unsigned long long)sz,
                       (unsigned long long)start, g->len);
        return kErrShape;
    }
    *data = g->data + start;
    *nbytes = (size_t)sz;
    return kOk;
}

void fill_info(const ferric_gguf* g, const TensorInfo& t, ferric_gguf_tensor* out)
{
    memset(out, 0, sizeof(*out));
    out->name = t.name.c_str();
    out->n_dims = (uint32_t)std::min<size_t>(t.dims.size(), 4);
    for (uint32_t k = 0; k < out->n_dims; k++) out->dims[k] = t.dims[k];
    out->ggml_type = t.ggml_type;
    out->offset = t.offset;
    out->n_elements = t.n_elements();
    uint64_t sz = 0;
    out->nbytes = type_bytes(t.ggml_type, t.n_elements(), &sz) ? sz : 0;
    (void)g;
}

const Meta* find_meta(const ferric_gguf* g, const char* key, int kind)
{
    if (!g || !key) {
        set_last_error("NULL file handle or key");
        return nullptr;
    }
    auto it = g->metadata.find(key);
    if (it == g->metadata.end()) {
        set_last_error("no metadata key '%s'", key);
        return nullptr;
    }
    if (kind >= 0 && it->second.kind != kind) {
        set_last_error("metadata key '%s' has kind %d, not %d", key, it->second.kind, kind);
        return nullptr;
    }
    return &it->second;
}

int32_t copy_str(const std::string& s, char* buf, size_t cap, size_t* len)
{
    if (len) *len = s.size();
    if (buf && cap > 0) {
        const size_t n = std::min(cap - 1, s.size());
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return kOk;
}

}  // namespace

extern "C" {

int32_t ferric_gguf_parse(const uint8_t* bytes, size_t len, ferric_gguf** out)
{
    if (!bytes || !out) {
        set_last_error("NULL bytes or output pointer");
        return kErrInvalidArg;
    }
    *out = nullptr;
    ferric_gguf* g = new (std::nothrow) ferric_gguf;
    if (!g) return kErrOom;
    const int32_t rc = parse_into(g, bytes, len);
    if (rc != kOk) {
        delete g;
        return rc;
    }
    *out = g;
    return kOk;
}

int32_t ferric_gguf_open(const char* path, ferric_gguf** out)
{
    if (!path || !out) {
        set_last_error("NULL path or output pointer");
        return kErrInvalidArg;
    }
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) {
        set_last_error("cannot open '%s': %s", path, strerror(errno));
        return kErrInvalidArg;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        set_last_error("cannot stat '%s' (or it is empty)", path);
        close(fd);
        return kErrInvalidArg;
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) {
        set_last_error("cannot map '%s': %s", path, strerror(errno));
        return kErrOom;
    }
    ferric_gguf* g = new (std::nothrow) ferric_gguf;
    if (!g) {
        munmap(map, (size_t)st.st_size);
        return kErrOom;
    }
    g->mapping = map;
    const int32_t rc = parse_into(g, reinterpret_cast<const uint8_t*>(map), (size_t)st.st_size);
    if (rc != kOk) {
        munmap(map, (size_t)st.st_size);
        delete g;
        return rc;
    }
    *out = g;
    return kOk;
}

void ferric_gguf_free(ferric_gguf* g)
{
    if (!g) return;
    if (g->mapping) munmap(g->mapping, g->len);
    delete g;
}

size_t ferric_gguf_n_tensors(const ferric_gguf* g) { return g ? g->tensors.size() : 0; }
size_t ferric_gguf_data_start(const ferric_gguf* g) { return g ? g->data_start : 0; }
size_t ferric_gguf_n_meta(const ferric_gguf* g) { return g ? g->keys.size() : 0; }

int32_t ferric_gguf_tensor_at(const ferric_gguf* g, size_t index, ferric_gguf_tensor* out)
{
    if (!g || !out || index >= g->tensors.size()) {
        set_last_error("NULL argument or tensor index out of range");
        return kErrInvalidArg;
    }
    fill_info(g, g->tensors[index], out);
    return kOk;
}

int32_t ferric_gguf_tensor_by_name(const ferric_gguf* g, const char* name, ferric_gguf_tensor* out)
{
    if (!g || !name || !out) {
        set_last_error("NULL argument");
        return kErrInvalidArg;
    }
    const TensorInfo* t = find_tensor(g, name);
    if (!t) {
        set_last_error("no tensor '%s'", name);
        return kErrInvalidArg;
    }
    fill_info(g, *t, out);
    return kOk;
}

int32_t ferric_gguf_raw(const ferric_gguf* g, const char* name, const uint8_t** data, size_t* nbytes)
{
    if (!g || !name || !data || !nbytes) {
        set_last_error("NULL argument");
        return kErrInvalidArg;
    }
    const TensorInfo* t = find_tensor(g, name);
    if (!t) {
        set_last_error("no tensor '%s'", name);
        return kErrInvalidArg;
    }
    return tensor_bytes(g, *t, data, nbytes);
}

int32_t ferric_gguf_meta_key_at(const ferric_gguf* g, size_t index, char* buf, size_t cap, size_t* len)
{
    if (!g || index >= g->keys.size()) {
        set_last_error("NULL handle or key index out of range");
        return kErrInvalidArg;
    }
    return copy_str(g->keys[index], buf, cap, len);
}

int32_t ferric_gguf_meta_kind(const ferric_gguf* g, const char* key, int32_t* kind)
{
    const Meta* m = find_meta(g, key, -1);
    if (!m || !kind) return kErrInvalidArg;
    *kind = m->kind;
    return kOk;
}

int32_t ferric_gguf_meta_u64(const ferric_gguf* g, const char* key, uint64_t* out)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_U);
    if (!m || !out) return kErrInvalidArg;
    *out = m->u;
    return kOk;
}

int32_t ferric_gguf_meta_i64(const ferric_gguf* g, const char* key, int64_t* out)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_I);
    if (!m || !out) return kErrInvalidArg;
    *out = m->i;
    return kOk;
}

int32_t ferric_gguf_meta_f64(const ferric_gguf* g, const char* key, double* out)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_F);
    if (!m || !out) return kErrInvalidArg;
    *out = m->f;
    return kOk;
}

int32_t ferric_gguf_meta_bool(const ferric_gguf* g, const char* key, int32_t* out)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_BOOL);
    if (!m || !out) return kErrInvalidArg;
    *out = m->b ? 1 : 0;
    return kOk;
}

int32_t ferric_gguf_meta_str(const ferric_gguf* g, const char* key, char* buf, size_t cap, size_t* len)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_STR);
    if (!m) return kErrInvalidArg;
    return copy_str(m->s, buf, cap, len);
}

int32_t ferric_gguf_meta_arr_len(const ferric_gguf* g, const char* key, size_t* n)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_ARR);
    if (!m || !n) return kErrInvalidArg;
    *n = m->arr.size();
    return kOk;
}

int32_t ferric_gguf_meta_arr_str(const ferric_gguf* g, const char* key, size_t index, char* buf, size_t cap, size_t* len)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_ARR);
    if (!m || index >= m->arr.size() || m->arr[index].kind != FERRIC_GGUF_META_STR) {
        if (m) set_last_error("array '%s' has no string element %zu", key, index);
        return kErrInvalidArg;
    }
    return copy_str(m->arr[index].s, buf, cap, len);
}

int32_t ferric_gguf_meta_arr_f64(const ferric_gguf* g, const char* key, size_t index, double* out)
{
    const Meta* m = find_meta(g, key, FERRIC_GGUF_META_ARR);
    if (!m || !out || index >= m->arr.size()) {
        if (m) set_last_error("array '%s' has no element %zu", key, index);
        return kErrInvalidArg;
    }
    const Meta& e = m->arr[index];
    switch (e.kind) {
    case FERRIC_GGUF_META_U: *out = (double)e.u; return kOk;
    case FERRIC_GGUF_META_I: *out = (double)e.i; return kOk;
    case FERRIC_GGUF_META_F: *out = e.f; return kOk;
    case FERRIC_GGUF_META_BOOL: *out = e.b ? 1.0 : 0.0; return kOk;
    default: set_last_error("element %zu of array '%s' is not a number", index, key); return kErrInvalidArg;
    }
}

// qm / qm_cat (crates/ferric-llama/src/qwen35.rs:366-402).
int32_t ferric_cuda_qmatrix_from_gguf(ferric_cuda_ctx* ctx, const ferric_gguf* g, const char* const* names, size_t n_names,
                                      ferric_qmatrix** out)
{
    if (!ctx || !g || !names || n_names == 0 || !out) {
        set_last_error("NULL argument or no tensor names");
        return kErrInvalidArg;
    }
    *out = nullptr;
    uint32_t ty = 0;
    size_t inn = 0, rows = 0, total = 0;
    std::vector<std::pair<const uint8_t*, size_t>> parts;
    for (size_t k = 0; k < n_names; k++) {
        const TensorInfo* t = names[k] ? find_tensor(g, names[k]) : nullptr;
        if (!t) {
            set_last_error("no tensor '%s'", names[k] ? names[k] : "(null)");
            return kErrInvalidArg;
        }
        if (t->dims.size() != 2) {
            set_last_error("%s: a weight matrix has two dims, this tensor has %zu", t->name.c_str(), t->dims.size());
            return kErrShape;
        }
        if (k == 0) {
            ty = t->ggml_type;
            inn = (size_t)t->dims[0];
        } else if (t->ggml_type != ty) {
            set_last_error("%s: mixed quant formats in one fused matmul", t->name.c_str());
            return kErrShape;
        } else if ((size_t)t->dims[0] != inn) {
            set_last_error("%s: input dim differs", t->name.c_str());
            return kErrShape;
        }
        rows += (size_t)t->dims[1];
        const uint8_t* p = nullptr;
        size_t nb = 0;
        const int32_t rc = tensor_bytes(g, *t, &p, &nb);
        if (rc != kOk) return rc;
        parts.emplace_back(p, nb);
        total += nb;
    }
    if (parts.size() == 1) return ferric_cuda_qmatrix_from_bytes(ctx, parts[0].first, parts[0].second, ty, rows, inn, out);
    std::vector<uint8_t> cat;
    cat.reserve(total);
    for (auto& pr : parts) cat.insert(cat.end(), pr.first, pr.first + pr.second);
    return ferric_cuda_qmatrix_from_bytes(ctx, cat.data(), cat.size(), ty, rows, inn, out);
}

// Proj::load (crates/ferric-llama/src/qwen3.rs:199-208).
int32_t ferric_cuda_proj_from_gguf(ferric_cuda_ctx* ctx, const ferric_gguf* g, const char* const* names, size_t n_names,
                                   ferric_proj** out)
{
    if (!ctx || !g || !names || n_names == 0 || n_names > 8 || !out) {
        set_last_error("NULL argument, or not 1..8 tensor names");
        return kErrInvalidArg;
    }
    *out = nullptr;
    bool same = true;
    uint32_t ty0 = 0;
    for (size_t k = 0; k < n_names; k++) {
        const TensorInfo* t = names[k] ? find_tensor(g, names[k]) : nullptr;
        if (!t) {
            set_last_error("no tensor '%s'", names[k] ? names[k] : "(null)");
            return kErrInvalidArg;
        }
        if (k == 0) ty0 = t->ggml_type;
        else if (t->ggml_type != ty0) same = false;
    }
    ferric_proj* p = new (std::nothrow) ferric_proj;
    if (!p) return kErrOom;
    int32_t rc = kOk;
    if (same) {   // Fused: the parts' bytes stacked into one matrix (qm_cat), or the single weight (qm)
        rc = ferric_cuda_qmatrix_from_gguf(ctx, g, names, n_names, &p->parts[0]);
        p->n_parts = rc == kOk ? 1 : 0;
    } else {      // Split: one matrix per part
        for (size_t k = 0; k < n_names && rc == kOk; k++) {
            rc = ferric_cuda_qmatrix_from_gguf(ctx, g, names + k, 1, &p->parts[k]);
            if (rc == kOk) p->n_parts++;
        }
    }
    if (rc == kOk) {
        p->cols = ferric_cuda_qmatrix_cols(p->parts[0]);
        for (size_t k = 0; k < p->n_parts; k++) {
            p->rows += ferric_cuda_qmatrix_rows(p->parts[k]);
            if (ferric_cuda_qmatrix_cols(p->parts[k]) != p->cols) {
                set_last_error("%s: input dim differs", names[k]);
                rc = kErrShape;
            }
        }
    }
    if (rc != kOk) {
        ferric_cuda_proj_free(p);
        return rc;
    }
    *out = p;
    return kOk;
}

}  // extern "C"
