// b200q_gguf.cpp -- the GGUF reader declared in b200q_gguf.h: mmap, one bounds-checked pass over the key/value
// section and the tensor table, nothing else. Plain C++ and POSIX, no ggml, no CUDA.
#include "b200q_gguf.h"

#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

namespace {

thread_local char g_error[256] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// value types of the kv section
enum { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64, T_COUNT };
const int SCALAR_BYTES[T_COUNT] = { 1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8 };

struct Kv {
    std::string key;
    uint32_t    type;
    uint64_t    pos;       // file offset of the value
};

struct Info {
    std::string name;
    int32_t     type, n_dims;
    int64_t     ne[4];
    uint64_t    offset;
};

// weights per block and bytes per block of the ggml types this path reads, and of plain f32 / f16 / i32
bool block_of(int32_t type, int *weights, int *bytes) {
    switch (type) {
    case B200Q_TYPE_F32:    *weights = 1;   *bytes = 4;   return true;
    case 1 /* F16 */:       *weights = 1;   *bytes = 2;   return true;
    case B200Q_TYPE_I32:    *weights = 1;   *bytes = 4;   return true;
    case B200Q_TYPE_Q4_0:   *weights = 32;  *bytes = 18;  return true;
    case B200Q_TYPE_Q8_0:   *weights = 32;  *bytes = 34;  return true;
    case B200Q_TYPE_IQ4_NL: *weights = 32;  *bytes = 18;  return true;
    case B200Q_TYPE_Q4_K:   *weights = 256; *bytes = 144; return true;
    case B200Q_TYPE_Q5_K:   *weights = 256; *bytes = 176; return true;
    case B200Q_TYPE_Q6_K:   *weights = 256; *bytes = 210; return true;
    case B200Q_TYPE_IQ4_XS: *weights = 256; *bytes = 136; return true;
    default: return false;
    }
}

struct Cursor {
    const uint8_t *base;
    uint64_t       size, pos;
    bool           ok;
    bool need(uint64_t n) {
        if (!ok || n > size - pos) { ok = false; return false; }
        return true;
    }
    template <typename T> T get() {
        T v = T();
        if (need(sizeof(T))) { memcpy(&v, base + pos, sizeof(T)); pos += sizeof(T); }
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        std::string s;
        if (n > (1u << 20)) { ok = false; return s; }          // keys and names are short; a huge length is a broken file
        if (need(n)) { s.assign((const char *)base + pos, (size_t)n); pos += n; }
        return s;
    }
    // steps over a value of the given type
    void skip(uint32_t type, int depth = 0) {
        if (type >= T_COUNT || depth > 4) { ok = false; return; }
        if (type == T_STR) { const uint64_t n = get<uint64_t>(); if (need(n)) pos += n; return; }
        if (type == T_ARR) {
            const uint32_t et = get<uint32_t>();
            const uint64_t cnt = get<uint64_t>();
            if (!ok || et >= T_COUNT) { ok = false; return; }
            if (et != T_STR && et != T_ARR) {
                const uint64_t eb = (uint64_t)SCALAR_BYTES[et];
                if (cnt > (size - pos) / eb) { ok = false; return; }
                pos += cnt * eb;
                return;
            }
            for (uint64_t i = 0; i < cnt && ok; ++i) skip(et, depth + 1);
            return;
        }
        if (need((uint64_t)SCALAR_BYTES[type])) pos += (uint64_t)SCALAR_BYTES[type];
    }
};

}  // namespace

struct b200q_gguf {
    int            fd = -1;
    const uint8_t *map = nullptr;
    uint64_t       size = 0;
    uint32_t       version = 0, alignment = 32;
    uint64_t       data_start = 0;
    std::vector<Kv>   kvs;
    std::vector<Info> infos;
};

extern "C" {

const char *b200q_gguf_error(void) { return g_error; }

void b200q_gguf_close(b200q_gguf *g) {
    if (!g) return;
    if (g->map) munmap((void *)g->map, (size_t)g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

b200q_gguf *b200q_gguf_open(const char *path) {
    if (!path) { set_error("null path"); return nullptr; }
    b200q_gguf *g = new b200q_gguf();
    g->fd = open(path, O_RDONLY);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        set_error("%s: cannot open, or shorter than a GGUF header", path);
        b200q_gguf_close(g);
        return nullptr;
    }
    g->size = (uint64_t)st.st_size;
    void *m = mmap(nullptr, (size_t)g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
        set_error("%s: mmap failed", path);
        b200q_gguf_close(g);
        return nullptr;
    }
    g->map = (const uint8_t *)m;
    Cursor c = { g->map, g->size, 0, true };
    if (memcmp(g->map, "GGUF", 4) != 0) {
        set_error("%s: not a GGUF file", path);
        b200q_gguf_close(g);
        return nullptr;
    }
    c.pos = 4;
    g->version = c.get<uint32_t>();
    if (g->version != 2 && g->version != 3) {
        set_error("%s: GGUF version %u (2 and 3 are read)", path, g->version);
        b200q_gguf_close(g);
        return nullptr;
    }
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (n_tensors > (1u << 24) || n_kv > (1u << 24)) c.ok = false;
    for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
        Kv kv;
        kv.key = c.str();
        kv.type = c.get<uint32_t>();
        kv.pos = c.pos;
        c.skip(kv.type);
        if (c.ok) g->kvs.push_back(kv);
    }
    for (uint64_t i = 0; i < n_tensors && c.ok; ++i) {
        Info t;
        t.name = c.str();
        t.n_dims = (int32_t)c.get<uint32_t>();
        if (t.n_dims < 0 || t.n_dims > 4) { c.ok = false; break; }
        for (int d = 0; d < 4; ++d) t.ne[d] = 1;
        for (int d = 0; d < t.n_dims; ++d) {
            t.ne[d] = (int64_t)c.get<uint64_t>();
            if (t.ne[d] < 0 || t.ne[d] > ((int64_t)1 << 40)) c.ok = false;
        }
        t.type = (int32_t)c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (c.ok) g->infos.push_back(t);
    }
    if (!c.ok) {
        set_error("%s: truncated or malformed header (stopped at byte %llu)", path, (unsigned long long)c.pos);
        b200q_gguf_close(g);
        return nullptr;
    }
    uint32_t al = 0;
    if (b200q_gguf_get_u32(g, "general.alignment", &al) == 0 && al >= 1 && al <= (1u << 20) && (al & (al - 1)) == 0) g->alignment = al;
    g->data_start = (c.pos + g->alignment - 1) / g->alignment * g->alignment;
    if (g->data_start > g->size) {
        set_error("%s: no data section", path);
        b200q_gguf_close(g);
        return nullptr;
    }
    return g;
}

uint32_t b200q_gguf_version(const b200q_gguf *g) { return g ? g->version : 0; }
uint32_t b200q_gguf_alignment(const b200q_gguf *g) { return g ? g->alignment : 0; }
int64_t b200q_gguf_tensor_count(const b200q_gguf *g) { return g ? (int64_t)g->infos.size() : 0; }
int64_t b200q_gguf_kv_count(const b200q_gguf *g) { return g ? (int64_t)g->kvs.size() : 0; }

size_t b200q_gguf_row_bytes(int32_t type, int64_t ne0) {
    int w = 0, b = 0;
    if (!block_of(type, &w, &b) || ne0 < 0 || ne0 % w) return 0;
    return (size_t)(ne0 / w) * (size_t)b;
}

int b200q_gguf_tensor_at(const b200q_gguf *g, int64_t i, b200q_gguf_tensor *out) {
    if (!g || !out || i < 0 || i >= (int64_t)g->infos.size()) return -1;
    const Info &t = g->infos[(size_t)i];
    out->name = t.name.c_str();
    out->type = t.type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->ne[d] = t.ne[d];
    out->offset = t.offset;
    const size_t rb = b200q_gguf_row_bytes(t.type, t.ne[0]);
    out->nbytes = (uint64_t)rb * (uint64_t)t.ne[1] * (uint64_t)t.ne[2] * (uint64_t)t.ne[3];
    out->data = nullptr;
    const uint64_t room = g->size - g->data_start;
    if (t.offset % g->alignment != 0 || t.offset > room || out->nbytes > room - t.offset) {
        set_error("tensor %s lies outside the file (offset %llu, %llu bytes)", t.name.c_str(), (unsigned long long)t.offset,
                  (unsigned long long)out->nbytes);
        return -2;
    }
    out->data = g->map + g->data_start + t.offset;
    return 0;
}

int b200q_gguf_find(const b200q_gguf *g, const char *name, b200q_gguf_tensor *out) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->infos.size(); ++i)
        if (g->infos[i].name == name) return b200q_gguf_tensor_at(g, (int64_t)i, out);
    return -1;
}

int b200q_gguf_get_u32(const b200q_gguf *g, const char *key, uint32_t *value) {
    if (!g || !key || !value) return -1;
    for (const Kv &kv : g->kvs)
        if (kv.key == key && kv.type == T_U32 && kv.pos + 4 <= g->size) {
            memcpy(value, g->map + kv.pos, 4);
            return 0;
        }
    return -1;
}

int b200q_gguf_get_str(const b200q_gguf *g, const char *key, const char **value, uint64_t *len) {
    if (!g || !key || !value || !len) return -1;
    for (const Kv &kv : g->kvs)
        if (kv.key == key && kv.type == T_STR && kv.pos + 8 <= g->size) {
            uint64_t n;
            memcpy(&n, g->map + kv.pos, 8);
            if (n > g->size - kv.pos - 8) return -1;
            *value = (const char *)g->map + kv.pos + 8;          // not NUL-terminated: use *len
            *len = n;
            return 0;
        }
    return -1;
}

b200q_status b200q_gguf_describe(const b200q_gguf_tensor *t, void *device_ptr, b200q_tensor *out) {
    if (!t || !out) return B200Q_INVALID;
    const size_t rb = b200q_gguf_row_bytes(t->type, t->ne[0]);
    int w = 0, b = 0;
    if (!rb || !block_of(t->type, &w, &b) || t->type == 1) return B200Q_UNSUPPORTED;
    out->type = t->type;
    for (int d = 0; d < 4; ++d) out->ne[d] = t->ne[d];
    out->nb[0] = (size_t)b;
    out->nb[1] = rb;
    out->nb[2] = rb * (size_t)t->ne[1];
    out->nb[3] = out->nb[2] * (size_t)t->ne[2];
    out->data = device_ptr;
    out->id = device_ptr;
    return B200Q_OK;
}

}  // extern "C"
