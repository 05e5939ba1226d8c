/*
 * b200q_gguf.h -- a small reader of GGUF files (versions 2 and 3) for callers that want to feed b200q without ggml:
 * it maps the file, walks the key/value section and the tensor table, and hands out each tensor's name, ggml type,
 * extents and a pointer to its bytes inside the mapping. The weights of this path are consumed as stored (GGUF
 * blocks, rows back to back), so "loading" a weight is one copy of [data, data + nbytes) to the device and a
 * b200q_tensor over it (b200q_gguf_describe fills one).
 *
 * The reference reads GGUF through llama.cpp's loader and repacks at set_tensor (marfrit/arcint
 * contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch:745-779); here nothing is repacked.
 *
 * File layout (the public GGUF specification): magic "GGUF", u32 version, u64 tensor count, u64 kv count; kv pairs
 * (string key, u32 value type, value; strings are u64 length + bytes, arrays are u32 element type + u64 count +
 * elements); tensor infos (string name, u32 n_dims, u64 dims[n_dims], u32 ggml type, u64 offset); then the data
 * section at the next multiple of general.alignment (default 32), tensor offsets relative to it.
 */
#ifndef B200Q_GGUF_H
#define B200Q_GGUF_H

#include <stddef.h>
#include <stdint.h>

#include "../../include/b200q.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200q_gguf b200q_gguf;

typedef struct {
    const char *name;        /* NUL-terminated copy owned by the reader */
    int32_t     type;        /* ggml type id as stored */
    int32_t     n_dims;
    int64_t     ne[4];       /* ne[0] fastest; 1 past n_dims */
    uint64_t    offset;      /* from the start of the data section */
    uint64_t    nbytes;      /* 0 when the type's block size is not known to this reader */
    const void *data;        /* inside the mapping; valid until b200q_gguf_close */
} b200q_gguf_tensor;

/* NULL on failure; b200q_gguf_error() says why (thread-local text). */
b200q_gguf *b200q_gguf_open(const char *path);
void        b200q_gguf_close(b200q_gguf *g);
const char *b200q_gguf_error(void);

uint32_t b200q_gguf_version(const b200q_gguf *g);
uint32_t b200q_gguf_alignment(const b200q_gguf *g);
int64_t  b200q_gguf_tensor_count(const b200q_gguf *g);
int64_t  b200q_gguf_kv_count(const b200q_gguf *g);
/* 0 on success */
int b200q_gguf_tensor_at(const b200q_gguf *g, int64_t i, b200q_gguf_tensor *out);
int b200q_gguf_find(const b200q_gguf *g, const char *name, b200q_gguf_tensor *out);
/* string and u32 values of the kv section by key; 0 on success */
int b200q_gguf_get_u32(const b200q_gguf *g, const char *key, uint32_t *value);
int b200q_gguf_get_str(const b200q_gguf *g, const char *key, const char **value, uint64_t *len);

/* bytes of one row of ne0 weights of a type b200q takes; 0 for other types */
size_t b200q_gguf_row_bytes(int32_t type, int64_t ne0);
/* A b200q_tensor over `device_ptr` (where the caller copied t->data .. + t->nbytes): packed rows, nb[1] = row bytes,
 * up to four dimensions (a stack of expert matrices is ne[2] > 1); id = device_ptr. B200Q_UNSUPPORTED for a type
 * outside the path, B200Q_INVALID for a null argument. */
b200q_status b200q_gguf_describe(const b200q_gguf_tensor *t, void *device_ptr, b200q_tensor *out);

#ifdef __cplusplus
}
#endif
#endif
