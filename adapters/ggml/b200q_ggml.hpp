// b200q_ggml.hpp -- the glue between ggml's graph and the b200q C ABI, for a ggml backend that hands its
// MUL_MAT / MUL_MAT_ID nodes to this library.
//
// The reference does this work inside its patched ggml-opencl.cpp (marfrit/arcint contrib/llama.cpp/patches/
// 0000-01-kquant-integer-dpas.patch: ggml_backend_opencl_graph_compute :609-614, ggml_opencl_supports_op
// :615-652, ggml_cl_mul_mat :1135-1158, ggml_cl_mul_mat_id :1316-1328). ggml's headers are not part of this
// repository, so the glue is written against the FIELDS of ggml_tensor the path reads (type, ne, nb, data,
// src[], op) as templates: include ggml.h first and instantiate with ggml_tensor, or -- as this repository's
// device-free test does -- with any struct that has those members. ggml_type ids are used as they are
// (Q4_0 = 2, Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14, IQ4_NL = 20, IQ4_XS = 23, F32 = 0, I32 = 26).
//
// What a backend built on this does:
//   supports_op(op)        -> b200q_ggml::supports_op(op, GGML_OP_MUL_MAT, GGML_OP_MUL_MAT_ID)
//   graph_compute(cgraph)  -> b200q_ggml::graph_compute(ctx, cgraph->nodes, cgraph->n_nodes, GGML_OP_MUL_MAT,
//                             GGML_OP_MUL_MAT_ID, &failed_node); nodes of other ops are skipped (another backend's)
//   buffers                -> b200q_buffer_alloc / b200q_tensor_set / _get / b200q_synchronize
// tensor->data must be the device address (ggml backend buffers keep it there; a view's offset is already in it).
#pragma once

#include "../../include/b200q.h"

namespace b200q_ggml {

// the ggml_tensor fields the path reads; the tensor's address is its identity for the per-graph caches
// (the reference keys its caches the same way: `c.src1 == src1`, P01:683-688)
template <class Tensor>
inline b200q_tensor view(const Tensor *t) {
    b200q_tensor o;
    o.type = (int32_t)t->type;
    for (int i = 0; i < 4; ++i) {
        o.ne[i] = (int64_t)t->ne[i];
        o.nb[i] = (size_t)t->nb[i];
    }
    o.data = t->data;
    o.id = (const void *)t;
    return o;
}

template <class Tensor>
inline bool supports_op(const Tensor *op, int op_mul_mat, int op_mul_mat_id) {
    const bool is_id = (int)op->op == op_mul_mat_id;
    if ((int)op->op != op_mul_mat && !is_id) return false;
    if (!op->src[0] || !op->src[1] || (is_id && !op->src[2])) return false;
    const b200q_tensor s0 = view(op->src[0]), s1 = view(op->src[1]), d = view(op);
    b200q_tensor ids;
    if (is_id) ids = view(op->src[2]);
    return b200q_supports(nullptr, is_id ? B200Q_OP_MUL_MAT_ID : B200Q_OP_MUL_MAT, &s0, &s1, is_id ? &ids : nullptr, &d) == B200Q_OK;
}

// one node; B200Q_UNSUPPORTED for an op that is not ours (the caller's scheduler never sends those)
template <class Tensor>
inline b200q_status compute_node(b200q_ctx *ctx, const Tensor *node, int op_mul_mat, int op_mul_mat_id) {
    const bool is_id = (int)node->op == op_mul_mat_id;
    if ((int)node->op != op_mul_mat && !is_id) return B200Q_UNSUPPORTED;
    const b200q_tensor s0 = view(node->src[0]), s1 = view(node->src[1]);
    b200q_tensor d = view(node);
    if (!is_id) return b200q_mul_mat(ctx, &s0, &s1, &d);
    const b200q_tensor ids = view(node->src[2]);
    return b200q_mul_mat_id(ctx, &s0, &s1, &ids, &d);
}

// a whole graph: one cache generation, every MUL_MAT / MUL_MAT_ID node in order, asynchronous on the context's
// stream. On an error *failed is the node's index and the context's last_error has the text.
template <class Tensor>
inline b200q_status graph_compute(b200q_ctx *ctx, Tensor *const *nodes, int n_nodes, int op_mul_mat, int op_mul_mat_id, int *failed) {
    b200q_status st = b200q_graph_begin(ctx);
    for (int i = 0; i < n_nodes && st == B200Q_OK; ++i) {
        if ((int)nodes[i]->op != op_mul_mat && (int)nodes[i]->op != op_mul_mat_id) continue;
        st = compute_node(ctx, nodes[i], op_mul_mat, op_mul_mat_id);
        if (st != B200Q_OK && failed) *failed = i;
    }
    return st;
}

}  // namespace b200q_ggml
