"""Device-free checks that the boundary is what it claims: include/b200q.h compiles as plain C and links against
the library (a C consumer, not only ctypes), and the ggml glue (adapters/ggml/b200q_ggml.hpp) compiles against a
struct with ggml_tensor's field names and answers supports_op like the reference's gate
(marfrit/arcint contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch:615-652)."""
import os
import shutil
import subprocess

import pytest

import arcint_b200 as A

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

C_SRC = r'''
#include <stdio.h>
#include <string.h>
#include "b200q.h"
int main(void) {
    b200q_tensor w, x, y;
    memset(&w, 0, sizeof w); memset(&x, 0, sizeof x); memset(&y, 0, sizeof y);
    w.type = B200Q_TYPE_Q4_K; w.ne[0] = 4096; w.ne[1] = 11008; w.ne[2] = w.ne[3] = 1;
    w.nb[0] = 144; w.nb[1] = 2304; w.nb[2] = w.nb[3] = 2304 * 11008; w.data = (void *)0x10000;
    x.type = B200Q_TYPE_F32; x.ne[0] = 4096; x.ne[1] = 8; x.ne[2] = x.ne[3] = 1;
    x.nb[0] = 4; x.nb[1] = 16384; x.nb[2] = x.nb[3] = 131072; x.data = (void *)0x20000;
    y.type = B200Q_TYPE_F32; y.ne[0] = 11008; y.ne[1] = 8; y.ne[2] = y.ne[3] = 1;
    y.nb[0] = 4; y.nb[1] = 44032; y.nb[2] = y.nb[3] = 352256; y.data = (void *)0x30000;
    if (b200q_supports(NULL, B200Q_OP_MUL_MAT, &w, &x, NULL, &y) != B200Q_OK) return 1;
    w.ne[0] = 4100;                                  /* K not a multiple of the block: refused, not guessed */
    if (b200q_supports(NULL, B200Q_OP_MUL_MAT, &w, &x, NULL, &y) != B200Q_UNSUPPORTED) return 2;
    printf("%s %d\n", b200q_version(), (int)sizeof(b200q_tensor));
    return 0;
}
'''

CPP_SRC = r'''
#include <stdint.h>
#include <stdio.h>
#include <string.h>
// a struct with the members of ggml_tensor the glue reads (ggml.h itself is not in this repository)
enum { OP_ADD = 2, OP_MUL_MAT = 27, OP_MUL_MAT_ID = 28 };
struct fake_tensor { int type; int op; int64_t ne[4]; size_t nb[4]; void *data; fake_tensor *src[3]; };
#include "adapters/ggml/b200q_ggml.hpp"
static fake_tensor make(int type, int64_t e0, int64_t e1, int64_t e2, size_t b0, void *data) {
    fake_tensor t; memset(&t, 0, sizeof t);
    t.type = type; t.ne[0] = e0; t.ne[1] = e1; t.ne[2] = e2; t.ne[3] = 1;
    t.nb[0] = b0; t.nb[1] = b0 * (size_t)(type == 0 || type == 26 ? e0 : e0 / 32); t.nb[2] = t.nb[1] * (size_t)e1; t.nb[3] = t.nb[2] * (size_t)e2;
    t.data = data; return t;
}
int main() {
    fake_tensor w = make(2, 4096, 512, 1, 18, (void *)0x10000), x = make(0, 4096, 4, 1, 4, (void *)0x20000), y = make(0, 512, 4, 1, 4, (void *)0x30000);
    y.op = OP_MUL_MAT; y.src[0] = &w; y.src[1] = &x;
    if (!b200q_ggml::supports_op(&y, OP_MUL_MAT, OP_MUL_MAT_ID)) return 1;
    y.op = OP_ADD;
    if (b200q_ggml::supports_op(&y, OP_MUL_MAT, OP_MUL_MAT_ID)) return 2;
    // MUL_MAT_ID: 8 experts, 2 used, 5 tokens
    fake_tensor we = make(2, 4096, 512, 8, 18, (void *)0x10000), xe = make(0, 4096, 1, 5, 4, (void *)0x20000);
    fake_tensor ids = make(26, 2, 5, 1, 4, (void *)0x40000), ye = make(0, 512, 2, 5, 4, (void *)0x30000);
    ye.op = OP_MUL_MAT_ID; ye.src[0] = &we; ye.src[1] = &xe; ye.src[2] = &ids;
    if (!b200q_ggml::supports_op(&ye, OP_MUL_MAT, OP_MUL_MAT_ID)) return 3;
    const b200q_tensor v = b200q_ggml::view(&we);
    if (v.id != (const void *)&we || v.ne[2] != 8 || v.type != B200Q_TYPE_Q4_0) return 4;
    // graph_compute and compute_node are instantiated (and so type-checked) without being run: no device here
    b200q_status (*gc)(b200q_ctx *, fake_tensor *const *, int, int, int, int *) = &b200q_ggml::graph_compute<fake_tensor>;
    printf("ok %p\n", (void *)gc);
    return 0;
}
'''


def _run(tmp_path, name, src, compiler, flags):
    cc = shutil.which(compiler)
    if not cc:
        pytest.skip(compiler + " not found")
    f = tmp_path / name
    f.write_text(src)
    exe = tmp_path / (name + ".exe")
    libdir = os.path.dirname(A.lib_path())
    cmd = [cc] + flags + ["-I", os.path.join(ROOT, "include"), "-I", ROOT, str(f), "-o", str(exe), "-L", libdir, "-lb200q",
                          "-Wl,-rpath," + libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    return r.stdout


def test_header_is_plain_c_and_links(tmp_path):
    A.lib()
    out = _run(tmp_path, "consumer.c", C_SRC, "gcc", ["-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic"])
    assert "sm_100a" in out and out.strip().endswith("88")


def test_ggml_glue_compiles_and_gates(tmp_path):
    A.lib()
    out = _run(tmp_path, "glue.cpp", CPP_SRC, "g++", ["-std=c++17", "-Wall", "-Wextra", "-Werror"])
    assert out.startswith("ok")


GGUF_C_SRC = r'''
#include <stdio.h>
#include <string.h>
#include "adapters/gguf/b200q_gguf.h"
#include "b200q_test.h"
int main(int argc, char **argv) {
    b200q_gguf *g = b200q_gguf_open(argc > 1 ? argv[1] : "");
    b200q_gguf_tensor t;
    b200q_tensor d;
    if (!g) { printf("open failed: %s\n", b200q_gguf_error()); return 1; }
    if (b200q_gguf_find(g, "blk.0.q4_K.weight", &t) != 0) return 2;
    if (b200q_gguf_describe(&t, (void *)0x1000, &d) != B200Q_OK || d.type != B200Q_TYPE_Q4_K || d.nb[1] != 288) return 3;
    printf("%d tensors, %s: %d x %d, %d bytes\n", (int)b200q_gguf_tensor_count(g), t.name, (int)t.ne[0], (int)t.ne[1], (int)t.nbytes);
    b200q_gguf_close(g);
    return 0;
}
'''


def test_gguf_reader_header_is_plain_c(tmp_path):
    """adapters/gguf/b200q_gguf.h (and include/b200q_test.h) compile as C99; a C program reads the fixture through the reader."""
    from arcint_b200 import build as B
    cc = shutil.which("gcc")
    if not cc:
        pytest.skip("gcc not found")
    so = B.build_gguf()
    f = tmp_path / "reader.c"
    f.write_text(GGUF_C_SRC)
    exe = tmp_path / "reader.exe"
    libdir = os.path.dirname(so)
    r = subprocess.run([cc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), "-I", ROOT, str(f), "-o",
                        str(exe), "-L", libdir, "-lb200q_gguf", "-Wl,-rpath," + libdir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe), os.path.join(ROOT, "tests", "golden", "tiny.gguf")], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "blk.0.q4_K.weight: 512 x 16, 4608 bytes" in r.stdout
