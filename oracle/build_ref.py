"""Builds oracle/_ref/libruquant_ref.so from the reference's own CPU code for the W4A4 MUL_MAT path.

TEST INFRASTRUCTURE ONLY.  Nothing on the product path may load what this script builds.

The reference ships its CPU path as added lines of a patch against ggml
(patches/llama.cpp-ruquant.patch: the `block_w4a4` struct in ggml/src/ggml-common.h, the quantizers and the
Hadamard in ggml/src/ggml-quants.c, `ggml_vec_dot_w4a4_a4` in ggml/src/ggml-cpu/quants.c).  ggml's own build
needs cmake, so instead this script takes those added lines from the patch *where it lies* (a path given on
the command line), writes them verbatim, between a small prelude and a threaded MUL_MAT driver of ours, to
`oracle/_ref/ruquant_ref.c` (git-ignored), and compiles that one file with gcc the way ggml-base is compiled
(-O3 -std=gnu11, no -march, so no FMA contraction).  No reference line is stored in this repository.

Usage: python oracle/build_ref.py [/path/to/reference]   (default: $RQ_REFERENCE_DIR, else a `reference` directory beside this repository)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# what ggml's headers give the extracted code; the enum ids are those of ggml/include/ggml.h in the patch
PRELUDE = r"""
#include <assert.h>
#include <math.h>
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#define GGML_RESTRICT restrict
#define GGML_API __attribute__((visibility("default")))
#define GGML_UNUSED(x) (void)(x)
#define UNUSED GGML_UNUSED
#define GGML_ABORT(...) do { fprintf(stderr, __VA_ARGS__); fputc('\n', stderr); abort(); } while (0)
#define GGML_ASSERT(x) do { if (!(x)) GGML_ABORT("GGML_ASSERT(%s) failed", #x); } while (0)
enum ggml_type { GGML_TYPE_W4A4 = 44, GGML_TYPE_W4A4H = 45, GGML_TYPE_A4 = 46, GGML_TYPE_A4H = 47 };
static size_t ggml_row_size(enum ggml_type type, int64_t ne) { (void) type; return (size_t) (ne / 256) * 144; }
"""

# the glue of ggml-cpu.c's mul_mat for these types (ggml/src/ggml-cpu/ggml-cpu.c hunk "ruquant A4 / A4H quantize
# per token"), restated over OpenMP threads: phase 1 quantizes token rows, phase 2 runs one vec_dot per output
DRIVER = r"""
GGML_API int rq_ref_mul_mat(const void * w, int type, int64_t K, int64_t N, const float * x, int64_t ldx, int64_t M,
                            float * y, int64_t ldy, int n_threads) {
    const bool had = type == GGML_TYPE_W4A4H;
    const float clip = ggml_rq_act_clip_for(ggml_rq_tensor_clip(w), had);
    const int64_t n_rot = had ? ggml_rq_tensor_rot(w, K) : 0;
    const size_t row = ggml_row_size(GGML_TYPE_W4A4, K);
    char * wdata = (char *) malloc(row * (size_t) M);
    if (!wdata) return -1;
    #pragma omp parallel for schedule(static) num_threads(n_threads)
    for (int64_t t = 0; t < M; ++t) {
        if (had) quantize_row_a4h_clip_n((float *) x + t*ldx, (block_w4a4 *) (wdata + t*row), K, clip, n_rot);
        else     quantize_row_a4_clip   ((float *) x + t*ldx, (block_w4a4 *) (wdata + t*row), K, clip);
    }
    #pragma omp parallel for schedule(dynamic, 16) num_threads(n_threads)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t t = 0; t < M; ++t) {
            ggml_vec_dot_w4a4_a4((int) K, y + t*ldy + n, 0, (const char *) w + n*row, 0, wdata + t*row, 0, 1);
        }
    }
    free(wdata);
    return 0;
}
GGML_API void rq_ref_quantize_act(const float * x, void * y, int64_t K, float clip, int64_t n_rot) {
    if (n_rot > 0) quantize_row_a4h_clip_n(x, (block_w4a4 *) y, K, clip, n_rot);
    else           quantize_row_a4_clip(x, (block_w4a4 *) y, K, clip);
}
GGML_API size_t rq_ref_quantize_weights(const float * src, void * dst, int64_t nrows, int64_t K, int type) {
    return type == GGML_TYPE_W4A4H ? quantize_w4a4h(src, dst, nrows, K, NULL) : quantize_w4a4(src, dst, nrows, K, NULL);
}
GGML_API float rq_ref_vec_dot(int64_t K, const void * w_row, const void * a_row) {
    float s;
    ggml_vec_dot_w4a4_a4((int) K, &s, 0, w_row, 0, a_row, 0, 1);
    return s;
}
"""


def added_lines(patch_lines, path, first_marker, last_marker):
    """The '+' lines of `path`'s diff from the one containing first_marker through the one equal to last_marker."""
    start = None
    for i, line in enumerate(patch_lines):
        if line.startswith("diff --git a/" + path + " "):
            start = i
            break
    if start is None:
        raise SystemExit("no diff for " + path)
    out, on = [], False
    for line in patch_lines[start + 1:]:
        if line.startswith("diff --git "):
            break
        if not line.startswith("+") or line.startswith("+++"):
            continue
        body = line[1:]
        if not on and first_marker in body:
            on = True
        if on:
            out.append(body)
            if body.rstrip() == last_marker:
                # the marker is a closing line that may repeat; the caller picks one that ends the span
                if last_marker != "}" or _balanced(out):
                    return out
    raise SystemExit("span not closed in " + path)


def _balanced(lines):
    text = "\n".join(lines)
    return text.count("{") == text.count("}")


REFERENCE_DIR = os.path.normpath(os.path.join(HERE, "..", "..", "reference"))      # the reference tree checked out beside this repository


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RQ_REFERENCE_DIR", REFERENCE_DIR)
    patch = os.path.join(ref, "patches", "llama.cpp-ruquant.patch")
    if not os.path.exists(patch):
        print("reference not present (%s): nothing built" % patch)
        return 1
    with open(patch, encoding="utf-8", errors="replace") as f:
        lines = f.read().split("\n")
    struct = added_lines(lines, "ggml/src/ggml-common.h", "#define QK_W4A4",
                         'static_assert(sizeof(block_w4a4) == 144, "wrong w4a4 block size/padding");')
    # ggml-quants.c: every added line of the first hunk, from rq_is_prime to the end of quantize_w4a4h
    start = next(i for i, l in enumerate(lines) if l.startswith("diff --git a/ggml/src/ggml-quants.c "))
    body = []
    for line in lines[start + 1:]:
        if line.startswith("diff --git "):
            break
        if line.startswith("@@") and body:
            break  # only the first hunk: the later one patches ggml_validate_row_data
        if line.startswith("+") and not line.startswith("+++"):
            body.append(line[1:])
    first = next(i for i, l in enumerate(body) if "static bool rq_is_prime" in l)
    quants = body[first:]
    vec_dot = added_lines(lines, "ggml/src/ggml-cpu/quants.c", "void ggml_vec_dot_w4a4_a4(", "}")
    # forward declarations the extracted code relies on (ggml-quants.h in the patch)
    protos = [l[1:] for l in lines if l.startswith("+GGML_API") and ("ggml_rq_" in l or "quantize_row_a4" in l
              or "quantize_row_w4a4" in l or "quantize_w4a4" in l)]
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(OUT, "ruquant_ref.c")
    with open(src, "w") as f:
        f.write("/* generated by oracle/build_ref.py from the reference patch; never committed */\n")
        f.write(PRELUDE)
        f.write("\n".join(struct) + "\n")
        f.write("\n".join(dict.fromkeys(protos)) + "\n")
        f.write("\n".join(quants) + "\n")
        f.write("\n".join(vec_dot) + "\n")
        f.write(DRIVER)
    so = os.path.join(OUT, "libruquant_ref.so")
    cmd = ["gcc", "-O3", "-std=gnu11", "-fPIC", "-shared", "-fopenmp", "-fvisibility=default", "-o", so, src, "-lm"]
    print(" ".join(cmd))
    subprocess.check_call(cmd)
    os.remove(src)   # keep only the library: the reference's lines do not stay on disk in this tree
    print("built", so)
    return 0


if __name__ == "__main__":
    sys.exit(main())
