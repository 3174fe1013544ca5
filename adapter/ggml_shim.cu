// Test harness for the ggml-cuda adapter (rq-w4a4.cu): the handful of ggml / ggml-cuda symbols the adapter links against,
// in their simplest form, and a C interface through which a test builds real `ggml_tensor` structs (ggml.h's own type,
// filled in by hand: no ggml allocator, no graph) and drives the six entry points and the custom1 hook the way
// ggml-cuda's dispatcher does (patches/llama.cpp-ruquant.patch:251-254, 282-287, 308-329).  TEST INFRASTRUCTURE: the
// product is rq-w4a4.cu + librq_b200.so; in a real build ggml itself provides everything defined here.
#include "rq-w4a4.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

// ---- what ggml.c / ggml-cuda.cu would provide

extern "C" void ggml_abort(const char * file, int line, const char * fmt, ...) {
    fprintf(stderr, "%s:%d: ", file, line);
    va_list ap;
    va_start(ap, fmt);
    vfprintf(stderr, fmt, ap);
    va_end(ap);
    fprintf(stderr, "\n");
    abort();
}

static size_t shim_row_bytes(const ggml_tensor * t) {
    if (t->type == GGML_TYPE_W4A4 || t->type == GGML_TYPE_W4A4H) return (size_t) (t->ne[0] / 256) * 144;
    return (size_t) t->ne[0] * t->nb[0];
}

extern "C" bool ggml_is_contiguous(const ggml_tensor * t) {
    return t->nb[1] == shim_row_bytes(t) && t->nb[2] == t->nb[1] * (size_t) t->ne[1] && t->nb[3] == t->nb[2] * (size_t) t->ne[2];
}

extern "C" int64_t ggml_nrows(const ggml_tensor * t) { return t->ne[1] * t->ne[2] * t->ne[3]; }

void ggml_cuda_set_device(int device) { cudaSetDevice(device); }

void ggml_cuda_error(const char * stmt, const char * func, const char * file, int line, const char * msg) {
    fprintf(stderr, "CUDA error: %s\n  in %s at %s:%d: %s\n", msg, func, file, line, stmt);
    abort();
}

// buffers are recycled in allocation order on one stream, like ggml-cuda's legacy pool
struct shim_pool : ggml_cuda_pool {
    struct buf { void * ptr; size_t size; };
    std::vector<buf> free_list;
    ~shim_pool() override { for (auto & b : free_list) cudaFree(b.ptr); }
    void * alloc(size_t size, size_t * actual_size) override {
        for (size_t i = 0; i < free_list.size(); ++i) {
            if (free_list[i].size >= size) {
                buf b = free_list[i];
                free_list.erase(free_list.begin() + (long) i);
                *actual_size = b.size;
                return b.ptr;
            }
        }
        void * p = nullptr;
        CUDA_CHECK(cudaMalloc(&p, size));
        *actual_size = size;
        return p;
    }
    void free(void * ptr, size_t size) override { free_list.push_back({ ptr, size }); }
};

std::unique_ptr<ggml_cuda_pool> ggml_backend_cuda_context::new_pool_for_device(int device, int stream_no) {
    GGML_UNUSED(device); GGML_UNUSED(stream_no);
    return std::unique_ptr<ggml_cuda_pool>(new shim_pool());
}

ggml_backend_cuda_context::~ggml_backend_cuda_context() {
    for (int d = 0; d < GGML_CUDA_MAX_DEVICES; ++d)
        for (int s = 0; s < GGML_CUDA_MAX_STREAMS; ++s)
            if (streams[d][s] != nullptr) cudaStreamDestroy(streams[d][s]);
}

// the hook of patch:263-272
typedef void (* ggml_cuda_custom1_fn)(cudaStream_t stream, struct ggml_tensor * dst);
static ggml_cuda_custom1_fn g_custom1 = nullptr;
extern "C" void ggml_cuda_set_custom1_hook(ggml_cuda_custom1_fn fn) { g_custom1 = fn; }

// ---- the test's interface

extern "C" {

void * shim_ctx_new(int device) { return new ggml_backend_cuda_context(device); }
void shim_ctx_free(void * ctx) { delete (ggml_backend_cuda_context *) ctx; }
void * shim_ctx_stream(void * ctx) { return ((ggml_backend_cuda_context *) ctx)->stream(); }
void shim_ctx_sync(void * ctx) { cudaStreamSynchronize(((ggml_backend_cuda_context *) ctx)->stream()); }

// a 2-D tensor over caller-owned device memory; nb1 = 0 means contiguous rows
void * shim_tensor_new(int type, int64_t ne0, int64_t ne1, void * data, size_t nb1) {
    ggml_tensor * t = new ggml_tensor();
    memset(t, 0, sizeof(*t));
    t->type = (ggml_type) type;
    t->ne[0] = ne0; t->ne[1] = ne1; t->ne[2] = 1; t->ne[3] = 1;
    t->nb[0] = (t->type == GGML_TYPE_W4A4 || t->type == GGML_TYPE_W4A4H) ? 144 : sizeof(float);
    t->nb[1] = nb1 ? nb1 : shim_row_bytes(t);
    t->nb[2] = t->nb[1] * (size_t) ne1;
    t->nb[3] = t->nb[2];
    t->op = GGML_OP_NONE;
    t->data = data;
    return t;
}
void shim_tensor_free(void * t) { delete (ggml_tensor *) t; }

// dst = mul_mat(w, x) (custom1 != 0: the same node as a GGML_OP_MAP_CUSTOM1 with src[0] = w, src[1] = x)
void * shim_node_new(void * w, void * x, void * ydata, size_t y_nb1, int custom1) {
    ggml_tensor * a = (ggml_tensor *) w, * b = (ggml_tensor *) x;
    ggml_tensor * d = (ggml_tensor *) shim_tensor_new(GGML_TYPE_F32, a->ne[1], b->ne[1], ydata, y_nb1);
    d->op = custom1 ? GGML_OP_MAP_CUSTOM1 : GGML_OP_MUL_MAT;
    d->src[0] = a;
    d->src[1] = b;
    return d;
}

int shim_supported(int cc, void * node) {
    ggml_tensor * d = (ggml_tensor *) node;
    return ggml_cuda_rq_w4a4_supported(cc, d->src[0], d->src[1], d) ? 1 : 0;
}
int shim_ready(void * w) { return ggml_cuda_rq_w4a4_ready((ggml_tensor *) w) ? 1 : 0; }
void shim_mul_mat(void * ctx, void * node) {
    ggml_tensor * d = (ggml_tensor *) node;
    ggml_cuda_mul_mat_rq_w4a4(*(ggml_backend_cuda_context *) ctx, d->src[0], d->src[1], d);
}
int shim_can_fuse(void * a, void * b) { return ggml_cuda_rq_w4a4_can_fuse((ggml_tensor *) a, (ggml_tensor *) b) ? 1 : 0; }
void shim_fused(void * ctx, void ** nodes, int n) {
    const ggml_tensor * src0s[3];
    ggml_tensor * dsts[3];
    for (int i = 0; i < n && i < 3; ++i) { dsts[i] = (ggml_tensor *) nodes[i]; src0s[i] = dsts[i]->src[0]; }
    ggml_cuda_mul_mat_rq_w4a4_fused(*(ggml_backend_cuda_context *) ctx, src0s, dsts, n, dsts[0]->src[1]);
}
void shim_graph_begin(void * ctx) { ggml_cuda_rq_graph_begin(*(ggml_backend_cuda_context *) ctx); }
// the dispatcher's case GGML_OP_MAP_CUSTOM1 (patch:282-287): 0 when no hook is registered
int shim_custom1(void * ctx, void * node) {
    if (g_custom1 == nullptr) return 0;
    g_custom1(((ggml_backend_cuda_context *) ctx)->stream(), (ggml_tensor *) node);
    return 1;
}
void shim_register_hook(void) { ggml_cuda_set_custom1_hook(rq_b200_custom1_mul_mat); }

}  // extern "C"
