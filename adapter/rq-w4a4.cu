// Replacement for the reference's ggml/src/ggml-cuda/rq-w4a4.cu (patches/llama.cpp-ruquant.patch:1589-2380): the six
// functions ggml-cuda's dispatcher calls, implemented on the C ABI of librq_b200.so (include/rq_b200.h).  The hooks in
// ggml-cuda.cu (patch:251-254, 295-299, 308-329, 338, 356-359) stay as the reference has them.
//
// Per-weight state lives in src0->extra, where the reference keeps its rq_tensor_info (patch:2027-2043).  The per-call
// scratch comes from the context's pool, as the reference's temporaries do, so nothing on the call path allocates.
#include "rq-w4a4.cuh"

#include "rq_b200.h"

#include <mutex>

namespace {

struct rq_b200_info {
    rq_weight_desc desc;
    void * prepack;
    float clip;
};

std::mutex g_prepare_mutex;      // several contexts (devices) may meet a weight for the first time at once

bool rq_is_w4a4(ggml_type t) { return t == GGML_TYPE_W4A4 || t == GGML_TYPE_W4A4H; }

// First use of a weight: the counterpart of rq_info + rq_repack_once (patch:2027-2075).  Not capture-safe, which is why
// ggml_cuda_rq_w4a4_ready exists.
rq_b200_info * rq_prepare_once(const ggml_tensor * src0, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_prepare_mutex);
    auto * info = (rq_b200_info *) src0->extra;
    if (info != nullptr) return info;
    info = new rq_b200_info{};
    const size_t n = rq_w4a4_prepack_bytes((int) src0->type, src0->ne[0], src0->ne[1], RQ_PREPACK_ALL);
    CUDA_CHECK(cudaMalloc(&info->prepack, n));
    const int rc = rq_w4a4_prepare(src0->data, (int) src0->type, src0->ne[0], src0->ne[1], info->prepack, n, RQ_PREPACK_ALL,
                                   &info->desc, stream);
    if (rc != RQ_OK) GGML_ABORT("W4A4: %s", rq_status_string(rc));     // the reference aborts on a bad rotation too (patch:2616)
    info->clip = rq_w4a4_resolve_clip(&info->desc);                    // environment, else header, else 1 (patch:2590-2600)
    const_cast<ggml_tensor *>(src0)->extra = info;
    return info;
}

void rq_mul_mat_n(const ggml_tensor * const * src0s, ggml_tensor * const * dsts, int n, const ggml_tensor * src1, void * ws,
                  size_t ws_bytes, cudaStream_t stream) {
    GGML_ASSERT(n >= 1 && n <= RQ_MAX_WEIGHTS);
    const rq_weight_desc * w[RQ_MAX_WEIGHTS];
    float * y[RQ_MAX_WEIGHTS];
    int64_t ldy[RQ_MAX_WEIGHTS];
    float clip = 1.0f;
    for (int i = 0; i < n; ++i) {
        rq_b200_info * info = rq_prepare_once(src0s[i], stream);
        w[i] = &info->desc;
        y[i] = (float *) dsts[i]->data;
        ldy[i] = (int64_t) (dsts[i]->nb[1] / sizeof(float));
        clip = info->clip;
    }
    const int64_t K = src1->ne[0], M = src1->ne[1];
    // pool memory is recycled: the workspace's status block (a sticky error word) starts every call at zero
    int rc = rq_w4a4_workspace_init(ws, K, M, stream);
    if (rc == RQ_OK) {
        rc = rq_w4a4_mul_mat(w, n, (const float *) src1->data, (int64_t) (src1->nb[1] / sizeof(float)), M, y, ldy, clip,
                             rq_w4a4_act_group(), RQ_PATH_AUTO, ws, ws_bytes, stream);
    }
    if (rc != RQ_OK) GGML_ABORT("W4A4: %s", rq_status_string(rc));
}

}  // namespace

// Admitted nodes, after ggml_cuda_rq_w4a4_supported of the reference (patch:1977-1994): 2-D, contiguous weight, f32
// activations with unit inner stride and 16-byte aligned rows, f32 output; Blackwell only (the library is sm_100a code).
// Unlike the reference any number of weight rows is admitted (it needs a multiple of 32).
bool ggml_cuda_rq_w4a4_supported(int cc, const ggml_tensor * src0, const ggml_tensor * src1, const ggml_tensor * dst) {
    if (!GGML_CUDA_CC_IS_NVIDIA(cc) || cc < 1000 || !rq_is_w4a4(src0->type)) return false;
    if (src1->type != GGML_TYPE_F32 || dst->type != GGML_TYPE_F32) return false;
    if (src0->ne[2] != 1 || src0->ne[3] != 1 || src1->ne[2] != 1 || src1->ne[3] != 1) return false;
    if (!ggml_is_contiguous(src0) || src1->nb[0] != sizeof(float) || dst->nb[0] != sizeof(float)) return false;
    if (dst->nb[1] % sizeof(float) != 0 || ((uintptr_t) src1->data & 15) != 0) return false;
    return rq_w4a4_supported((int) src0->type, src0->ne[0], src0->ne[1], src1->ne[1], (int64_t) src1->nb[1]) != 0;
}

bool ggml_cuda_rq_w4a4_ready(const ggml_tensor * src0) { return src0->extra != nullptr; }

void ggml_cuda_mul_mat_rq_w4a4_fused(ggml_backend_cuda_context & ctx, const ggml_tensor * const * src0s, ggml_tensor * const * dsts,
                                     int n, const ggml_tensor * src1) {
    const size_t ws_bytes = rq_w4a4_workspace_bytes(src1->ne[0], src1->ne[1]);
    ggml_cuda_pool_alloc<uint8_t> ws(ctx.pool(), ws_bytes + 256);       // stream-ordered pool; 256 for the alignment
    void * ws256 = (void *) (((uintptr_t) ws.get() + 255) & ~(uintptr_t) 255);
    rq_mul_mat_n(src0s, dsts, n, src1, ws256, ws_bytes, ctx.stream());
}

void ggml_cuda_mul_mat_rq_w4a4(ggml_backend_cuda_context & ctx, const ggml_tensor * src0, const ggml_tensor * src1, ggml_tensor * dst) {
    ggml_cuda_mul_mat_rq_w4a4_fused(ctx, &src0, &dst, 1, src1);
}

// The reference's predicate (patch:2350-2368) with its kernel-specific part replaced: there "both run the skinny kernel",
// here "both have been prepared" (which also implies both were seen outside a capture).  The width limit of 16 tokens is
// kept: wider inputs gain nothing from one launch over all rows.
bool ggml_cuda_rq_w4a4_can_fuse(const ggml_tensor * a, const ggml_tensor * b) {
    const ggml_tensor * wa = a->src[0];
    const ggml_tensor * wb = b->src[0];
    const ggml_tensor * x = a->src[1];
    if (a->op != GGML_OP_MUL_MAT || b->op != GGML_OP_MUL_MAT || b->src[1] != x || !rq_is_w4a4(wa->type) || wb->type != wa->type ||
        wb->ne[0] != wa->ne[0] || x->type != GGML_TYPE_F32 || ggml_nrows(x) != x->ne[1] || x->ne[1] > 16 ||
        a->type != GGML_TYPE_F32 || b->type != GGML_TYPE_F32) {
        return false;
    }
    const auto * ia = (const rq_b200_info *) wa->extra;
    const auto * ib = (const rq_b200_info *) wb->extra;
    return ia != nullptr && ib != nullptr && ia->clip == ib->clip && ia->desc.n_rot == ib->desc.n_rot &&
           ia->desc.wk_mode == ib->desc.wk_mode;
}

void ggml_cuda_rq_graph_begin(ggml_backend_cuda_context & ctx) { GGML_UNUSED(ctx); }

// The custom1 route has no backend context, hence no pool.  Up to 16 tokens it uses the library's entry point that needs
// no scratch from the caller; wider inputs use a per-device scratch that grows on demand -- growing allocates, so a host
// that captures graphs runs its widest input once before capturing, as it must for the weights' first use anyway.
extern "C" void rq_b200_custom1_mul_mat(cudaStream_t stream, ggml_tensor * dst) {
    const ggml_tensor * src0 = dst->src[0];
    const ggml_tensor * src1 = dst->src[1];
    GGML_ASSERT(src0 != nullptr && src1 != nullptr && rq_is_w4a4(src0->type));
    const int64_t K = src1->ne[0], M = src1->ne[1];
    if (M <= 16) {
        rq_b200_info * info = rq_prepare_once(src0, stream);
        const int rc = rq_w4a4_mul_mat_static(&info->desc, (const float *) src1->data, (int64_t) (src1->nb[1] / sizeof(float)), M,
                                              (float *) dst->data, (int64_t) (dst->nb[1] / sizeof(float)), info->clip,
                                              rq_w4a4_act_group(), RQ_PATH_AUTO, stream);
        if (rc != RQ_OK) GGML_ABORT("W4A4: %s", rq_status_string(rc));
        return;
    }
    static std::mutex mu;
    static void * scratch[GGML_CUDA_MAX_DEVICES] = {};
    static size_t scratch_bytes[GGML_CUDA_MAX_DEVICES] = {};
    int dev = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    const size_t need = rq_w4a4_workspace_bytes(K, M);
    void * ws;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (scratch_bytes[dev] < need) {
            CUDA_CHECK(cudaStreamSynchronize(stream));
            if (scratch[dev] != nullptr) CUDA_CHECK(cudaFree(scratch[dev]));
            CUDA_CHECK(cudaMalloc(&scratch[dev], need));
            scratch_bytes[dev] = need;
        }
        ws = scratch[dev];
    }
    rq_mul_mat_n(&src0, &dst, 1, src1, ws, need, stream);
}
