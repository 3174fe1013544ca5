// C ABI of the library (declared in include/rq_b200.h): argument checks, header decoding, layout bookkeeping and
// kernel dispatch.  Mirrors the host logic of the reference's ggml/src/ggml-cuda/rq-w4a4.cu
// (patches/llama.cpp-ruquant.patch:1977-2043 supported / first-use header read, 2145-2338 dispatch) with status
// codes in place of aborts and with every first-use step moved into rq_w4a4_prepare.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "rq_common.cuh"

static thread_local int g_last_cuda = 0;

#define RQ_CUDA(call)                                             \
    do {                                                          \
        const cudaError_t e_ = (call);                            \
        if (e_ != cudaSuccess) { g_last_cuda = (int) e_; return RQ_ERR_CUDA; } \
    } while (0)

extern "C" __attribute__((visibility("default"))) int rq_last_cuda_error(void) { return g_last_cuda; }

extern "C" __attribute__((visibility("default"))) const char * rq_status_string(int status) {
    switch (status) {
        case RQ_OK:            return "ok";
        case RQ_ERR_ARG:       return "bad argument (null pointer, type id or count)";
        case RQ_ERR_SHAPE:     return "unsupported shape (K must be a multiple of 256 and <= 32768; rows 16-byte aligned)";
        case RQ_ERR_ROTATION:  return "W4A4H: Hadamard length does not divide K or does not factor (ruquant convert --rot-blocks)";
        case RQ_ERR_GROUP:     return "activation group must be 64, 128 or 256 (64 with weight groups of 64)";
        case RQ_ERR_WORKSPACE: return "workspace or prepack buffer too small or misaligned";
        case RQ_ERR_CUDA:      return "CUDA call failed (see rq_last_cuda_error)";
        case RQ_ERR_MISMATCH:  return "weights of one call differ in K, type or rotation";
        case RQ_ERR_DEVICE:    return "a kernel gave up on a bounded wait";
        case RQ_ERR_CLIP:      return "clip must be finite and > 0";
        case RQ_ERR_LIMIT:     return "size beyond a fixed maximum";
        default:               return "unknown status";
    }
}

static bool rq_is_prime(int q) {
    if (q < 2) return false;
    for (int d = 2; d * d <= q; ++d) if (q % d == 0) return false;
    return true;
}

// ggml_rq_hadamard_factor, ggml/src/ggml-quants.c in patch:2419-2430
extern "C" __attribute__((visibility("default"))) int rq_hadamard_factor(int64_t n, int * p, int * m) {
    for (int c = 1; c <= 128 && c <= n; ++c) {
        if (c > 1 && !(c % 4 == 0 && rq_is_prime(c - 1) && (c - 1) % 4 == 3)) continue;
        if (n % c != 0) continue;
        const int64_t rest = n / c;
        if (rest & (rest - 1)) continue;
        if (p) *p = c;
        if (m) *m = (int) rest;
        return 1;
    }
    return 0;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_supported(int type, int64_t K, int64_t N, int64_t M, int64_t ldx_bytes) {
    if (type != RQ_TYPE_W4A4 && type != RQ_TYPE_W4A4H) return 0;
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || K > RQ_MAX_K || N < 1 || M < 1) return 0;
    if (ldx_bytes < K * 4 || ldx_bytes % 16 != 0) return 0;
    if (type == RQ_TYPE_W4A4H && !rq_hadamard_factor(K, nullptr, nullptr)) return 0;
    return 1;
}

// ggml_rq_act_clip_for, patch:2590-2600: RQ_ACT_CLIP (and RQ_ACT_CLIP_H for rotated inputs, defaulting to
// RQ_ACT_CLIP) win over the tensor's own clip, which wins over 1
// A header clip that is not > 0 counts as unset there, NaN included; +infinity is treated as unset here as well (the
// reference would scale every range by infinity).
struct rq_env_clips { float plain, hadamard; };
extern "C" __attribute__((visibility("default"))) float rq_w4a4_resolve_clip(const rq_weight_desc * w) {
    static const rq_env_clips env = []() {          // read once; -1: not set (thread-safe static initialisation)
        const char * e = getenv("RQ_ACT_CLIP");
        const char * eh = getenv("RQ_ACT_CLIP_H");
        rq_env_clips c;
        c.plain = e ? (float) atof(e) : -1.0f;
        c.hadamard = eh ? (float) atof(eh) : c.plain;
        return c;
    }();
    const bool had = w != nullptr && w->type == RQ_TYPE_W4A4H;
    const float e = had ? env.hadamard : env.plain;
    const float t = w != nullptr ? w->header_clip : 0.0f;
    if (e > 0.0f && !isinf(e)) return e;
    return (t > 0.0f && !isinf(t)) ? t : 1.0f;
}

// ggml_rq_act_group, patch:2623-2631
extern "C" __attribute__((visibility("default"))) int rq_w4a4_act_group(void) {
    static const int g = []() {
        const char * e = getenv("RQ_ACT_GROUP");
        const int v = e ? atoi(e) : 64;
        return (v == 128 || v == 256) ? v : 64;
    }();
    return g;
}

struct rq_pp_layout {
    uint64_t off_sw, off_w4, off_w8, off_wk, bytes;
};
static rq_pp_layout rq_pp(int64_t K, int64_t N, int layouts) {
    rq_pp_layout l;
    l.off_sw = 0;
    l.off_wk = rq_align256((uint64_t) N * 4);
    l.off_w4 = l.off_wk + rq_align256((uint64_t) N * (K / 64));
    l.off_w8 = l.off_w4 + ((layouts & RQ_PREPACK_DECODE) ? rq_align256((uint64_t) ((N + 15) / 16) * 16 * K / 2) : 0);
    l.bytes = l.off_w8 + ((layouts & RQ_PREPACK_PREFILL) ? rq_align256((uint64_t) N * K) : 0);
    return l;
}

extern "C" __attribute__((visibility("default"))) size_t rq_w4a4_prepack_bytes(int type, int64_t K, int64_t N, int layouts) {
    if ((type != RQ_TYPE_W4A4 && type != RQ_TYPE_W4A4H) || K <= 0 || K % RQ_BLOCK_CODES != 0 || N < 1) return 0;
    return (size_t) rq_pp(K, N, layouts & RQ_PREPACK_ALL).bytes;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_prepare(const void * w_blocks_dev, int type, int64_t K, int64_t N, void * prepack_dev,
                               size_t prepack_bytes, int layouts, rq_weight_desc * out, void * stream_) {
    cudaStream_t stream = (cudaStream_t) stream_;
    if (w_blocks_dev == nullptr || prepack_dev == nullptr || out == nullptr) return RQ_ERR_ARG;
    if (type != RQ_TYPE_W4A4 && type != RQ_TYPE_W4A4H) return RQ_ERR_ARG;
    layouts &= RQ_PREPACK_ALL;
    if (layouts == 0) return RQ_ERR_ARG;
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || K > RQ_MAX_K || N < 1) return RQ_ERR_SHAPE;
    const rq_pp_layout l = rq_pp(K, N, layouts);
    if (prepack_bytes < l.bytes || (reinterpret_cast<uintptr_t>(prepack_dev) & 255) != 0) return RQ_ERR_WORKSPACE;

    // block 0 of row 0 carries the tensor's switches (ggml_rq_tensor_clip / ggml_rq_tensor_rot, patch:2602-2610;
    // rq_info, patch:2027-2043): sum -> weight-group mode, pad[0] -> Hadamard length, pad[1] -> clip
    RQ_CUDA(rq_configure_act());
    RQ_CUDA(rq_configure_gemm_tc());
    rq_block hdr;
    uint8_t * pp = static_cast<uint8_t *>(prepack_dev);
    int32_t * flag_dev = reinterpret_cast<int32_t *>(pp + l.off_wk);   // scratch until the pack kernel overwrites it
    int32_t flag = 0;
    RQ_CUDA(cudaMemcpyAsync(&hdr, w_blocks_dev, 16, cudaMemcpyDeviceToHost, stream));
    RQ_CUDA(cudaMemsetAsync(flag_dev, 0, 4, stream));
    RQ_CUDA(rq_launch_scan_wk(static_cast<const rq_block *>(w_blocks_dev), N * (K / RQ_BLOCK_CODES), flag_dev, stream));
    RQ_CUDA(cudaMemcpyAsync(&flag, flag_dev, 4, cudaMemcpyDeviceToHost, stream));
    RQ_CUDA(cudaStreamSynchronize(stream));

    memset(out, 0, sizeof(*out));
    out->type = type;
    out->layouts = layouts;
    out->K = K;
    out->N = N;
    memcpy(&out->header_clip, &hdr.pad[1], 4);      // kept as read; rq_w4a4_resolve_clip decides whether it counts
    out->wg64 = (((uint32_t) hdr.sum) >> 29) == 3u ? 1 : 0;
    out->wk_mode = flag ? 1 : 0;
    out->had_p = 1;
    if (type == RQ_TYPE_W4A4H) {
        const int32_t n = hdr.pad[0];   // ggml_rq_rot_check, patch:2612-2620
        int p = 0, m = 0;
        if (n <= 0 || K % n != 0 || !rq_hadamard_factor(n, &p, &m)) return RQ_ERR_ROTATION;
        out->n_rot = n;
        out->had_p = p;
        out->had_m = m;
    }
    out->blocks = w_blocks_dev;
    out->prepack = prepack_dev;
    out->off_sw = l.off_sw;
    out->off_w4 = l.off_w4;
    out->off_w8 = l.off_w8;
    out->off_wk = l.off_wk;

    RQ_CUDA(rq_launch_prepack(static_cast<const rq_block *>(w_blocks_dev), K, N, reinterpret_cast<float *>(pp + l.off_sw),
                              (layouts & RQ_PREPACK_DECODE) ? pp + l.off_w4 : nullptr,
                              (layouts & RQ_PREPACK_PREFILL) ? reinterpret_cast<int8_t *>(pp + l.off_w8) : nullptr,
                              reinterpret_cast<int8_t *>(pp + l.off_wk), out->wk_mode, stream));
    if (layouts & RQ_PREPACK_PREFILL) {
        if (rq_encode_tmap_i8(out->tmap_w8, pp + l.off_w8, K, N, 128)   /* box: half a tile of weight rows */ != 0) return RQ_ERR_CUDA;
    }
    RQ_CUDA(cudaStreamSynchronize(stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) size_t rq_w4a4_workspace_bytes(int64_t K, int64_t M) {
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || M < 1) return 0;
    return (size_t) rq_ws(K, M).bytes;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_workspace_layout(int64_t K, int64_t M, int act_group, uint64_t * off_a8, uint64_t * off_msh,
                                        uint64_t * off_u, uint64_t * off_status) {
    (void) act_group;
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || M < 1) return RQ_ERR_SHAPE;
    const rq_ws_layout l = rq_ws(K, M);
    if (off_a8) *off_a8 = l.off_a8;
    if (off_msh) *off_msh = l.off_msh;
    if (off_u) *off_u = l.off_u;
    if (off_status) *off_status = l.off_status;
    return RQ_OK;
}

static int rq_check_x(const float * x, int64_t ldx, int64_t M, int64_t K) {
    if (x == nullptr) return RQ_ERR_ARG;
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || K > RQ_MAX_K || M < 1) return RQ_ERR_SHAPE;
    if (ldx < K || (ldx * 4) % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return RQ_ERR_SHAPE;
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_rotate(const float * x_dev, int64_t ldx, int64_t M, int64_t K, int64_t n_rot, float * out_dev,
                              int64_t ldo, void * stream) {
    int rc = rq_check_x(x_dev, ldx, M, K);
    if (rc != RQ_OK) return rc;
    rc = rq_check_x(out_dev, ldo, M, K);
    if (rc != RQ_OK) return rc;
    int p = 0, m = 0;
    if (n_rot <= 0 || K % n_rot != 0 || !rq_hadamard_factor(n_rot, &p, &m)) return RQ_ERR_ROTATION;
    const float scale = 1.0f / sqrtf((float) n_rot);
    RQ_CUDA(rq_launch_act(x_dev, ldx, M, K, (int) n_rot, p, m, scale, 1.0f, 64, RQ_FMT_I8, nullptr, nullptr, nullptr, out_dev, ldo,
                          nullptr, (cudaStream_t) stream));
    return RQ_OK;
}

// scratch of the weight quantizer: [rotated rows, W4A4H only][one scale per row or per weight group]
static void rq_wq_scratch(int type, int64_t K, int64_t N, int wgroup, uint64_t * off_sg, uint64_t * bytes) {
    const uint64_t rot = type == RQ_TYPE_W4A4H ? rq_align256((uint64_t) N * K * 4) : 0;
    const uint64_t ng = wgroup ? (uint64_t) (K / wgroup) : 1;
    *off_sg = rot;
    *bytes = rot + rq_align256((uint64_t) N * ng * 4);
}

extern "C" __attribute__((visibility("default"))) size_t rq_w4a4_quantize_weights_scratch_bytes(int type, int64_t K, int64_t N, int wgroup) {
    if ((type != RQ_TYPE_W4A4 && type != RQ_TYPE_W4A4H) || K <= 0 || K % RQ_BLOCK_CODES != 0 || K > RQ_MAX_K || N < 1 ||
        (wgroup != 0 && wgroup != 64 && wgroup != 256)) return 0;
    uint64_t off = 0, bytes = 0;
    rq_wq_scratch(type, K, N, wgroup, &off, &bytes);
    return (size_t) bytes;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_quantize_weights(const float * w_dev, int64_t ldw, int type, int64_t K, int64_t N, int wgroup,
                                        int rot_blocks, void * blocks_dev, void * scratch_dev, size_t scratch_bytes,
                                        void * stream) {
    if (type != RQ_TYPE_W4A4 && type != RQ_TYPE_W4A4H) return RQ_ERR_ARG;
    int rc = rq_check_x(w_dev, ldw, N, K);
    if (rc != RQ_OK) return rc;
    if (wgroup != 0 && wgroup != 64 && wgroup != 256) return RQ_ERR_GROUP;
    if (blocks_dev == nullptr || scratch_dev == nullptr || (reinterpret_cast<uintptr_t>(scratch_dev) & 255) != 0) return RQ_ERR_ARG;
    uint64_t off_sg = 0, need = 0;
    rq_wq_scratch(type, K, N, wgroup, &off_sg, &need);
    if (scratch_bytes < need) return RQ_ERR_WORKSPACE;
    uint8_t * sc = static_cast<uint8_t *>(scratch_dev);
    const float * rows = w_dev;
    int64_t ld = ldw;
    int pad0 = (int) K;
    if (type == RQ_TYPE_W4A4H) {
        // block-diagonal rotation of K / rot_blocks wide blocks when that divides K (rq_rot_len, patch:2687-2694)
        const int64_t n_rot = (rot_blocks > 1 && K % rot_blocks == 0) ? K / rot_blocks : K;
        int p = 0, m = 0;
        if (!rq_hadamard_factor(n_rot, &p, &m)) return RQ_ERR_ROTATION;
        float * rot = reinterpret_cast<float *>(sc);
        RQ_CUDA(rq_launch_act(w_dev, ldw, N, K, (int) n_rot, p, m, 1.0f / sqrtf((float) n_rot), 1.0f, 64, RQ_FMT_I8, nullptr, nullptr,
                              nullptr, rot, K, nullptr, (cudaStream_t) stream));
        rows = rot;
        ld = K;
        pad0 = (int) n_rot;
    }
    RQ_CUDA(rq_launch_wquant(rows, ld, N, K, wgroup, pad0, reinterpret_cast<float *>(sc + off_sg),
                             static_cast<rq_block *>(blocks_dev), (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_quantize(const float * x_dev, int64_t ldx, int64_t M, int64_t K, int64_t n_rot, float clip,
                                int act_group, int act_format, void * workspace_dev, size_t workspace_bytes, void * stream) {
    if (act_format != RQ_FMT_I8 && act_format != RQ_FMT_E4M3) return RQ_ERR_ARG;
    int rc = rq_check_x(x_dev, ldx, M, K);
    if (rc != RQ_OK) return rc;
    if (act_group != 64 && act_group != 128 && act_group != 256) return RQ_ERR_GROUP;
    if (!(clip > 0.0f) || isinf(clip)) return RQ_ERR_CLIP;
    const rq_ws_layout l = rq_ws(K, M);
    if (workspace_dev == nullptr || workspace_bytes < l.bytes || (reinterpret_cast<uintptr_t>(workspace_dev) & 255) != 0)
        return RQ_ERR_WORKSPACE;
    int p = 1, m = 0;
    float scale = 1.0f;
    if (n_rot > 0) {
        if (K % n_rot != 0 || !rq_hadamard_factor(n_rot, &p, &m)) return RQ_ERR_ROTATION;
        scale = 1.0f / sqrtf((float) n_rot);
    } else if (n_rot < 0) {
        return RQ_ERR_ROTATION;
    }
    uint8_t * ws = static_cast<uint8_t *>(workspace_dev);
    RQ_CUDA(rq_launch_act(x_dev, ldx, M, K, (int) n_rot, p, m, scale, clip, act_group, act_format, reinterpret_cast<int8_t *>(ws + l.off_a8),
                          reinterpret_cast<int32_t *>(ws + l.off_msh), reinterpret_cast<float *>(ws + l.off_u), nullptr, 0,
                          reinterpret_cast<int32_t *>(ws + l.off_status), (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_quantize_rows(const float * x_rows_dev, int64_t ldx, int64_t M_total, int64_t first, int64_t count,
                                     int64_t K, int64_t n_rot, float clip, int act_group, int act_format, void * workspace_dev,
                                     size_t workspace_bytes, void * stream) {
    if (act_format != RQ_FMT_I8 && act_format != RQ_FMT_E4M3) return RQ_ERR_ARG;
    if (first < 0 || count < 1 || first + count > M_total) return RQ_ERR_SHAPE;
    int rc = rq_check_x(x_rows_dev, ldx, count, K);
    if (rc != RQ_OK) return rc;
    if (act_group != 64 && act_group != 128 && act_group != 256) return RQ_ERR_GROUP;
    if (!(clip > 0.0f) || isinf(clip)) return RQ_ERR_CLIP;
    const rq_ws_layout l = rq_ws(K, M_total);
    if (workspace_dev == nullptr || workspace_bytes < l.bytes || (reinterpret_cast<uintptr_t>(workspace_dev) & 255) != 0)
        return RQ_ERR_WORKSPACE;
    int p = 1, m = 0;
    float scale = 1.0f;
    if (n_rot > 0) {
        if (K % n_rot != 0 || !rq_hadamard_factor(n_rot, &p, &m)) return RQ_ERR_ROTATION;
        scale = 1.0f / sqrtf((float) n_rot);
    } else if (n_rot < 0) {
        return RQ_ERR_ROTATION;
    }
    uint8_t * ws = static_cast<uint8_t *>(workspace_dev);
    RQ_CUDA(rq_launch_act(x_rows_dev, ldx, count, K, (int) n_rot, p, m, scale, clip, act_group, act_format,
                          reinterpret_cast<int8_t *>(ws + l.off_a8) + first * K,
                          reinterpret_cast<int32_t *>(ws + l.off_msh) + first * (K / act_group),
                          reinterpret_cast<float *>(ws + l.off_u) + first, nullptr, 0,
                          reinterpret_cast<int32_t *>(ws + l.off_status), (cudaStream_t) stream));
    return RQ_OK;
}

// which kernel a weight takes at M tokens: true = tcgen05 GEMM, false = GEMV passes; -1 on a bad request
static int rq_use_tc(const rq_weight_desc * w, int64_t M, int path) {
    const bool has_dec = (w->layouts & RQ_PREPACK_DECODE) != 0, has_pre = (w->layouts & RQ_PREPACK_PREFILL) != 0;
    if (path == RQ_PATH_GEMV) return has_dec ? 0 : -1;
    if (path == RQ_PATH_TC) return has_pre ? 1 : -1;
    // up to 64 tokens the GEMV in passes of 16 (the later passes read the stream from L2) beats a 128-token MMA tile
    if (path == RQ_PATH_AUTO) return (has_pre && (M > 64 || !has_dec)) ? 1 : (has_dec ? 0 : -1);
    return -1;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_act_format(const rq_weight_desc * const * w, int n_w, int64_t M, int path) {
    if (w == nullptr || n_w < 1 || n_w > RQ_MAX_WEIGHTS) return RQ_ERR_ARG;
    int fmt = -1;
    for (int i = 0; i < n_w; ++i) {
        if (w[i] == nullptr) return RQ_ERR_ARG;
        const int tc = rq_use_tc(w[i], M, path);
        if (tc < 0) return RQ_ERR_ARG;
        const int f = (tc && !w[i]->wk_mode) ? RQ_FMT_E4M3 : RQ_FMT_I8;
        if (fmt >= 0 && f != fmt) return RQ_ERR_MISMATCH;   // one activation cannot serve both formats
        fmt = f;
    }
    return fmt;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_mul_mat_quantized(const rq_weight_desc * w, int64_t M, float * y_dev, int64_t ldy, int act_group,
                                         int path, void * workspace_dev, size_t workspace_bytes, void * stream_) {
    cudaStream_t stream = (cudaStream_t) stream_;
    if (w == nullptr || y_dev == nullptr || w->prepack == nullptr) return RQ_ERR_ARG;
    if (M < 1 || ldy < w->N) return RQ_ERR_SHAPE;
    if (act_group != 64 && act_group != 128 && act_group != 256) return RQ_ERR_GROUP;
    if (w->wg64 && act_group != 64) return RQ_ERR_GROUP;   // ggml_vec_dot_w4a4_a4's assert, patch:171
    const rq_ws_layout l = rq_ws(w->K, M);
    if (workspace_dev == nullptr || workspace_bytes < l.bytes) return RQ_ERR_WORKSPACE;
    const uint8_t * ws = static_cast<const uint8_t *>(workspace_dev);
    const uint8_t * pp = static_cast<const uint8_t *>(w->prepack);
    const int8_t * a8 = reinterpret_cast<const int8_t *>(ws + l.off_a8);
    const int32_t * msh = reinterpret_cast<const int32_t *>(ws + l.off_msh);
    const float * u = reinterpret_cast<const float *>(ws + l.off_u);
    const float * sw = reinterpret_cast<const float *>(pp + w->off_sw);
    const int use_tc = rq_use_tc(w, M, path);
    if (use_tc < 0) return RQ_ERR_ARG;
    const bool tc = use_tc != 0;
    int32_t * status = reinterpret_cast<int32_t *>(const_cast<uint8_t *>(ws) + l.off_status);
    if (tc) {
        RQ_CUDA(rq_launch_gemm_tc(w->tmap_w8, sw, w->wk_mode ? RQ_FMT_I8 : RQ_FMT_E4M3, w->K, w->N, a8, msh, u, M, act_group, y_dev, ldy, status, stream));
    } else {
        rq_gemv_job job;
        job.w4 = pp + w->off_w4; job.sw = sw; job.N = w->N; job.y = y_dev; job.ldy = ldy; job.n_more = 0;
        job.wk = w->wk_mode ? reinterpret_cast<const int8_t *>(pp + w->off_wk) : nullptr;
        RQ_CUDA(rq_launch_gemv(&job, 1, w->K, a8, msh, u, M, act_group, status, stream));
    }
    return RQ_OK;
}

// Measurement aid: the tcgen05 kernel with the whole of K in ONE accumulator per output, i.e. without the per-group
// hand-over from tensor memory and without the fold.  The numbers it writes are not the MUL_MAT (the reference's
// per-group shift is skipped); a benchmark times it to see what the same kernel reaches when nothing leaves tensor
// memory between the first and the last input.
extern "C" __attribute__((visibility("default"))) int rq_w4a4_tc_nofold_probe(const rq_weight_desc * w, int64_t M, float * y_dev, int64_t ldy,
                                                                           void * workspace_dev, size_t workspace_bytes, void * stream) {
    if (w == nullptr || y_dev == nullptr || w->prepack == nullptr || (w->layouts & RQ_PREPACK_PREFILL) == 0) return RQ_ERR_ARG;
    if (M < 1 || ldy < w->N) return RQ_ERR_SHAPE;
    const rq_ws_layout l = rq_ws(w->K, M);
    if (workspace_dev == nullptr || workspace_bytes < l.bytes) return RQ_ERR_WORKSPACE;
    const uint8_t * ws = static_cast<const uint8_t *>(workspace_dev);
    const uint8_t * pp = static_cast<const uint8_t *>(w->prepack);
    RQ_CUDA(rq_launch_gemm_tc(w->tmap_w8, reinterpret_cast<const float *>(pp + w->off_sw), w->wk_mode ? RQ_FMT_I8 : RQ_FMT_E4M3, w->K, w->N,
                              reinterpret_cast<const int8_t *>(ws + l.off_a8), reinterpret_cast<const int32_t *>(ws + l.off_msh),
                              reinterpret_cast<const float *>(ws + l.off_u), M, (int) w->K, y_dev, ldy,
                              reinterpret_cast<int32_t *>(const_cast<uint8_t *>(ws) + l.off_status), (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_mul_mat_quantized_n(const rq_weight_desc * const * w, int n_w, int64_t M,
                                           float * const * y_dev, const int64_t * ldy, int act_group, int path,
                                           void * workspace_dev, size_t workspace_bytes, void * stream) {
    if (w == nullptr || y_dev == nullptr || ldy == nullptr || n_w < 1 || n_w > RQ_MAX_WEIGHTS) return RQ_ERR_ARG;
    for (int i = 0; i < n_w; ++i) {
        if (w[i] == nullptr || y_dev[i] == nullptr) return RQ_ERR_ARG;
        if (w[i]->K != w[0]->K || w[i]->type != w[0]->type || w[i]->n_rot != w[0]->n_rot) return RQ_ERR_MISMATCH;
    }
    if (M < 1) return RQ_ERR_SHAPE;
    if (act_group != 64 && act_group != 128 && act_group != 256) return RQ_ERR_GROUP;
    int rc;
    // decode widths: the weights' row tiles become one GEMV launch when they all have the decode stream and agree on
    // the weight-multiplier mode (the reference fuses up to three skinny matmuls the same way, patch:308-329)
    bool one_launch = n_w > 1 && path != RQ_PATH_TC && M <= 64;
    for (int i = 0; i < n_w && one_launch; ++i) {
        one_launch = (w[i]->layouts & RQ_PREPACK_DECODE) != 0 && w[i]->wk_mode == w[0]->wk_mode && w[i]->prepack != nullptr &&
                     ldy[i] >= w[i]->N && !(w[i]->wg64 && act_group != 64);
    }
    if (one_launch) {
        const rq_ws_layout l = rq_ws(w[0]->K, M);
        if (workspace_dev == nullptr || workspace_bytes < l.bytes) return RQ_ERR_WORKSPACE;
        uint8_t * ws = static_cast<uint8_t *>(workspace_dev);
        rq_gemv_job jobs[RQ_MAX_WEIGHTS];
        for (int i = 0; i < n_w; ++i) {
            const uint8_t * pp = static_cast<const uint8_t *>(w[i]->prepack);
            jobs[i].w4 = pp + w[i]->off_w4;
            jobs[i].sw = reinterpret_cast<const float *>(pp + w[i]->off_sw);
            jobs[i].wk = w[i]->wk_mode ? reinterpret_cast<const int8_t *>(pp + w[i]->off_wk) : nullptr;
            jobs[i].N = w[i]->N; jobs[i].y = y_dev[i]; jobs[i].ldy = ldy[i]; jobs[i].n_more = 0;
        }
        RQ_CUDA(rq_launch_gemv(jobs, n_w, w[0]->K, reinterpret_cast<const int8_t *>(ws + l.off_a8),
                               reinterpret_cast<const int32_t *>(ws + l.off_msh), reinterpret_cast<const float *>(ws + l.off_u), M,
                               act_group, reinterpret_cast<int32_t *>(ws + l.off_status), (cudaStream_t) stream));
        return RQ_OK;
    }
    for (int i = 0; i < n_w; ++i) {
        rc = rq_w4a4_mul_mat_quantized(w[i], M, y_dev[i], ldy[i], act_group, path, workspace_dev, workspace_bytes, stream);
        if (rc != RQ_OK) return rc;
    }
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_mul_mat(const rq_weight_desc * const * w, int n_w, const float * x_dev, int64_t ldx, int64_t M,
                               float * const * y_dev, const int64_t * ldy, float clip, int act_group, int path,
                               void * workspace_dev, size_t workspace_bytes, void * stream) {
    if (w == nullptr || y_dev == nullptr || ldy == nullptr || n_w < 1 || n_w > RQ_MAX_WEIGHTS) return RQ_ERR_ARG;
    for (int i = 0; i < n_w; ++i) {
        if (w[i] == nullptr || y_dev[i] == nullptr) return RQ_ERR_ARG;
        // one activation serves all: same input width, type and rotation (ggml_cuda_rq_w4a4_can_fuse, patch:2394-2397)
        if (w[i]->K != w[0]->K || w[i]->type != w[0]->type || w[i]->n_rot != w[0]->n_rot) return RQ_ERR_MISMATCH;
    }
    const int fmt = rq_w4a4_act_format(w, n_w, M, path);
    if (fmt < 0) return fmt;
    int rc = rq_w4a4_quantize(x_dev, ldx, M, w[0]->K, w[0]->type == RQ_TYPE_W4A4H ? w[0]->n_rot : 0, clip, act_group, fmt,
                              workspace_dev, workspace_bytes, stream);
    if (rc != RQ_OK) return rc;
    return rq_w4a4_mul_mat_quantized_n(w, n_w, M, y_dev, ldy, act_group, path, workspace_dev, workspace_bytes, stream);
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_mul_mat_push(const rq_weight_desc * const * w, int n_w, const float * x_dev, int64_t ldx,
                                    int64_t M, float * const * y_dst, int n_dst, const int64_t * ldy, float clip,
                                    int act_group, void * workspace_dev, size_t workspace_bytes, void * stream) {
    if (w == nullptr || y_dst == nullptr || ldy == nullptr || n_w < 1 || n_w > RQ_MAX_WEIGHTS || n_dst < 1 || n_dst > RQ_MAX_RANKS)
        return RQ_ERR_ARG;
    if (M < 1) return RQ_ERR_SHAPE;
    const bool tc = M > 64;          // wider inputs: the tcgen05 kernel's final store pushes instead
    for (int i = 0; i < n_w; ++i) {
        if (w[i] == nullptr) return RQ_ERR_ARG;
        if (w[i]->K != w[0]->K || w[i]->type != w[0]->type || w[i]->n_rot != w[0]->n_rot || w[i]->wk_mode != w[0]->wk_mode)
            return RQ_ERR_MISMATCH;
        if ((w[i]->layouts & (tc ? RQ_PREPACK_PREFILL : RQ_PREPACK_DECODE)) == 0 || w[i]->prepack == nullptr || ldy[i] < w[i]->N)
            return RQ_ERR_ARG;
        if (w[i]->wg64 && act_group != 64) return RQ_ERR_GROUP;
        for (int d = 0; d < n_dst; ++d) if (y_dst[d * n_w + i] == nullptr) return RQ_ERR_ARG;
    }
    const int fmt = tc && !w[0]->wk_mode ? RQ_FMT_E4M3 : RQ_FMT_I8;
    const rq_ws_layout l = rq_ws(w[0]->K, M);
    if (x_dev != nullptr) {
        int rc = rq_w4a4_quantize(x_dev, ldx, M, w[0]->K, w[0]->type == RQ_TYPE_W4A4H ? w[0]->n_rot : 0, clip, act_group, fmt,
                                  workspace_dev, workspace_bytes, stream);
        if (rc != RQ_OK) return rc;
    } else if (workspace_dev == nullptr || workspace_bytes < l.bytes) {     // the activation is already in the workspace
        return RQ_ERR_WORKSPACE;
    }
    uint8_t * ws = static_cast<uint8_t *>(workspace_dev);
    if (tc) {
        for (int i = 0; i < n_w; ++i) {
            const uint8_t * pp = static_cast<const uint8_t *>(w[i]->prepack);
            float * more[RQ_MAX_RANKS - 1];
            for (int d = 1; d < n_dst; ++d) more[d - 1] = y_dst[d * n_w + i];
            RQ_CUDA(rq_launch_gemm_tc(w[i]->tmap_w8, reinterpret_cast<const float *>(pp + w[i]->off_sw), fmt, w[i]->K, w[i]->N,
                                      reinterpret_cast<const int8_t *>(ws + l.off_a8), reinterpret_cast<const int32_t *>(ws + l.off_msh),
                                      reinterpret_cast<const float *>(ws + l.off_u), M, act_group, y_dst[i], ldy[i],
                                      reinterpret_cast<int32_t *>(ws + l.off_status), (cudaStream_t) stream, more, n_dst - 1));
        }
        return RQ_OK;
    }
    rq_gemv_job jobs[RQ_MAX_WEIGHTS];
    for (int i = 0; i < n_w; ++i) {
        const uint8_t * pp = static_cast<const uint8_t *>(w[i]->prepack);
        jobs[i].w4 = pp + w[i]->off_w4;
        jobs[i].sw = reinterpret_cast<const float *>(pp + w[i]->off_sw);
        jobs[i].wk = w[i]->wk_mode ? reinterpret_cast<const int8_t *>(pp + w[i]->off_wk) : nullptr;
        jobs[i].N = w[i]->N; jobs[i].y = y_dst[i]; jobs[i].ldy = ldy[i];
        jobs[i].n_more = n_dst - 1;
        for (int d = 1; d < n_dst; ++d) jobs[i].y_more[d - 1] = y_dst[d * n_w + i];
    }
    RQ_CUDA(rq_launch_gemv(jobs, n_w, w[0]->K, reinterpret_cast<const int8_t *>(ws + l.off_a8),
                           reinterpret_cast<const int32_t *>(ws + l.off_msh), reinterpret_cast<const float *>(ws + l.off_u), M,
                           act_group, reinterpret_cast<int32_t *>(ws + l.off_status), (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_rank_barrier(uint32_t * const * flags_of_rank, int rank, int n_ranks, uint32_t * epoch_dev,
                               int32_t * status_dev, void * stream) {
    if (flags_of_rank == nullptr || epoch_dev == nullptr || n_ranks < 1 || n_ranks > RQ_MAX_RANKS || rank < 0 || rank >= n_ranks)
        return RQ_ERR_ARG;
    for (int p = 0; p < n_ranks; ++p) if (flags_of_rank[p] == nullptr) return RQ_ERR_ARG;
    RQ_CUDA(rq_launch_rank_barrier(flags_of_rank, rank, n_ranks, epoch_dev, status_dev, (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_sum_partials(const float * const * partials_of_rank, int rank, int n_ranks, int64_t count,
                                                                         float * const * y_of_rank, int two_shot, void * stream) {
    if (partials_of_rank == nullptr || y_of_rank == nullptr || n_ranks < 1 || n_ranks > RQ_MAX_RANKS || rank < 0 || rank >= n_ranks)
        return RQ_ERR_ARG;
    if (count < 1) return RQ_ERR_SHAPE;
    for (int r = 0; r < n_ranks; ++r) {
        if (partials_of_rank[r] == nullptr || (reinterpret_cast<uintptr_t>(partials_of_rank[r]) & 15) != 0) return RQ_ERR_ARG;
    }
    if (!two_shot) {
        if (y_of_rank[rank] == nullptr || (reinterpret_cast<uintptr_t>(y_of_rank[rank]) & 15) != 0) return RQ_ERR_ARG;
        float * out[1] = { y_of_rank[rank] };
        RQ_CUDA(rq_launch_partial_sum(partials_of_rank, n_ranks, 0, count, out, 1, (cudaStream_t) stream));
        return RQ_OK;
    }
    for (int r = 0; r < n_ranks; ++r) {
        if (y_of_rank[r] == nullptr || (reinterpret_cast<uintptr_t>(y_of_rank[r]) & 15) != 0) return RQ_ERR_ARG;
    }
    // pieces of whole 4-element vectors; the last rank takes the remainder
    const int64_t per = ((count / n_ranks) / 4) * 4;
    const int64_t lo = per * rank, hi = rank == n_ranks - 1 ? count : per * (rank + 1);
    RQ_CUDA(rq_launch_partial_sum(partials_of_rank, n_ranks, lo, hi, y_of_rank, n_ranks, (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_share_rows(void * const * workspace_of_rank, int rank, int n_ranks,
                                                                       size_t workspace_bytes, int64_t K, int64_t M_total, int act_group,
                                                                       int64_t first, int64_t count, void * stream) {
    if (workspace_of_rank == nullptr || n_ranks < 1 || n_ranks > RQ_MAX_RANKS || rank < 0 || rank >= n_ranks) return RQ_ERR_ARG;
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || K > RQ_MAX_K || M_total < 1) return RQ_ERR_SHAPE;
    if (act_group != 64 && act_group != 128 && act_group != 256) return RQ_ERR_ARG;
    if (first < 0 || count < 1 || first + count > M_total) return RQ_ERR_SHAPE;
    const rq_ws_layout l = rq_ws(K, M_total);
    if (workspace_bytes < l.bytes) return RQ_ERR_WORKSPACE;
    void * dst[RQ_MAX_RANKS - 1];
    int n_dst = 0;
    for (int r = 0; r < n_ranks; ++r) {
        if (workspace_of_rank[r] == nullptr || (reinterpret_cast<uintptr_t>(workspace_of_rank[r]) & 15) != 0) return RQ_ERR_ARG;
        if (r != rank) dst[n_dst++] = workspace_of_rank[r];
    }
    const uint64_t n_ag = (uint64_t) (K / act_group);
    const uint64_t off[3] = { l.off_a8 + (uint64_t) first * (uint64_t) K, l.off_msh + (uint64_t) first * n_ag * 4, l.off_u + (uint64_t) first * 4 };
    const uint64_t bytes[3] = { (uint64_t) count * (uint64_t) K, (uint64_t) count * n_ag * 4, (uint64_t) count * 4 };
    RQ_CUDA(rq_launch_share_rows(workspace_of_rank[rank], dst, n_dst, off, bytes, (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_workspace_init(void * workspace_dev, int64_t K, int64_t M, void * stream) {
    if (workspace_dev == nullptr) return RQ_ERR_ARG;
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || M < 1) return RQ_ERR_SHAPE;
    RQ_CUDA(cudaMemsetAsync(static_cast<uint8_t *>(workspace_dev) + rq_ws(K, M).off_status, 0, 256, (cudaStream_t) stream));
    return RQ_OK;
}

extern "C" __attribute__((visibility("default"))) int rq_w4a4_device_status(void * workspace_dev, int64_t K, int64_t M, void * stream) {
    if (workspace_dev == nullptr) return RQ_ERR_ARG;
    if (K <= 0 || K % RQ_BLOCK_CODES != 0 || M < 1) return RQ_ERR_SHAPE;
    const rq_ws_layout l = rq_ws(K, M);
    int32_t st = 0;
    uint8_t * word = static_cast<uint8_t *>(workspace_dev) + l.off_status;
    RQ_CUDA(cudaMemcpyAsync(&st, word, 4, cudaMemcpyDeviceToHost, (cudaStream_t) stream));
    RQ_CUDA(cudaStreamSynchronize((cudaStream_t) stream));
    // the word is sticky (no kernel clears it): reading a report takes it away
    if (st != 0) RQ_CUDA(cudaMemsetAsync(word, 0, 4, (cudaStream_t) stream));
    // 1: a bounded wait expired; 2: the activation was quantized in the other kernel's format
    return st == 0 ? RQ_OK : st == 2 ? RQ_ERR_MISMATCH : RQ_ERR_DEVICE;
}
