// rq_w4a4_mul_mat_static: the MUL_MAT node for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc: a ggml backend hands out memory only from buffers
// sized at graph-planning time, and a plug-in running inside someone else's captured stream or inside a process
// whose allocator is owned by another runtime must not allocate either.  rq_w4a4_mul_mat needs a scratch buffer
// for the quantized activation (int8 codes, group multipliers, token units, a status word); this variant keeps
// that scratch in a fixed array inside the library image instead, so the caller passes only inputs and outputs.
//
// Limits and rules:
//   * M * K <= RQ_STATIC_MAX_TOKENS * RQ_MAX_K is not enough: each of M <= 16 and K <= 32768 is checked, and one
//     weight per call.  Beyond that the call returns RQ_ERR_LIMIT and does nothing.
//   * Every GPU that loads the library holds the array (about 0.6 MB) until the process exits.
//   * All calls on a device share the one array and it keeps the previous call's contents.  The status word is
//     cleared at the start of each call; everything else is overwritten before it is read.  Two calls that may run
//     on the GPU at the same time (different streams, or graph branches) race on it: serialise them.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress); make that first
//     call outside any stream capture.
#include <mutex>

#include "rq_common.cuh"

#define RQ_STATIC_MAX_TOKENS 16
// rq_ws(RQ_MAX_K, 16): 16*32768 codes + 16*512*4 multipliers + 256 (units) + 256 (status)
#define RQ_STATIC_WS_BYTES (16 * 32768 + 16 * 512 * 4 + 256 + 256)

static __device__ __align__(256) unsigned char rq_static_scratch[RQ_STATIC_WS_BYTES];

namespace {
std::mutex g_mu;
void * g_scratch_ptr[64] = {};   // device address of rq_static_scratch, per device ordinal
}

extern "C" __attribute__((visibility("default")))
int rq_w4a4_mul_mat_static(const rq_weight_desc * w, const float * x_dev, int64_t ldx, int64_t M, float * y_dev, int64_t ldy,
                           float clip, int act_group, int path, void * stream) {
    if (w == nullptr || x_dev == nullptr || y_dev == nullptr) return RQ_ERR_ARG;
    if (M < 1 || M > RQ_STATIC_MAX_TOKENS || w->K > RQ_MAX_K) return RQ_ERR_LIMIT;
    if (rq_ws(w->K, M).bytes > RQ_STATIC_WS_BYTES) return RQ_ERR_LIMIT;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return RQ_ERR_CUDA;
    void * ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (g_scratch_ptr[dev] == nullptr) {
            // in host code the array's name is only a handle: the kernels need the address the device sees
            void * p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, rq_static_scratch);
            if (e != cudaSuccess || p == nullptr) return RQ_ERR_CUDA;
            g_scratch_ptr[dev] = p;
        }
        ptr = g_scratch_ptr[dev];
    }
    const rq_weight_desc * ws[1] = { w };
    float * ys[1] = { y_dev };
    const int64_t ldys[1] = { ldy };
    return rq_w4a4_mul_mat(ws, 1, x_dev, ldx, M, ys, ldys, clip, act_group, path, ptr, RQ_STATIC_WS_BYTES, stream);
}
