// Shared declarations of the sm_100a W4A4 / W4A4H MUL_MAT library (internal; the public face is include/rq_b200.h).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/rq_b200.h"

// 144-byte block of 256 int4 codes: element 8w+j in bits [4j+3:4j] of qs[w], two's complement
// (block_w4a4, ggml/src/ggml-common.h in patches/llama.cpp-ruquant.patch:26-50 of the reference).
struct rq_block {
    float    d;        // weights: the row's unit s_w
    int32_t  sum;      // weights: legacy code sum, or 1<<30 | k_b, or 3<<29 | k0 | k1<<4 | k2<<8 | k3<<12
    int32_t  pad[2];   // weights: pad[0] = row length (W4A4) / Hadamard length (W4A4H), pad[1] = clip as float bits
    uint32_t qs[32];
};
static_assert(sizeof(rq_block) == RQ_BLOCK_BYTES, "block layout");

// weight multiplier of the g-th run of 64 inputs of a block (RQ_W_MULT_G, patch:40-43)
__host__ __device__ inline int rq_wmult(int32_t sum, int g) {
    const uint32_t s = (uint32_t) sum;
    if ((s >> 29) == 3u) return (int) ((s >> (4 * g)) & 0xF);
    if ((s >> 30) == 1u) return (int) (s & 0xF);
    return 1;
}

// The contraction delivers D = 128 * S_g (weights as 16*c, activations as 8*(q-z)); the reference's term
// (m_g * S_g) >> 4 (RQ_TERM_SHIFT, patch:39 and ggml_vec_dot_w4a4_a4, patch:173) is then (m_g * D) >> 11, exact,
// and m_g * D stays below 2^31 for every group width (255 * 128 * 120 * 256 < 2^30).
#define RQ_FOLD_SHIFT 11
// Inside every run of 64 inputs both int8 operands (activations a8, tensor-core weights w8) are stored permuted:
// the 4 inputs 16*i + 4*t .. +3 (i, t in 0..3) sit at bytes 16*t + 4*i .. +3, so that the 16 bytes at 16*t are the
// B fragment (k = {0,16,32,48} + 4*t .. +3) of the two m16n8k32 MMAs that cover the run.  A dot product over the run
// does not care about the order as long as both operands agree.
__host__ __device__ inline int rq_perm64(int k4) {   // k4: offset of a 4-input piece inside the run (multiple of 4)
    return ((k4 & 15) >> 2) * 16 + (k4 >> 4) * 4;
}
// e4m3 byte of a small integer (|v| <= 15: at most four significant bits, so the conversion is exact)
__host__ __device__ inline uint32_t rq_e4m3_of_int(int v) {
    const uint32_t sign = v < 0 ? 0x80u : 0u;
    const uint32_t a = (uint32_t) (v < 0 ? -v : v);
    if (a == 0) return 0u;
    const int e = a >= 8 ? 3 : a >= 4 ? 2 : a >= 2 ? 1 : 0;
    return sign | (uint32_t) ((e + 7) << 3) | ((a << (3 - e)) & 7u);
}
#define RQ_ACT_SCALE 8     // activations are stored as 8*(q - z), |.| <= 120
#define RQ_W_SCALE   16    // weights with multiplier 1 are stored as 16*c, in [-128, 112]

// Workspace of one call: [a8 int8 M*K][msh int32 M*(K/64)][u f32 M][status int32 x 64], each part 256-byte aligned.
struct rq_ws_layout {
    uint64_t off_a8, off_msh, off_u, off_status, bytes;
};
static inline uint64_t rq_align256(uint64_t v) { return (v + 255) & ~(uint64_t) 255; }
static inline rq_ws_layout rq_ws(int64_t K, int64_t M) {
    rq_ws_layout l;
    l.off_a8 = 0;
    l.off_msh = rq_align256((uint64_t) M * K);
    l.off_u = l.off_msh + rq_align256((uint64_t) M * (K / 64) * 4);
    l.off_status = l.off_u + rq_align256((uint64_t) M * 4);
    l.bytes = l.off_status + 256;
    return l;
}

// Timeline diagnostics, compiled in with -DRQ_TRACE only: when the 64-bit word at status[2..3] holds a device
// pointer, every call appends (global timer in ns, tag << 32 | CTA) to the buffer behind it ([0] = event count).
#if defined(RQ_TRACE) && defined(__CUDACC__)
__device__ __forceinline__ void rq_trace(const int32_t * status, unsigned tag) {
    if (status == nullptr) return;
    unsigned long long * buf = *reinterpret_cast<unsigned long long * const *>(status + 2);
    if (buf == nullptr) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned long long i = atomicAdd(buf, 1ull);
    if (i < (1ull << 16)) { buf[2 + 2 * i] = t; buf[3 + 2 * i] = ((unsigned long long) tag << 32) | blockIdx.x; }
}
// cheaper form for phases inside one kernel: time stamps collected in registers and appended at the end
struct rq_stamps {
    unsigned long long t[12];
    int n;
    __device__ __forceinline__ rq_stamps() : n(0) {}
    __device__ __forceinline__ void mark() {
        unsigned long long v;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
        if (n < 12) t[n++] = v;
    }
    __device__ __forceinline__ void flush(const int32_t * status, unsigned tag) {
        if (status == nullptr) return;
        unsigned long long * buf = *reinterpret_cast<unsigned long long * const *>(status + 2);
        if (buf == nullptr) return;
        const unsigned long long i = atomicAdd(buf, (unsigned long long) n);
        for (int k = 0; k < n; ++k)
            if (i + k < (1ull << 16)) { buf[2 + 2 * (i + k)] = t[k]; buf[3 + 2 * (i + k)] = ((unsigned long long) (tag + k) << 32) | blockIdx.x; }
    }
};
// cycle counters around waits: RQ_CYC_REPORT appends (cycles, tag << 32 | CTA)
#define RQ_CYC_DECL(name) long long name = 0, name##_t0 = 0
#define RQ_CYC_BEGIN(name) name##_t0 = clock64()
#define RQ_CYC_END(name) name += clock64() - name##_t0
#define RQ_CYC_REPORT(status, tag, name) rq_trace_value(status, tag, (unsigned long long) (name))
__device__ __forceinline__ void rq_trace_value(const int32_t * status, unsigned tag, unsigned long long value) {
    if (status == nullptr) return;
    unsigned long long * buf = *reinterpret_cast<unsigned long long * const *>(status + 2);
    if (buf == nullptr) return;
    const unsigned long long i = atomicAdd(buf, 1ull);
    if (i < (1ull << 16)) { buf[2 + 2 * i] = value; buf[3 + 2 * i] = ((unsigned long long) tag << 32) | (blockIdx.x + gridDim.x * blockIdx.y); }
}
#define RQ_STAMP_DECL rq_stamps rq_st
#define RQ_STAMP(cond) do { if (cond) rq_st.mark(); } while (0)
#define RQ_STAMP_FLUSH(cond, status, tag) do { if (cond) rq_st.flush(status, tag); } while (0)
#else
#define rq_trace(status, tag) ((void) 0)
#define RQ_CYC_DECL(name)
#define RQ_CYC_BEGIN(name) ((void) 0)
#define RQ_CYC_END(name) ((void) 0)
#define RQ_CYC_REPORT(status, tag, name) ((void) 0)
#define RQ_STAMP_DECL
#define RQ_STAMP(cond) ((void) 0)
#define RQ_STAMP_FLUSH(cond, status, tag) ((void) 0)
#endif

// an integer tuning knob from the environment (call sites cache the result in a function-local static: read once)
static inline int rq_env_int(const char * name, int fallback) {
    const char * v = getenv(name);
    return v != nullptr ? atoi(v) : fallback;
}

// Launchers (one per .cu file).  All enqueue on `stream` and return a cudaError_t.
cudaError_t rq_launch_act(const float * x, int64_t ldx, int64_t M, int64_t K, int n_rot, int p, int m, float rot_scale,
                          float clip, int G, int fmt, int8_t * a8, int32_t * msh, float * u, float * rot_out, int64_t ldo,
                          int32_t * status, cudaStream_t stream);
cudaError_t rq_launch_prepack(const rq_block * blocks, int64_t K, int64_t N, float * sw, uint8_t * w4, int8_t * w8,
                              int8_t * wk, int wk_mode, cudaStream_t stream);
cudaError_t rq_launch_scan_wk(const rq_block * blocks, int64_t n_blocks, int32_t * flag, cudaStream_t stream);
// one weight of a GEMV launch; all jobs of a launch share K, the activation and the weight-multiplier mode
struct rq_gemv_job {
    const uint8_t * w4;
    const float * sw;
    const int8_t * wk;     // null when every multiplier is 1 (then null for every job of the launch)
    int64_t N;
    float * y;
    int64_t ldy;
    float * y_more[RQ_MAX_RANKS - 1];   // further destinations of the same output (peer-mapped buffers of other ranks)
    int n_more;
};
cudaError_t rq_launch_gemv(const rq_gemv_job * jobs, int n_jobs, int64_t K, const int8_t * a8, const int32_t * msh,
                           const float * u, int64_t M, int G, int32_t * status, cudaStream_t stream);
cudaError_t rq_launch_gemm_tc(const void * tmap_w8, const float * sw, int fmt, int64_t K, int64_t N,
                              const int8_t * a8, const int32_t * msh, const float * u, int64_t M, int G,
                              float * y, int64_t ldy, int32_t * status, cudaStream_t stream, float * const * y_more = nullptr,
                              int n_more = 0);
// all-ranks barrier over peer-mapped flag words (rq_rank.cu)
cudaError_t rq_launch_rank_barrier(uint32_t * const * flags_of_rank, int rank, int n_ranks, uint32_t * epoch, int32_t * status,
                                   cudaStream_t stream);
// rank-ordered sum of the ranks' partial outputs over elements [lo, hi), stored into n_out destinations (rq_rank.cu)
cudaError_t rq_launch_partial_sum(const float * const * partials, int n_ranks, int64_t lo, int64_t hi, float * const * outs, int n_out,
                                  cudaStream_t stream);
cudaError_t rq_launch_share_rows(const void * src, void * const * dst, int n_dst, const uint64_t * off, const uint64_t * bytes,
                                 cudaStream_t stream);
// weight quantizer: scale search + pack of already-rotated rows (rq_wquant.cu)
cudaError_t rq_launch_wquant(const float * x, int64_t ldx, int64_t n_rows, int64_t K, int wgroup, int pad0, float * sg,
                             rq_block * out, cudaStream_t stream);
// per-device kernel attributes (large dynamic shared memory); called from rq_w4a4_prepare so that the first
// launch inside a stream capture has nothing left to set up
cudaError_t rq_configure_act();
cudaError_t rq_configure_gemm_tc();
// host-side: encodes the 2-D tensor map of a row-major int8 [rows][K] operand with a {128, box_rows} box, 128B swizzle
int rq_encode_tmap_i8(void * tmap_out, const void * base, int64_t K, int64_t rows, int box_rows);
