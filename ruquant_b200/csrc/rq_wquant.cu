// Weight quantizer on the GPU: rows of fp32 -> rows of 144-byte W4A4 / W4A4H blocks, bit-identical to the reference's
// CPU quantizer (quantize_row_w4a4_ref / quantize_row_w4a4h_ref, rq_quantize_row_w, rq_scale_search, rq_pack in
// patches/llama.cpp-ruquant.patch:2489-2580, 2681-2710 of the reference).  Not on the MUL_MAT path: it makes the
// path's input (model conversion, test and benchmark tensors) without the CPU's 0.5 ms per row.
//
// Bit-parity contract
//   scale search  per row (or per block of 256 / per 64 inputs with weight groups): amax = max |x|; thirteen candidates
//                 s_r = (amax * (1.0f - 0.025f * r)) / 7.0f; for each, err_r = sum over the inputs IN ORDER, in double, of
//                 e*e with e = (double)(q*s) - (double)x, q = clamp(rintf(x / s), -8, 7); the first smallest err wins.
//                 The sum's order is part of the result (which candidate wins a near-tie), so one thread owns one
//                 (group, candidate) pair and walks its inputs sequentially; the parallelism is rows x groups x 13.
//                 The multiply and the add of err += e*e are separate roundings (the reference is built without fused
//                 multiply-add contraction on its baseline x86-64 target).
//   weight groups smax = max of the group scales, v = smax / 15, k_g = clamp(rintf(s_g / v), 1, 15), codes with k_g * v;
//                 header d = v, sum = 1<<30 | k_b (per block) or 3<<29 | k0 | k1<<4 | k2<<8 | k3<<12 (per 64 inputs).
//   no groups     header d = s, sum = the row's code sum.
//   pad[0] = row length K (W4A4) or Hadamard length n (W4A4H), pad[1] = 0 (activation clip unset).
// W4A4H rows are rotated first by the activation path's own rotation kernel (same operations, same order).
#include <math.h>

#include "rq_common.cuh"

namespace {

constexpr int CAND = 13;

__device__ __forceinline__ float candidate_scale(float amax, int r) {
    return __fdiv_rn(__fmul_rn(amax, __fsub_rn(1.0f, __fmul_rn(0.025f, (float) r))), 7.0f);
}
__device__ __forceinline__ float code_of(float x, float s) {
    return fminf(fmaxf(rintf(__fdiv_rn(x, s)), -8.0f), 7.0f);
}

// One half-warp per (row, group): lanes 0..12 each walk the group's inputs for one candidate; lanes of a half-warp
// read the same address (a broadcast), consecutive iterations the next float of the same 32-byte sector.
// sg[row * ng + g] receives the winning scale (0 for an all-zero group).
__global__ void __launch_bounds__(256) rq_wsearch_kernel(const float * __restrict__ x, int64_t ldx, int64_t n_rows, int K, int gs,
                                                         float * __restrict__ sg) {
    const int ng = K / gs;
    const int64_t unit = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 4;     // (row, group) index
    const int r = threadIdx.x & 15;
    const bool live = unit < n_rows * ng;
    const int64_t row = live ? unit / ng : 0;
    const int g = live ? (int) (unit - row * ng) : 0;
    const float * xg = x + row * ldx + (int64_t) g * gs;

    // amax: every lane of the half-warp takes a stride-16 share, then a max over the 16 lanes (exact in any order)
    float amax = 0.0f;
    for (int i = r; i < gs; i += 16) amax = fmaxf(amax, fabsf(__ldg(xg + i)));
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));

    double err = INFINITY;
    float s = 0.0f;
    if (amax > 0.0f && r < CAND) {
        s = candidate_scale(amax, r);
        err = 0.0;
        for (int i = 0; i < gs; ++i) {
            const float v = __ldg(xg + i);
            const float q = code_of(v, s);
            const double e = __dsub_rn((double) __fmul_rn(q, s), (double) v);
            err = __dadd_rn(err, __dmul_rn(e, e));
        }
    }
    // the first smallest error: walk the candidates in order, as the reference's loop does
    double best_err = INFINITY;
    float best_s = 0.0f;
    const int base = (threadIdx.x & 31) & 16;
    for (int c = 0; c < CAND; ++c) {
        const double ec = __shfl_sync(0xffffffffu, err, base + c);
        const float sc = __shfl_sync(0xffffffffu, s, base + c);
        if (ec < best_err) { best_err = ec; best_s = sc; }
    }
    if (live && r == 0) sg[unit] = amax > 0.0f ? best_s : 0.0f;
}

// One CTA per row: group multipliers (if any), codes, headers.
__global__ void __launch_bounds__(256) rq_wpack_kernel(const float * __restrict__ x, int64_t ldx, int K, int gs, int wgroup,
                                                       int pad0, const float * __restrict__ sg, rq_block * __restrict__ out) {
    __shared__ float red[8];
    __shared__ int red_i[8];
    __shared__ float unit_s;
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x, ng = K / gs;
    const float * xr = x + row * ldx;
    const float * sr = sg + row * ng;
    rq_block * yr = out + row * (K / RQ_BLOCK_CODES);

    float unit = 0.0f;
    if (wgroup) {
        float smax = 0.0f;
        for (int g = tid; g < ng; g += blockDim.x) smax = fmaxf(smax, sr[g]);
        for (int o = 16; o > 0; o >>= 1) smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, o));
        if ((tid & 31) == 0) red[tid >> 5] = smax;
        __syncthreads();
        if (tid == 0) {
            float v = 0.0f;
            for (int i = 0; i < (int) (blockDim.x >> 5); ++i) v = fmaxf(v, red[i]);
            unit_s = __fdiv_rn(v, 15.0f);
        }
        __syncthreads();
        unit = unit_s;
    }
    // a thread packs whole words of 8 codes
    int code_sum = 0;
    for (int w = tid; w < K / 8; w += blockDim.x) {
        const int g = (w * 8) / gs;
        float s;
        if (wgroup) {
            const float kf = unit > 0.0f ? fminf(fmaxf(rintf(__fdiv_rn(sr[g], unit)), 1.0f), 15.0f) : 1.0f;
            s = __fmul_rn((float) (int) kf, unit);
        } else {
            s = sr[0];
        }
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = s > 0.0f ? (int) code_of(xr[w * 8 + j], s) : 0;
            code_sum += c;
            word |= (uint32_t) (c & 0xF) << (4 * j);
        }
        yr[w >> 5].qs[w & 31] = word;
    }
    int32_t row_sum = 0;
    if (!wgroup) {
        for (int o = 16; o > 0; o >>= 1) code_sum += __shfl_xor_sync(0xffffffffu, code_sum, o);
        if ((tid & 31) == 0) red_i[tid >> 5] = code_sum;
        __syncthreads();
        for (int i = 0; i < (int) (blockDim.x >> 5); ++i) row_sum += red_i[i];
    }
    for (int b = tid; b < K / RQ_BLOCK_CODES; b += blockDim.x) {
        int32_t sum;
        if (!wgroup) {
            sum = row_sum;
        } else {
            auto mult = [&](int g) -> uint32_t {
                const float kf = unit > 0.0f ? fminf(fmaxf(rintf(__fdiv_rn(sr[g], unit)), 1.0f), 15.0f) : 1.0f;
                return (uint32_t) (int) kf;
            };
            sum = gs == RQ_BLOCK_CODES ? (int32_t) (1u << 30 | mult(b))
                                       : (int32_t) (3u << 29 | mult(4 * b) | mult(4 * b + 1) << 4 | mult(4 * b + 2) << 8 | mult(4 * b + 3) << 12);
        }
        yr[b].d = wgroup ? unit : sr[0];
        yr[b].sum = sum;
        yr[b].pad[0] = pad0;
        yr[b].pad[1] = 0;
    }
}

}  // namespace

// x: [n_rows][K] fp32 rows ldx apart, already rotated for W4A4H.  wgroup: 0, 256 or 64.  sg: n_rows * (K / gs) floats
// of scratch (gs = K without weight groups).  pad0: what the headers' pad[0] records.
cudaError_t rq_launch_wquant(const float * x, int64_t ldx, int64_t n_rows, int64_t K, int wgroup, int pad0, float * sg,
                             rq_block * out, cudaStream_t stream) {
    const int gs = wgroup ? wgroup : (int) K;
    const int64_t units = n_rows * (K / gs);
    const int64_t threads = units * 16;
    rq_wsearch_kernel<<<(unsigned) ((threads + 255) / 256), 256, 0, stream>>>(x, ldx, n_rows, (int) K, gs, sg);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    rq_wpack_kernel<<<(unsigned) n_rows, 256, 0, stream>>>(x, ldx, (int) K, gs, wgroup, pad0, sg, out);
    return cudaGetLastError();
}
