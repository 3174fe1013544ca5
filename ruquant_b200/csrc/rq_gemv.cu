// Decode-width contraction (M <= 16 tokens per pass): an HBM-bound GEMV over the int4 decode stream.
//
// A lane owns 32 consecutive inputs of a row per step (one 128-bit load of the stream), a warp 1024; G/32
// neighbouring lanes make up one activation group and combine their partial sums with shuffles, so every group of
// every (row, token) pair is folded on its own, as the reference's dot product does
// (ggml_vec_dot_w4a4_a4, ggml/src/ggml-cpu/quants.c in patches/llama.cpp-ruquant.patch:148-177):
//     total += (k * m_g * S_g) >> 4,   S_g = sum c * (q - z_g)       (int32, arithmetic shift)
//     y = ((float(total) * 16) * u) * s_w                             (three separate fp32 multiplies)
// Weights arrive as int8 16*c (two logic ops per word, see rq_prepack.cu), activations as int8 8*(q - z), so a
// group's dp4a sum is 128*S_g and the shift by 7 that recovers S_g is exact.
#include "rq_common.cuh"

namespace {

constexpr int GEMV_WARPS = 4;

__device__ __forceinline__ uint4 ld_stream(const void * p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

struct GemvParams {
    const uint8_t * w4;
    const float * sw;
    const int8_t * wk;
    const int8_t * a8;
    const int32_t * msh;
    const float * u;
    float * y;
    int64_t ldy;
    int K, N, M, G;
};

// TT tokens per pass, R rows per warp, KS warps of the CTA splitting K (1 or GEMV_WARPS)
template <int TT, int R, int KS, bool HAS_K>
__global__ void __launch_bounds__(GEMV_WARPS * 32) rq_gemv_kernel(const GemvParams prm) {
    __shared__ int32_t part[GEMV_WARPS][R][TT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = prm.K, N = prm.N, M = prm.M;
    const int units = K >> 5;                 // 32-input lane units per row
    const int n_it = (units + 31) >> 5;
    const int lpg = prm.G >> 5;               // lanes per activation group: 2, 4 or 8
    const int ngrp = K / prm.G;
    const int rows_per_cta = KS == 1 ? R * GEMV_WARPS : R;
    const int row0 = blockIdx.x * rows_per_cta + (KS == 1 ? warp * R : 0);
    const int ks = KS == 1 ? 0 : warp;

    int32_t tot[R][TT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) tot[r][t] = 0;

    const size_t row_bytes = (size_t) K >> 1;
    uint4 wv[R];
    {
        const int unit = ks * 32 + lane;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            wv[r] = make_uint4(0u, 0u, 0u, 0u);
            if (ks < n_it && unit < units && row0 + r < N) wv[r] = ld_stream(prm.w4 + (size_t) (row0 + r) * row_bytes + (size_t) unit * 16);
        }
    }
    for (int it = ks; it < n_it; it += KS) {
        const int unit = it * 32 + lane;
        const bool active = unit < units;
        uint4 wn[R];
        {
            const int nu = unit + KS * 32;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                wn[r] = make_uint4(0u, 0u, 0u, 0u);
                if (it + KS < n_it && nu < units && row0 + r < N) wn[r] = ld_stream(prm.w4 + (size_t) (row0 + r) * row_bytes + (size_t) nu * 16);
            }
        }
        const int g = active ? unit / lpg : 0;
        int kk[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            kk[r] = 1;
            if (HAS_K) kk[r] = (active && row0 + r < N) ? (int) prm.wk[(size_t) (row0 + r) * (K >> 6) + (unit >> 1)] : 1;
        }
        // the int8 views of this lane's 32 codes: lo[j] = 16*(c[8j..8j+3]), hi[j] = 16*(c[8j+4..8j+7])
        int lo[R][4], hi[R][4];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t w[4] = { wv[r].x, wv[r].y, wv[r].z, wv[r].w };
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                lo[r][j] = (int) ((w[j] << 4) & 0xF0F0F0F0u);
                hi[r][j] = (int) (w[j] & 0xF0F0F0F0u);
            }
        }
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            uint4 a0 = make_uint4(0u, 0u, 0u, 0u), a1 = a0;
            int mval = 0;
            if (active && t < M) {
                const uint4 * ap = reinterpret_cast<const uint4 *>(prm.a8 + (size_t) t * K + (size_t) unit * 32);
                a0 = __ldg(ap);
                a1 = __ldg(ap + 1);
                mval = __ldg(prm.msh + (size_t) t * ngrp + g) >> RQ_MSH_SHIFT;
            }
            const int aw[8] = { (int) a0.x, (int) a0.y, (int) a0.z, (int) a0.w, (int) a1.x, (int) a1.y, (int) a1.z, (int) a1.w };
#pragma unroll
            for (int r = 0; r < R; ++r) {
                int s = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s = __dp4a(lo[r][j], aw[2 * j], s);
                    s = __dp4a(hi[r][j], aw[2 * j + 1], s);
                }
                for (int o = 1; o < lpg; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if ((lane & (lpg - 1)) == 0) tot[r][t] += (kk[r] * mval * (s >> 7)) >> 4;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) wv[r] = wn[r];
    }

    // integer sums are exact in any order: lanes first, then (KS > 1) the warps that split K
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            int v = tot[r][t];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            tot[r][t] = v;
        }
    if (KS > 1) {
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int t = 0; t < TT; ++t) part[warp][r][t] = tot[r][t];
        }
        __syncthreads();
        if (warp != 0) return;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int t = 0; t < TT; ++t) {
                int v = 0;
                for (int w = 0; w < GEMV_WARPS; ++w) v += part[w][r][t];
                tot[r][t] = v;
            }
    }
    // epilogue: lane (r, t) pairs spread over the warp
    for (int i = lane; i < R * TT; i += 32) {
        const int r = i / TT, t = i - r * TT;
        int v = 0;
#pragma unroll
        for (int rr = 0; rr < R; ++rr)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) if (rr == r && tt == t) v = tot[rr][tt];
        if (row0 + r < N && t < M) {
            const float f = __fmul_rn(__fmul_rn(__fmul_rn((float) v, 16.0f), __ldg(prm.u + t)), __ldg(prm.sw + row0 + r));
            prm.y[(size_t) t * prm.ldy + row0 + r] = f;
        }
    }
}

template <int TT, int R>
cudaError_t launch_tt(const GemvParams & prm, bool has_k, cudaStream_t stream) {
    // few rows: let the CTA's warps split K so that enough warps are in flight to cover HBM latency
    const bool split = (int64_t) prm.N / R < 148 * 16;
    const int rows_per_cta = split ? R : R * GEMV_WARPS;
    const unsigned grid = (unsigned) ((prm.N + rows_per_cta - 1) / rows_per_cta);
    if (split) {
        if (has_k) rq_gemv_kernel<TT, R, GEMV_WARPS, true><<<grid, GEMV_WARPS * 32, 0, stream>>>(prm);
        else       rq_gemv_kernel<TT, R, GEMV_WARPS, false><<<grid, GEMV_WARPS * 32, 0, stream>>>(prm);
    } else {
        if (has_k) rq_gemv_kernel<TT, R, 1, true><<<grid, GEMV_WARPS * 32, 0, stream>>>(prm);
        else       rq_gemv_kernel<TT, R, 1, false><<<grid, GEMV_WARPS * 32, 0, stream>>>(prm);
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t rq_launch_gemv(const uint8_t * w4, const float * sw, const int8_t * wk, int64_t K, int64_t N,
                           const int8_t * a8, const int32_t * msh, const float * u, int64_t M, int G,
                           float * y, int64_t ldy, cudaStream_t stream) {
    // wider inputs go through in passes of 16 tokens, each re-reading the stream
    for (int64_t t0 = 0; t0 < M; t0 += 16) {
        const int mt = (int) (M - t0 < 16 ? M - t0 : 16);
        GemvParams prm;
        prm.w4 = w4; prm.sw = sw; prm.wk = wk; prm.K = (int) K; prm.N = (int) N; prm.M = mt; prm.G = G;
        prm.a8 = a8 + t0 * K; prm.msh = msh + t0 * (K / G); prm.u = u + t0; prm.y = y + t0 * ldy; prm.ldy = ldy;
        cudaError_t e;
        const bool has_k = wk != nullptr;
        if (mt == 1) e = launch_tt<1, 4>(prm, has_k, stream);
        else if (mt == 2) e = launch_tt<2, 4>(prm, has_k, stream);
        else if (mt <= 4) e = launch_tt<4, 4>(prm, has_k, stream);
        else if (mt <= 8) e = launch_tt<8, 2>(prm, has_k, stream);
        else e = launch_tt<16, 2>(prm, has_k, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}
