// Activation side of the W4A4 / W4A4H MUL_MAT node: online Hadamard rotation + per-token grouped int4 quantizer.
//
// Bit-parity contract (reference: patches/llama.cpp-ruquant.patch, "patch" below):
//   rotation   ggml_rq_hadamard, patch:2450-2485 -- Sylvester butterflies in increasing stride over each chunk of m,
//              then every Paley output summed from 0.0f over ascending i with one add or subtract per term, then one
//              multiply by 1/sqrtf(n).  Every fp32 operation here is an explicit round-to-nearest intrinsic.  A term
//              is applied as fma(x, +-1.0f, acc): the product is exact, so the result is the same single rounding as
//              acc + x / acc - x, and the sign becomes data (a table in shared memory) instead of code.
//   quantizer  rq_quantize_row_a, patch:2639-2679.
// Output layout (what the contraction kernels consume): int8 8*(q - z_g) [M][K] (permuted inside each run of 64
// inputs, see rq_perm64), int32 m_g [M][K/G], f32 u [M]; for the fp8 tensor-core path instead the e4m3 byte of
// (q - z_g) and the f32 bits of m_g / 16.
//
// Two kernels:
//   rq_act_kernel<P>          one CTA per token, the token's row resident in shared memory (prefill widths, any G).
//   rq_act_cluster_kernel<P>  a thread-block cluster per token for decode widths: every CTA transforms the whole row
//                             (redundant, but it spares a gather through distributed shared memory), the Paley outputs
//                             are split between the CTAs, and one cluster barrier agrees on the token's range.
// Both start their successor early (programmatic dependent launch) and build the sign table before they wait for
// the kernel that produced x.
#include <cooperative_groups.h>

#include <stdlib.h>

#include <mutex>
#include <type_traits>

#include "rq_common.cuh"
#include "rq_act_dev.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int ACT_THREADS = 256;
// threads of a cluster CTA: every phase is latency, so as many warps as the Paley stage's registers allow (it reads its
// P inputs once each, the compiler keeps them at about 55-64 registers)
constexpr int cluster_threads(int p) { return p <= 72 ? 1024 : 512; }

using namespace rq_act_dev;


struct ActParams {
    const float * x;
    int64_t ldx;
    int K, n_rot, p, m, G, fmt;
    float rot_scale, clip;
    int8_t * a8;
    int32_t * msh;
    float * u;
    float * rot_out;
    int64_t ldo;
    int32_t * status;
};

// =====================================================================================  one CTA per token
// P > 1: Paley order (compile time); P == 1: no Paley stage (plain W4A4, or a power-of-two rotation).
// shared memory: [K floats row][P*P floats sign table]
// three CTAs (tokens) per SM where the row fits three times in shared memory: caps the 256-thread form at 85 registers
#ifndef RQ_ACT_MIN_CTAS
#define RQ_ACT_MIN_CTAS 3
#endif
template <int P, int THREADS>
__global__ void __launch_bounds__(THREADS, THREADS <= 256 ? RQ_ACT_MIN_CTAS : 1) rq_act_kernel(const ActParams prm) {
    extern __shared__ __align__(16) float buf[];
    __shared__ float g_lo[512], g_hi[512];
    __shared__ float red[THREADS / 32];
    __shared__ signed char chi[128];
    __shared__ uint64_t row_bar;
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int K = prm.K;
    float * table = buf + K;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"((uint32_t) __cvta_generic_to_shared(&row_bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    constexpr bool NEED_TABLE = P > 1 && THREADS > 256;       // the 256-thread form takes every sign from code or constant memory

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    RQ_STAMP_DECL;
    RQ_STAMP(tid == 0);                                     // 0: start
    if constexpr (NEED_TABLE) build_sign_table(table, chi, P, tid, nt);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (t == 0 && tid == 0 && prm.status != nullptr) prm.status[1] = prm.fmt;     // word 0 (errors) is sticky: only the host clears it
    RQ_STAMP(tid == 0);                                     // 1: after the wait

    // the row arrives in one bulk copy (thousands of tokens: what counts is trips to memory per token, and this is one)
    const float * xrow = prm.x + (int64_t) t * prm.ldx;
    if (!bulk_load_row(buf, xrow, (uint32_t) K * 4u, &row_bar, tid)) {
        if (tid == 0 && prm.status != nullptr) atomicExch(prm.status, 1);
        return;
    }
    if (prm.n_rot > 0) {
        fwht_resident(buf, K, prm.m, tid, nt);
        RQ_STAMP(tid == 0);                                 // 2: chunks transformed
    }

    if (prm.n_rot > 0) {
        const int m = prm.m;
        if constexpr (P > 1) {
            const int ncol = K / P, n = prm.n_rot;
            if constexpr (P <= 20 && THREADS <= 256) {
                // many tokens in flight (one CTA each): the adds themselves are the work, signs folded into the code
                for (int c = tid; c < ncol; c += nt) {
                    const int blk = c / m, j = c - blk * m;
                    float * b = buf + (size_t) blk * n + j;
                    float acc[P];
#pragma unroll
                    for (int a = 0; a < P; ++a) acc[a] = 0.0f;
                    paley_static<P>(b, m, acc, std::make_index_sequence<P>{});
#pragma unroll
                    for (int a = 0; a < P; ++a) b[a * m] = __fmul_rn(acc[a], prm.rot_scale);
                }
            } else
            for (int c = tid; c < ncol; c += nt) {
                const int blk = c / m, j = c - blk * m;
                float * b = buf + (size_t) blk * n + j;
                float col[P];
#pragma unroll
                for (int i = 0; i < P; ++i) col[i] = b[i * m];
                for (int a0 = 0; a0 < P; a0 += 4) {
                    float out[4];
                    if constexpr (THREADS <= 256) {
                        if (a0 > 0) paley_block4_const<P>(col, a0, prm.rot_scale, out);
                        else paley_block4_first<P>(col, prm.rot_scale, out, std::make_index_sequence<P>{});      // holds the irregular output 0
                    } else {
                        paley_block4<P>(col, table, a0, prm.rot_scale, out);
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) b[(a0 + k) * m] = out[k];
                }
            }
        } else {
            for (int i = tid; i < K; i += nt) buf[i] = __fmul_rn(buf[i], prm.rot_scale);
        }
        __syncthreads();
        if (prm.rot_out != nullptr) {
            float4 * o = reinterpret_cast<float4 *>(prm.rot_out + (int64_t) t * prm.ldo);
            for (int i = tid; i < K / 4; i += nt) o[i] = reinterpret_cast<float4 *>(buf)[i];
        }
    }
    if (prm.a8 == nullptr) return;
    RQ_STAMP(tid == 0);                                     // 3: Paley done

    // ---- quantizer: a thread owns a word of 8 values, G/8 neighbouring lanes own a group
    const int lpg = prm.G >> 3, nwords = K >> 3;
    const int llpg = __ffs(lpg) - 1;                        // G / 8 is a power of two: a shift, not a division, per word
    float tmax = 0.0f;
    for (int w = tid; w < nwords; w += nt) {
        float lo, hi;
        group_range(reinterpret_cast<float4 *>(buf)[2 * w], reinterpret_cast<float4 *>(buf)[2 * w + 1], lpg, prm.clip, lo, hi);
        if ((w & (lpg - 1)) == 0) {
            g_lo[w >> llpg] = lo;
            g_hi[w >> llpg] = hi;
        }
        tmax = fmaxf(tmax, __fsub_rn(hi, lo));
    }
    tmax = cta_max_warp0(tmax, red, tid, nt);
    if (tid == 0) red[0] = tmax;
    __syncthreads();
    float R = red[0];
    if (R == 0.0f) R = 2.0f;
    const float unit = __fdiv_rn(R, 15.0f * 255.0f);
    if (tid == 0) prm.u[t] = unit;
    RQ_STAMP(tid == 0);                                     // 4: ranges reduced

    int8_t * arow = prm.a8 + (int64_t) t * K;
    int32_t * mrow = prm.msh + (int64_t) t * (K / prm.G);
    auto store_codes = [&](auto f8) {
        constexpr bool F8 = decltype(f8)::value;
        for (int w = tid; w < nwords; w += nt) {
            const int g = w >> llpg;
            float mi;
            const uint2 pk = encode_word<F8>(reinterpret_cast<float4 *>(buf)[2 * w], reinterpret_cast<float4 *>(buf)[2 * w + 1],
                                             g_lo[g], g_hi[g], R, unit, mi);
            const int kw = w * 8, run = kw & ~63, off = kw & 63;   // two 4-input pieces, permuted inside their run of 64
            *reinterpret_cast<uint32_t *>(arow + run + rq_perm64(off)) = pk.x;
            *reinterpret_cast<uint32_t *>(arow + run + rq_perm64(off + 4)) = pk.y;
            if ((w & (lpg - 1)) == 0) mrow[g] = multiplier_word<F8>(mi);
        }
    };
    if (prm.fmt == RQ_FMT_E4M3) store_codes(std::true_type{});
    else store_codes(std::false_type{});
    RQ_STAMP(tid == 0);                                     // 5: codes stored
    RQ_STAMP_FLUSH(tid == 0, prm.status, 0x30);
}

// =====================================================================================  a cluster per token
// For G = 64, m a multiple of 64 and P > 1: decode widths, where one SM is too slow and every hand-over between CTAs
// costs about as much as a whole phase.  C = gridDim.x CTAs per token.  Every CTA loads the whole row and transforms
// all its chunks (cheap, and it spares a cluster barrier and a gather through distributed shared memory); the Paley
// outputs are dealt out in units of 4 output chunks x 64 columns -- unit v = (blk * (m/64) + js) * (P/4) + ab covers
// outputs blk*n + (4 ab + k)*m + 64 js + col, k < 4, col < 64: four activation groups -- round-robin, unit v to CTA
// v % C.  A thread = (column, unit slot) forms the unit's 4 outputs of its column from registers.  The only exchange
// is the token's range: one float per CTA written into every peer's shared memory, one cluster barrier.
// shared memory: [K row][P*P sign table][units_max * 4 * 64 outputs]
template <int P, int THREADS>
__global__ void __launch_bounds__(THREADS) rq_act_cluster_kernel(const ActParams prm, int units_max) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[THREADS / 32];
    __shared__ float peer_max[16];
    __shared__ signed char chi[128];
    cg::cluster_group cluster = cg::this_cluster();
    const int C = gridDim.x, rank = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, nt = THREADS;
    const int K = prm.K, m = prm.m, n = prm.n_rot;
    constexpr int NB = P / 4;
    const int nq = m >> 6, units = (K / n) * nq * NB;
    const int lq = __ffs(nq) - 1;                           // m is a power of two: shifts and masks instead of divisions by nq
    const int nl = (units - rank + C - 1) / C;              // units of this CTA: rank, rank + C, ...
    float * row = smem;
    float * table = row + K;
    float * outs = table + P * P;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    RQ_STAMP_DECL;
    RQ_STAMP(tid == 0);                                     // 0: start
    // pull the row towards L2 while the kernel ahead may still be running (a hint: no value is read before the wait)
    for (int i = rank * nt + tid; i < K / 32; i += C * nt) asm volatile("prefetch.global.L2 [%0];" :: "l"(prm.x + (int64_t) t * prm.ldx + i * 32));
    build_sign_table(table, chi, P, tid, nt);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    RQ_STAMP(tid == 0);                                     // 1: after the wait
    if (t == 0 && rank == 0 && tid == 0 && prm.status != nullptr) prm.status[1] = prm.fmt;

    // ---- Sylvester transform of every chunk of the row
    load_fwht(prm.x + (int64_t) t * prm.ldx, row, K, m, tid, nt);
    RQ_STAMP(tid == 0);                                     // 2: chunks transformed

    // ---- Paley: this CTA's units, THREADS / 64 of them side by side
    const int col = tid & 63;
    for (int l = tid >> 6; l < nl; l += THREADS / 64) {
        const int v = rank + l * C;
        const int ab = v % NB, sl = v / NB, js = sl & (nq - 1), blk = sl >> lq;
        const float * b = row + (size_t) blk * n + js * 64 + col;
        float colv[P];
#pragma unroll
        for (int i = 0; i < P; ++i) colv[i] = b[i * m];
        float out[4];
        paley_block4<P>(colv, table, ab * 4, prm.rot_scale, out);
#pragma unroll
        for (int k = 0; k < 4; ++k) outs[(l * 4 + k) * 64 + col] = out[k];
    }
    __syncthreads();
    RQ_STAMP(tid == 0);                                     // 3: Paley done

    // ---- group ranges: a row of 64 outputs is one activation group (8 lanes x 8 values); nl * 32 words, so a warp is
    // inside or outside the loop as a whole
    const int words = nl * 32;
    float tmax = 0.0f;
    for (int w = tid; w < words; w += nt) {
        float lo, hi;
        group_range(reinterpret_cast<float4 *>(outs)[2 * w], reinterpret_cast<float4 *>(outs)[2 * w + 1], 8, prm.clip, lo, hi);
        tmax = fmaxf(tmax, __fsub_rn(hi, lo));
    }
    tmax = cta_max_warp0(tmax, red, tid, nt);
    if (tid < C) cluster.map_shared_rank(peer_max, tid)[rank] = tmax;     // my maximum into slot `rank` of CTA tid
    RQ_STAMP(tid == 0);                                     // 4: ranges reduced
    cluster.sync();
    RQ_STAMP(tid == 0);                                     // 5: cluster barrier
    float R = 0.0f;
    for (int i = 0; i < C; ++i) R = fmaxf(R, peer_max[i]);
    if (R == 0.0f) R = 2.0f;
    const float unit = __fdiv_rn(R, 15.0f * 255.0f);
    if (rank == 0 && tid == 0) prm.u[t] = unit;

    // ---- codes
    int8_t * arow = prm.a8 + (int64_t) t * K;
    int32_t * mrow = prm.msh + (int64_t) t * (K / 64);
    auto store_codes = [&](auto f8) {
        constexpr bool F8 = decltype(f8)::value;
        for (int w = tid; w < words; w += nt) {
            const int r = w >> 3, l = r >> 2, k = r & 3;
            const int v = rank + l * C;
            const int ab = v % NB, sl = v / NB, js = sl & (nq - 1), blk = sl >> lq;
            const int kbase = blk * n + (ab * 4 + k) * m + js * 64;         // first input of this group in the row
            const float4 a = reinterpret_cast<float4 *>(outs)[2 * w], b = reinterpret_cast<float4 *>(outs)[2 * w + 1];
            float lo, hi;
            group_range(a, b, 8, prm.clip, lo, hi);
            float mi;
            const uint2 pk = encode_word<F8>(a, b, lo, hi, R, unit, mi);
            const int off = (w & 7) * 8;
            *reinterpret_cast<uint32_t *>(arow + kbase + rq_perm64(off)) = pk.x;
            *reinterpret_cast<uint32_t *>(arow + kbase + rq_perm64(off + 4)) = pk.y;
            if ((w & 7) == 0) mrow[kbase >> 6] = multiplier_word<F8>(mi);
        }
    };
    if (prm.fmt == RQ_FMT_E4M3) store_codes(std::true_type{});
    else store_codes(std::false_type{});
    RQ_STAMP(tid == 0);                                     // 6: codes stored
    RQ_STAMP_FLUSH(tid == 0, prm.status, 0x20);
}

template <typename Kern, typename... Args>
cudaError_t launch_ex(Kern kern, dim3 grid, dim3 block, size_t smem, int cluster_x, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    static const int pdl = getenv("RQ_NO_PDL") ? 0 : 1;      // read once
    attr[na].val.programmaticStreamSerializationAllowed = pdl;
    ++na;
    if (cluster_x > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned) cluster_x;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

constexpr size_t SMEM_LIMIT = 220 * 1024;

template <typename Kern>
cudaError_t configure_kernel(Kern kern) {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) SMEM_LIMIT);
}

template <int P>
cudaError_t configure() {
    cudaError_t e = configure_kernel(rq_act_kernel<P, ACT_THREADS>);
    if (e != cudaSuccess) return e;
    if (P <= 20) {
        e = configure_kernel(rq_act_kernel<(P <= 20 ? P : 1), 1024>);
        if (e != cudaSuccess) return e;
    }
    if (P == 1) return e;
    return configure_kernel(rq_act_cluster_kernel<(P > 1 ? P : 12), cluster_threads(P > 1 ? P : 12)>);
}

template <int P>
cudaError_t launch(const ActParams & prm, int64_t M, cudaStream_t stream) {
    // first use on a device (normally rq_w4a4_prepare's); several host threads may get here at once
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev]) {
            e = configure<P>();
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
    }
    const int K = prm.K;
    static const int min_p = rq_env_int("RQ_TUNE_ACT_MINP", 0);
    if (P > 1 && P >= min_p && prm.a8 != nullptr && prm.rot_out == nullptr && prm.G == 64 && prm.m % 64 == 0 && M <= 32) {
        // decode widths: a cluster per token
        constexpr int CP = P > 1 ? P : 12, CT = cluster_threads(CP);
        const int units = (K / prm.n_rot) * (prm.m / 64) * (CP / 4);
        static const int c_max = rq_env_int("RQ_TUNE_ACT_CMAX", 8);
        int C = c_max;
        while (C > 1 && units < 2 * C) C >>= 1;
        const int units_max = (units + C - 1) / C;
        const size_t smem = ((size_t) K + (size_t) CP * CP + (size_t) units_max * 4 * 64) * sizeof(float);
        if (C > 1 && smem <= SMEM_LIMIT) {
            return launch_ex(rq_act_cluster_kernel<CP, CT>, dim3((unsigned) C, (unsigned) M), dim3(CT), smem, C, stream, prm, units_max);
        }
    }
    const size_t smem_row = (size_t) K * sizeof(float);
    const size_t smem = smem_row + (P > 1 ? (size_t) P * P : 0) * sizeof(float);       // the wide CTA keeps a sign table
    if (smem > SMEM_LIMIT) return cudaErrorInvalidValue;
    // few tokens and a cheap Paley stage: one big CTA per token keeps every phase short
    static const int wide = rq_env_int("RQ_TUNE_ACT_WIDE", 1);
    if (P <= 20 && M <= 64 && wide) return launch_ex(rq_act_kernel<(P <= 20 ? P : 1), 1024>, dim3((unsigned) M), dim3(1024), smem, 1, stream, prm);
    return launch_ex(rq_act_kernel<P, ACT_THREADS>, dim3((unsigned) M), dim3(ACT_THREADS), smem_row, 1, stream, prm);
}

}  // namespace

// opt every instantiation into the large dynamic shared memory carve-out (done by rq_w4a4_prepare, outside capture)
cudaError_t rq_configure_act() {
    cudaError_t e;
    if ((e = configure<1>()) != cudaSuccess) return e;
    if ((e = configure<12>()) != cudaSuccess) return e;
    if ((e = configure<20>()) != cudaSuccess) return e;
    if ((e = configure<44>()) != cudaSuccess) return e;
    if ((e = configure<60>()) != cudaSuccess) return e;
    if ((e = configure<68>()) != cudaSuccess) return e;
    if ((e = configure<72>()) != cudaSuccess) return e;
    if ((e = configure<84>()) != cudaSuccess) return e;
    if ((e = configure<104>()) != cudaSuccess) return e;
    return configure<108>();
}

cudaError_t rq_launch_act(const float * x, int64_t ldx, int64_t M, int64_t K, int n_rot, int p, int m, float rot_scale,
                          float clip, int G, int fmt, int8_t * a8, int32_t * msh, float * u, float * rot_out, int64_t ldo,
                          int32_t * status, cudaStream_t stream) {
    ActParams prm;
    prm.x = x; prm.ldx = ldx; prm.K = (int) K; prm.n_rot = n_rot; prm.p = p; prm.m = m; prm.G = G; prm.fmt = fmt;
    prm.rot_scale = rot_scale; prm.clip = clip; prm.a8 = a8; prm.msh = msh; prm.u = u; prm.rot_out = rot_out; prm.ldo = ldo;
    prm.status = status;
    if (n_rot <= 0 || p == 1) return launch<1>(prm, M, stream);
    switch (p) {   // every order the factorisation can return (ggml_rq_hadamard_factor, patch:2419-2430)
        case 12:  return launch<12>(prm, M, stream);
        case 20:  return launch<20>(prm, M, stream);
        case 44:  return launch<44>(prm, M, stream);
        case 60:  return launch<60>(prm, M, stream);
        case 68:  return launch<68>(prm, M, stream);
        case 72:  return launch<72>(prm, M, stream);
        case 84:  return launch<84>(prm, M, stream);
        case 104: return launch<104>(prm, M, stream);
        case 108: return launch<108>(prm, M, stream);
        default:  return cudaErrorInvalidValue;
    }
}
