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
//   rq_act_cluster_kernel<P>  a thread-block cluster per token for decode widths: the CTAs transform disjoint chunks,
//                             exchange columns through distributed shared memory, split the Paley outputs between
//                             them and agree on the token's range with one more cluster barrier.
// Both start their successor early (programmatic dependent launch) and build the sign table before they wait for
// the kernel that produced x.
#include <cooperative_groups.h>

#include <stdlib.h>

#include "rq_common.cuh"
#include "rq_act_dev.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int ACT_THREADS = 256;

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
template <int P, int THREADS>
__global__ void __launch_bounds__(THREADS) rq_act_kernel(const ActParams prm) {
    extern __shared__ __align__(16) float buf[];
    __shared__ float g_lo[512], g_hi[512];
    __shared__ float red[THREADS / 32];
    __shared__ signed char chi[128];
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int K = prm.K;
    float * table = buf + K;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if constexpr (P > 1) build_sign_table(table, chi, P, tid, nt);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (t == 0 && tid == 0 && prm.status != nullptr) { prm.status[0] = 0; prm.status[1] = prm.fmt; }

    const float * xrow = prm.x + (int64_t) t * prm.ldx;
    if (prm.n_rot > 0) {
        load_fwht(xrow, buf, K, prm.m, tid, nt);
    } else {
        for (int i = tid; i < K / 4; i += nt) reinterpret_cast<float4 *>(buf)[i] = __ldg(reinterpret_cast<const float4 *>(xrow) + i);
        __syncthreads();
    }

    if (prm.n_rot > 0) {
        const int m = prm.m;
        if constexpr (P > 1) {
            const int ncol = K / P, n = prm.n_rot;
            for (int c = tid; c < ncol; c += nt) {
                const int blk = c / m, j = c - blk * m;
                float * b = buf + (size_t) blk * n + j;
                float col[P];
#pragma unroll
                for (int i = 0; i < P; ++i) col[i] = b[i * m];
                for (int a0 = 0; a0 < P; a0 += 4) {
                    float out[4];
                    paley_block4<P>(col, table, a0, prm.rot_scale, out);
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

    // ---- quantizer: a thread owns a word of 8 values, G/8 neighbouring lanes own a group
    const int lpg = prm.G >> 3, nwords = K >> 3;
    float tmax = 0.0f;
    for (int w = tid; w < nwords; w += nt) {
        float lo, hi;
        group_range(reinterpret_cast<float4 *>(buf)[2 * w], reinterpret_cast<float4 *>(buf)[2 * w + 1], lpg, prm.clip, lo, hi);
        if ((w & (lpg - 1)) == 0) {
            g_lo[w / lpg] = lo;
            g_hi[w / lpg] = hi;
        }
        tmax = fmaxf(tmax, __fsub_rn(hi, lo));
    }
    for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    if ((tid & 31) == 0) red[tid >> 5] = tmax;
    __syncthreads();
    float R = 0.0f;
    for (int i = 0; i < nt / 32; ++i) R = fmaxf(R, red[i]);
    if (R == 0.0f) R = 2.0f;
    const float unit = __fdiv_rn(R, 15.0f * 255.0f);
    if (tid == 0) prm.u[t] = unit;

    int8_t * arow = prm.a8 + (int64_t) t * K;
    int32_t * mrow = prm.msh + (int64_t) t * (K / prm.G);
    for (int w = tid; w < nwords; w += nt) {
        const int g = w / lpg;
        int mi;
        const uint2 pk = encode_word(reinterpret_cast<float4 *>(buf)[2 * w], reinterpret_cast<float4 *>(buf)[2 * w + 1],
                                     g_lo[g], g_hi[g], R, unit, prm.fmt, mi);
        const int kw = w * 8, run = kw & ~63, off = kw & 63;   // two 4-input pieces, permuted inside their run of 64
        *reinterpret_cast<uint32_t *>(arow + run + rq_perm64(off)) = pk.x;
        *reinterpret_cast<uint32_t *>(arow + run + rq_perm64(off + 4)) = pk.y;
        if ((w & (lpg - 1)) == 0) mrow[g] = prm.fmt == RQ_FMT_E4M3 ? __float_as_int(__fmul_rn((float) mi, 0.0625f)) : mi;
    }
}

// =====================================================================================  a cluster per token
// For G = 64, m a multiple of 64 and P > 1.  C = gridDim.x CTAs per token (8 or a smaller power of two).
//   chunk ch = blk * P + i (m floats) is loaded and transformed by CTA ch % C into its slot ch / C;
//   slice sl = blk * (m/64) + js owns columns [64 js, 64 js + 64) of block blk; T = K / (64 P) slices.
//   With C >= T, cps = C / T CTAs share a slice and deal its NB = P / 4 blocks of 4 outputs round-robin; with C < T a
//   CTA walks nsl = T / C slices and forms all their outputs.  Per slice the CTA first copies the slice's P x 64
//   inputs out of the owners' shared memory (distributed shared memory, 256-byte rows), then a thread = (column,
//   block slot) forms 4 outputs from registers; a row of 64 outputs is one activation group.
// shared memory: [slots * m chunks][P*P sign table][P * 64 slice][nsl * nb_max * 4 * 64 outputs]
template <int P>
__global__ void __launch_bounds__(ACT_THREADS) rq_act_cluster_kernel(const ActParams prm, int slots, int cps, int nsl, int nb_max) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[ACT_THREADS / 32];
    __shared__ float peer_max[8];
    __shared__ signed char chi[128];
    cg::cluster_group cluster = cg::this_cluster();
    const int C = gridDim.x, rank = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
    const int K = prm.K, m = prm.m, n = prm.n_rot;
    const int nchunks = K / m, spb = m / 64, NB = P / 4;
    float * chunks = smem;
    float * table = chunks + (size_t) slots * m;
    float * slice = table + P * P;
    float * outs = slice + P * 64;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    build_sign_table(table, chi, P, tid, nt);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (t == 0 && rank == 0 && tid == 0 && prm.status != nullptr) { prm.status[0] = 0; prm.status[1] = prm.fmt; }

    // ---- Sylvester transform of this CTA's chunks (chunk rank + C*s lands in slot s)
    const float * xrow = prm.x + (int64_t) t * prm.ldx;
    {
        int nloc = 0;
        for (int ch = rank; ch < nchunks; ch += C) ++nloc;
        switch (m < 1024 ? m : 1024) {
            case 64:   cluster_chunks<2>(xrow, chunks, rank, C, nloc, m, tid, nt); break;
            case 128:  cluster_chunks<4>(xrow, chunks, rank, C, nloc, m, tid, nt); break;
            case 256:  cluster_chunks<8>(xrow, chunks, rank, C, nloc, m, tid, nt); break;
            case 512:  cluster_chunks<16>(xrow, chunks, rank, C, nloc, m, tid, nt); break;
            default:   cluster_chunks<32>(xrow, chunks, rank, C, nloc, m, tid, nt); break;
        }
        __syncthreads();
        for (int ls = 10; (1 << ls) < m; ls += 3) {
            const int rem = m >> ls;
            if (rem >= 8) fwht_pass<8>(chunks, nloc * m, ls, tid, nt);
            else if (rem == 4) fwht_pass<4>(chunks, nloc * m, ls, tid, nt);
            else fwht_pass<2>(chunks, nloc * m, ls, tid, nt);
            __syncthreads();
        }
    }
    cluster.sync();

    // ---- Paley, slice by slice
    const int col = tid & 63, bslot = tid >> 6;            // 4 block slots run side by side
    const int sub = C >= (K / (64 * P)) ? rank % cps : 0;
    float tmax = 0.0f;
    for (int si = 0; si < nsl; ++si) {
        const int sl = cps > 1 || nsl == 1 ? rank / cps : rank + si * C;
        const int blk = sl / spb, js = sl - blk * spb;
        for (int idx = tid; idx < P * 16; idx += nt) {      // the slice's P rows of 64 floats, as float4
            const int i = idx >> 4, q4 = idx & 15;
            const int ch = blk * P + i;
            const float * remote = cluster.map_shared_rank(chunks, ch % C);
            reinterpret_cast<float4 *>(slice)[idx] = *reinterpret_cast<const float4 *>(remote + (size_t) (ch / C) * m + js * 64 + q4 * 4);
        }
        __syncthreads();
        float colv[P];
#pragma unroll
        for (int i = 0; i < P; ++i) colv[i] = slice[i * 64 + col];
        for (int lb = bslot; lb * cps + sub < NB; lb += 4) {
            const int ab = lb * cps + sub;
            float out[4];
            paley_block4<P>(colv, table, ab * 4, prm.rot_scale, out);
#pragma unroll
            for (int k = 0; k < 4; ++k) outs[((si * nb_max + lb) * 4 + k) * 64 + col] = out[k];
        }
        __syncthreads();
    }

    // ---- group ranges: a row of 64 outputs is one activation group (8 lanes x 8 values)
    int my_nb = 0;
    for (int ab = sub; ab < NB; ab += cps) ++my_nb;
    const int words_per_slice = my_nb * 32;                 // 4 rows x 8 words per block
    for (int si = 0; si < nsl; ++si) {
        for (int w = tid; w < words_per_slice; w += nt) {
            const int wi = (si * nb_max * 4) * 8 + w;
            float lo, hi;
            group_range(reinterpret_cast<float4 *>(outs)[2 * wi], reinterpret_cast<float4 *>(outs)[2 * wi + 1], 8, prm.clip, lo, hi);
            tmax = fmaxf(tmax, __fsub_rn(hi, lo));
        }
    }
    for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    if ((tid & 31) == 0) red[tid >> 5] = tmax;
    __syncthreads();
    if (tid < C) {
        float v = 0.0f;
        for (int i = 0; i < nt / 32; ++i) v = fmaxf(v, red[i]);
        float * remote = cluster.map_shared_rank(peer_max, tid);   // my maximum into slot `rank` of CTA tid
        remote[rank] = v;
    }
    cluster.sync();
    float R = 0.0f;
    for (int i = 0; i < C; ++i) R = fmaxf(R, peer_max[i]);
    if (R == 0.0f) R = 2.0f;
    const float unit = __fdiv_rn(R, 15.0f * 255.0f);
    if (rank == 0 && tid == 0) prm.u[t] = unit;

    // ---- codes
    int8_t * arow = prm.a8 + (int64_t) t * K;
    int32_t * mrow = prm.msh + (int64_t) t * (K / 64);
    for (int si = 0; si < nsl; ++si) {
        const int sl = cps > 1 || nsl == 1 ? rank / cps : rank + si * C;
        const int blk = sl / spb, js = sl - blk * spb;
        for (int w = tid; w < words_per_slice; w += nt) {
            const int row = w >> 3, lb = row >> 2, k = row & 3;
            const int ab = lb * cps + sub;
            const int kbase = blk * n + (ab * 4 + k) * m + js * 64;      // first input of this group in the row
            const int wi = (si * nb_max * 4) * 8 + w;
            const float4 a = reinterpret_cast<float4 *>(outs)[2 * wi], b = reinterpret_cast<float4 *>(outs)[2 * wi + 1];
            float lo, hi;
            group_range(a, b, 8, prm.clip, lo, hi);
            int mi;
            const uint2 pk = encode_word(a, b, lo, hi, R, unit, prm.fmt, mi);
            const int off = (w & 7) * 8;
            *reinterpret_cast<uint32_t *>(arow + kbase + rq_perm64(off)) = pk.x;
            *reinterpret_cast<uint32_t *>(arow + kbase + rq_perm64(off + 4)) = pk.y;
            if ((w & 7) == 0) mrow[kbase >> 6] = prm.fmt == RQ_FMT_E4M3 ? __float_as_int(__fmul_rn((float) mi, 0.0625f)) : mi;
        }
    }
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
    attr[na].val.programmaticStreamSerializationAllowed = getenv("RQ_NO_PDL") ? 0 : 1;
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

template <int P>
cudaError_t configure() {
    cudaError_t e = cudaFuncSetAttribute(rq_act_kernel<P, ACT_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) SMEM_LIMIT);
    if (e != cudaSuccess) return e;
    if (P <= 20) {
        e = cudaFuncSetAttribute(rq_act_kernel<(P <= 20 ? P : 1), 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) SMEM_LIMIT);
        if (e != cudaSuccess) return e;
    }
    if (P == 1) return e;
    return cudaFuncSetAttribute(rq_act_cluster_kernel<(P > 1 ? P : 12)>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) SMEM_LIMIT);
}

template <int P>
cudaError_t launch(const ActParams & prm, int64_t M, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = configure<P>();
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int K = prm.K;
    static const int min_p = getenv("RQ_TUNE_ACT_MINP") ? atoi(getenv("RQ_TUNE_ACT_MINP")) : 0;
    if (P > 1 && P >= min_p && prm.a8 != nullptr && prm.rot_out == nullptr && prm.G == 64 && prm.m % 64 == 0 && M <= 32) {
        // decode widths: a cluster per token
        const int T = K / (64 * P), NB = P / 4, nchunks = K / prm.m;
        int C = 8;
        while (C > 1 && !((C % T == 0 && C / T <= NB) || T % C == 0)) C >>= 1;
        const int cps = C >= T ? C / T : 1, nsl = C >= T ? 1 : T / C;
        const int slots = (nchunks + C - 1) / C, nb_max = (NB + cps - 1) / cps;
        const size_t smem = ((size_t) slots * prm.m + (size_t) P * P + (size_t) P * 64 + (size_t) nsl * nb_max * 4 * 64) * sizeof(float);
        if (C > 1 && smem <= SMEM_LIMIT) {
            return launch_ex(rq_act_cluster_kernel<(P > 1 ? P : 12)>, dim3((unsigned) C, (unsigned) M), dim3(ACT_THREADS), smem, C,
                             stream, prm, slots, cps, nsl, nb_max);
        }
    }
    const size_t smem = ((size_t) K + (P > 1 ? (size_t) P * P : 0)) * sizeof(float);
    if (smem > SMEM_LIMIT) return cudaErrorInvalidValue;
    // few tokens and a cheap Paley stage: one big CTA per token keeps every phase short
    static const int wide = getenv("RQ_TUNE_ACT_WIDE") ? atoi(getenv("RQ_TUNE_ACT_WIDE")) : 1;
    if (P <= 20 && M <= 64 && wide) return launch_ex(rq_act_kernel<(P <= 20 ? P : 1), 1024>, dim3((unsigned) M), dim3(1024), smem, 1, stream, prm);
    return launch_ex(rq_act_kernel<P, ACT_THREADS>, dim3((unsigned) M), dim3(ACT_THREADS), smem, 1, stream, prm);
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
