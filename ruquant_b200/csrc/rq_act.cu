// Activation side of the W4A4 / W4A4H MUL_MAT node: online Hadamard rotation + per-token grouped int4 quantizer,
// one kernel, one CTA per token, the token's row resident in shared memory from load to store.
//
// Bit-parity contract (reference: patches/llama.cpp-ruquant.patch, "patch" below):
//   rotation   ggml_rq_hadamard, patch:2450-2485 -- Sylvester butterflies in increasing stride over each chunk of m,
//              then every Paley output summed from 0.0f over ascending i with one add or subtract per term, then one
//              multiply by 1/sqrtf(n).  Every fp32 operation here is an explicit round-to-nearest intrinsic so that
//              nothing is contracted or reassociated.
//   quantizer  rq_quantize_row_a, patch:2639-2679.
// The kernel writes the activation in the layout the contraction kernels consume: int8 8*(q - z_g) [M][K],
// int32 m_g << 21 [M][K/G], f32 u [M].
#include <utility>

#include "rq_common.cuh"

namespace {

constexpr int ACT_THREADS = 256;

// bit r of (LO, HI) is set when r is a non-zero square mod q: the Legendre symbol chi(r) = +1
constexpr unsigned long long qr_bits(int q, int half) {
    unsigned long long b = 0;
    for (int i = 1; i < q; ++i) {
        const int r = (i * i) % q;
        if (r / 64 == half) b |= 1ull << (r % 64);
    }
    return b;
}

// Sign of entry (i, a) of the Paley-I matrix A = I + S of order P (rq_paley, patch:2432-2448):
// S[0][a>0] = +1, S[i>0][0] = -1, S[i][a] = chi((a - i) mod q), and the diagonal of A is +1.
template <int P, int I, int A>
struct PaleySign {
    static constexpr int Q = P - 1;
    static constexpr int R = ((A - I) % Q + Q) % Q;
    static constexpr bool plus = (I == A) ? true : (I == 0) ? true : (A == 0) ? false
                                 : ((R < 64 ? (qr_bits(Q, 0) >> (R % 64)) : (qr_bits(Q, 1) >> (R % 64))) & 1ull) != 0;
};

template <int P, int A, int... I>
__device__ __forceinline__ float paley_output(const float (&col)[P], std::integer_sequence<int, I...>) {
    float acc = 0.0f;
    ((acc = PaleySign<P, I, A>::plus ? __fadd_rn(acc, col[I]) : __fsub_rn(acc, col[I])), ...);
    return acc;
}

template <int P, int... A>
__device__ __forceinline__ void paley_column(const float (&col)[P], float * b, int m, float scale,
                                             std::integer_sequence<int, A...>) {
    ((b[A * m] = __fmul_rn(paley_output<P, A>(col, std::make_integer_sequence<int, P>{}), scale)), ...);
}

// Paley stage for a compile-time order: a thread owns column j of one rotation block, holds its P inputs in
// registers and emits the P outputs with every sign folded at compile time (one FADD per term).
template <int P>
__device__ __forceinline__ void paley_fixed(float * buf, int K, int n, int m, float scale, int tid, int nt) {
    const int ncol = K / P;
    for (int c = tid; c < ncol; c += nt) {
        const int blk = c / m, j = c - blk * m;
        float * b = buf + (size_t) blk * n + j;
        float col[P];
#pragma unroll
        for (int i = 0; i < P; ++i) col[i] = b[i * m];
        paley_column<P>(col, b, m, scale, std::make_integer_sequence<int, P>{});
    }
}

// Any order up to 128 (the factorisation admits 12, 20, 44, 60, 68, 72, 84, 104, 108): signs from a Legendre table
// in shared memory, outputs parked in local memory until the column has been read for the last time.
__device__ void paley_generic(float * buf, int K, int n, int p, int m, float scale, const signed char * chi, int tid,
                              int nt) {
    const int ncol = K / p, q = p - 1;
    float out[128];
    for (int c = tid; c < ncol; c += nt) {
        const int blk = c / m, j = c - blk * m;
        float * b = buf + (size_t) blk * n + j;
        for (int a = 0; a < p; ++a) {
            float acc = 0.0f;
            for (int i = 0; i < p; ++i) {
                bool plus;
                if (i == a || i == 0) plus = true;
                else if (a == 0) plus = false;
                else plus = chi[(((a - i) % q) + q) % q] > 0;
                const float v = b[i * m];
                acc = plus ? __fadd_rn(acc, v) : __fsub_rn(acc, v);
            }
            out[a] = acc;
        }
        for (int a = 0; a < p; ++a) b[a * m] = __fmul_rn(out[a], scale);
    }
}

// One radix-R pass of the Sylvester transform over every chunk: elements base + j*s, j < R, go through log2(R)
// butterfly stages of strides s, 2s, 4s (the reference's order, h ascending; each stage is c[k] = a + b,
// c[k+h] = a - b with k the lower index, patch:2456-2463).
template <int R>
__device__ __forceinline__ void fwht_pass(float * buf, int K, int ls, int tid, int nt) {
    const int s = 1 << ls;
    for (int q = tid; q < K / R; q += nt) {
        const int hi = q >> ls, lo = q & (s - 1);
        float * b = buf + (size_t) hi * s * R + lo;
        float v[R];
#pragma unroll
        for (int j = 0; j < R; ++j) v[j] = b[j * s];
#pragma unroll
        for (int d = 1; d < R; d <<= 1) {
#pragma unroll
            for (int j = 0; j < R; ++j) {
                if ((j & d) == 0) {
                    const float a = v[j], c = v[j + d];
                    v[j] = __fadd_rn(a, c);
                    v[j + d] = __fsub_rn(a, c);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < R; ++j) b[j * s] = v[j];
    }
}

struct ActParams {
    const float * x;
    int64_t ldx;
    int K, n_rot, p, m, G;
    float rot_scale, clip;
    int8_t * a8;
    int32_t * msh;
    float * u;
    float * rot_out;
    int64_t ldo;
};

// P > 1: compile-time Paley order; P == 1: no Paley stage (plain W4A4, or a power-of-two rotation);
// P == 0: run-time order prm.p.
template <int P>
__global__ void __launch_bounds__(ACT_THREADS) rq_act_kernel(const ActParams prm) {
    extern __shared__ __align__(16) float buf[];
    __shared__ float g_lo[512], g_hi[512];
    __shared__ float red[ACT_THREADS / 32];
    __shared__ signed char chi[128];
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int K = prm.K;

    const float4 * xr = reinterpret_cast<const float4 *>(prm.x + (int64_t) t * prm.ldx);
    for (int i = tid; i < K / 4; i += nt) reinterpret_cast<float4 *>(buf)[i] = __ldg(xr + i);
    if (P == 0) {
        const int q = prm.p - 1;
        if (tid < 128) chi[tid] = tid == 0 ? 0 : -1;
        __syncthreads();
        if (tid >= 1 && tid < q) chi[(tid * tid) % q] = 1;
    }
    __syncthreads();

    if (prm.n_rot > 0) {
        const int m = prm.m;
        for (int ls = 0; (1 << ls) < m; ls += 3) {
            const int rem = m >> ls;
            if (rem >= 8) fwht_pass<8>(buf, K, ls, tid, nt);
            else if (rem == 4) fwht_pass<4>(buf, K, ls, tid, nt);
            else fwht_pass<2>(buf, K, ls, tid, nt);
            __syncthreads();
        }
        if (P > 1) {
            paley_fixed<(P > 1 ? P : 12)>(buf, K, prm.n_rot, m, prm.rot_scale, tid, nt);
        } else if (P == 0) {
            paley_generic(buf, K, prm.n_rot, prm.p, m, prm.rot_scale, chi, tid, nt);
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
    const float clip = prm.clip;
    float tmax = 0.0f;
    for (int w = tid; w < nwords; w += nt) {
        const float4 a = reinterpret_cast<float4 *>(buf)[2 * w], b = reinterpret_cast<float4 *>(buf)[2 * w + 1];
        float mn = fminf(fminf(fminf(a.x, a.y), fminf(a.z, a.w)), fminf(fminf(b.x, b.y), fminf(b.z, b.w)));
        float mx = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
        mn = fminf(mn, 0.0f);
        mx = fmaxf(mx, 0.0f);
        for (int o = 1; o < lpg; o <<= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const float lo = __fmul_rn(mn, clip), hi = __fmul_rn(mx, clip);
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
        const float lo = g_lo[g], hi = g_hi[g];
        const float mf = fminf(fmaxf(ceilf(__fdiv_rn(__fmul_rn(__fsub_rn(hi, lo), 255.0f), R)), 1.0f), 255.0f);
        const int mi = (int) mf;
        const float inv = __fdiv_rn(1.0f, __fmul_rn((float) mi, unit));
        const float zf = fminf(fmaxf(rintf(__fmul_rn(-lo, inv)), 0.0f), 15.0f);
        const float4 a = reinterpret_cast<float4 *>(buf)[2 * w], b = reinterpret_cast<float4 *>(buf)[2 * w + 1];
        const float v[8] = { a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w };
        uint32_t pk[2] = { 0u, 0u };
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float qf = fminf(fmaxf(__fadd_rn(rintf(__fmul_rn(v[j], inv)), zf), 0.0f), 15.0f);
            const int d = RQ_ACT_SCALE * ((int) qf - (int) zf);   // 8*(q - z) in [-120, 120]
            pk[j >> 2] |= (uint32_t) (d & 0xFF) << (8 * (j & 3));
        }
        reinterpret_cast<uint2 *>(arow)[w] = make_uint2(pk[0], pk[1]);
        if ((w & (lpg - 1)) == 0) mrow[g] = mi << RQ_MSH_SHIFT;
    }
}

template <int P>
cudaError_t configure() {
    return cudaFuncSetAttribute(rq_act_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, RQ_MAX_K * 4);
}

template <int P>
cudaError_t launch(const ActParams & prm, int64_t M, size_t smem, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = configure<P>();
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    rq_act_kernel<P><<<(unsigned) M, ACT_THREADS, smem, stream>>>(prm);
    return cudaGetLastError();
}

}  // namespace

// opt every instantiation into the large dynamic shared memory carve-out (done by rq_w4a4_prepare, outside capture)
cudaError_t rq_configure_act() {
    cudaError_t e;
    if ((e = configure<0>()) != cudaSuccess) return e;
    if ((e = configure<1>()) != cudaSuccess) return e;
    if ((e = configure<12>()) != cudaSuccess) return e;
    if ((e = configure<20>()) != cudaSuccess) return e;
    return configure<68>();
}

cudaError_t rq_launch_act(const float * x, int64_t ldx, int64_t M, int64_t K, int n_rot, int p, int m, float rot_scale,
                          float clip, int G, int8_t * a8, int32_t * msh, float * u, float * rot_out, int64_t ldo,
                          cudaStream_t stream) {
    ActParams prm;
    prm.x = x; prm.ldx = ldx; prm.K = (int) K; prm.n_rot = n_rot; prm.p = p; prm.m = m; prm.G = G;
    prm.rot_scale = rot_scale; prm.clip = clip; prm.a8 = a8; prm.msh = msh; prm.u = u; prm.rot_out = rot_out; prm.ldo = ldo;
    const size_t smem = (size_t) K * sizeof(float);
    if (n_rot <= 0 || p == 1) return launch<1>(prm, M, smem, stream);
    switch (p) {
        case 12: return launch<12>(prm, M, smem, stream);
        case 20: return launch<20>(prm, M, smem, stream);
        case 68: return launch<68>(prm, M, smem, stream);
        default: return launch<0>(prm, M, smem, stream);
    }
}
