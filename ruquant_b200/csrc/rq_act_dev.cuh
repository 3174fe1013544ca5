// Device-side building blocks of the activation path (rotation + quantizer) used by the kernels of rq_act.cu.
// Bit-parity contract: see rq_act.cu.
#pragma once

#include <utility>

#include "rq_common.cuh"

namespace rq_act_dev {

// barrier over the calling group of threads: the whole CTA (bar == 0) or a named barrier over nt threads
__device__ __forceinline__ void rq_cta_sync(int bar, int nt) {
    if (bar == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" :: "r"(bar), "r"(nt) : "memory");
}

// ---- Paley-I signs: A = I + S, S[0][a>0] = +1, S[i>0][0] = -1, S[i][a] = chi((a - i) mod q)   (rq_paley, patch:2432-2448)
// table[i * p + a] = +1.0f / -1.0f for "add" / "subtract" of input chunk i into output chunk a
__device__ __forceinline__ void build_sign_table(float * table, signed char * chi, int p, int tid, int nt, int bar = 0) {
    const int q = p - 1;
    for (int r = tid; r < q; r += nt) chi[r] = r == 0 ? 0 : -1;
    rq_cta_sync(bar, nt);
    for (int r = tid + 1; r < q; r += nt) chi[(r * r) % q] = 1;
    rq_cta_sync(bar, nt);
    for (int e = tid; e < p * p; e += nt) {
        const int i = e / p, a = e - i * p;
        bool plus;
        if (i == a || i == 0) plus = true;
        else if (a == 0) plus = false;
        else plus = chi[(((a - i) % q) + q) % q] > 0;
        table[e] = plus ? 1.0f : -1.0f;
    }
}

// ---- the same signs at compile time.  chi(r) = +1 when r is a non-zero square mod q = P - 1.
template <int P>
__host__ __device__ constexpr bool paley_plus(int i, int a) {
    if (i == a || i == 0) return true;
    if (a == 0) return false;
    const int q = P - 1;
    const int r = (((a - i) % q) + q) % q;
    for (int t = 1; t < q; ++t) if ((t * t) % q == r) return true;
    return false;
}
// All P outputs of one column, fully unrolled: acc[a] += x_i or acc[a] -= x_i with the choice made by the compiler, so
// a term is one add and nothing else (the table-driven form spends a shared-memory wavefront per 32-bit sign, which is
// what bounds it when thousands of tokens are rotated).  Ascending i per output, from 0.0f, as the reference sums.
template <int P, int I, size_t... A>
__device__ __forceinline__ void paley_static_row(float x, float (&acc)[P], std::index_sequence<A...>) {
    ((acc[A] = paley_plus<P>(I, (int) A) ? __fadd_rn(acc[A], x) : __fsub_rn(acc[A], x)), ...);
}
template <int P, size_t... I>
__device__ __forceinline__ void paley_static(const float * b, int m, float (&acc)[P], std::index_sequence<I...>) {
    (paley_static_row<P, (int) I>(b[I * m], acc, std::make_index_sequence<P>{}), ...);
}

// The Paley matrix is circulant away from its first row and column: for i, a >= 1 the sign of input chunk i in output
// chunk a depends only on a - i.  ext[d + q - 1], d = a - i in (-q, q), holds it (+1 at d = 0, the identity's share), a
// table of 2q - 1 floats that lives in constant memory: a warp walks the output blocks together, so the index is
// warp-uniform and the sign comes through the constant cache instead of costing a shared-memory wavefront per term.
template <int P>
struct PaleyExt {
    float v[2 * (P - 1) - 1];
    constexpr PaleyExt() : v() {
        const int q = P - 1;
        for (int d = -(q - 1); d <= q - 1; ++d) {
            const int r = ((d % q) + q) % q;
            bool plus = d == 0;
            for (int t = 1; t < q && !plus; ++t) plus = (t * t) % q == r;
            v[d + q - 1] = plus ? 1.0f : -1.0f;
        }
    }
};
template <int P> __constant__ PaleyExt<P> c_paley_ext = PaleyExt<P>();

// outputs a0 .. a0+3 (a0 >= 1, warp-uniform) of one column held in registers, signs from the constant table
template <int P>
__device__ __forceinline__ void paley_block4_const(const float (&col)[P], int a0, float scale, float (&out)[4]) {
    // i = 0 enters every output with +
    float acc0 = __fadd_rn(0.0f, col[0]), acc1 = acc0, acc2 = acc0, acc3 = acc0;
    const float * e = c_paley_ext<P>.v + (a0 + P - 2);          // e[k - i] = sign of input i in output a0 + k
#pragma unroll
    for (int i = 1; i < P; ++i) {
        acc0 = __fmaf_rn(col[i], e[0 - i], acc0);
        acc1 = __fmaf_rn(col[i], e[1 - i], acc1);
        acc2 = __fmaf_rn(col[i], e[2 - i], acc2);
        acc3 = __fmaf_rn(col[i], e[3 - i], acc3);
    }
    out[0] = __fmul_rn(acc0, scale);
    out[1] = __fmul_rn(acc1, scale);
    out[2] = __fmul_rn(acc2, scale);
    out[3] = __fmul_rn(acc3, scale);
}

// outputs 0 .. 3 of one column held in registers (the block with the matrix's irregular first row and column): the signs
// are compile-time, so a term is one add or subtract and no table is needed
template <int P, size_t... I>
__device__ __forceinline__ void paley_block4_first(const float (&col)[P], float scale, float (&out)[4], std::index_sequence<I...>) {
    float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
    ((acc0 = paley_plus<P>((int) I, 0) ? __fadd_rn(acc0, col[I]) : __fsub_rn(acc0, col[I]),
      acc1 = paley_plus<P>((int) I, 1) ? __fadd_rn(acc1, col[I]) : __fsub_rn(acc1, col[I]),
      acc2 = paley_plus<P>((int) I, 2) ? __fadd_rn(acc2, col[I]) : __fsub_rn(acc2, col[I]),
      acc3 = paley_plus<P>((int) I, 3) ? __fadd_rn(acc3, col[I]) : __fsub_rn(acc3, col[I])), ...);
    out[0] = __fmul_rn(acc0, scale);
    out[1] = __fmul_rn(acc1, scale);
    out[2] = __fmul_rn(acc2, scale);
    out[3] = __fmul_rn(acc3, scale);
}

// outputs a0 .. a0+3 of one column held in registers: four independent chains, terms in ascending i
template <int P>
__device__ __forceinline__ void paley_block4(const float (&col)[P], const float * __restrict__ table, int a0, float scale,
                                             float (&out)[4]) {
    float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
#pragma unroll
    for (int i = 0; i < P; ++i) {
        const float4 s = *reinterpret_cast<const float4 *>(table + i * P + a0);
        acc0 = __fmaf_rn(col[i], s.x, acc0);
        acc1 = __fmaf_rn(col[i], s.y, acc1);
        acc2 = __fmaf_rn(col[i], s.z, acc2);
        acc3 = __fmaf_rn(col[i], s.w, acc3);
    }
    out[0] = __fmul_rn(acc0, scale);
    out[1] = __fmul_rn(acc1, scale);
    out[2] = __fmul_rn(acc2, scale);
    out[3] = __fmul_rn(acc3, scale);
}

// One radix-R pass of the Sylvester transform over a buffer of whole chunks: elements base + j*s, j < R, go through
// log2(R) butterfly stages of strides s, 2s, 4s (the reference's order, h ascending; each stage is c[k] = a + b,
// c[k+h] = a - b with k the lower index, patch:2456-2463).
template <int R>
__device__ __forceinline__ void fwht_pass(float * buf, int len, int ls, int tid, int nt) {
    const int s = 1 << ls;
    for (int q = tid; q < len / R; q += nt) {
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

__device__ __forceinline__ void fwht_chunks(float * buf, int len, int m, int tid, int nt, int bar = 0) {
    for (int ls = 0; (1 << ls) < m; ls += 3) {
        const int rem = m >> ls;
        if (rem >= 8) fwht_pass<8>(buf, len, ls, tid, nt);
        else if (rem == 4) fwht_pass<4>(buf, len, ls, tid, nt);
        else fwht_pass<2>(buf, len, ls, tid, nt);
        rq_cta_sync(bar, nt);
    }
}

// Sylvester transform of 32*EPT consecutive values held by one warp, lane l owning values [l*EPT, (l+1)*EPT): the
// strides below EPT are butterflies between a lane's own registers, the strides EPT .. 16*EPT are exchanges with lane
// l ^ d (the lower lane forms a + b, the upper lane a - b with a the lower lane's value) -- the same operations in the
// same order as the reference's loop, without touching shared memory.
template <int EPT>
__device__ __forceinline__ void fwht_warp(float (&v)[EPT], int lane) {
#pragma unroll
    for (int d = 1; d < EPT; d <<= 1) {
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            if ((j & d) == 0) {
                const float a = v[j], c = v[j + d];
                v[j] = __fadd_rn(a, c);
                v[j + d] = __fsub_rn(a, c);
            }
        }
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const bool upper = (lane & d) != 0;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], d);
            v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
        }
    }
}

// global -> (transform) -> shared for `count` runs of 32*EPT floats, one warp per run
template <int EPT>
__device__ __forceinline__ void load_transform_runs(const float * __restrict__ src, float * dst, int count, bool transform,
                                                    int warp, int nwarps, int lane) {
    for (int r = warp; r < count; r += nwarps) {
        const float * s = src + (size_t) r * 32 * EPT + lane * EPT;
        float * d = dst + (size_t) r * 32 * EPT + lane * EPT;
        float v[EPT];
        if constexpr (EPT >= 4) {
#pragma unroll
            for (int j = 0; j < EPT; j += 4) {
                const float4 q = __ldg(reinterpret_cast<const float4 *>(s + j));
                v[j] = q.x; v[j + 1] = q.y; v[j + 2] = q.z; v[j + 3] = q.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < EPT; ++j) v[j] = __ldg(s + j);
        }
        if (transform) fwht_warp<EPT>(v, lane);
        if constexpr (EPT >= 4) {
#pragma unroll
            for (int j = 0; j < EPT; j += 4) *reinterpret_cast<float4 *>(d + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < EPT; ++j) d[j] = v[j];
        }
    }
}

// the same for runs that already lie in shared memory (a bulk copy brought the row): transformed in place
template <int EPT>
__device__ __forceinline__ void transform_runs_inplace(float * buf, int count, int warp, int nwarps, int lane) {
    for (int r = warp; r < count; r += nwarps) {
        float * d = buf + (size_t) r * 32 * EPT + lane * EPT;
        float v[EPT];
        if constexpr (EPT >= 4) {
#pragma unroll
            for (int j = 0; j < EPT; j += 4) {
                const float4 q = *reinterpret_cast<const float4 *>(d + j);
                v[j] = q.x; v[j + 1] = q.y; v[j + 2] = q.z; v[j + 3] = q.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < EPT; ++j) v[j] = d[j];
        }
        fwht_warp<EPT>(v, lane);
        if constexpr (EPT >= 4) {
#pragma unroll
            for (int j = 0; j < EPT; j += 4) *reinterpret_cast<float4 *>(d + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < EPT; ++j) d[j] = v[j];
        }
    }
}

// Sylvester transform, chunk by chunk, of a row that is already in shared memory.  Ends with a CTA barrier.
__device__ __forceinline__ void fwht_resident(float * buf, int len, int m, int tid, int nt, int bar = 0) {
    const int warp = tid >> 5, nwarps = nt >> 5, lane = tid & 31;
    const int run = m < 1024 ? m : 1024;
    switch (run) {
        case 32:   if (m > 1) transform_runs_inplace<1>(buf, len / 32, warp, nwarps, lane); break;
        case 64:   transform_runs_inplace<2>(buf, len / 64, warp, nwarps, lane); break;
        case 128:  transform_runs_inplace<4>(buf, len / 128, warp, nwarps, lane); break;
        case 256:  transform_runs_inplace<8>(buf, len / 256, warp, nwarps, lane); break;
        case 512:  transform_runs_inplace<16>(buf, len / 512, warp, nwarps, lane); break;
        case 1024: transform_runs_inplace<32>(buf, len / 1024, warp, nwarps, lane); break;
        default:   fwht_chunks(buf, len, m, tid, nt, bar); return;      // m < 32: the generic passes
    }
    rq_cta_sync(bar, nt);
    for (int ls = 10; (1 << ls) < m; ls += 3) {
        const int rem = m >> ls;
        if (rem >= 8) fwht_pass<8>(buf, len, ls, tid, nt);
        else if (rem == 4) fwht_pass<4>(buf, len, ls, tid, nt);
        else fwht_pass<2>(buf, len, ls, tid, nt);
        rq_cta_sync(bar, nt);
    }
}

// One bulk asynchronous copy of a row (bytes a multiple of 16, both ends 16-byte aligned) into shared memory, issued by
// one thread, awaited by all: a single trip to memory for the whole row, where per-run loads expose one trip per round of
// runs a warp takes.  The wait is bounded (about a second); false when it ran out.
__device__ __forceinline__ bool bulk_load_row(float * dst, const float * src, uint32_t bytes, uint64_t * bar, int tid) {
    const uint32_t b = (uint32_t) __cvta_generic_to_shared(bar);
    if (tid == 0) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(b), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"((uint32_t) __cvta_generic_to_shared(dst)), "l"(src), "r"(bytes), "r"(b) : "memory");
    }
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(b) : "memory");
        if (ok) return true;
        if ((i & 63u) == 63u && clock64() - t0 > 2000000000ll) return false;
    }
}

// A buffer of `len` floats made of whole chunks of m: loaded from global memory and Sylvester-transformed chunk by
// chunk.  Chunks up to 1024 wide are done entirely in registers and shuffles; wider chunks finish their upper
// strides (1024 and above, conflict-free) in shared memory.  Ends with a CTA barrier.
__device__ __forceinline__ void load_fwht(const float * __restrict__ src, float * dst, int len, int m, int tid, int nt, int bar = 0) {
    const int warp = tid >> 5, nwarps = nt >> 5, lane = tid & 31;
    const int run = m < 1024 ? m : 1024;
    switch (run) {
        case 32:   load_transform_runs<1>(src, dst, len / 32, m > 1, warp, nwarps, lane); break;
        case 64:   load_transform_runs<2>(src, dst, len / 64, true, warp, nwarps, lane); break;
        case 128:  load_transform_runs<4>(src, dst, len / 128, true, warp, nwarps, lane); break;
        case 256:  load_transform_runs<8>(src, dst, len / 256, true, warp, nwarps, lane); break;
        case 512:  load_transform_runs<16>(src, dst, len / 512, true, warp, nwarps, lane); break;
        case 1024: load_transform_runs<32>(src, dst, len / 1024, true, warp, nwarps, lane); break;
        default: {   // m < 32 (1 .. 16): plain copy, then the generic passes
            for (int i = tid; i < len; i += nt) dst[i] = __ldg(src + i);
            rq_cta_sync(bar, nt);
            fwht_chunks(dst, len, m, tid, nt, bar);
            return;
        }
    }
    rq_cta_sync(bar, nt);
    for (int ls = 10; (1 << ls) < m; ls += 3) {
        const int rem = m >> ls;
        if (rem >= 8) fwht_pass<8>(dst, len, ls, tid, nt);
        else if (rem == 4) fwht_pass<4>(dst, len, ls, tid, nt);
        else fwht_pass<2>(dst, len, ls, tid, nt);
        rq_cta_sync(bar, nt);
    }
}

// ---- quantizer pieces shared by both kernels

// range of a word of 8 values reduced over the lpg lanes that share its group
__device__ __forceinline__ void group_range(const float4 a, const float4 b, int lpg, float clip, float & lo, float & hi) {
    float mn = fminf(fminf(fminf(a.x, a.y), fminf(a.z, a.w)), fminf(fminf(b.x, b.y), fminf(b.z, b.w)));
    float mx = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
    mn = fminf(mn, 0.0f);
    mx = fmaxf(mx, 0.0f);
    for (int o = 1; o < lpg; o <<= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    lo = __fmul_rn(mn, clip);
    hi = __fmul_rn(mx, clip);
}

// the 8 codes of a word and the group's multiplier.  F8 false: int8 8*(q - z) (RQ_FMT_I8); true: the e4m3 byte of
// (q - z), exact (RQ_FMT_E4M3, the fp8 tensor-core path).  Everything stays in float registers: conversions between
// float and int run at a quarter of the FMA rate on this part and integer logic at half of it, and this loop runs once
// per input value.
//   rint(t)        (t + 1.5*2^23) - 1.5*2^23: round-to-nearest-even of the add, exact for |t| < 2^22; beyond that the
//                  result may be off by one, at magnitudes the clamp to [0, 15] that follows maps to the same end
//   byte, int8     the low mantissa byte of 8*(q - z) + 1.5*2^23 is the value's two's-complement byte
//   byte, e4m3     cvt.rn.satfinite.e4m3x2.f32 on two values at once (|q - z| <= 15 has four significant bits: exact)
template <bool F8>
__device__ __forceinline__ uint2 encode_word(const float4 a, const float4 b, float lo, float hi, float R, float unit, float & mf_out) {
    const float mf = fminf(fmaxf(ceilf(__fdiv_rn(__fmul_rn(__fsub_rn(hi, lo), 255.0f), R)), 1.0f), 255.0f);
    mf_out = mf;
    const float inv = __fdiv_rn(1.0f, __fmul_rn(mf, unit));
    constexpr float MAGIC = 12582912.0f;
    const float zf = fminf(fmaxf(__fsub_rn(__fadd_rn(__fmul_rn(-lo, inv), MAGIC), MAGIC), 0.0f), 15.0f);
    const float v[8] = { a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w };
    float dz[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float r = __fsub_rn(__fadd_rn(__fmul_rn(v[j], inv), MAGIC), MAGIC);
        const float qf = fminf(fmaxf(__fadd_rn(r, zf), 0.0f), 15.0f);
        dz[j] = __fsub_rn(qf, zf);                                           // q - z in [-15, 15]
    }
    uint32_t pk[2];
    if constexpr (F8) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint16_t p01, p23;      // the second source operand lands in the low byte
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(p01) : "f"(dz[4 * h + 1]), "f"(dz[4 * h]));
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(p23) : "f"(dz[4 * h + 3]), "f"(dz[4 * h + 2]));
            pk[h] = (uint32_t) p01 | ((uint32_t) p23 << 16);
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = __float_as_uint(__fmaf_rn(dz[4 * h + j], (float) RQ_ACT_SCALE, MAGIC));
            uint32_t lo01, lo23;
            asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo01) : "r"(w[0]), "r"(w[1]));      // {w0.b0, w1.b0, ., .}
            asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo23) : "r"(w[2]), "r"(w[3]));
            asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(pk[h]) : "r"(lo01), "r"(lo23));     // {lo01.b0, lo01.b1, lo23.b0, lo23.b1}
        }
    }
    return make_uint2(pk[0], pk[1]);
}
// what the multiplier word holds: m_g as an integer, or for the fp8 path the f32 bits of m_g / 16 (exact)
template <bool F8>
__device__ __forceinline__ int multiplier_word(float mf) {
    return F8 ? __float_as_int(__fmul_rn(mf, 0.0625f)) : (int) mf;
}

// maximum over the CTA of a per-thread value >= 0: warp shuffles, one shared-memory round, result in every thread of
// warp 0 (other warps get an unspecified value).  red: one float per warp.  Contains one CTA barrier.
__device__ __forceinline__ float cta_max_warp0(float v, float * red, int tid, int nt) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
        v = tid < (nt >> 5) ? red[tid] : 0.0f;
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    }
    return v;
}

}  // namespace rq_act_dev
