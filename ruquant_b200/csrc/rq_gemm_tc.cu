// Prefill-width contraction on the sm_100a tensor cores: tcgen05.mma kind::i8 with the accumulator in tensor memory,
// operands staged by TMA, and the reference's per-group integer fold done by the epilogue warps straight out of
// tensor memory while the tensor pipe works on the next group.
//
// Why the accumulator leaves tensor memory every G inputs: the reference shifts each group's term right by 4 before
// the int32 sum (ggml_vec_dot_w4a4_a4, ggml/src/ggml-cpu/quants.c in patches/llama.cpp-ruquant.patch:173), which is
// not linear, so groups cannot be accumulated together.  Operand scaling makes that fold one instruction:
//   A = activations, int8 8*(q - z_g), [M][K] K-major      (tokens are the MMA's M = 128 rows = TMEM lanes)
//   B = weights,     int8 16*c,        [N][K] K-major      (weight rows are the MMA's N = 256 = TMEM columns)
//   D = 128 * S_g after G/32 instructions of K = 32;   total += (m_g * D) >> 11   ( = (m_g*S_g) >> 4, exact)
// An epilogue thread owns one token (one TMEM lane), so m_g is a single register per group.  Weights with
// multipliers k != 1 are stored as k*c instead and folded as (D * m_g) >> 7.
//
// CTA = 128 tokens x 256 weight rows.  Warp 0 lane 0: TMA producer over a 4-stage ring of 128-input K slices
// (16 KB of A + 32 KB of B, 128B swizzle).  Warp 1: TMEM allocation, lane 0 issues the MMAs into two 256-column
// accumulator buffers.  Warps 4-11: fold + final fp32 epilogue y = ((float(total) * 16) * u) * s_w.
// Every wait is bounded: on expiry the waiter raises a CTA-wide abort flag and a status word in global memory,
// everyone leaves the pipeline, outstanding TMA transactions are drained and tensor memory is released.
#include <cuda.h>

#include "rq_common.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4;
constexpr int TC_THREADS = 384;
constexpr uint32_t A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + slack to align the ring to 1024 bytes
constexpr long long WAIT_CYCLES = 2000000000ll;                // about a second at B200 clocks
constexpr uint32_t TMEM_COLS = 512;

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the barrier did not flip within WAIT_CYCLES or another role already gave up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int * abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_CYCLES) { *abort_flag = 1; return false; }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap * map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// K-major operand tile in the canonical 128B-swizzled layout TMA writes: rows of 128 bytes, 8-row atoms 1024 bytes
// apart.  Fields: start address >> 4 [0,14), leading byte offset >> 4 [16,30) (unused for swizzled K-major, 1),
// stride byte offset >> 4 [32,46), descriptor version 1 [46,48), layout type SWIZZLE_128B = 2 [61,64).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t) (1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::i8: D = s32 (2 at [4,6)), A and B signed int8 (1 at [7,10) and [10,13)), both
// K-major (0 at 15, 16), N >> 3 at [17,23), M >> 4 at [24,29)
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (BN >> 3) << 17) | ((uint32_t) (BM >> 4) << 24);
// kind::f8f6f4: D = f32 (1 at [4,6)), A and B e4m3 (0 at [7,10) and [10,13)), K-major, same N and M fields
constexpr uint32_t IDESC_F8 = (1u << 4) | ((uint32_t) (BN >> 3) << 17) | ((uint32_t) (BM >> 4) << 24);

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(da), "l"(db), "r"(IDESC_F8), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
}
// completes this thread's outstanding tensor-memory loads; the values are threaded through as read-write operands
// so that no use of them can be scheduled above the wait
__device__ __forceinline__ void tmem_ld_wait(int (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                   "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
                   "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :: "memory");
}

// one integer multiply and one shift-add per output per group (measured on B200: 50+ outputs per clock per SM,
// against 30 for a high multiply-add)
// integer path (weights k*c, activations 8*(q - z)): D = 8*k*S, term = (D * m) >> 7
__device__ __forceinline__ void fold32(int (&tot)[128], int base, const int (&v)[32], int mm) {
#pragma unroll
    for (int i = 0; i < 32; ++i) tot[base + i] += (v[i] * mm) >> 7;
}

// fp8 path: D = S exactly (fp32 accumulation of products of small integers).  The running total lives in a float
// kept inside [2^23, 2^24), where the spacing of floats is 1: a round-down fused multiply-add
//     t <- fma.rm(S, m/16, t)
// adds floor(S*m/16) = (m*S) >> 4 exactly (S*m/16 has at most 21 + 4 significant bits below 2^23, the sum is rounded
// once, downwards, to an integer) -- the reference's shifted term in ONE instruction at the full fp32 rate.
constexpr float FOLD_MAGIC = 12582912.0f;        // 1.5 * 2^23
constexpr int FOLD_MAGIC_BITS = 0x4B400000;
__device__ __forceinline__ float fma_rm(float a, float b, float c) {
    float d;
    asm("fma.rm.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void fold32_f8(float (&tf)[128], int base, const int (&v)[32], float mf) {
#pragma unroll
    for (int i = 0; i < 32; ++i) tf[base + i] = fma_rm(__int_as_float(v[i]), mf, tf[base + i]);
}
// Every 1024 inputs the float is re-centred: what it holds above +-2^19 moves, in units of 2^20, into a signed byte
// of a packed carry word (at most 32 re-centrings of at most +-3 each), so the float never leaves its window.
__device__ __forceinline__ void recenter(float (&tf)[128], int (&carry)[32]) {
#pragma unroll
    for (int i = 0; i < 128; ++i) {
        const int k = __float_as_int(tf[i]) - FOLD_MAGIC_BITS;
        const int c = (k + (1 << 19)) >> 20;
        tf[i] = __int_as_float(FOLD_MAGIC_BITS + (k - (c << 20)));
        carry[i >> 2] += c << (8 * (i & 3));
    }
}

struct TcParams {
    const float * sw;
    const int32_t * msh;
    const float * u;
    float * y;
    int64_t ldy;
    int32_t * status;
    int K, N, M, G;
};

struct __align__(8) TcShared {
    uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// F8 = true: multipliers all 1, operands are e4m3 bytes of c and (q - z), fp8 MMA with fp32 accumulators, float fold.
// F8 = false: weight multipliers present, B holds int8 k*c, A int8 8*(q - z), integer MMA and integer fold.
template <bool F8>
__global__ void __launch_bounds__(TC_THREADS, 1)
rq_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const TcParams prm) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcShared sh;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tile = blockIdx.x, n_tile = blockIdx.y;
    const int n_ks = prm.K / BK;          // ring slices of 128 inputs
    const int gsteps = prm.G / 64;        // 64-input steps per activation group: 1, 2 or 4
    const int n_ag = prm.K / prm.G;       // activation groups
    volatile int * abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&sh.full[s]), 1); mbar_init(smem_u32(&sh.empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&sh.tmem_full[b]), 1); mbar_init(smem_u32(&sh.tmem_empty[b]), 8); }
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&sh.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_base;

    // warps 0-3 (TMA, MMA, two idle) give registers back; the two epilogue warpgroups take them
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int ks = 0; ks < n_ks; ++ks) {
                const int s = ks % STAGES;
                if (!mbar_wait(smem_u32(&sh.empty[s]), ((ks / STAGES) & 1) ^ 1, abort_flag)) break;
                const uint32_t bar = smem_u32(&sh.full[s]);
                mbar_expect_tx(bar, STAGE_BYTES);
                tma_load_2d(ring + s * STAGE_BYTES, &tmap_a, bar, ks * BK, m_tile * BM);
                tma_load_2d(ring + s * STAGE_BYTES + A_BYTES, &tmap_b, bar, ks * BK, n_tile * BN);
                issued = ks + 1;
            }
            if (*abort_flag) {
                // drain: every slice that was issued must land before the CTA's shared memory is given back
                for (int ks = issued > STAGES ? issued - STAGES : 0; ks < issued; ++ks) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&sh.full[ks % STAGES]), (ks / STAGES) & 1) && clock64() - t0 < WAIT_CYCLES) { }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int ks = 0; ks < n_ks && ok; ++ks) {
                const int s = ks % STAGES;
                if (!mbar_wait(smem_u32(&sh.full[s]), (ks / STAGES) & 1, abort_flag)) break;
                tc_fence_after();
                const uint64_t da = umma_desc(ring + s * STAGE_BYTES), db = umma_desc(ring + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int step = 2 * ks + h;              // 64-input step
                    const int ag = step / gsteps, gs = step - ag * gsteps;
                    const int buf = ag & 1;
                    if (gs == 0) {
                        if (!mbar_wait(smem_u32(&sh.tmem_empty[buf]), ((ag >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                    }
                    const uint32_t d = tmem_base + (uint32_t) buf * BN;
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        const uint32_t koff = (uint32_t) ((h * 64 + kk * 32) >> 4);   // bytes >> 4 inside the swizzled row
                        if (F8) umma_f8(d, da + koff, db + koff, (gs | kk) != 0 ? 1u : 0u);
                        else    umma_i8(d, da + koff, db + koff, (gs | kk) != 0 ? 1u : 0u);
                    }
                    if (gs == gsteps - 1) umma_commit(smem_u32(&sh.tmem_full[buf]));
                }
                umma_commit(smem_u32(&sh.empty[s]));
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
        const int e = warp - 4, quarter = warp & 3, half = e >> 2;
        const int row = m_tile * BM + quarter * 32 + lane;
        const bool row_ok = row < prm.M;
        const uint32_t lane_base = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (half * 128);
        const int32_t * mrow = prm.msh + (size_t) (row_ok ? row : 0) * n_ag;
        // the quantizer records the format it wrote: refuse to multiply the wrong one
        const bool fmt_ok = prm.status == nullptr || prm.status[1] == (F8 ? RQ_FMT_E4M3 : RQ_FMT_I8);
        int tot[F8 ? 1 : 128];
        float tf[F8 ? 128 : 1];
        int carry[F8 ? 32 : 1];
        if (F8) {
#pragma unroll
            for (int i = 0; i < 128; ++i) tf[F8 ? i : 0] = FOLD_MAGIC;
#pragma unroll
            for (int i = 0; i < 32; ++i) carry[F8 ? i : 0] = 0;
        } else {
#pragma unroll
            for (int i = 0; i < 128; ++i) tot[F8 ? 0 : i] = 0;
        }
        const int recenter_every = prm.G >= 1024 ? 1 : 1024 / prm.G;
        int since = 0;
        int mnext = row_ok ? __ldg(mrow) : 0;
        bool ok = true;
        for (int ag = 0; ag < n_ag; ++ag) {
            const int buf = ag & 1;
            const int mm = mnext;
            if (ag + 1 < n_ag) mnext = row_ok ? __ldg(mrow + ag + 1) : 0;
            // the loads below are warp-collective: leave the loop together or not at all
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh.tmem_full[buf]), (ag >> 1) & 1, abort_flag))) { ok = false; break; }
            tc_fence_after();
            const uint32_t t0 = lane_base + (uint32_t) buf * BN;
            if constexpr (F8) {
                const float mf = __int_as_float(mm);          // m / 16
                int va[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    tmem_ld32(t0 + c * 32, va);
                    tmem_ld_wait(va);
                    if (c == 0) fold32_f8(tf, 0, va, mf);
                    else if (c == 1) fold32_f8(tf, 32, va, mf);
                    else if (c == 2) fold32_f8(tf, 64, va, mf);
                    else fold32_f8(tf, 96, va, mf);
                }
            } else {
                // software pipeline over the four 32-column chunks: the load of chunk c+1 is in flight while chunk c folds
                int va[32], vb[32];
                tmem_ld32(t0, va);
                tmem_ld_wait(va);
                tmem_ld32(t0 + 32, vb);
                fold32(tot, 0, va, mm);
                tmem_ld_wait(vb);
                tmem_ld32(t0 + 64, va);
                fold32(tot, 32, vb, mm);
                tmem_ld_wait(va);
                tmem_ld32(t0 + 96, vb);
                fold32(tot, 64, va, mm);
                tmem_ld_wait(vb);
                fold32(tot, 96, vb, mm);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[buf]));
            if constexpr (F8) {
                if (++since == recenter_every || ag == n_ag - 1) { recenter(tf, carry); since = 0; }
            }
        }
        if (!fmt_ok) {
            ok = false;
            if (lane == 0 && prm.status != nullptr) atomicExch(prm.status, 2);
        }
        if (ok && row_ok) {
            const float ut = __ldg(prm.u + row);
            float * yr = prm.y + (size_t) row * prm.ldy;
            const int n0 = n_tile * BN + half * 128;
            const bool vec = ((prm.ldy & 3) == 0) && ((reinterpret_cast<uintptr_t>(prm.y) & 15) == 0);
#pragma unroll
            for (int i = 0; i < 128; i += 4) {
                float f[4];
                int P = F8 ? carry[F8 ? i >> 2 : 0] : 0;      // four signed byte digits, units of 2^20
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = n0 + i + j;
                    const float s = n < prm.N ? __ldg(prm.sw + n) : 0.0f;
                    int total;
                    if (F8) {
                        const int d = (int) (signed char) (P & 0xFF);
                        total = d * (1 << 20) + (__float_as_int(tf[F8 ? i + j : 0]) - FOLD_MAGIC_BITS);
                        P = (P - d) >> 8;
                    } else {
                        total = tot[F8 ? 0 : i + j];
                    }
                    f[j] = __fmul_rn(__fmul_rn(__fmul_rn((float) total, 16.0f), ut), s);
                }
                if (vec && n0 + i + 3 < prm.N) {
                    *reinterpret_cast<float4 *>(yr + n0 + i) = make_float4(f[0], f[1], f[2], f[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) if (n0 + i + j < prm.N) yr[n0 + i + j] = f[j];
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_flag && prm.status != nullptr) atomicExch(prm.status, 1);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*encode_fn_t)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_fn_t get_encode() {
    static encode_fn_t fn = nullptr;
    if (fn == nullptr) {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<encode_fn_t>(p);
        }
    }
    return fn;
}

}  // namespace

int rq_encode_tmap_i8(void * tmap_out, const void * base, int64_t K, int64_t rows, int box_rows) {
    encode_fn_t fn = get_encode();
    if (fn == nullptr) return -1;
    alignas(64) CUtensorMap map;
    const cuuint64_t dims[2] = { (cuuint64_t) K, (cuuint64_t) rows };
    const cuuint64_t strides[1] = { (cuuint64_t) K };       // bytes between rows
    const cuuint32_t box[2] = { (cuuint32_t) BK, (cuuint32_t) box_rows };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
    memcpy(tmap_out, &map, sizeof(map));
    return 0;
}

cudaError_t rq_configure_gemm_tc() {
    // <true>: fp8 operands (no weight multipliers); <false>: int8 operands
    cudaError_t e = cudaFuncSetAttribute(rq_gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(rq_gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
}

cudaError_t rq_launch_gemm_tc(const void * tmap_w8, const float * sw, int fmt, int64_t K, int64_t N,
                              const int8_t * a8, const int32_t * msh, const float * u, int64_t M, int G,
                              float * y, int64_t ldy, int32_t * status, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = rq_configure_gemm_tc();
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    alignas(64) CUtensorMap ta, tb;
    if (rq_encode_tmap_i8(&ta, a8, K, M, BM) != 0) return cudaErrorInvalidValue;
    memcpy(&tb, tmap_w8, sizeof(tb));
    TcParams prm;
    prm.sw = sw; prm.msh = msh; prm.u = u; prm.y = y; prm.ldy = ldy; prm.status = status;
    prm.K = (int) K; prm.N = (int) N; prm.M = (int) M; prm.G = G;
    const dim3 grid((unsigned) ((M + BM - 1) / BM), (unsigned) ((N + BN - 1) / BN));
    if (fmt == RQ_FMT_E4M3) rq_gemm_tc_kernel<true><<<grid, TC_THREADS, SMEM_BYTES, stream>>>(ta, tb, prm);
    else                    rq_gemm_tc_kernel<false><<<grid, TC_THREADS, SMEM_BYTES, stream>>>(ta, tb, prm);
    return cudaGetLastError();
}
