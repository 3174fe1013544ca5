// Decode-width contraction (M <= 16 tokens per pass): an HBM-bound GEMV over the int4 decode stream.
//
// The stream is stored in the order the warp consumes it (rq_prepack.cu): for every tile of 16 weight rows and every
// run of 64 inputs, 512 contiguous bytes = one 128-bit load per lane, whose four words unpack (two logic ops each)
// into the eight int8 A-fragment registers of two m16n8k32 integer MMAs.  The MMAs do the multiply-accumulate for
// up to 8 tokens at once, so the instruction count per byte of weights does not grow with M and the kernel stays
// bandwidth-bound from M = 1 to 16.  Every activation group of every (row, token) pair is folded on its own, as
// the reference's dot product does (ggml_vec_dot_w4a4_a4, ggml/src/ggml-cpu/quants.c in
// patches/llama.cpp-ruquant.patch:148-177):
//     total += (k * m_g * S_g) >> 4,   S_g = sum c * (q - z_g)       (int32, arithmetic shift)
//     y = ((float(total) * 16) * u) * s_w                             (three separate fp32 multiplies)
// Weights arrive as int8 16*c, activations as int8 8*(q - z), so the MMA delivers 128*S_g and the fold is
// (m_g * 128*S_g) >> 11, exact.  The stream reaches shared memory through bulk asynchronous copies issued by a
// producer warp (deep, register-free prefetch: HBM on this part needs > 100 KB in flight per SM); the consumer warps
// of a CTA split K (integer sums are exact in any order) and combine through shared memory.  The kernel is launched
// with programmatic stream serialization: it lets its successor start at once and fills its ring before waiting for
// the quantizer that precedes it.
#include <stdlib.h>

#include <mutex>

#include "rq_common.cuh"

namespace {


__device__ __forceinline__ void mma_s8(int (&d)[4], const int (&a)[4], int b0, int b1, const int (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

struct GemvJob {            // one weight of the launch
    const uint4 * w4t;      // [tiles][K/64][32 lanes] x 16 B
    const float * sw;
    const int8_t * wk;      // [N][K/64] or null
    float * y;
    float * y_more[RQ_MAX_RANKS - 1];   // further copies of the output (other ranks' buffers, peer-mapped), same layout
    int64_t ldy;
    int N;
    int n_more;
};

// Up to three weights that share the activation (q/k/v, gate/up) are one launch: their row tiles form one list
// (the reference's multi-weight launch: rq_jobs, ggml/src/ggml-cuda/rq-w4a4-skinny.cuh in patch:1168-1179).
struct GemvParams {
    GemvJob job[RQ_MAX_WEIGHTS];
    int tile_start[RQ_MAX_WEIGHTS + 1];
    int n_jobs;
    const int8_t * a8;      // [M][K]  8*(q - z)
    const int32_t * msh;    // [M][K/G]  m_g
    const float * u;
    int32_t * status;       // set to 1 when a bounded wait expires
    int K, M, G;
};

__device__ __forceinline__ int job_of_tile(const GemvParams & prm, int tile) {
    int w = 0;
#pragma unroll
    for (int i = 1; i < RQ_MAX_WEIGHTS; ++i) if (i < prm.n_jobs && tile >= prm.tile_start[i]) w = i;
    return w;
}

constexpr int CH_STEPS = 4;                 // 64-input steps per chunk of the stream
constexpr int CH_BYTES = CH_STEPS * 512;    // 2 KB: the unit one consumer warp works on
constexpr int SUBS = 4;                     // chunks per bulk copy
constexpr int ST_BYTES = SUBS * CH_BYTES;   // 8 KB per bulk copy: few enough copies for a single issuing thread
constexpr int STAGES = 8;                   // 64 KB ring per CTA
constexpr int CONSUMERS = 8;                // consumer warps; warp CONSUMERS is the producer
constexpr long long WAIT_CYCLES = 2000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the barrier did not flip in about a second or another warp already gave up
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

// Persistent CTAs, three per SM, each walking tiles of 16 weight rows (tile = blockIdx.x, += gridDim.x).  The producer
// warp streams the tiles' K/64 * 512 bytes back to back into a shared-memory ring with bulk copies (it starts at once:
// the weights do not depend on the preceding kernel, and it never drains between tiles); the consumer warps take the
// chunks of that stream round-robin, so 64 KB per CTA stay in flight or resident from the first cycle to the last.
// NT: token tiles of 8 (1 or 2).  GS: 64-input steps per activation group (1, 2, 4).  HAS_K: weight multipliers.
// ONE: M == 1 (only token 0 is folded and stored).  PUSH: outputs also go to the jobs' further destinations.
template <int NT, int GS, bool HAS_K, bool ONE, bool PUSH>
__global__ void __launch_bounds__((CONSUMERS + 1) * 32) rq_gemv_mma_kernel(const GemvParams prm) {
    extern __shared__ __align__(128) uint8_t dyn[];
    __shared__ uint64_t full[STAGES], empty[STAGES];
    __shared__ int abort_word;
    __shared__ int fmt_word;     // the activation format the quantizer recorded (-1 until a spare producer lane has read it)
    uint8_t * ring = dyn;
    int * part = reinterpret_cast<int *>(dyn + STAGES * ST_BYTES);      // [2][CONSUMERS][32][4 * NT]
    volatile int * abort_flag = &abort_word;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const int K = prm.K, M = prm.M;
    const int ng64 = K >> 6, n_ag = ng64 / GS, nchunks = ng64 / CH_STEPS, nst = (nchunks + SUBS - 1) / SUBS;
    const int tiles = prm.tile_start[prm.n_jobs];

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(&empty[s])), "r"(SUBS) : "memory");
        }
        abort_word = 0;
        fmt_word = -1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) rq_trace(prm.status, 0x10);

    if (warp == CONSUMERS) {
        // ---- producer: bulk copies of up to 8 KB, gated only by ring space
        if (lane == 0) {
            int issued = 0;       // stages of this CTA's stream, all tiles
            bool ok = true;
            // This kernel multiplies int8 activations; one quantized for the fp8 tensor-core path is refused (status 2, no
            // stores).  The word is read here, off the consumers' path: they look at it only when a tile is complete.
            auto read_format = [&]() {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                *reinterpret_cast<volatile int *>(&fmt_word) = prm.status != nullptr ? prm.status[1] : RQ_FMT_I8;
            };
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int wi = job_of_tile(prm, tile);
                const uint8_t * src = reinterpret_cast<const uint8_t *>(prm.job[wi].w4t) + (size_t) (tile - prm.tile_start[wi]) * ng64 * 512;
                for (int st = 0; st < nst; ++st) {
                    const int s = issued % STAGES;
                    const int left = nchunks - st * SUBS;
                    const uint32_t bytes = (uint32_t) (left < SUBS ? left : SUBS) * CH_BYTES;
                    if (!mbar_wait(smem_u32(&empty[s]), ((issued / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full[s]);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 :: "r"(smem_u32(ring + (size_t) s * ST_BYTES)), "l"(src + (size_t) st * ST_BYTES), "r"(bytes), "r"(bar) : "memory");
                    ++issued;
                    // (asking L2 for the stream behind the ring at this point -- per line or with bulk prefetches -- made the pass
                    // slower: 3.86 against 3.72 ms with 128 KB per CTA)
                    if (issued == STAGES) read_format();      // the ring is full: nothing to issue until the consumers run
                }
            }
            if (issued < STAGES) read_format();
            if (*abort_flag) {   // let every copy that was issued land before the CTA's shared memory goes away
                for (int c = issued > STAGES ? issued - STAGES : 0; c < issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&full[c % STAGES]), (c / STAGES) & 1) && clock64() - t0 < WAIT_CYCLES) { }
                }
                if (prm.status != nullptr) atomicExch(prm.status, 1);
            }
        }
        return;
    }

    // ---- consumers.  Everything below reads what the preceding kernel (the quantizer) wrote.  With the ring full, the
    // trip to L2 for the quantized token is the one latency left on the path: a pass over the 64-layer stack takes 3.40 ms
    // with these loads replaced by constants against 3.68 ms.  Neither asking L1 for the whole token at once (3.81 ms) nor
    // staging it in shared memory with one round of asynchronous copies (3.72 against 3.67 ms) shortens it: the CTAs of an
    // SM already share the lines through L1, what remains is the first trip itself.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) rq_trace(prm.status, 0x11);

    // B fragments: token gid (+8 for the second tile); the quantizer stores each run of 64 inputs so that the 16
    // bytes at offset tig*16 are inputs {0,16,32,48} + tig*4 .. +3: b0, b1 of both MMAs in one 128-bit load.
    // Token slots beyond M read token 0's data: their columns of the product are never stored.
    const uint4 * ap[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t)
        ap[t] = reinterpret_cast<const uint4 *>(prm.a8 + (size_t) (gid + 8 * t < M ? gid + 8 * t : 0) * K) + tig;
    const int32_t * mp[NT][2];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int tok = 8 * t + 2 * tig + c;
            mp[t][c] = prm.msh + (size_t) (tok < M ? tok : 0) * n_ag;
        }

    int it = 0;                                    // tiles done by this CTA
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
        const int wi = job_of_tile(prm, tile);
        const GemvJob & jb = prm.job[wi];
        const int row_lo = (tile - prm.tile_start[wi]) * 16 + gid, row_hi = row_lo + 8;
        const int8_t * kp_lo = nullptr, * kp_hi = nullptr;
        if (HAS_K) {
            kp_lo = jb.wk + (size_t) (row_lo < jb.N ? row_lo : 0) * ng64;
            kp_hi = jb.wk + (size_t) (row_hi < jb.N ? row_hi : 0) * ng64;
        }
        int tot[NT][4];
        int acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) { tot[t][i] = 0; acc[t][i] = 0; }

        // stage gs of the CTA's stream (all tiles) is shared by four consumer warps, one chunk each: warps 0-3 take
        // the even stages, warps 4-7 the odd ones
        const int gs0 = it * nst, sc = warp & 3;
        bool ok = true;
        for (int st = ((warp >> 2) - gs0) & 1; st < nst; st += 2) {
            const int gs = gs0 + st, s = gs % STAGES;
            const int c = st * SUBS + sc;                 // this warp's chunk of the tile (may lie beyond its end)
            // the activations do not depend on the weights: fetch them while the stage is still in flight
            uint4 bq[CH_STEPS][NT];
            if (c < nchunks) {
#pragma unroll
                for (int q = 0; q < CH_STEPS; ++q)
#pragma unroll
                    for (int t = 0; t < NT; ++t) bq[q][t] = __ldg(ap[t] + (c * CH_STEPS + q) * 4);
            }
            // the MMAs below are warp-collective: leave the loop together or not at all
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&full[s]), (gs / STAGES) & 1, abort_flag))) { ok = false; break; }
            if (c < nchunks) {
            const uint4 * sp_ = reinterpret_cast<const uint4 *>(ring + (size_t) s * ST_BYTES + (size_t) sc * CH_BYTES) + lane;
            // The integer MMA of this part has a long latency: issue the MMAs of SP steps (two per step, on
            // independent zero-initialised accumulators) before touching any result.
            constexpr int SP = NT == 1 ? 4 : 2;
#pragma unroll
            for (int h = 0; h < CH_STEPS; h += SP) {
                int pa[SP][2][NT][4];
#pragma unroll
                for (int sp = 0; sp < SP; ++sp) {
                    const uint4 wv = sp_[(h + sp) * 32];
                    uint4 b[NT];
#pragma unroll
                    for (int t = 0; t < NT; ++t) b[t] = bq[h + sp][t];
                    // words 0,1 -> first 32 inputs (a0..a3), words 2,3 -> second 32 inputs
                    int a0[4], a1[4];
                    a0[0] = (int) ((wv.x << 4) & 0xF0F0F0F0u); a0[1] = (int) (wv.x & 0xF0F0F0F0u);
                    a0[2] = (int) ((wv.y << 4) & 0xF0F0F0F0u); a0[3] = (int) (wv.y & 0xF0F0F0F0u);
                    a1[0] = (int) ((wv.z << 4) & 0xF0F0F0F0u); a1[1] = (int) (wv.z & 0xF0F0F0F0u);
                    a1[2] = (int) ((wv.w << 4) & 0xF0F0F0F0u); a1[3] = (int) (wv.w & 0xF0F0F0F0u);
                    const int zero[4] = { 0, 0, 0, 0 };
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        mma_s8(pa[sp][0][t], a0, (int) b[t].x, (int) b[t].y, zero);
                        mma_s8(pa[sp][1][t], a1, (int) b[t].z, (int) b[t].w, zero);
                    }
                }
#pragma unroll
                for (int sp = 0; sp < SP; ++sp) {
                    const int st = h + sp, j = c * CH_STEPS + st;
#pragma unroll
                    for (int t = 0; t < NT; ++t)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (ONE && (i & 1)) continue;                 // token 1 of the pair does not exist
                            if (GS == 1) acc[t][i] = pa[sp][0][t][i] + pa[sp][1][t][i];
                            else         acc[t][i] += pa[sp][0][t][i] + pa[sp][1][t][i];
                        }
                    if ((st % GS) == GS - 1) {
                        const int ag = j / GS;
                        int klo = 1, khi = 1;
                        if (HAS_K) { klo = kp_lo[j]; khi = kp_hi[j]; }
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            const int m0 = __ldg(mp[t][0] + ag);
                            const int m1 = ONE ? 0 : __ldg(mp[t][1] + ag);
                            if (HAS_K) {
                                tot[t][0] += (klo * m0 * (acc[t][0] >> 7)) >> 4;
                                tot[t][2] += (khi * m0 * (acc[t][2] >> 7)) >> 4;
                                if (!ONE) {
                                    tot[t][1] += (klo * m1 * (acc[t][1] >> 7)) >> 4;
                                    tot[t][3] += (khi * m1 * (acc[t][3] >> 7)) >> 4;
                                }
                            } else {
                                tot[t][0] += (m0 * acc[t][0]) >> RQ_FOLD_SHIFT;
                                tot[t][2] += (m0 * acc[t][2]) >> RQ_FOLD_SHIFT;
                                if (!ONE) {
                                    tot[t][1] += (m1 * acc[t][1]) >> RQ_FOLD_SHIFT;
                                    tot[t][3] += (m1 * acc[t][3]) >> RQ_FOLD_SHIFT;
                                }
                            }
                            if (GS > 1) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) acc[t][i] = 0;
                            }
                        }
                    }
                }
            }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(&empty[s])) : "memory");
        }

        // combine the consumer warps (integer sums are exact in any order); partials are double-buffered by tile
        // parity, and the warp that reduces and stores rotates from tile to tile
        int * pt = part + (it & 1) * (CONSUMERS * 32 * 4 * NT);
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) pt[(warp * 32 + lane) * 4 * NT + t * 4 + i] = tot[t][i];
        asm volatile("bar.sync 1, %0;" :: "n"(CONSUMERS * 32) : "memory");
        if (!ok || *abort_flag) return;
        if (warp != it % CONSUMERS) continue;
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int v = 0;
                for (int w = 0; w < CONSUMERS; ++w) v += pt[(w * 32 + lane) * 4 * NT + t * 4 + i];
                tot[t][i] = v;
            }
        int fmt = *reinterpret_cast<volatile int *>(&fmt_word);
        for (int spin = 0; fmt < 0 && spin < (1 << 20); ++spin) fmt = *reinterpret_cast<volatile int *>(&fmt_word);
        const bool fmt_ok = fmt == RQ_FMT_I8;
        if (!fmt_ok && lane == 0) atomicExch(prm.status, 2);
        const float s_lo = row_lo < jb.N ? __ldg(jb.sw + row_lo) : 0.0f;
        const float s_hi = row_hi < jb.N ? __ldg(jb.sw + row_hi) : 0.0f;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int tok = 8 * t + 2 * tig + c;
                if (tok < M && fmt_ok) {
                    const float ut = __ldg(prm.u + tok);
                    const float v_lo = __fmul_rn(__fmul_rn(__fmul_rn((float) tot[t][c], 16.0f), ut), s_lo);
                    const float v_hi = __fmul_rn(__fmul_rn(__fmul_rn((float) tot[t][2 + c], 16.0f), ut), s_hi);
                    if (row_lo < jb.N) jb.y[(size_t) tok * jb.ldy + row_lo] = v_lo;
                    if (row_hi < jb.N) jb.y[(size_t) tok * jb.ldy + row_hi] = v_hi;
                    // N-sharded ranks: the same values straight into every other rank's copy of the output
                    if constexpr (PUSH) {
                    for (int d = 0; d < jb.n_more; ++d) {
                        if (row_lo < jb.N) jb.y_more[d][(size_t) tok * jb.ldy + row_lo] = v_lo;
                        if (row_hi < jb.N) jb.y_more[d][(size_t) tok * jb.ldy + row_hi] = v_hi;
                    }
                    }
                }
            }
        }
    }
    if (threadIdx.x == 0) rq_trace(prm.status, 0x13);
}

template <int NT, int GS, bool HAS_K, bool ONE, bool PUSH>
cudaError_t launch_one(const GemvParams & prm, cudaStream_t stream) {
    // first use of this instantiation on a device; several host threads may get here at once
    static std::mutex mu;
    static bool configured[64] = {};
    static int per_sm[64] = {};
    const size_t smem = (size_t) STAGES * ST_BYTES + 2 * (size_t) CONSUMERS * 32 * 4 * NT * sizeof(int);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    int resident_slots;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev]) {
            e = cudaFuncSetAttribute(rq_gemv_mma_kernel<NT, GS, HAS_K, ONE, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
            if (e != cudaSuccess) return e;
            // persistent grid: as many CTAs as are resident at once
            int nb = 0, sms = 148;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, rq_gemv_mma_kernel<NT, GS, HAS_K, ONE, PUSH>, (CONSUMERS + 1) * 32, smem);
            if (e != cudaSuccess) return e;
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            per_sm[dev] = (nb > 0 ? nb : 1) * sms;
            configured[dev] = true;
        }
        resident_slots = per_sm[dev];
    }
    cudaLaunchConfig_t cfg = {};
    const int tiles = prm.tile_start[prm.n_jobs];
    // The quantizer ahead of this kernel (a cluster of up to 8 CTAs per token) still holds its shared memory when this
    // grid starts: CTAs beyond the free slots would start only after it, with their whole share of tiles still to do.
    static const int reserve = rq_env_int("RQ_TUNE_GEMV_RESERVE", 8);
    const int resident = resident_slots - reserve;
    // (an evenly divided grid -- every CTA the same number of tiles -- measured slower: 3.79 against 3.68 ms per pass)
    cfg.gridDim = dim3((unsigned) (tiles < resident ? tiles : resident));
    cfg.blockDim = dim3((CONSUMERS + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    static const int pdl = getenv("RQ_NO_PDL") ? 0 : 1;      // read once
    attr[0].val.programmaticStreamSerializationAllowed = pdl;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, rq_gemv_mma_kernel<NT, GS, HAS_K, ONE, PUSH>, prm);
}

template <int NT, int GS, bool HAS_K>
cudaError_t launch(const GemvParams & prm, cudaStream_t stream) {
    bool push = false;
    for (int i = 0; i < prm.n_jobs; ++i) push = push || prm.job[i].n_more > 0;
    if (NT == 1 && prm.M == 1) return push ? launch_one<1, GS, HAS_K, true, true>(prm, stream) : launch_one<1, GS, HAS_K, true, false>(prm, stream);
    return push ? launch_one<NT, GS, HAS_K, false, true>(prm, stream) : launch_one<NT, GS, HAS_K, false, false>(prm, stream);
}

template <int NT>
cudaError_t launch_nt(const GemvParams & prm, bool has_k, cudaStream_t stream) {
    const int gs = prm.G / 64;
    if (has_k) {
        if (gs == 1) return launch<NT, 1, true>(prm, stream);
        if (gs == 2) return launch<NT, 2, true>(prm, stream);
        return launch<NT, 4, true>(prm, stream);
    }
    if (gs == 1) return launch<NT, 1, false>(prm, stream);
    if (gs == 2) return launch<NT, 2, false>(prm, stream);
    return launch<NT, 4, false>(prm, stream);
}

}  // namespace

cudaError_t rq_launch_gemv(const rq_gemv_job * jobs, int n_jobs, int64_t K, const int8_t * a8, const int32_t * msh,
                           const float * u, int64_t M, int G, int32_t * status, cudaStream_t stream) {
    if (n_jobs < 1 || n_jobs > RQ_MAX_WEIGHTS) return cudaErrorInvalidValue;
    // wider inputs go through in passes of 16 tokens, each re-reading the stream
    for (int64_t t0 = 0; t0 < M; t0 += 16) {
        const int mt = (int) (M - t0 < 16 ? M - t0 : 16);
        GemvParams prm = {};
        prm.n_jobs = n_jobs;
        for (int i = 0; i < n_jobs; ++i) {
            prm.job[i].w4t = reinterpret_cast<const uint4 *>(jobs[i].w4);
            prm.job[i].sw = jobs[i].sw;
            prm.job[i].wk = jobs[i].wk;
            prm.job[i].y = jobs[i].y + t0 * jobs[i].ldy;
            prm.job[i].n_more = jobs[i].n_more;
            for (int d = 0; d < jobs[i].n_more; ++d) prm.job[i].y_more[d] = jobs[i].y_more[d] + t0 * jobs[i].ldy;
            prm.job[i].ldy = jobs[i].ldy;
            prm.job[i].N = (int) jobs[i].N;
            prm.tile_start[i + 1] = prm.tile_start[i] + (int) ((jobs[i].N + 15) / 16);
        }
        prm.K = (int) K; prm.M = mt; prm.G = G;
        prm.a8 = a8 + t0 * K; prm.msh = msh + t0 * (K / G); prm.u = u + t0; prm.status = status;
        const bool has_k = jobs[0].wk != nullptr;
        const cudaError_t e = mt <= 8 ? launch_nt<1>(prm, has_k, stream) : launch_nt<2>(prm, has_k, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}
