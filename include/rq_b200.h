/*
 * rq_b200.h -- C ABI of the B200 (sm_100a) W4A4 / W4A4H MUL_MAT path.
 *
 * One ggml MUL_MAT node whose weight is of type W4A4 (44) or W4A4H (45): activations f32 [M tokens][K], weight
 * [N rows][K] in the reference's 144-byte blocks of 256 int4 codes, output f32 [M][N].  The library computes, with
 * bit-identical results, what the reference's CPU path computes: the online Hadamard rotation of each token
 * (W4A4H), the per-token grouped asymmetric int4 activation quantizer, the int4 x int4 -> int32 contraction with
 * the per-group integer fold, and the three-multiply fp32 epilogue.
 *
 * Conventions (the same as the reference's GPU entry points, ggml/src/ggml-cuda/rq-w4a4.cuh in
 * patches/llama.cpp-ruquant.patch:2389-2401, and its demo launcher kernels/rq_scale.cu:11-15): raw device
 * pointers, the caller's stream, nothing synchronises or allocates on the call path.  Unlike the reference,
 * which aborts the process on a bad input, every function returns a status (0 = success, negative = rq_status).
 * Everything first-use (header read, weight re-layout) happens in rq_w4a4_prepare, outside stream capture; the
 * 144-byte blocks are left untouched (the reference re-packs them in place on first use, rq-w4a4.cu in
 * patch:2046-2075).
 */
#ifndef RQ_B200_H
#define RQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids of the weight (ggml/include/ggml.h in patch:10-11) */
#define RQ_TYPE_W4A4  44
#define RQ_TYPE_W4A4H 45

#define RQ_BLOCK_CODES 256   /* QK_W4A4, ggml/src/ggml-common.h in patch:38 */
#define RQ_BLOCK_BYTES 144   /* sizeof(block_w4a4), patch:44-50 */
#define RQ_MAX_K       32768 /* the reference admits K <= 256 * 128 blocks (rq-w4a4.cu in patch:1981) */
#define RQ_MAX_WEIGHTS 3     /* weights sharing one activation in a single call (ggml_cuda_try_fuse, patch:308-329) */

typedef enum rq_status {
    RQ_OK             =  0,
    RQ_ERR_ARG        = -1,  /* null pointer, bad type id, bad count */
    RQ_ERR_SHAPE      = -2,  /* K not a multiple of 256 or above RQ_MAX_K, N or M < 1, misaligned row stride */
    RQ_ERR_ROTATION   = -3,  /* W4A4H: header rotation length does not divide K or has no H_p x H_m factorisation */
    RQ_ERR_GROUP      = -4,  /* activation group not 64/128/256, or weight groups of 64 with a group other than 64 */
    RQ_ERR_WORKSPACE  = -5,  /* workspace or prepack buffer too small or misaligned */
    RQ_ERR_CUDA       = -6,  /* a CUDA runtime / driver call failed (rq_last_cuda_error has the code) */
    RQ_ERR_MISMATCH   = -7,  /* weights of one call differ in K, type, rotation length */
    RQ_ERR_DEVICE     = -8,  /* a kernel gave up on a bounded wait (read by rq_w4a4_device_status) */
    RQ_ERR_CLIP       = -9,  /* clip not finite or <= 0 */
    RQ_ERR_LIMIT      = -10  /* a size beyond a stated fixed maximum */
} rq_status;

#define RQ_MAX_RANKS 8   /* ranks of one node whose output buffers a push call can address */

/* which kernel-side layouts rq_w4a4_prepare builds */
#define RQ_PREPACK_DECODE  1   /* int4 stream for the M <= 16 GEMV            (K*N/2 bytes) */
#define RQ_PREPACK_PREFILL 2   /* int8 operand for the tcgen05 GEMM           (K*N bytes)   */
#define RQ_PREPACK_ALL     3

/* how rq_w4a4_quantize stores the activation: int8 8*(q - z) for the GEMV and the integer tensor-core kernel,
 * or e4m3 (q - z) for the fp8 tensor-core kernel (weights without multipliers, the usual case) */
#define RQ_FMT_I8   0
#define RQ_FMT_E4M3 1

/* kernel selection of rq_w4a4_mul_mat */
#define RQ_PATH_AUTO  0        /* M <= 64: GEMV in passes of 16 tokens; else tcgen05 GEMM if prepacked for it */
#define RQ_PATH_GEMV  1
#define RQ_PATH_TC    2

/* A prepared weight.  Plain data: filled by rq_w4a4_prepare, read by rq_w4a4_mul_mat; the caller may copy it.
 * All pointers are device pointers owned by the caller. */
typedef struct rq_weight_desc {
    int32_t  type;          /* RQ_TYPE_W4A4 / RQ_TYPE_W4A4H */
    int32_t  layouts;       /* RQ_PREPACK_* bits present in `prepack` */
    int64_t  K, N;
    int32_t  n_rot;         /* W4A4H: Hadamard length from block 0's pad[0]; 0 for W4A4 */
    int32_t  had_p, had_m;  /* n_rot = had_p * had_m, had_m a power of two */
    int32_t  wk_mode;       /* 0: every weight multiplier is 1; 1: multipliers present (per block or per 64 inputs) */
    int32_t  wg64;          /* block 0's header selects weight groups of 64 (needs activation groups of 64) */
    float    header_clip;   /* block 0's pad[1] as a float; 0 = unset */
    const void * blocks;    /* the 144-byte blocks as given */
    void *   prepack;       /* base of the prepack buffer */
    uint64_t off_sw;        /* f32  [N]        row units s_w */
    uint64_t off_w4;        /* u8   [N][K/2]   decode stream (if RQ_PREPACK_DECODE) */
    uint64_t off_w8;        /* i8   [N][K]     prefill operand (if RQ_PREPACK_PREFILL) */
    uint64_t off_wk;        /* i8   [N][K/64]  weight multipliers (if wk_mode) */
    uint64_t tmap_w8[16];   /* CUtensorMap of the prefill operand (128 bytes, 64-byte aligned copy is made at launch) */
} rq_weight_desc;

/* Admitted shapes.  Mirrors ggml_cuda_rq_w4a4_supported (rq-w4a4.cu in patch:1977-1994): K a multiple of 256 and
 * <= 32768, x rows 16-byte aligned, W4A4H needs a factorable K -- but any N >= 1 and any M >= 1 are accepted
 * (the reference needs N a multiple of 32).  Returns 1 if supported, 0 if not. */
int rq_w4a4_supported(int type, int64_t K, int64_t N, int64_t M, int64_t ldx_bytes);

/* The reference's factorisation of a Hadamard length (ggml_rq_hadamard_factor, ggml/src/ggml-quants.c in
 * patch:2419-2430).  Returns 1 and fills p, m, or 0. */
int rq_hadamard_factor(int64_t n, int * p, int * m);

/* Resolution of the run-time switches exactly as the reference does it, environment included:
 * clip = RQ_ACT_CLIP / RQ_ACT_CLIP_H if > 0, else the tensor's header clip if > 0, else 1
 * (ggml_rq_act_clip_for, patch:2590-2600); group = RQ_ACT_GROUP if 128 or 256, else 64 (ggml_rq_act_group,
 * patch:2623-2631). */
float rq_w4a4_resolve_clip(const rq_weight_desc * w);
int   rq_w4a4_act_group(void);

/* Bytes of the caller-owned prepack buffer for one weight. */
size_t rq_w4a4_prepack_bytes(int type, int64_t K, int64_t N, int layouts);

/* First use of a weight; NOT capture-safe (copies block 0's header to the host and synchronises `stream`, as
 * rq_info does in patch:2027-2043).  Reads clip, rotation length and weight-group mode, validates them, builds the
 * kernel-side layouts in `prepack_dev` (256-byte aligned, rq_w4a4_prepack_bytes large).  The blocks stay valid and
 * untouched. */
int rq_w4a4_prepare(const void * w_blocks_dev, int type, int64_t K, int64_t N, void * prepack_dev, size_t prepack_bytes,
                    int layouts, rq_weight_desc * out_desc, void * stream);

/* Bytes of the per-call workspace (quantized activations and a 256-byte status block) for M tokens of width K. */
size_t rq_w4a4_workspace_bytes(int64_t K, int64_t M);

/* Zeroes the workspace's status block (a memset node: capture-safe).  Call it once after allocating a workspace --
 * or before each use when the memory comes from a pool, as ggml-cuda's does -- because the error word of the block is
 * sticky: kernels only ever set it, so that a report survives later calls until rq_w4a4_device_status reads it.  A
 * build with -DRQ_TRACE also reads a buffer address from the block; garbage there would be dereferenced. */
int rq_w4a4_workspace_init(void * workspace_dev, int64_t K, int64_t M, void * stream);

/* The MUL_MAT node.  Capture-safe: only enqueues on `stream`.  y[i][t*ldy[i] + n] for n_w (1..3) weights that
 * share the activation x (f32, row stride ldx floats, rows 16-byte aligned): rotate (W4A4H) -> quantize -> GEMV
 * or tcgen05 GEMM with the per-group fold -> epilogue.  clip and act_group are the resolved values (see
 * rq_w4a4_resolve_clip / rq_w4a4_act_group).  Replaces ggml_cuda_mul_mat_rq_w4a4 and ggml_cuda_mul_mat_rq_w4a4_fused
 * (rq-w4a4.cu in patch:2341-2380). */
int rq_w4a4_mul_mat(const rq_weight_desc * const * w, int n_w, const float * x_dev, int64_t ldx, int64_t M,
                    float * const * y_dev, const int64_t * ldy, float clip, int act_group, int path,
                    void * workspace_dev, size_t workspace_bytes, void * stream);

/* The GEMM / GEMV stage alone on an activation that rq_w4a4_quantize already left in `workspace_dev` (the
 * explicit form of the reference's activation cache, rq-w4a4.cu in patch:1996-2023). */
int rq_w4a4_mul_mat_quantized(const rq_weight_desc * w, int64_t M, float * y_dev, int64_t ldy, int act_group, int path,
                              void * workspace_dev, size_t workspace_bytes, void * stream);

/* The same for 1..3 weights sharing that activation: at decode widths their row tiles form a single GEMV launch
 * (the reference's fused skinny launch, ggml_cuda_mul_mat_rq_w4a4_fused, patch:2370-2380). */
int rq_w4a4_mul_mat_quantized_n(const rq_weight_desc * const * w, int n_w, int64_t M, float * const * y_dev,
                                const int64_t * ldy, int act_group, int path, void * workspace_dev, size_t workspace_bytes,
                                void * stream);

/* Stage entry points (also used by the parity tests).
 * rq_w4a4_rotate: out[t][:] = x[t][:] * diag(H, H, ...) with H = (H_p kron H_m)/sqrt(n_rot)
 *   (ggml_rq_hadamard per block of n_rot, patch:2450-2485, 2697-2699).
 * rq_w4a4_quantize: rotate (n_rot > 0) and quantize M tokens into the workspace
 *   (quantize_row_a4_clip / quantize_row_a4h_clip_n, patch:2639-2679, 2720-2736); act_format as returned by
 *   rq_w4a4_act_format.  The contraction kernels check the recorded format and refuse a mismatch (status). */
int rq_w4a4_rotate(const float * x_dev, int64_t ldx, int64_t M, int64_t K, int64_t n_rot, float * out_dev, int64_t ldo,
                   void * stream);
int rq_w4a4_quantize(const float * x_dev, int64_t ldx, int64_t M, int64_t K, int64_t n_rot, float clip, int act_group,
                     int act_format, void * workspace_dev, size_t workspace_bytes, void * stream);

/* The same for `count` tokens starting at token `first` of a workspace laid out for M_total tokens (x_rows_dev points at
 * the first of those rows).  Ranks that share the quantizer's work each do a range of tokens this way and exchange the
 * results -- the three regions of rq_w4a4_workspace_layout are contiguous per token range: count * K bytes of codes,
 * count * (K / act_group) multipliers, count units -- before every rank multiplies by its own rows
 * (rq_w4a4_mul_mat_quantized, or rq_w4a4_mul_mat_push with x_dev = NULL). */
int rq_w4a4_quantize_rows(const float * x_rows_dev, int64_t ldx, int64_t M_total, int64_t first, int64_t count, int64_t K,
                          int64_t n_rot, float clip, int act_group, int act_format, void * workspace_dev,
                          size_t workspace_bytes, void * stream);

/* The exchange for ranks whose workspaces are mapped into one another (cudaIpc / symmetric memory): one copy kernel
 * stores rows [first, first + count) of this rank's three regions into the same rows of every other rank's workspace.
 * workspace_of_rank[r]: rank r's workspace as mapped on this device, all laid out for the same K and M_total;
 * workspace_of_rank[rank] is the source.  An rq_rank_barrier after the call makes every rank's rows visible everywhere;
 * a workspace must not be quantized into again before the ranks that read it have passed a later barrier.  The reference
 * has no counterpart: its ranks each rotate and quantize every token.  Capture-safe. */
int rq_w4a4_share_rows(void * const * workspace_of_rank, int rank, int n_ranks, size_t workspace_bytes, int64_t K,
                       int64_t M_total, int act_group, int64_t first, int64_t count, void * stream);

/* The activation format (RQ_FMT_*) the contraction of these weights at M tokens wants -- what rq_w4a4_mul_mat passes
 * to the quantizer itself; for callers that run rq_w4a4_quantize and rq_w4a4_mul_mat_quantized separately.
 * Negative rq_status on a request that cannot be served (missing layout, weights that need different formats). */
int rq_w4a4_act_format(const rq_weight_desc * const * w, int n_w, int64_t M, int path);

/* Where the quantized activation sits in the workspace (RQ_FMT_I8): a8 = int8 [M][K] holding 8*(q - z_g),
 * permuted inside each run of 64 inputs (piece 16*i + 4*t .. +3 at byte 16*t + 4*i); msh = int32
 * [M][K/act_group] holding m_g; u = f32 [M] token units. */
int rq_w4a4_workspace_layout(int64_t K, int64_t M, int act_group, uint64_t * off_a8, uint64_t * off_msh, uint64_t * off_u,
                             uint64_t * off_status);

/* Synchronises `stream` and returns RQ_OK, RQ_ERR_DEVICE if a kernel of ANY earlier call on this workspace gave up on
 * a bounded wait, or RQ_ERR_MISMATCH if a contraction kernel met an activation quantized in the other format.  The
 * report is sticky until this call reads it (and clears it).  Not capture-safe. */
int rq_w4a4_device_status(void * workspace_dev, int64_t K, int64_t M, void * stream);

/* N-sharded ranks of one node (the reference assembles the outputs with a collective after the node; here the node
 * writes them itself).  rq_w4a4_mul_mat_push is rq_w4a4_mul_mat (GEMV up to 64 tokens: needs the decode layout; tcgen05
 * kernel above: needs the prefill layout) that leaves every output value in n_dst buffers instead of one (the GEMV's epilogue
 * stores it into each; in the tcgen05 kernel two warps copy every finished unit from the first buffer into the others while
 * the next units are computed): y_dst[d * n_w + i] is weight i's output in destination d
 * -- this rank's own buffer and the peer-mapped buffers of the other ranks (cudaIpc / symmetric memory), all with the
 * same row stride ldy[i].  x_dev may be NULL: the workspace then already holds the quantized activation of all M tokens
 * (rq_w4a4_quantize / rq_w4a4_quantize_rows in the format rq_w4a4_act_format names).  No collective kernel follows.  rq_rank_barrier then makes the pushed data of all ranks
 * visible: rank r stores a fresh epoch into word r of every rank's flag array (flags_of_rank[p] = rank p's array of
 * n_ranks words, peer-mapped, zero-initialised) and waits, bounded, until its own array shows that epoch from every
 * rank; the epoch counts up in *epoch_dev (local device memory, zero-initialised), so a captured graph replays
 * correctly.  On expiry of the wait *status_dev becomes 3 and the kernel returns.  One barrier kernel per GPU; ranks
 * are separate processes or threads, one per GPU.
 * Rules the caller keeps:
 *  - every rank calls the barrier the same number of times, in the same places: a rank whose epoch lags behind passes
 *    without waiting (the comparison is "at least this epoch"), it does not wait for the others to catch up;
 *  - a rank leaves barrier k as soon as all flags show epoch k, and may then push again while its peers still run
 *    what they placed between barrier k and barrier k+1.  So a destination pushed to after barrier k must not alias
 *    memory that any peer still reads before ITS barrier k+1: keep two copies of such an output and alternate
 *    (double-buffering), or place a second barrier after the readers.  ggml reuses graph buffers, so an adapter that
 *    pushes straight into dst tensors needs one of the two;
 *  - all y_dst[d * n_w + i] of a call must be 4-byte aligned; 16-byte stores are used only when every destination
 *    (and ldy) allows them. */
int rq_w4a4_mul_mat_push(const rq_weight_desc * const * w, int n_w, const float * x_dev, int64_t ldx, int64_t M,
                         float * const * y_dst, int n_dst, const int64_t * ldy, float clip, int act_group,
                         void * workspace_dev, size_t workspace_bytes, void * stream);
int rq_rank_barrier(uint32_t * const * flags_of_rank, int rank, int n_ranks, uint32_t * epoch_dev, int32_t * status_dev,
                    void * stream);

/* K-split ranks of one node (the reference's tensor-parallel mode for attn_output / ffn_down: `ruquant convert
 * --rot-blocks`, src/convert.rs:120-128; every rank multiplies its block columns by its slice of x and the partial
 * outputs are added by a peer-write all-reduce, patches/mx-llama.cpp-ruquant.patch:5293-5374).  Each rank's partial
 * [count] f32 lies in a buffer every rank has mapped: partials_of_rank[r] is rank r's as mapped here, 16-byte aligned.
 * The sum is taken in rank order, ((p0 + p1) + p2) + ..., so every rank gets the same bits.  two_shot = 0: this rank adds
 * all `count` elements into y_of_rank[rank] (its own, local) -- one kernel, nothing after it.  two_shot = 1: this rank
 * adds its 1/n_ranks piece and stores it into every y_of_rank[d] (peer-mapped outputs); an rq_rank_barrier after it makes
 * all pieces visible on all ranks.  Either way an rq_rank_barrier must stand between the MUL_MATs that wrote the
 * partials and this call, and the partials must not be overwritten before every rank's sum has run (a second barrier,
 * or two sets of buffers).  Capture-safe. */
int rq_w4a4_sum_partials(const float * const * partials_of_rank, int rank, int n_ranks, int64_t count,
                         float * const * y_of_rank, int two_shot, void * stream);

/* The reference's weight quantizer on the GPU: N rows of K fp32 (rows ldw floats apart) -> N rows of K/256 blocks,
 * byte for byte what quantize_w4a4 / quantize_w4a4h write (patch:2775-2789; per row quantize_row_w4a4_ref /
 * quantize_row_w4a4h_ref, patch:2681-2710; scale search and packing rq_scale_search, rq_quantize_row_w, rq_pack,
 * patch:2489-2580).  wgroup: 0 = one scale per row, 256 / 64 = the reference's RQ_WGROUP=1 / 64 (a multiplier per block
 * / per 64 inputs).  rot_blocks: RQ_ROT_BLOCKS (W4A4H rows are rotated in blocks of K / rot_blocks when that divides
 * K).  The activation clip in the headers is left unset (0), as the reference leaves it.  scratch: caller-owned,
 * 256-byte aligned, rq_w4a4_quantize_weights_scratch_bytes (0 on a bad request).  Enqueues on stream. */
size_t rq_w4a4_quantize_weights_scratch_bytes(int type, int64_t K, int64_t N, int wgroup);
int rq_w4a4_quantize_weights(const float * w_dev, int64_t ldw, int type, int64_t K, int64_t N, int wgroup, int rot_blocks,
                             void * blocks_dev, void * scratch_dev, size_t scratch_bytes, void * stream);

/* No counterpart in the reference.  The MUL_MAT node for callers that may not allocate device memory (a backend
 * whose buffers are planned ahead of time, a plug-in inside another runtime's stream): the scratch that
 * rq_w4a4_mul_mat takes from the caller lives in a fixed array inside the library instead.  One weight, M <= 16
 * tokens, K <= 32768, else RQ_ERR_LIMIT.  Calls no cudaMalloc / cudaFree.  All calls on a device share the array:
 * calls that can overlap on the GPU race.  The first call on a device resolves the array's device address and
 * should be made outside stream capture. */
int rq_w4a4_mul_mat_static(const rq_weight_desc * w, const float * x_dev, int64_t ldx, int64_t M, float * y_dev, int64_t ldy,
                           float clip, int act_group, int path, void * stream);

/* Measurement aid, not the MUL_MAT: the tcgen05 kernel run with the whole of K in one accumulator per output (no
 * per-group hand-over out of tensor memory, no fold), on an activation already quantized into the workspace.  A
 * benchmark times it next to rq_w4a4_mul_mat_quantized to see what the per-group fold of the reference's format costs
 * on this kernel.  The values written to y_dev are meaningless. */
int rq_w4a4_tc_nofold_probe(const rq_weight_desc * w, int64_t M, float * y_dev, int64_t ldy, void * workspace_dev,
                            size_t workspace_bytes, void * stream);

const char * rq_status_string(int status);
int rq_last_cuda_error(void);   /* cudaError_t of the last failed runtime call on this thread */

#ifdef __cplusplus
}
#endif
#endif /* RQ_B200_H */
