// Entry points ggml-cuda calls for MUL_MAT nodes whose weight is W4A4 / W4A4H: the declarations of the reference's
// ggml/src/ggml-cuda/rq-w4a4.cuh (patches/llama.cpp-ruquant.patch:2389-2401), served here by librq_b200.so.
#pragma once

#include "common.cuh"

// The vendored ggml tree this adapter is compile-checked against predates the patch's type rows; a patched tree
// (ggml/include/ggml.h in patch:10-14) defines the enumerators itself: build with -DRQ_GGML_HAS_W4A4 there.
#ifndef RQ_GGML_HAS_W4A4
static const ggml_type GGML_TYPE_W4A4  = (ggml_type) 44;
static const ggml_type GGML_TYPE_W4A4H = (ggml_type) 45;
#endif

bool ggml_cuda_rq_w4a4_supported(int cc, const ggml_tensor * src0, const ggml_tensor * src1, const ggml_tensor * dst);
// false until the weight has been prepared (its header read, its kernel-side layouts built), which copies to the host
// and synchronizes and so must not happen inside a stream capture: ggml-cuda keeps CUDA graphs off while any W4A4
// weight of the graph is not ready (patch:295-299)
bool ggml_cuda_rq_w4a4_ready(const ggml_tensor * src0);
void ggml_cuda_mul_mat_rq_w4a4(ggml_backend_cuda_context & ctx, const ggml_tensor * src0, const ggml_tensor * src1, ggml_tensor * dst);
// b = W_b x can share a's quantized activation: same x, type, K, clip and rotation, decode widths (patch:2350-2368)
bool ggml_cuda_rq_w4a4_can_fuse(const ggml_tensor * a, const ggml_tensor * b);
// n <= 3 such matmuls as one call: one rotate+quantize, one GEMV launch over all their rows
void ggml_cuda_mul_mat_rq_w4a4_fused(ggml_backend_cuda_context & ctx, const ggml_tensor * const * src0s, ggml_tensor * const * dsts,
                                     int n, const ggml_tensor * src1);
// start of a graph evaluation (patch:338).  The reference drops its hidden activation cache here; this library shares an
// activation only inside one call, so there is nothing to drop.
void ggml_cuda_rq_graph_begin(ggml_backend_cuda_context & ctx);

// The Rust host's route (src/kernels.rs:12-43): a launcher with the signature ggml_cuda_set_custom1_hook takes
// (patch:263-272).  dst is a GGML_OP_MAP_CUSTOM1 node whose src[0] is the W4A4 / W4A4H weight and src[1] the f32
// activation; enqueues the MUL_MAT on `stream`.
extern "C" void rq_b200_custom1_mul_mat(cudaStream_t stream, ggml_tensor * dst);
