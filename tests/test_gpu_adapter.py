"""GPU: the ggml-cuda adapter (adapter/rq-w4a4.cu, compiled against the reference's own ggml headers) driven the way
ggml-cuda's dispatcher drives the reference's rq-w4a4.cu: real `ggml_tensor` structs, a real `ggml_backend_cuda_context`
(stream and pool), the six entry points of patches/llama.cpp-ruquant.patch:2389-2401 and the custom1 hook of
patch:263-287 -- outputs bit for bit against the oracle."""
import ctypes
import os

import numpy as np
import pytest

from tests import inputs
from tests.test_gpu_parity import assert_bits, dev

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

SHIM = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "adapter", "_build", "librq_ggml_shim.so")
GGML_TYPE_F32, W4A4, W4A4H = 0, 44, 45


@pytest.fixture(scope="module")
def shim():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not os.path.exists(SHIM):
        pytest.skip("adapter/_build/librq_ggml_shim.so is not built (python adapter/build.py needs the reference's ggml headers)")
    import ruquant_b200
    ruquant_b200.lib()
    L = ctypes.CDLL(SHIM)
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    L.shim_ctx_new.restype = vp
    L.shim_ctx_new.argtypes = [i32]
    L.shim_ctx_free.argtypes = [vp]
    L.shim_ctx_sync.argtypes = [vp]
    L.shim_tensor_new.restype = vp
    L.shim_tensor_new.argtypes = [i32, i64, i64, vp, sz]
    L.shim_tensor_free.argtypes = [vp]
    L.shim_node_new.restype = vp
    L.shim_node_new.argtypes = [vp, vp, vp, sz, i32]
    L.shim_supported.argtypes = [i32, vp]
    L.shim_ready.argtypes = [vp]
    L.shim_mul_mat.argtypes = [vp, vp]
    L.shim_can_fuse.argtypes = [vp, vp]
    L.shim_fused.argtypes = [vp, ctypes.POINTER(vp), i32]
    L.shim_graph_begin.argtypes = [vp]
    L.shim_custom1.argtypes = [vp, vp]
    return L


def _weight(shim, port, N, K, type_, seed, clip=0.0):
    import oracle
    wb = port.quantize_weights(inputs.normal_weights(N, K, seed), type_)
    if clip:
        wb = oracle.set_clip(wb, clip)
    wd = dev(wb)
    return wb, wd, shim.shim_tensor_new(type_, K, N, wd.data_ptr(), 0)


def test_adapter_single_node_and_first_use(shim, port):
    K, N = 5120, 384
    ctx = shim.shim_ctx_new(0)
    wb, wd, w = _weight(shim, port, N, K, W4A4H, 9900, clip=0.9)
    assert shim.shim_ready(w) == 0                       # not prepared yet: ggml-cuda keeps graphs off (patch:295-299)
    for M in (1, 5, 200):
        x = inputs.outlier_activations(M, K, 9901 + M)
        xd = dev(x)
        y = torch.full((M, N + 4), -3.0, dtype=torch.float32, device="cuda")
        xt = shim.shim_tensor_new(GGML_TYPE_F32, K, M, xd.data_ptr(), 0)
        node = shim.shim_node_new(w, xt, y.data_ptr(), (N + 4) * 4, 0)
        assert shim.shim_supported(1000, node) == 1
        assert shim.shim_supported(900, node) == 0       # the library is sm_100a code
        shim.shim_graph_begin(ctx)
        shim.shim_mul_mat(ctx, node)
        shim.shim_ctx_sync(ctx)
        assert shim.shim_ready(w) == 1
        got = y.cpu().numpy()
        assert_bits(np.ascontiguousarray(got[:, :N]), port.mul_mat(wb, W4A4H, K, x), "adapter M=%d" % M)   # header clip 0.9 applies
        assert (got[:, N:] == -3.0).all()
    shim.shim_ctx_free(ctx)


def test_adapter_fused_nodes_share_the_activation(shim, port):
    K, M = 5120, 3
    ctx = shim.shim_ctx_new(0)
    x = inputs.outlier_activations(M, K, 9920)
    xd = dev(x)
    xt = shim.shim_tensor_new(GGML_TYPE_F32, K, M, xd.data_ptr(), 0)
    weights, nodes, outs = [], [], []
    for i, N in enumerate((768, 128, 128)):
        wb, wd, w = _weight(shim, port, N, K, W4A4H, 9930 + i)
        y = torch.zeros((M, N), dtype=torch.float32, device="cuda")
        weights.append((wb, wd, w))
        outs.append(y)
        nodes.append(shim.shim_node_new(w, xt, y.data_ptr(), 0, 0))
    assert shim.shim_can_fuse(nodes[0], nodes[1]) == 0   # the weights have not been seen yet: first use stays unfused
    for n in nodes:
        shim.shim_mul_mat(ctx, n)
    shim.shim_ctx_sync(ctx)
    assert shim.shim_can_fuse(nodes[0], nodes[1]) == 1 and shim.shim_can_fuse(nodes[0], nodes[2]) == 1
    other = shim.shim_tensor_new(GGML_TYPE_F32, K, M, xd.data_ptr(), 0)                 # same data, another tensor: not the same src1
    stranger = shim.shim_node_new(weights[1][2], other, outs[1].data_ptr(), 0, 0)
    assert shim.shim_can_fuse(nodes[0], stranger) == 0
    for y in outs:
        y.zero_()
    arr = (ctypes.c_void_p * 3)(*nodes)
    shim.shim_fused(ctx, arr, 3)
    shim.shim_ctx_sync(ctx)
    for (wb, _wd, _w), y in zip(weights, outs):
        assert_bits(y.cpu().numpy(), port.mul_mat(wb, W4A4H, K, x), "fused N=%d" % wb.shape[0])
    shim.shim_ctx_free(ctx)


def test_adapter_custom1_hook(shim, port):
    """The Rust host's route: a launcher registered through ggml_cuda_set_custom1_hook, called by the dispatcher with its
    stream and the GGML_OP_MAP_CUSTOM1 node (src[0] the weight, src[1] the activation)."""
    K, N = 4096, 256
    ctx = shim.shim_ctx_new(0)
    wb, wd, w = _weight(shim, port, N, K, W4A4, 9950)
    x1 = inputs.outlier_activations(2, K, 9951)
    x1d = dev(x1)
    xt = shim.shim_tensor_new(GGML_TYPE_F32, K, 2, x1d.data_ptr(), 0)
    y = torch.zeros((2, N), dtype=torch.float32, device="cuda")
    node = shim.shim_node_new(w, xt, y.data_ptr(), 0, 1)
    assert shim.shim_custom1(ctx, node) == 0             # nothing registered: the node would fall back to the CPU
    shim.shim_register_hook()
    assert shim.shim_custom1(ctx, node) == 1
    shim.shim_ctx_sync(ctx)
    assert_bits(y.cpu().numpy(), port.mul_mat(wb, W4A4, K, x1), "custom1 M=2")
    x2 = inputs.outlier_activations(40, K, 9952)          # wider than the library's built-in scratch serves
    x2d = dev(x2)
    xt2 = shim.shim_tensor_new(GGML_TYPE_F32, K, 40, x2d.data_ptr(), 0)
    y2 = torch.zeros((40, N), dtype=torch.float32, device="cuda")
    node2 = shim.shim_node_new(w, xt2, y2.data_ptr(), 0, 1)
    assert shim.shim_custom1(ctx, node2) == 1
    shim.shim_ctx_sync(ctx)
    assert_bits(y2.cpu().numpy(), port.mul_mat(wb, W4A4, K, x2), "custom1 M=40")
    shim.shim_ctx_free(ctx)
