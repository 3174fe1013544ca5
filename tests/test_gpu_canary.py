"""GPU: guard bands around every buffer the library writes -- the workspace, the prepack buffer and the outputs -- checked
on the host after calls on every kernel path.  compute-sanitizer is not available where these tests run; the bands catch
a write outside a region, whichever kernel made it.  The reference's own substitute is the same idea (outputs filled with
garbage before a launch to prove they are overwritten and nothing else is, gfx906/test_skinny.cu:86-88)."""
import ctypes

import numpy as np
import pytest

from tests import inputs
from tests.test_gpu_parity import assert_bits, dev

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

BAND = 4096
FILL = 0xA5


@pytest.fixture(scope="module")
def rq():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ruquant_b200
    ruquant_b200.lib()
    return ruquant_b200


class Guarded:
    """`nbytes` of device memory, 256-byte aligned, with a band of a known byte on either side."""

    def __init__(self, nbytes):
        self.nbytes = nbytes
        self.raw = torch.full((nbytes + 2 * BAND + 256,), FILL, dtype=torch.uint8, device="cuda")
        self.off = (-(self.raw.data_ptr() + BAND)) % 256 + BAND
        self.view = self.raw[self.off:self.off + nbytes]

    def intact(self):
        before = self.raw[:self.off]
        after = self.raw[self.off + self.nbytes:]
        return bool((before == FILL).all().item()) and bool((after == FILL).all().item())


@pytest.mark.parametrize("M,path,wgroup", [(1, 0, 0), (7, 1, 0), (16, 1, 64), (40, 1, 0), (100, 2, 0), (200, 2, 0), (130, 2, 64)])
def test_nothing_is_written_outside_the_buffers(rq, port, M, path, wgroup):
    K, N = 5120, 200                      # N neither a multiple of the 256-row tile nor of 16
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9990 + wgroup), 45, wgroup=wgroup)
    blocks = dev(wb).view(-1)
    L = rq.lib()
    # the prepack buffer, guarded
    pp = Guarded(L.rq_w4a4_prepack_bytes(45, K, N, rq.PREPACK_ALL))
    desc = rq.WeightDesc()
    rc = L.rq_w4a4_prepare(blocks.data_ptr(), 45, K, N, pp.view.data_ptr(), pp.nbytes, rq.PREPACK_ALL, ctypes.byref(desc),
                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    # workspace and output, guarded; the output also has unused columns at the end of every row
    ws = Guarded(rq.workspace_bytes(K, M))
    assert L.rq_w4a4_workspace_init(ws.view.data_ptr(), K, M, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    ld = N + 5
    y = Guarded(M * ld * 4)
    x = inputs.outlier_activations(M, K, 9991 + M)
    xd = dev(x)
    pd = ctypes.POINTER(rq.WeightDesc)
    descs = (pd * 1)(ctypes.pointer(desc))
    ys = (ctypes.c_void_p * 1)(y.view.data_ptr())
    lds = (ctypes.c_int64 * 1)(ld)
    rc = L.rq_w4a4_mul_mat(descs, 1, xd.data_ptr(), K, M, ys, lds, 1.0, 64, path, ws.view.data_ptr(), ws.nbytes,
                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert L.rq_w4a4_device_status(ws.view.data_ptr(), K, M, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    assert pp.intact(), "prepack buffer overrun"
    assert ws.intact(), "workspace overrun"
    assert y.intact(), "output overrun"
    got = y.view.view(torch.float32).view(M, ld).cpu().numpy()
    assert_bits(np.ascontiguousarray(got[:, :N]), port.mul_mat(wb, 45, K, x), "M=%d path=%d" % (M, path))
    tail = y.view.view(torch.uint8).view(M, ld * 4)[:, N * 4:]
    assert bool((tail == FILL).all().item()), "wrote past N inside a row"
