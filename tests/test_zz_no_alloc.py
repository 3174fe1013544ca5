"""GPU: rq_w4a4_mul_mat_static -- the entry point for hosts that cannot allocate device memory (planned-buffer
backends, plug-ins inside another runtime's stream).  Its scratch is a fixed array inside the library; the test calls
it through the C ABI twice in a row and wants the very bits rq_w4a4_mul_mat produces with a caller workspace.
Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import numpy as np
import pytest

from tests import inputs

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_static_scratch_matches_workspace_call_twice(port):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ruquant_b200 as rq
    rq.lib()
    K, N = 5120, 768
    wb = port.quantize_weights(inputs.normal_weights(N, K, 900), 45)
    w = rq.Weight(torch.from_numpy(wb).cuda().view(-1), 45, K, N=N)
    for M, seed in ((3, 901), (16, 902)):      # two calls in a row, the second one larger: stale contents must not leak
        x = torch.from_numpy(inputs.outlier_activations(M, K, seed)).cuda()
        want = rq.mul_mat(w, x)
        got = rq.mul_mat_static(w, x)
        torch.cuda.synchronize()
        assert (got.view(torch.int32) == want.view(torch.int32)).all(), "M=%d" % M
        assert (inputs.bits(got.cpu().numpy()) == inputs.bits(port.mul_mat(wb, 45, K, x.cpu().numpy()))).all()
    # beyond the fixed maximum: a clear status, nothing launched
    x = torch.zeros((17, K), dtype=torch.float32, device="cuda")
    with pytest.raises(rq.RqError) as e:
        rq.mul_mat_static(w, x)
    assert e.value.status == -10
