"""GPU weight quantizer (rq_w4a4_quantize_weights) against the oracle and the reference's golden blocks: tolerance 0,
every byte of every block (codes, row unit, header sum / multipliers, pad words)."""
import numpy as np
import pytest
import torch

import oracle
from tests import inputs
from tests.test_oracle_golden import CASE_CLIP, CASE_TYPES, ENV_SETTINGS, cases_of, load

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rq():
    import ruquant_b200
    ruquant_b200.lib()
    return ruquant_b200


def gpu_blocks(rq, w, type_, wgroup=0, rot_blocks=1):
    out = rq.quantize_weights(torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32)).cuda(), type_, wgroup, rot_blocks)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("env", sorted(ENV_SETTINGS))
def test_golden_weight_blocks(rq, env):
    """Where the fixtures hold the fp32 weights, the GPU must reproduce the blocks the reference's own code wrote."""
    _group, wgroup, rot_blocks = ENV_SETTINGS[env]
    g, base = load(env), load("default")
    seen = 0
    for name in cases_of(g):
        wf = base[name + "_wf"]
        if not wf.size:
            continue
        mine = gpu_blocks(rq, wf, CASE_TYPES[name], wgroup, rot_blocks)
        if name in CASE_CLIP:
            oracle.set_clip(mine, CASE_CLIP[name])
        assert (mine == g[name + "_w"]).all(), (env, name)
        seen += 1
    assert seen > 0


@pytest.mark.parametrize("type_", [44, 45])
@pytest.mark.parametrize("wgroup", [0, 256, 64])
def test_random_rows_match_the_oracle(rq, port, type_, wgroup):
    for K, N, seed in [(256, 5, 1), (1024, 33, 2), (5120, 48, 3), (6144, 17, 4), (17408, 12, 5)]:
        w = inputs.normal_weights(N, K, 7000 + seed)
        w[0] = 0.0                              # an all-zero row: scale 0, codes 0
        if N > 2:
            w[1, :K // 2] = 0.0                 # all-zero groups inside a row
            w[2] *= 1e-20                       # tiny magnitudes
        want = port.quantize_weights(w, type_, wgroup=wgroup)
        got = gpu_blocks(rq, w, type_, wgroup)
        assert (got == want).all(), (type_, wgroup, K, N, np.argwhere(got != want)[:4])


def test_rotation_blocks_and_strided_rows(rq, port):
    K, N = 5120, 24
    w = inputs.normal_weights(N, K + 64, 7100)[:, :K]          # rows 5184 floats apart
    for rot_blocks in (2, 4):
        want = port.quantize_weights(np.ascontiguousarray(w), 45, rot_blocks=rot_blocks)
        wt = torch.from_numpy(np.ascontiguousarray(inputs.normal_weights(N, K + 64, 7100))).cuda()[:, :K]
        got = rq.quantize_weights(wt, 45, 0, rot_blocks)
        torch.cuda.synchronize()
        assert (got.cpu().numpy() == want).all(), rot_blocks


def test_quantized_weights_feed_the_mul_mat(rq, port):
    """End to end on the GPU: quantize on the GPU, multiply on the GPU, compare with the oracle's node on its own blocks."""
    K, N, M = 5120, 64, 3
    w = inputs.normal_weights(N, K, 7200)
    x = inputs.outlier_activations(M, K, 7201)
    blocks = rq.quantize_weights(torch.from_numpy(w).cuda(), 45)
    weight = rq.Weight(blocks.view(-1), 45, K, N=N)
    y = rq.mul_mat(weight, torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    want = port.mul_mat(port.quantize_weights(w, 45), 45, K, x)
    assert (y.cpu().numpy().view(np.uint32) == want.view(np.uint32)).all()


def test_bad_requests(rq):
    w = torch.zeros((4, 512), dtype=torch.float32, device="cuda")
    with pytest.raises(rq.RqError):
        rq.quantize_weights(w, 44, wgroup=32)
    with pytest.raises(rq.RqError) as e:
        rq.quantize_weights(torch.zeros((4, 1792), dtype=torch.float32, device="cuda"), 45)    # 7 * 256 does not factor
    assert e.value.status == -3


def test_gguf_tensor_to_mul_mat(rq, port, tmp_path):
    """A converted model's tensor: GGUF file -> GPU weight -> MUL_MAT, against the oracle on the same blocks."""
    from ruquant_b200 import gguf
    K, N, M = 5120, 96, 2
    wb = port.quantize_weights(inputs.normal_weights(N, K, 7300), 45)
    oracle.set_clip(wb, 0.9)
    path = str(tmp_path / "m.gguf")
    gguf.write(path, {"general.alignment": 64}, [("pad", (7,), gguf.F32, np.zeros(7, np.float32)),
                                                 ("blk.3.ffn_gate.weight", (K, N), gguf.W4A4H, wb)])
    g = gguf.Gguf.open(path)
    w = g.weight("blk.3.ffn_gate.weight")
    assert abs(w.clip() - 0.9) < 1e-7
    x = inputs.outlier_activations(M, K, 7301)
    y = rq.mul_mat(w, torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    want = port.mul_mat(wb, 45, K, x)
    assert (y.cpu().numpy().view(np.uint32) == want.view(np.uint32)).all()
