"""CPU: the oracle restatement (oracle/rq_oracle.c) against the golden vectors generated from the reference's own
compiled code, and -- where that compiled reference is present -- against it directly on fresh random inputs."""
import os

import numpy as np
import pytest

import oracle
from tests import inputs

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ENV_SETTINGS = {   # name -> (activation group, weight group mode, rotation blocks)
    "default": (64, 0, 1), "g128": (128, 0, 1), "g256": (256, 0, 1), "wg256": (64, 256, 1), "wg64": (64, 64, 1),
    "wg256_g256": (256, 256, 1), "rot2": (64, 0, 2), "rot4": (64, 0, 4),
}
CASE_TYPES = {"cfg1_w4a4": 44, "cfg2_w4a4h": 45, "cfg4_w4a4h": 45, "o_w4a4h": 45, "adv_w4a4": 44, "adv_w4a4h": 45,
              "adv_w4a4_long": 44, "zero_row": 44}
CASE_CLIP = {"cfg1_w4a4": 1.0, "cfg2_w4a4h": 0.9, "cfg4_w4a4h": 0.85}


def load(env):
    return np.load(os.path.join(GOLD, "golden_%s.npz" % env))


def cases_of(g):
    return sorted(k[:-2] for k in g.files if k.endswith("_y") and not k.startswith("rot"))


def test_hadamard_factor(port):
    # ggml_rq_hadamard_factor: the factorisations the reference picks for the model's widths
    assert port.hadamard_factor(4096) == (1, 4096)
    assert port.hadamard_factor(5120) == (20, 256)
    assert port.hadamard_factor(6144) == (12, 512)
    assert port.hadamard_factor(17408) == (68, 256)
    assert port.hadamard_factor(11264) == (44, 256)
    assert port.hadamard_factor(1792) is None          # 7 * 256: no Paley order fits


def test_paley_is_hadamard(port):
    for p in (12, 20, 44, 60, 68, 72, 84, 104, 108):
        A = port.paley(p).astype(np.int32)
        assert (np.abs(A) == 1).all()
        assert (A @ A.T == p * np.eye(p, dtype=np.int32)).all()


def test_rotation_golden(port):
    g = load("default")
    for n in (256, 1536, 5120, 6144, 11264, 17408):
        got = port.rotate(g["rot%d_x" % n], n)
        assert (inputs.bits(got) == g["rot%d_y" % n]).all(), n


@pytest.mark.parametrize("env", sorted(ENV_SETTINGS))
def test_quantizers_and_mul_mat_golden(port, env):
    group, wgroup, rot_blocks = ENV_SETTINGS[env]
    g, base = load(env), load("default")
    for name in cases_of(g):
        type_ = CASE_TYPES[name]
        x, wb = base[name + "_x"], g[name + "_w"]
        K = x.shape[1]
        wf = base[name + "_wf"]
        if wf.size:   # weight quantizer (scale search, packing, headers) where the fp32 weights are stored
            mine = port.quantize_weights(wf, type_, wgroup=wgroup, rot_blocks=rot_blocks, threads=2)
            if name in CASE_CLIP:
                oracle.set_clip(mine, CASE_CLIP[name])
            assert (mine == wb).all(), (env, name, "weights")
        clip = CASE_CLIP.get(name, 1.0)
        n_rot = int(wb[0, 8:12].copy().view(np.int32)[0]) if type_ == 45 else 0
        if type_ == 45:
            assert n_rot == K // rot_blocks
        a = port.quantize_act(x, clip, group, n_rot)
        assert (a == g[name + "_a"]).all(), (env, name, "activations")
        y = port.mul_mat(wb, type_, K, x, group=group, threads=2)
        assert (inputs.bits(y) == g[name + "_y"]).all(), (env, name, "mul_mat")
        # the per-output form (the reference's own loop structure) agrees with the widened form
        d = port.vec_dot(K, wb[wb.shape[0] - 1], a[0])
        assert np.float32(d).view(np.uint32) == g[name + "_y"][0, -1]


def test_header_clip_of_other_rows_is_ignored(port):
    # the reference reads the clip from block 0 of row 0 only (ggml_rq_tensor_clip): other rows' headers are inert
    g = load("default")
    x, wb = g["cfg2_w4a4h_x"], g["cfg2_w4a4h_w"].copy()
    y0 = port.mul_mat(wb, 45, 5120, x)
    v = wb.reshape(wb.shape[0], -1, 144)
    v[1:, :, 12:16] = np.frombuffer(np.float32(0.5).tobytes(), dtype=np.uint8)
    v[0, 1:, 12:16] = np.frombuffer(np.float32(0.7).tobytes(), dtype=np.uint8)
    assert (inputs.bits(port.mul_mat(wb, 45, 5120, x)) == inputs.bits(y0)).all()
    assert (inputs.bits(y0) == g["cfg2_w4a4h_y"]).all()


def test_bad_rotation_length_is_rejected(port):
    g = load("default")
    wb = g["o_w4a4h_w"].copy()
    wb.reshape(wb.shape[0], -1, 144)[0, 0, 8:12] = np.frombuffer(np.int32(1792).tobytes(), dtype=np.uint8)
    with pytest.raises(ValueError):
        port.mul_mat(wb, 45, 6144, g["o_w4a4h_x"])


def test_port_against_compiled_reference(port, ref):
    rng = np.random.default_rng(42)
    for K, N, M, type_ in [(256, 8, 2, 44), (512, 8, 3, 45), (2560, 16, 5, 45), (4096, 16, 2, 45), (11264, 8, 2, 45)]:
        w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
        x = rng.standard_t(3, (M, K)).astype(np.float32)
        wb = ref.quantize_weights(w, type_)
        assert (port.quantize_weights(w, type_) == wb).all()
        assert (inputs.bits(port.mul_mat(wb, type_, K, x)) == inputs.bits(ref.mul_mat(wb, type_, K, x))).all()
