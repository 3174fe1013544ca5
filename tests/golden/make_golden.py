"""Generates the golden vectors under tests/golden/ from the reference's own compiled CPU code.

Run where the reference tree is present:  python oracle/build_ref.py && python tests/golden/make_golden.py
Each environment setting of the reference (RQ_ACT_GROUP, RQ_WGROUP, RQ_ROT_BLOCKS are read once per process) gets
its own child process and its own .npz.  Stored per case: the fp32 inputs, the weight blocks, and the reference's
outputs as raw bits (rotated rows, activation blocks, MUL_MAT results).
"""
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

ENVS = {
    "default": {},
    "g128": {"RQ_ACT_GROUP": "128"},
    "g256": {"RQ_ACT_GROUP": "256"},
    "wg256": {"RQ_WGROUP": "1"},
    "wg64": {"RQ_WGROUP": "64"},
    "wg256_g256": {"RQ_WGROUP": "1", "RQ_ACT_GROUP": "256"},
    "rot2": {"RQ_ROT_BLOCKS": "2"},
    "rot4": {"RQ_ROT_BLOCKS": "4"},
}

# (name, type, K, N, M, kind, header clip or 0)
CASES = [
    ("cfg1_w4a4", 44, 4096, 32, 1, "normal", 1.0),
    ("cfg2_w4a4h", 45, 5120, 32, 4, "outlier", 0.9),
    ("cfg4_w4a4h", 45, 17408, 16, 2, "spiky", 0.85),
    ("o_w4a4h", 45, 6144, 16, 3, "normal", 0.0),
    ("adv_w4a4", 44, 512, 40, 17, "adversarial", 0.0),
    ("adv_w4a4h", 45, 1536, 24, 6, "adversarial", 0.0),
    ("adv_w4a4_long", 44, 17408, 8, 6, "adversarial", 0.0),
    ("zero_row", 44, 256, 8, 3, "zeros", 0.0),
]
ROT_LENGTHS = [256, 1536, 5120, 6144, 11264, 17408]


def make_inputs(name, type_, K, N, M, kind, seed):
    from tests import inputs
    if kind == "adversarial":
        w = inputs.reference_test_weights(N, K)
        x = inputs.reference_test_activations(M, K, w, type_ == 44, seed)
    elif kind == "zeros":
        w = inputs.normal_weights(N, K, seed)
        w[1] = 0.0
        x = inputs.outlier_activations(M, K, seed + 1)
        x[0] = 0.0
        x[2, :128] = 0.0
    else:
        w = inputs.normal_weights(N, K, seed)
        x = {"normal": lambda: np.random.default_rng(seed + 1).normal(0, 1, (M, K)).astype(np.float32),
             "outlier": lambda: inputs.outlier_activations(M, K, seed + 1),
             "spiky": lambda: inputs.spiky_activations(M, K, seed + 1)}[kind]()
    return w, x


def child(env_name):
    import oracle
    R = oracle.Ref()
    out = {}
    if env_name == "default":
        rng = np.random.default_rng(7)
        for n in ROT_LENGTHS:
            x = rng.normal(0, 1, (2, n)).astype(np.float32)
            x[1, ::3] *= 17.0
            out["rot%d_x" % n] = x
            out["rot%d_y" % n] = R.rotate(x, n).view(np.uint32)
    for ci, (name, type_, K, N, M, kind, clip) in enumerate(CASES):
        if env_name.startswith("rot") and type_ != 45:
            continue
        if name == "adv_w4a4_long" and env_name not in ("default", "g256"):
            continue
        w, x = make_inputs(name, type_, K, N, M, kind, 1000 + ci)
        wb = R.quantize_weights(w, type_)
        if clip > 0:
            oracle.set_clip(wb, clip)
        n_rot = int(wb[0, 8:12].view(np.int32)[0]) if type_ == 45 else 0
        eff_clip = clip if clip > 0 else 1.0
        if env_name == "default":   # the fp32 inputs are the same in every environment: stored once
            out[name + "_wf"] = w if K * N <= 1 << 16 else np.zeros(0, np.float32)   # fp32 weights only where small
            out[name + "_x"] = x
        out[name + "_w"] = wb
        out[name + "_a"] = R.quantize_act(x, eff_clip, n_rot)
        out[name + "_y"] = R.mul_mat(wb, type_, K, x, threads=4).view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "golden_%s.npz" % env_name), **out)
    print(env_name, "ok", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) > 1:
        child(sys.argv[1])
    else:
        for name, env in ENVS.items():
            e = dict(os.environ)
            for k in ("RQ_ACT_GROUP", "RQ_WGROUP", "RQ_ROT_BLOCKS", "RQ_ACT_CLIP", "RQ_ACT_CLIP_H"):
                e.pop(k, None)
            e.update(env)
            subprocess.check_call([sys.executable, os.path.abspath(__file__), name], env=e, cwd=ROOT)
