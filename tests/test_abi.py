"""CPU: the C-ABI library loads and exports every symbol include/rq_b200.h declares; host-only entry points behave."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rq_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from ruquant_b200 import build
    build.build()
    import ruquant_b200
    return ruquant_b200.lib()


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    import ruquant_b200
    assert sorted(ruquant_b200.EXPORTS) == [n for n in names if n in ruquant_b200.EXPORTS]
    assert set(names) == set(ruquant_b200.EXPORTS)


def test_supported_mirrors_reference_shape_rules(lib):
    import ruquant_b200 as rq
    assert rq.supported(44, 4096, 1024, 1)
    assert rq.supported(45, 17408, 5120, 4096)
    assert not rq.supported(45, 1792, 64, 1)          # no H_p x H_m factorisation
    assert rq.supported(44, 1792, 64, 1)              # plain W4A4 does not rotate
    assert not rq.supported(44, 4096 + 128, 64, 1)    # K not a multiple of 256
    assert not rq.supported(44, 32768 + 256, 64, 1)   # K above the reference's 128 blocks
    assert not rq.supported(43, 4096, 64, 1)
    assert not rq.supported(44, 4096, 64, 1, ldx_bytes=4096 * 4 + 4)   # rows must stay 16-byte aligned
    assert rq.supported(44, 4096, 136, 3)             # any N (the reference needs N % 32 == 0)


def test_factor_and_sizes(lib):
    import ruquant_b200 as rq
    assert rq.hadamard_factor(5120) == (20, 256)
    assert rq.hadamard_factor(17408) == (68, 256)
    assert rq.hadamard_factor(1792) is None
    K, N = 5120, 5120
    assert lib.rq_w4a4_prepack_bytes(45, K, N, rq.PREPACK_DECODE) >= N * K // 2 + N * 4
    assert lib.rq_w4a4_prepack_bytes(45, K, N, rq.PREPACK_ALL) >= N * K * 3 // 2
    assert lib.rq_w4a4_prepack_bytes(45, K + 1, N, rq.PREPACK_ALL) == 0
    assert rq.workspace_bytes(K, 64) >= 64 * K + 64 * (K // 64) * 4 + 64 * 4
    assert lib.rq_status_string(-3).decode().startswith("W4A4H")


def test_null_arguments_return_status_not_crash(lib):
    # error behaviour: status codes where the reference aborts
    assert lib.rq_w4a4_prepare(None, 44, 4096, 64, None, 0, 3, None, None) == -1
    assert lib.rq_w4a4_mul_mat(None, 1, None, 0, 1, None, None, 1.0, 64, 0, None, 0, None) == -1
    assert lib.rq_w4a4_quantize(None, 4096, 1, 4096, 0, 1.0, 64, 0, None, 0, None) == -1
    assert lib.rq_w4a4_rotate(None, 4096, 1, 4096, 4096, None, 4096, None) == -1
    # the multi-rank entry points check their arguments before they touch a device
    import ctypes
    two = (ctypes.c_void_p * 2)(None, None)
    assert lib.rq_w4a4_share_rows(None, 0, 2, 1 << 20, 4096, 8, 64, 0, 4, None) == -1
    assert lib.rq_w4a4_share_rows(two, 2, 2, 1 << 20, 4096, 8, 64, 0, 4, None) == -1          # rank out of range
    assert lib.rq_w4a4_share_rows(two, 0, 2, 1 << 20, 4000, 8, 64, 0, 4, None) == -2          # K not a multiple of 256
    assert lib.rq_w4a4_share_rows(two, 0, 2, 1 << 20, 4096, 8, 64, 6, 4, None) == -2          # rows beyond M_total
    assert lib.rq_w4a4_share_rows(two, 0, 2, 16, 4096, 8, 64, 0, 4, None) == -5               # workspace too small
    assert lib.rq_w4a4_share_rows(two, 0, 2, 1 << 20, 4096, 8, 64, 0, 4, None) == -1          # null workspaces
    assert lib.rq_w4a4_sum_partials(None, 0, 2, 16, None, 0, None) == -1
    assert lib.rq_w4a4_sum_partials(two, 0, 9, 16, two, 0, None) == -1                        # more ranks than RQ_MAX_RANKS
    assert lib.rq_rank_barrier(None, 0, 2, None, None, None) == -1


ENV_PROBE = r"""
import ctypes, sys
import ruquant_b200 as rq
L = rq.lib()
out = []
for type_, header in [(44, 0.0), (44, 0.9), (45, 0.0), (45, 0.85)]:
    d = rq.WeightDesc()
    d.type, d.header_clip = type_, header
    out.append("%.4f" % L.rq_w4a4_resolve_clip(ctypes.byref(d)))
out.append(str(L.rq_w4a4_act_group()))
print(" ".join(out))
"""


@pytest.mark.parametrize("env,want", [
    ({}, "1.0000 0.9000 1.0000 0.8500 64"),                                    # unset: header clip, else 1; groups of 64
    ({"RQ_ACT_CLIP": "0.7"}, "0.7000 0.7000 0.7000 0.7000 64"),                # one switch serves both types
    ({"RQ_ACT_CLIP": "0.7", "RQ_ACT_CLIP_H": "0.6"}, "0.7000 0.7000 0.6000 0.6000 64"),
    ({"RQ_ACT_CLIP_H": "0.6"}, "1.0000 0.9000 0.6000 0.6000 64"),
    ({"RQ_ACT_CLIP": "0"}, "1.0000 0.9000 1.0000 0.8500 64"),                  # not positive: ignored
    ({"RQ_ACT_GROUP": "128"}, "1.0000 0.9000 1.0000 0.8500 128"),
    ({"RQ_ACT_GROUP": "256"}, "1.0000 0.9000 1.0000 0.8500 256"),
    ({"RQ_ACT_GROUP": "100"}, "1.0000 0.9000 1.0000 0.8500 64"),               # anything else: 64
])
def test_environment_switches_resolve_as_in_the_reference(env, want):
    """ggml_rq_act_clip_for and ggml_rq_act_group (patch:2590-2600, 2623-2631): read once per process, so each setting
    gets its own interpreter."""
    import subprocess
    import sys
    e = {k: v for k, v in os.environ.items() if not k.startswith("RQ_ACT_")}
    e.update(env)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    got = subprocess.run([sys.executable, "-c", ENV_PROBE], env=e, cwd=root, capture_output=True, text=True, check=True).stdout.strip()
    assert got == want


def test_adapter_exports_the_reference_entry_points():
    """adapter/rq-w4a4.cu compiled against the reference's ggml headers: the six functions ggml-cuda's dispatcher calls
    (patches/llama.cpp-ruquant.patch:2389-2401) and the custom1 launcher are defined in the object."""
    import os
    import subprocess
    obj = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "adapter", "_build", "rq-w4a4.o")
    if not os.path.exists(obj):
        pytest.skip("adapter/_build is not built (needs the reference's ggml headers)")
    syms = subprocess.check_output(["nm", "-C", "--defined-only", obj], text=True)
    for name in ("ggml_cuda_rq_w4a4_supported(", "ggml_cuda_rq_w4a4_ready(", "ggml_cuda_mul_mat_rq_w4a4(", "ggml_cuda_rq_w4a4_can_fuse(",
                 "ggml_cuda_mul_mat_rq_w4a4_fused(", "ggml_cuda_rq_graph_begin(", "rq_b200_custom1_mul_mat"):
        assert name in syms, name
