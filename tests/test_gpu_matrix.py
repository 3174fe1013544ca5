"""GPU: the reference's environment matrix over its whole backend-test shape list, and the benchmark's configurations at
their full token counts -- every kernel variant the library can launch, bit for bit against the oracle.

The reference runs its MUL_MAT test list (tests/test-backend-ops.cpp hunk in patches/llama.cpp-ruquant.patch:3024-3040)
under RQ_WGROUP=1|64, RQ_ACT_GROUP=128|256 and RQ_ROT_BLOCKS (patch:2529-2538, 2623-2631, 2685-2694; RESULTS.md:142).
Here the switches are arguments: weight groups decide whether the contraction runs on fp8 operands (no multipliers) or
on int8 ones, activation groups decide how many 64-input steps share an accumulator.
"""
import numpy as np
import pytest

from tests import inputs
from tests.test_gpu_parity import assert_bits, dev, gpu_mul_mat, ref_shape_list

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def rq():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ruquant_b200
    ruquant_b200.lib()
    return ruquant_b200


# name -> (activation group, weight group mode: 0 = none, 256 = RQ_WGROUP=1 (per block), 64 = RQ_WGROUP=64)
MATRIX = {"wg256": (64, 256), "wg64": (64, 64), "g128": (128, 0), "g256": (256, 0), "wg256_g128": (128, 256), "wg256_g256": (256, 256)}


@pytest.mark.parametrize("type_", [44, 45])
@pytest.mark.parametrize("env", sorted(MATRIX))
def test_reference_shape_list_under_the_environment_matrix(rq, port, env, type_):
    group, wgroup = MATRIX[env]
    cache = {}
    for rows, tokens, K in ref_shape_list():
        if (rows, K) not in cache:      # the weights of the reference's initialiser depend on (rows, K) only
            w = inputs.reference_test_weights(rows, K)
            cache[(rows, K)] = (w, port.quantize_weights(w, type_, wgroup=wgroup))
        w, wb = cache[(rows, K)]
        x = inputs.reference_test_activations(tokens, K, w, type_ == 44, 77)
        want = port.mul_mat(wb, type_, K, x, group=group)
        what = "%s type=%d rows=%d tokens=%d K=%d" % (env, type_, rows, tokens, K)
        assert_bits(gpu_mul_mat(rq, wb, type_, K, x, group=group), want, what)
        if 17 <= tokens <= 64:          # below 65 tokens the library prefers the GEMV: drive the tensor-core kernel too
            assert_bits(gpu_mul_mat(rq, wb, type_, K, x, group=group, path=2), want, what + " tcgen05")


def _sampled(M, n, seed):
    return np.arange(M) if M <= n else np.sort(np.random.default_rng(seed).choice(M, n, replace=False))


@pytest.mark.parametrize("M", [4, 16, 64, 256, 1024, 2048, 4096])
def test_config4_down_projection_remaining_powers_of_two(rq, port, M):
    """K = 17408 (68 x 256 rotation), N = 5120, the token counts of the sweep that test_config4_down_projection leaves
    out, up to the 4096 tokens the benchmark times; the oracle checks every output of a seeded sample of 64 tokens and
    the tiled weight rows give a full-size property check."""
    K, N = 17408, 5120
    wf = inputs.normal_weights(512, K, 4000)
    wb = np.tile(port.quantize_weights(wf, 45), (N // 512, 1))
    x = inputs.spiky_activations(M, K, 4100 + M)
    got = gpu_mul_mat(rq, wb, 45, K, x)
    pick = _sampled(M, 64, 4200 + M)
    assert_bits(got[pick], port.mul_mat(wb, 45, K, x[pick]), "config 4 M=%d sample" % M)
    assert (inputs.bits(got).reshape(M, N // 512, 512) == inputs.bits(got)[:, None, :512]).all()


@pytest.mark.parametrize("layer_seed", [5100, 5200])
def test_config5_prefill_layer_at_4096_tokens(rq, port, layer_seed):
    """The seven projections of a decoder layer at M = 4096 (two layers' worth of weights), full N; the oracle checks
    every output of 32 sampled tokens."""
    M = 4096
    for i, (name, K, N) in enumerate([("q", 5120, 6144), ("k", 5120, 1024), ("v", 5120, 1024), ("o", 6144, 5120),
                                      ("gate", 5120, 17408), ("up", 5120, 17408), ("down", 17408, 5120)]):
        wf = inputs.normal_weights(128, K, layer_seed + i)
        wb = np.tile(port.quantize_weights(wf, 45), (N // 128, 1))
        x = np.random.default_rng(layer_seed + 50 + i).normal(0, 1, (M, K)).astype(np.float32)
        got = gpu_mul_mat(rq, wb, 45, K, x)
        pick = _sampled(M, 32, layer_seed + 70 + i)
        assert_bits(got[pick], port.mul_mat(wb, 45, K, x[pick]), "%s M=4096 sample" % name)
        assert (inputs.bits(got).reshape(M, N // 128, 128) == inputs.bits(got)[:, None, :128]).all()
        del got


@pytest.mark.parametrize("type_", [44, 45])
@pytest.mark.parametrize("wgroup", [0, 64])
def test_longest_row_on_the_tensor_core_path(rq, port, type_, wgroup):
    """K = 32768, the longest row the format admits: the widest running totals, the most re-centrings of the float fold
    (fp8 operands) and the reference's adversarial initialiser (sign-aligned tokens, flat rows), one CTA and a pair."""
    K, N = 32768, 264
    w = inputs.reference_test_weights(N, K)
    wb = port.quantize_weights(w, type_, wgroup=wgroup)
    for M in (70, 130):
        x = inputs.reference_test_activations(M, K, w, type_ == 44, 88 + M)
        for group in ((64,) if wgroup == 64 else (64, 256)):
            want = port.mul_mat(wb, type_, K, x, group=group)
            assert_bits(gpu_mul_mat(rq, wb, type_, K, x, group=group, path=2), want, "K=32768 M=%d group=%d" % (M, group))


@pytest.mark.parametrize("wgroup", [0, 64])
@pytest.mark.parametrize("M", [100, 200])
def test_push_from_every_tensor_core_variant(rq, port, wgroup, M):
    """rq_w4a4_mul_mat_push above 64 tokens: fp8 and int8 operands, one CTA (M = 100) and pairs (M = 200), two
    destinations on one GPU; the second destination starts 4 bytes off a 16-byte boundary, so the kernel may not use
    16-byte stores for it."""
    K, N = 1536, 328
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9800 + wgroup), 45, wgroup=wgroup)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    assert w.desc.wk_mode == (1 if wgroup else 0)
    x = inputs.outlier_activations(M, K, 9810 + M)
    ld = N + 8
    a = torch.full((M, ld), -1.0, dtype=torch.float32, device="cuda")
    b = torch.full((M * ld + 1,), -1.0, dtype=torch.float32, device="cuda")
    ws = rq.new_workspace(K, M)
    rq.mul_mat_push([w], dev(x), [[a.data_ptr()], [b.data_ptr() + 4]], [ld], workspace=ws)
    torch.cuda.synchronize()
    rq.device_status(ws, K, M)
    want = port.mul_mat(wb, 45, K, x)
    ga, gb = a.cpu().numpy(), b[1:].view(M, ld).cpu().numpy()
    for got in (ga, gb):
        assert_bits(np.ascontiguousarray(got[:, :N]), want, "push wgroup=%d M=%d" % (wgroup, M))
        assert (got[:, N:] == -1.0).all()
    assert float(b[0].item()) == -1.0


def test_push_refuses_the_wrong_activation_format_at_once(rq, port):
    """Tokens quantized for the integer GEMV handed to the pushing tensor-core kernel: status -7, nothing stored in either
    destination, and no warp of the kernel sits out a bounded wait for the stores that never come."""
    import time
    K, N, M = 1536, 328, 200
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9830), 45)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    x = dev(inputs.outlier_activations(M, K, 9831))
    ws = rq.new_workspace(K, M)
    rq.quantize_rows(x, M, 0, w.n_rot, 1.0, 64, rq.FMT_I8, ws)
    bufs = [torch.full((M, N), 7.0, dtype=torch.float32, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rq.mul_mat_push([w], None, [[b.data_ptr()] for b in bufs], [N], act_group=64, workspace=ws, M=M)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5
    with pytest.raises(rq.RqError) as e:
        rq.device_status(ws, K, M)
    assert e.value.status == -7
    for b in bufs:
        assert (b == 7.0).all()


@pytest.mark.parametrize("M", [12, 200])
def test_token_ranges_quantized_apart_multiply_like_the_whole(rq, port, M):
    """Ranks that share the quantizer's work: token ranges rotated and quantized by separate rq_w4a4_quantize_rows calls
    into one workspace (here one GPU makes both calls), then the contraction on the whole -- through
    rq_w4a4_mul_mat_quantized and through the pushing node with no x."""
    K, N = 5120, 320
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9850), 45)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    x = inputs.outlier_activations(M, K, 9851 + M)
    xd = dev(x)
    cut = M // 3
    ws = rq.new_workspace(K, M)
    fmt = rq.act_format(w, M)
    rq.quantize_rows(xd[cut:], M, cut, w.n_rot, 1.0, 64, fmt, ws)          # the ranges in any order
    rq.quantize_rows(xd[:cut], M, 0, w.n_rot, 1.0, 64, fmt, ws)
    want = port.mul_mat(wb, 45, K, x)
    y = rq.mul_mat_quantized(w, M, ws, act_group=64)
    torch.cuda.synchronize()
    assert_bits(y.cpu().numpy(), want, "ranges, M=%d" % M)
    bufs = [torch.full((M, N), -1.0, dtype=torch.float32, device="cuda") for _ in range(2)]
    rq.mul_mat_push([w], None, [[b.data_ptr()] for b in bufs], [N], act_group=64, workspace=ws, M=M)
    torch.cuda.synchronize()
    rq.device_status(ws, K, M)
    for b in bufs:
        assert_bits(b.cpu().numpy(), want, "ranges pushed, M=%d" % M)


@pytest.mark.parametrize("group", [64, 256])
def test_shared_rows_make_every_workspace_whole(rq, port, group):
    """rq_w4a4_share_rows between three workspaces on one GPU standing for three ranks: each quantizes its own range of
    tokens, copies it into the others, and every workspace must then equal, byte for byte in all three regions, the one a
    single quantizer call fills -- and multiply like it."""
    K, N, M = 5120, 192, 70
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9870), 45)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    x = inputs.outlier_activations(M, K, 9871)
    xd = dev(x)
    fmt = rq.act_format(w, M)
    whole = rq.new_workspace(K, M)
    rq.quantize_rows(xd, M, 0, w.n_rot, 1.0, group, fmt, whole)
    cuts = [0, 23, 24, M]                       # ragged ranges, one of a single token
    wss = [rq.new_workspace(K, M) for _ in range(3)]
    for ws in wss:
        ws[:ws.numel() - 256].fill_(0xA5)       # what a range does not write must come from its owner
    ptrs = [ws.data_ptr() for ws in wss]
    for r in range(3):
        rq.quantize_rows(xd[cuts[r]:cuts[r + 1]], M, cuts[r], w.n_rot, 1.0, group, fmt, wss[r])
    for r in range(3):
        rq.share_rows(ptrs, r, wss[r].numel(), K, M, group, cuts[r], cuts[r + 1] - cuts[r])
    torch.cuda.synchronize()
    want_regions = rq.workspace_views(whole, K, M, group)
    for r in range(3):
        for got, want, name in zip(rq.workspace_views(wss[r], K, M, group), want_regions, ("codes", "multipliers", "units")):
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), "%s of workspace %d" % (name, r)
    want = port.mul_mat(wb, 45, K, x, group=group)
    y = rq.mul_mat_quantized(w, M, wss[2], act_group=group)
    torch.cuda.synchronize()
    assert_bits(y.cpu().numpy(), want, "shared rows, group=%d" % group)


@pytest.mark.parametrize("M", [5, 300])
def test_push_of_a_shard_narrower_than_a_unit(rq, port, M):
    """An eighth of a 1024-row tensor: 128 weight rows, half a 256-row unit of the tensor-core kernel, pushed into columns
    384..511 of two gathered [M][1024] outputs; nothing outside those columns may change."""
    K, N = 5120, 128
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9880), 45)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    x = inputs.outlier_activations(M, K, 9881 + M)
    full = [torch.full((M, 1024), -1.0, dtype=torch.float32, device="cuda") for _ in range(2)]
    ws = rq.new_workspace(K, M)
    rq.mul_mat_push([w], dev(x), [[f.data_ptr() + 4 * 384] for f in full], [1024], workspace=ws)
    torch.cuda.synchronize()
    rq.device_status(ws, K, M)
    want = port.mul_mat(wb, 45, K, x)
    for f in full:
        g = f.cpu().numpy()
        assert_bits(np.ascontiguousarray(g[:, 384:512]), want, "narrow shard, M=%d" % M)
        assert (g[:, :384] == -1.0).all() and (g[:, 512:] == -1.0).all()

