"""GPU: the CUDA path, called through the C ABI, against the oracle and the golden vectors -- bit for bit
(tolerance 0, like the reference's own backend test: max_nmse_err() == 0.0 for W4A4 / W4A4H,
tests/test-backend-ops.cpp hunk in patches/llama.cpp-ruquant.patch:2946-2948)."""
import os

import numpy as np
import pytest

import oracle
from tests import inputs
from tests.test_oracle_golden import CASE_CLIP, CASE_TYPES, ENV_SETTINGS, cases_of, load

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def rq():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ruquant_b200
    ruquant_b200.lib()       # raises if the extension is missing: there is no fallback to test
    return ruquant_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def gpu_mul_mat(rq, wb, type_, K, x, group=64, path=0, clip=None):
    w = rq.Weight(dev(wb).view(-1), type_, K, N=wb.shape[0])
    M = x.shape[0]
    ws = rq.new_workspace(K, M)
    y = rq.mul_mat(w, dev(x), act_group=group, path=path, clip=clip, workspace=ws)
    torch.cuda.synchronize()
    rq.device_status(ws, K, M)
    return y.cpu().numpy()


def assert_bits(got, want, what):
    g, w = inputs.bits(got), inputs.bits(want) if want.dtype != np.uint32 else want
    bad = np.argwhere(g != w)
    assert bad.size == 0, "%s: %d of %d outputs differ, first at %s: got %r want %r" % (
        what, len(bad), g.size, bad[0], got[tuple(bad[0])], w[tuple(bad[0])].view(np.float32))


# ------------------------------------------------------------------------------------------- stages

def test_rotation_matches_golden(rq):
    g = load("default")
    for n in (256, 1536, 5120, 6144, 11264, 17408):
        got = rq.rotate(dev(g["rot%d_x" % n]), n).cpu().numpy()
        assert_bits(got, g["rot%d_y" % n], "rotation n=%d" % n)


def test_block_diagonal_rotation(rq, port):
    # RQ_ROT_BLOCKS files: the Hadamard length is a divisor of K and each run of n_rot inputs rotates on its own
    rng = np.random.default_rng(3)
    for K, n_rot in [(5120, 2560), (6144, 1536), (4096, 1024), (17408, 4352)]:
        x = rng.normal(0, 1, (3, K)).astype(np.float32)
        assert_bits(rq.rotate(dev(x), n_rot).cpu().numpy(), port.rotate(x, n_rot), "K=%d n_rot=%d" % (K, n_rot))


@pytest.mark.parametrize("group", [64, 128, 256])
def test_activation_quantizer_fields(rq, port, group):
    rng = np.random.default_rng(5)
    for K, n_rot, clip in [(4096, 0, 1.0), (5120, 5120, 0.9), (6144, 6144, 1.0), (17408, 17408, 0.8), (256, 0, 0.7)]:
        x = inputs.outlier_activations(5, K, 11)
        x[1] = 0.0                      # an all-zero token: R == 0 -> 2
        x[2, :K // 2] = 0.0             # groups with an empty range: m = 1
        x[3] = np.abs(x[3])             # no negative values: z = 0
        x[4] = rng.uniform(-1e-30, 1e-30, K).astype(np.float32)
        ws, a8, msh, u = rq.quantize(dev(x), n_rot, clip, group)
        torch.cuda.synchronize()
        uo, mo, zo, qo = oracle.act_fields(port.quantize_act(x, clip, group, n_rot), group)
        assert_bits(u.cpu().numpy(), uo, "unit")
        assert (msh.cpu().numpy() == mo).all(), "multipliers"
        want = 8 * (qo - np.repeat(zo, group, axis=1))
        # stored permuted inside each run of 64 inputs: the piece 16*i + 4*t .. +3 sits at 16*t + 4*i
        k = np.arange(K)
        off = k % 64
        pos = (k - off) + ((off % 16) // 4) * 16 + (off // 16) * 4 + off % 4
        got = a8.cpu().numpy().astype(np.int32)[:, pos]
        assert (got == want).all(), "codes"


def _e4m3_value(b):
    """Value of an e4m3 byte (no NaN/inf codes occur for |v| <= 15)."""
    b = b.astype(np.int32)
    e, mant = (b >> 3) & 15, b & 7
    mag = np.where(e == 0, mant / 8.0 * 2.0 ** -6, (1 + mant / 8.0) * 2.0 ** (e - 7))
    return np.where(b & 0x80, -mag, mag)


def test_activation_quantizer_e4m3_format(rq, port):
    """The tcgen05 fp8 path's activation: bytes are e4m3 of (q - z), multipliers are float bits of m/16."""
    for K, n_rot, clip, group in [(4096, 0, 1.0, 64), (5120, 5120, 0.9, 128), (2048, 2048, 0.8, 256)]:
        x = inputs.outlier_activations(3, K, 12)
        x[1] = 0.0
        ws, a8, msh, u = rq.quantize(dev(x), n_rot, clip, group, fmt=rq.FMT_E4M3)
        torch.cuda.synchronize()
        uo, mo, zo, qo = oracle.act_fields(port.quantize_act(x, clip, group, n_rot), group)
        assert_bits(u.cpu().numpy(), uo, "unit")
        assert_bits(msh.cpu().numpy().view(np.float32), (mo / 16.0).astype(np.float32), "multipliers")
        want = qo - np.repeat(zo, group, axis=1)
        k = np.arange(K)
        off = k % 64
        pos = (k - off) + ((off % 16) // 4) * 16 + (off // 16) * 4 + off % 4
        got = _e4m3_value(a8.cpu().numpy().view(np.uint8)[:, pos])
        assert (got == want).all(), "codes"


def test_activation_format_mismatch_is_refused(rq, port):
    K, N = 1024, 48
    wb = port.quantize_weights(inputs.normal_weights(N, K, 130), 44)
    w = rq.Weight(dev(wb).view(-1), 44, K, N=N)
    assert rq.act_format(w, 4, rq.PATH_GEMV) == rq.FMT_I8 and rq.act_format(w, 4, rq.PATH_TC) == rq.FMT_E4M3
    x = dev(inputs.outlier_activations(4, K, 131))
    y = torch.full((4, N), 7.0, dtype=torch.float32, device="cuda")
    for fmt, path in [(rq.FMT_E4M3, rq.PATH_GEMV), (rq.FMT_I8, rq.PATH_TC)]:
        ws, *_ = rq.quantize(x, 0, 1.0, 64, fmt=fmt)
        rq.mul_mat_quantized(w, 4, ws, out=y, act_group=64, path=path)
        with pytest.raises(rq.RqError) as e:
            rq.device_status(ws, K, 4)
        assert e.value.status == -7
        assert (y == 7.0).all()           # nothing was stored


# ------------------------------------------------------------------------------------------- golden MUL_MAT

@pytest.mark.parametrize("path", [1, 2], ids=["gemv", "tcgen05"])
@pytest.mark.parametrize("env", sorted(ENV_SETTINGS))
def test_mul_mat_matches_golden(rq, env, path):
    group = ENV_SETTINGS[env][0]
    g, base = load(env), load("default")
    for name in cases_of(g):
        x, wb = base[name + "_x"], g[name + "_w"]
        got = gpu_mul_mat(rq, wb, CASE_TYPES[name], x.shape[1], x, group=group, path=path)
        assert_bits(got, g[name + "_y"], "%s/%s" % (env, name))


# ------------------------------------------------------------------------------------------- the reference's own test shapes

def ref_shape_list():
    shapes = []
    for n in (1, 3, 8, 17, 64, 200):
        for k in (256, 512, 1536, 5120, 6144):
            shapes.append((136, n, k))
    shapes.append((5120, 32, 17408))
    for n in (1, 2, 4, 5, 8, 16, 24, 32, 48, 64, 65, 130):
        for k in (256, 6144):
            shapes.append((256, n, k))
    shapes += [(192, 8, 5120), (1024, 8, 5120), (5120, 8, 17408)]
    return shapes


@pytest.mark.parametrize("type_", [44, 45])
def test_reference_backend_test_shapes(rq, port, type_):
    # every (rows, tokens, K) of the reference's test list, with its adversarial initialiser, tolerance 0
    for rows, tokens, K in ref_shape_list():
        w = inputs.reference_test_weights(rows, K)
        x = inputs.reference_test_activations(tokens, K, w, type_ == 44, 77)
        wb = port.quantize_weights(w, type_)
        want = port.mul_mat(wb, type_, K, x)
        assert_bits(gpu_mul_mat(rq, wb, type_, K, x), want, "rows=%d tokens=%d K=%d" % (rows, tokens, K))


# ------------------------------------------------------------------------------------------- configurations of the benchmark

def test_config1_w4a4_decode(rq, port):
    K, N = 4096, 1024
    wb = oracle.set_clip(port.quantize_weights(inputs.normal_weights(N, K, 1000), 44), 1.0)
    x = np.random.default_rng(1001).normal(0, 1, (1, K)).astype(np.float32)
    assert_bits(gpu_mul_mat(rq, wb, 44, K, x), port.mul_mat(wb, 44, K, x), "config 1")


@pytest.mark.parametrize("M", [1, 4, 16, 64])
def test_config2_w4a4h_sweep(rq, port, M):
    K = N = 5120
    wb = oracle.set_clip(port.quantize_weights(inputs.normal_weights(N, K, 2000), 45), 0.9)
    x = inputs.outlier_activations(M, K, 2001, 8, 40.0)
    want = port.mul_mat(wb, 45, K, x)
    assert_bits(gpu_mul_mat(rq, wb, 45, K, x), want, "config 2 M=%d auto" % M)
    assert_bits(gpu_mul_mat(rq, wb, 45, K, x, path=1), want, "config 2 M=%d gemv" % M)
    assert_bits(gpu_mul_mat(rq, wb, 45, K, x, path=2), want, "config 2 M=%d tcgen05" % M)


def test_config3_prefill_full_size_sampled(rq, port):
    # full K=5120 N=17408 M=4096 on the GPU; the oracle checks every output of a seeded sample of 192 tokens
    K, N, M = 5120, 17408, 4096
    wf = inputs.normal_weights(256, K, 3000)                 # 256 distinct rows, tiled
    wb = np.tile(port.quantize_weights(wf, 45), (N // 256, 1))
    x = inputs.student_t_activations(M, K, 3001, 16, 50.0)
    got = gpu_mul_mat(rq, wb, 45, K, x)
    pick = np.sort(np.random.default_rng(3002).choice(M, 192, replace=False))
    assert_bits(got[pick], port.mul_mat(wb, 45, K, x[pick]), "config 3 sample")
    # size-independent property: tiled weight rows give tiled outputs
    assert (inputs.bits(got).reshape(M, N // 256, 256) == inputs.bits(got)[:, None, :256]).all()


@pytest.mark.parametrize("M", [1, 2, 8, 32, 128, 512])
def test_config4_down_projection(rq, port, M):
    K, N = 17408, 5120
    wf = inputs.normal_weights(512, K, 4000)
    wb = np.tile(port.quantize_weights(wf, 45), (N // 512, 1))
    v = wb.reshape(N, -1, 144)
    clips = np.random.default_rng(4002).uniform(0.8, 1.0, N).astype(np.float32)
    for r in range(N):    # per-row clips in the headers: only block 0 of row 0 counts (ggml_rq_tensor_clip)
        v[r, :, 12:16] = np.frombuffer(clips[r].tobytes(), dtype=np.uint8)
    x = inputs.spiky_activations(M, K, 4001)
    want = port.mul_mat(wb, 45, K, x)
    assert_bits(gpu_mul_mat(rq, wb, 45, K, x), want, "config 4 M=%d" % M)
    if M == 8:
        assert_bits(gpu_mul_mat(rq, wb, 45, K, x, clip=float(clips[0])), want, "explicit clip == row 0's clip")


def test_config5_layer_shapes(rq, port):
    # one decoder layer's seven projections, M = 1 and M = 80 (reduced N keeps the oracle quick; K is full size)
    for name, K, N in [("q", 5120, 6144), ("k", 5120, 1024), ("v", 5120, 1024), ("o", 6144, 5120), ("gate", 5120, 17408),
                       ("up", 5120, 17408), ("down", 17408, 5120)]:
        wf = inputs.normal_weights(128, K, 5000 + N)
        wb = np.tile(port.quantize_weights(wf, 45), (N // 128, 1))
        for M in (1, 80):
            x = np.random.default_rng(5001 + M).normal(0, 1, (M, K)).astype(np.float32)
            assert_bits(gpu_mul_mat(rq, wb, 45, K, x), port.mul_mat(wb, 45, K, x), "%s M=%d" % (name, M))


# ------------------------------------------------------------------------------------------- properties and edges

def test_token_permutation_and_path_agreement(rq, port):
    K, N, M = 6144, 768, 48
    wb = port.quantize_weights(inputs.normal_weights(N, K, 60), 45)
    x = inputs.outlier_activations(M, K, 61)
    perm = np.random.default_rng(62).permutation(M)
    y = gpu_mul_mat(rq, wb, 45, K, x, path=2)
    assert_bits(gpu_mul_mat(rq, wb, 45, K, x[perm], path=2), y[perm], "token permutation")
    assert_bits(gpu_mul_mat(rq, wb, 45, K, x, path=1), y, "gemv == tcgen05")


def test_row_sharding_is_exact(rq, port):
    # weights sharded along N: each shard's output equals the matching columns of the unsharded result
    K, N, M = 5120, 1024, 5
    wb = port.quantize_weights(inputs.normal_weights(N, K, 70), 45)
    x = inputs.outlier_activations(M, K, 71)
    full = gpu_mul_mat(rq, wb, 45, K, x)
    for g in (2, 4, 8):
        for r in range(g):
            part = gpu_mul_mat(rq, wb[r * N // g:(r + 1) * N // g], 45, K, x)
            assert_bits(part, full[:, r * N // g:(r + 1) * N // g], "shard %d/%d" % (r, g))


def test_ragged_rows_strides_and_fused_weights(rq, port):
    K, M = 1536, 7
    x = inputs.outlier_activations(M, K, 81)
    xs = torch.zeros((M, K + 64), dtype=torch.float32, device="cuda")
    xs[:, :K] = dev(x)
    weights, wants = [], []
    for i, N in enumerate((8, 100, 260)):          # N not a multiple of the 256-row tile, nor of 4
        wb = port.quantize_weights(inputs.normal_weights(N, K, 90 + i), 45)
        weights.append(rq.Weight(dev(wb).view(-1), 45, K, N=N))
        wants.append(port.mul_mat(wb, 45, K, x))
    for path in (1, 2):
        outs = [torch.full((M, w.N + 3), -7.0, dtype=torch.float32, device="cuda") for w in weights]
        rq.mul_mat(weights, xs[:, :K], out=[o[:, :w.N] for o, w in zip(outs, weights)], path=path)
        torch.cuda.synchronize()
        for o, w, want in zip(outs, weights, wants):
            assert_bits(o[:, :w.N].cpu().numpy(), want, "fused N=%d path=%d" % (w.N, path))
            assert (o[:, w.N:] == -7.0).all(), "wrote past N"


@pytest.mark.parametrize("M", [1, 2, 9, 16])
def test_shared_activation_single_launch(rq, port, M):
    # q / k / v and gate / up read one activation: one rotate+quantize and one GEMV launch over all their row tiles
    for K, Ns in [(5120, (6144, 1024, 1024)), (5120, (2176, 2176))]:
        x = inputs.outlier_activations(M, K, 300 + M)
        wbs = [port.quantize_weights(inputs.normal_weights(N, K, 310 + i), 45) for i, N in enumerate(Ns)]
        weights = [rq.Weight(dev(wb).view(-1), 45, K, N=wb.shape[0], layouts=rq.PREPACK_DECODE) for wb in wbs]
        outs = rq.mul_mat(weights, dev(x))
        torch.cuda.synchronize()
        for o, wb in zip(outs, wbs):
            assert_bits(o.cpu().numpy(), port.mul_mat(wb, 45, K, x), "shared activation M=%d N=%d" % (M, wb.shape[0]))


def test_cuda_graph_capture_and_replay(rq, port):
    K, N, M = 5120, 512, 4
    wb = port.quantize_weights(inputs.normal_weights(N, K, 100), 45)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    x = torch.empty((M, K), dtype=torch.float32, device="cuda")
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    ws = rq.new_workspace(K, M)
    s = torch.cuda.Stream()
    graphs = {}
    for path in (1, 2):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                rq.mul_mat(w, x, out=y, workspace=ws, path=path, stream=s)
        graphs[path] = g
    for seed in (101, 102):
        xh = inputs.outlier_activations(M, K, seed)
        want = port.mul_mat(wb, 45, K, xh)
        for path, g in graphs.items():
            x.copy_(dev(xh))
            y.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert_bits(y.cpu().numpy(), want, "graph replay path=%d" % path)


def test_status_codes(rq, port):
    K, N = 1792, 16          # 7 * 256: W4A4H cannot rotate this width
    wb = port.quantize_weights(inputs.normal_weights(N, K, 110), 44)
    with pytest.raises(rq.RqError) as e:
        rq.Weight(dev(wb).view(-1), 45, K, N=N)
    assert e.value.status == -3
    w = rq.Weight(dev(wb).view(-1), 44, K, N=N)
    x = torch.zeros((2, K), dtype=torch.float32, device="cuda")
    with pytest.raises(rq.RqError) as e:
        rq.mul_mat(w, x, act_group=32)
    assert e.value.status == -4
    with pytest.raises(rq.RqError) as e:
        rq.mul_mat(w, x, clip=-1.0)
    assert e.value.status == -9
    with pytest.raises(rq.RqError) as e:
        rq.mul_mat(w, x, workspace=torch.empty(256, dtype=torch.uint8, device="cuda"))
    assert e.value.status == -5
    g = load("wg64")
    w64 = rq.Weight(dev(g["adv_w4a4_w"]).view(-1), 44, 512, N=40)
    assert w64.desc.wg64 == 1 and w64.desc.wk_mode == 1
    with pytest.raises(rq.RqError) as e:      # weight groups of 64 need activation groups of 64
        rq.mul_mat(w64, torch.zeros((1, 512), dtype=torch.float32, device="cuda"), act_group=128)
    assert e.value.status == -4


# ------------------------------------------------------------------------------------------- column (K) split

@pytest.mark.parametrize("world", [2, 4])
def test_column_split_partials_sum_in_rank_order(rq, port, world):
    """The reference's tensor-parallel mode for attn_output / ffn_down: every rank multiplies its block columns by its
    slice of x (quantized on its own) and the partials are added in rank order by rq_w4a4_sum_partials, in one shot (every
    rank adds everything) and in two (a rank adds its piece and stores it into every rank's output).  One GPU plays all
    ranks in turn; 5 x 97 outputs do not divide into whole vectors per rank, so the last piece's tail is covered."""
    from ruquant_b200 import shard
    K, N, M = 5120 * 2, 97, 5
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9300), 45, rot_blocks=world)    # rotation length K / world
    x = inputs.outlier_activations(M, K, 9301)
    ks = K // world
    parts, want = [], None
    for r in range(world):
        cols = np.ascontiguousarray(shard.col_shard(wb, N, K, r, world))
        xs = np.ascontiguousarray(x[:, r * ks:(r + 1) * ks])
        parts.append(dev(gpu_mul_mat(rq, cols, 45, ks, xs)))            # rank r's partial, "mapped" on every rank
        p_cpu = port.mul_mat(cols, 45, ks, xs)
        want = p_cpu if want is None else want + p_cpu
    ptrs = [p.data_ptr() for p in parts]
    for rank in range(world):                                            # one shot: every rank by itself
        y = torch.full((M, N), -1.0, dtype=torch.float32, device="cuda")
        rq.sum_partials(ptrs, rank, M * N, [y.data_ptr() if r == rank else 0 for r in range(world)])
        torch.cuda.synchronize()
        assert_bits(y.cpu().numpy(), want, "column split over %d, one shot, rank %d" % (world, rank))
    ys = [torch.full((M, N), -1.0, dtype=torch.float32, device="cuda") for _ in range(world)]
    for rank in range(world):                                            # two shots: each rank its piece into every output
        rq.sum_partials(ptrs, rank, M * N, [t.data_ptr() for t in ys], two_shot=True)
    torch.cuda.synchronize()
    for rank in range(world):
        assert_bits(ys[rank].cpu().numpy(), want, "column split over %d, two shots, rank %d" % (world, rank))


def test_column_split_needs_rotation_blocks(rq, port):
    from ruquant_b200 import shard
    K, N = 2048, 32
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9310), 45)         # rotated over the whole row
    cols = np.ascontiguousarray(shard.col_shard(wb, N, K, 0, 2))
    with pytest.raises(rq.RqError) as e:
        rq.Weight(dev(cols).view(-1), 45, K // 2, N=N)
    assert e.value.status == -3


# ------------------------------------------------------------------------------------------- push to several buffers

def test_push_writes_every_destination(rq, port):
    """rq_w4a4_mul_mat_push: the decode node storing its outputs into several buffers (other ranks' copies of Y); here all
    destinations live on one GPU.  Three weights sharing x, strided destinations, bits against the oracle."""
    K, M = 5120, 3
    Ns = [96, 32, 48]
    wbs = [port.quantize_weights(inputs.normal_weights(n, K, 9400 + i), 45) for i, n in enumerate(Ns)]
    ws = [rq.Weight(dev(wb).view(-1), 45, K, N=n, layouts=rq.PREPACK_DECODE) for wb, n in zip(wbs, Ns)]
    x = inputs.outlier_activations(M, K, 9410)
    total = sum(Ns)
    bufs = [torch.full((M, total + 8), -1.0, dtype=torch.float32, device="cuda") for _ in range(3)]
    cols = np.concatenate([[0], np.cumsum(Ns)[:-1]])
    dst = [[b.data_ptr() + 4 * int(c) for c in cols] for b in bufs]
    rq.mul_mat_push(ws, dev(x), dst, [total + 8] * 3)
    torch.cuda.synchronize()
    want = np.concatenate([port.mul_mat(wb, 45, K, x) for wb in wbs], axis=1)
    for b in bufs:
        got = b.cpu().numpy()
        assert_bits(got[:, :total], want, "push destination")
        assert (got[:, total:] == -1.0).all()


def test_rank_barrier_single_rank_and_expiry(rq):
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(3):                       # one rank: the kernel sees its own flag at once; the epoch counts up
        rq.rank_barrier([flags.data_ptr()], 0, epoch, status)
    torch.cuda.synchronize()
    assert int(epoch.item()) == 3 and int(flags[0].item()) == 3 and int(status.item()) == 0
    # two ranks, the other one never arrives: the bounded wait runs out, the status word says so, the context lives on
    other = torch.zeros(8, dtype=torch.int32, device="cuda")
    rq.rank_barrier([flags.data_ptr(), other.data_ptr()], 0, epoch, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 3 and int(other[0].item()) == 4
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0


def test_push_from_the_tcgen05_kernel(rq, port):
    """Above 64 tokens the push variant runs the tcgen05 kernel, whose final store writes every destination."""
    K, N, M = 1024, 320, 200
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9500), 45)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    x = inputs.outlier_activations(M, K, 9501)
    bufs = [torch.full((M, 2 * N), -1.0, dtype=torch.float32, device="cuda") for _ in range(2)]
    rq.mul_mat_push([w], dev(x), [[b.data_ptr() + 4 * N] for b in bufs], [2 * N])      # the right half of a wider Y
    torch.cuda.synchronize()
    want = port.mul_mat(wb, 45, K, x)
    for b in bufs:
        got = b.cpu().numpy()
        assert_bits(got[:, N:], want, "tcgen05 push")
        assert (got[:, :N] == -1.0).all()


def test_eight_rotation_blocks(rq, port):
    """RQ_ROT_BLOCKS = 8 (the widest split the reference's converter documents): K = 8 x 2560 is rotated in blocks of
    2560 = 20 x 128; weights from the GPU quantizer and from the oracle agree, and so do the products on every path."""
    K, N = 8 * 2560, 48
    wf = inputs.normal_weights(N, K, 9600)
    wb = port.quantize_weights(wf, 45, rot_blocks=8)
    got = rq.quantize_weights(dev(wf), 45, 0, 8)
    torch.cuda.synchronize()
    assert (got.cpu().numpy() == wb).all()
    for M, path in [(1, 1), (5, 1), (70, 2)]:
        x = inputs.outlier_activations(M, K, 9601 + M)
        assert_bits(gpu_mul_mat(rq, wb, 45, K, x, path=path), port.mul_mat(wb, 45, K, x), "rot8 M=%d" % M)


@pytest.mark.parametrize("M", [129, 257, 300])
def test_pairs_with_ragged_token_and_row_counts(rq, port, M):
    """CTA pairs (above 128 tokens) when the last pair's second CTA holds one token, none, or a partial tile, the weight
    rows do not fill their last 256-row tile, and y has a row stride that is not a multiple of 4 floats."""
    K, N = 1024, 300
    wb = port.quantize_weights(inputs.normal_weights(N, K, 9700), 45)
    w = rq.Weight(dev(wb).view(-1), 45, K, N=N)
    x = inputs.outlier_activations(M, K, 9700 + M)
    ybuf = torch.full((M, N + 3), -2.0, dtype=torch.float32, device="cuda")
    ws = rq.new_workspace(K, M)
    rq.mul_mat(w, dev(x), out=ybuf[:, :N], path=2, workspace=ws)
    torch.cuda.synchronize()
    rq.device_status(ws, K, M)
    got = ybuf.cpu().numpy()
    assert_bits(np.ascontiguousarray(got[:, :N]), port.mul_mat(wb, 45, K, x), "ragged pair M=%d" % M)
    assert (got[:, N:] == -2.0).all()
