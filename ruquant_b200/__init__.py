"""ruquant_b200 -- B200 (sm_100a) W4A4 / W4A4H MUL_MAT behind ruquant's ggml operator surface.

The product is the C-ABI library `librq_b200.so` (declared in include/rq_b200.h, built in-tree by
`python -m ruquant_b200.build`).  This package is its Python host side: ctypes bindings plus thin helpers that use
torch only for device memory and streams.  There is no CPU or PyTorch fallback: importing the bindings without the
built library raises, and every compute call goes through the library's CUDA kernels.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("RQ_B200_LIB") or os.path.join(HERE, "librq_b200.so")

TYPE_W4A4, TYPE_W4A4H = 44, 45
BLOCK_CODES, BLOCK_BYTES = 256, 144
PREPACK_DECODE, PREPACK_PREFILL, PREPACK_ALL = 1, 2, 3
PATH_AUTO, PATH_GEMV, PATH_TC = 0, 1, 2
FMT_I8, FMT_E4M3 = 0, 1

EXPORTS = [
    "rq_w4a4_supported", "rq_hadamard_factor", "rq_w4a4_resolve_clip", "rq_w4a4_act_group", "rq_w4a4_prepack_bytes",
    "rq_w4a4_prepare", "rq_w4a4_workspace_bytes", "rq_w4a4_mul_mat", "rq_w4a4_mul_mat_quantized", "rq_w4a4_rotate",
    "rq_w4a4_quantize", "rq_w4a4_workspace_layout", "rq_w4a4_device_status", "rq_status_string", "rq_last_cuda_error",
    "rq_w4a4_mul_mat_static", "rq_w4a4_mul_mat_quantized_n", "rq_w4a4_act_format",
    "rq_w4a4_quantize_weights", "rq_w4a4_quantize_weights_scratch_bytes", "rq_w4a4_mul_mat_push", "rq_rank_barrier",
    "rq_w4a4_workspace_init", "rq_w4a4_tc_nofold_probe", "rq_w4a4_sum_partials", "rq_w4a4_quantize_rows",
    "rq_w4a4_share_rows",
]


class RqError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__("%s: %s (status %d)" % (what, lib().rq_status_string(status).decode(), status))


class WeightDesc(ctypes.Structure):
    """rq_weight_desc of include/rq_b200.h."""
    _fields_ = [
        ("type", ctypes.c_int32), ("layouts", ctypes.c_int32), ("K", ctypes.c_int64), ("N", ctypes.c_int64),
        ("n_rot", ctypes.c_int32), ("had_p", ctypes.c_int32), ("had_m", ctypes.c_int32), ("wk_mode", ctypes.c_int32),
        ("wg64", ctypes.c_int32), ("header_clip", ctypes.c_float), ("blocks", ctypes.c_void_p), ("prepack", ctypes.c_void_p),
        ("off_sw", ctypes.c_uint64), ("off_w4", ctypes.c_uint64), ("off_w8", ctypes.c_uint64), ("off_wk", ctypes.c_uint64),
        ("tmap_w8", ctypes.c_uint64 * 16),
    ]


_lib = None


def lib():
    """The loaded C-ABI library.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("librq_b200.so is not built (run `python -m ruquant_b200.build`); "
                              "ruquant_b200 has no CPU or PyTorch fallback")
        L = ctypes.CDLL(LIB_PATH)
        i64, i32, vp, f32, sz = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_size_t
        pd = ctypes.POINTER(WeightDesc)
        L.rq_w4a4_supported.argtypes = [i32, i64, i64, i64, i64]
        L.rq_hadamard_factor.argtypes = [i64, ctypes.POINTER(i32), ctypes.POINTER(i32)]
        L.rq_w4a4_resolve_clip.argtypes = [pd]
        L.rq_w4a4_resolve_clip.restype = f32
        L.rq_w4a4_act_group.argtypes = []
        L.rq_w4a4_prepack_bytes.argtypes = [i32, i64, i64, i32]
        L.rq_w4a4_prepack_bytes.restype = sz
        L.rq_w4a4_prepare.argtypes = [vp, i32, i64, i64, vp, sz, i32, pd, vp]
        L.rq_w4a4_workspace_bytes.argtypes = [i64, i64]
        L.rq_w4a4_workspace_bytes.restype = sz
        L.rq_w4a4_mul_mat.argtypes = [ctypes.POINTER(pd), i32, vp, i64, i64, ctypes.POINTER(vp), ctypes.POINTER(i64), f32, i32,
                                      i32, vp, sz, vp]
        L.rq_w4a4_mul_mat_static.argtypes = [pd, vp, i64, i64, vp, i64, f32, i32, i32, vp]
        L.rq_w4a4_mul_mat_quantized_n.argtypes = [ctypes.POINTER(pd), i32, i64, ctypes.POINTER(vp), ctypes.POINTER(i64), i32, i32,
                                                  vp, sz, vp]
        L.rq_w4a4_mul_mat_quantized.argtypes = [pd, i64, vp, i64, i32, i32, vp, sz, vp]
        L.rq_w4a4_rotate.argtypes = [vp, i64, i64, i64, i64, vp, i64, vp]
        L.rq_w4a4_quantize.argtypes = [vp, i64, i64, i64, i64, f32, i32, i32, vp, sz, vp]
        L.rq_w4a4_act_format.argtypes = [ctypes.POINTER(pd), i32, i64, i32]
        L.rq_w4a4_quantize_rows.argtypes = [vp, i64, i64, i64, i64, i64, i64, f32, i32, i32, vp, sz, vp]
        L.rq_w4a4_share_rows.argtypes = [vp, i32, i32, sz, i64, i64, i32, i64, i64, vp]
        L.rq_w4a4_mul_mat_push.argtypes = [ctypes.POINTER(pd), i32, vp, i64, i64, ctypes.POINTER(vp), i32, ctypes.POINTER(i64), f32,
                                           i32, vp, sz, vp]
        L.rq_rank_barrier.argtypes = [ctypes.POINTER(vp), i32, i32, vp, vp, vp]
        L.rq_w4a4_quantize_weights_scratch_bytes.argtypes = [i32, i64, i64, i32]
        L.rq_w4a4_quantize_weights_scratch_bytes.restype = sz
        L.rq_w4a4_quantize_weights.argtypes = [vp, i64, i32, i64, i64, i32, i32, vp, vp, sz, vp]
        u64p = ctypes.POINTER(ctypes.c_uint64)
        L.rq_w4a4_workspace_layout.argtypes = [i64, i64, i32, u64p, u64p, u64p, u64p]
        L.rq_w4a4_device_status.argtypes = [vp, i64, i64, vp]
        L.rq_w4a4_workspace_init.argtypes = [vp, i64, i64, vp]
        L.rq_w4a4_sum_partials.argtypes = [ctypes.POINTER(vp), i32, i32, i64, ctypes.POINTER(vp), i32, vp]
        L.rq_w4a4_tc_nofold_probe.argtypes = [pd, i64, vp, i64, vp, sz, vp]
        L.rq_status_string.argtypes = [i32]
        L.rq_status_string.restype = ctypes.c_char_p
        L.rq_last_cuda_error.argtypes = []
        _lib = L
    return _lib


def _check(status, what):
    if status != 0:
        raise RqError(status, what)


def hadamard_factor(n):
    p, m = ctypes.c_int(0), ctypes.c_int(0)
    return (p.value, m.value) if lib().rq_hadamard_factor(n, ctypes.byref(p), ctypes.byref(m)) else None


def supported(type_, K, N, M, ldx_bytes=None):
    return bool(lib().rq_w4a4_supported(type_, K, N, M, ldx_bytes if ldx_bytes is not None else 4 * K))


def _stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


class Weight:
    """A W4A4 / W4A4H weight prepared for the kernels.

    blocks: torch.uint8 CUDA tensor holding N rows of K/256 144-byte blocks (the ggml tensor's data).  It is only
    read; the kernel-side layouts live in a separate prepack tensor owned by this object."""

    def __init__(self, blocks, type_, K, N=None, layouts=PREPACK_ALL, stream=None):
        import torch
        if not blocks.is_cuda or blocks.dtype != torch.uint8 or not blocks.is_contiguous():
            raise ValueError("blocks must be a contiguous uint8 CUDA tensor")
        row_bytes = K // BLOCK_CODES * BLOCK_BYTES
        if N is None:
            N = blocks.numel() // row_bytes
        if blocks.numel() != N * row_bytes:
            raise ValueError("blocks has %d bytes, expected %d" % (blocks.numel(), N * row_bytes))
        self.blocks, self.type, self.K, self.N = blocks, type_, K, N
        nbytes = lib().rq_w4a4_prepack_bytes(type_, K, N, layouts)
        if nbytes == 0:
            raise RqError(-2, "rq_w4a4_prepack_bytes")
        self.prepack = torch.empty(nbytes, dtype=torch.uint8, device=blocks.device)
        self.desc = WeightDesc()
        with torch.cuda.device(blocks.device):
            _check(lib().rq_w4a4_prepare(blocks.data_ptr(), type_, K, N, self.prepack.data_ptr(), nbytes, layouts,
                                         ctypes.byref(self.desc), _stream_ptr(stream)), "rq_w4a4_prepare")

    @property
    def n_rot(self):
        return self.desc.n_rot

    def clip(self):
        """The activation clip the reference would use: environment, else header, else 1."""
        return lib().rq_w4a4_resolve_clip(ctypes.byref(self.desc))


def workspace_bytes(K, M):
    return lib().rq_w4a4_workspace_bytes(K, M)


def init_workspace(ws, K, M):
    """Zero the status block of a workspace the caller allocated (uint8 CUDA tensor of workspace_bytes(K, M), e.g. in
    memory mapped into other ranks); waits for the zeroing, so that the workspace may be used on any stream afterwards."""
    import torch
    with torch.cuda.device(ws.device):
        _check(lib().rq_w4a4_workspace_init(ws.data_ptr(), K, M, _stream_ptr()), "rq_w4a4_workspace_init")
        torch.cuda.current_stream().synchronize()
    return ws


def new_workspace(K, M, device="cuda"):
    """A workspace for M tokens of width K with its status block zeroed (the error word in it is sticky).  Waits for
    the zeroing to finish, so that the workspace may be used on any stream afterwards."""
    import torch
    return init_workspace(torch.empty(workspace_bytes(K, M), dtype=torch.uint8, device=device), K, M)


def workspace_views(ws, K, M, group):
    """(a8 int8 [M, K], msh int32 [M, K/group], u f32 [M]) views into a workspace tensor."""
    import torch
    o = [ctypes.c_uint64(0) for _ in range(4)]
    _check(lib().rq_w4a4_workspace_layout(K, M, group, *[ctypes.byref(v) for v in o]), "rq_w4a4_workspace_layout")
    a8 = ws[o[0].value:o[0].value + M * K].view(torch.int8).view(M, K)
    ng = K // group
    msh = ws[o[1].value:o[1].value + M * ng * 4].view(torch.int32).view(M, ng)
    u = ws[o[2].value:o[2].value + M * 4].view(torch.float32)
    return a8, msh, u


def mul_mat(weights, x, out=None, clip=None, act_group=None, path=PATH_AUTO, workspace=None, stream=None):
    """The MUL_MAT node: y[i] = x @ W[i]^T for 1..3 prepared weights sharing the f32 activation x [M, K].
    Returns one tensor [M, N] (single weight) or a list.  Only enqueues on the stream."""
    import torch
    single = isinstance(weights, Weight)
    ws_list = [weights] if single else list(weights)
    if x.dtype != torch.float32 or not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a 2-D f32 CUDA tensor with unit inner stride")
    M, K = x.shape
    n_w = len(ws_list)
    if out is None:
        outs = [torch.empty((M, w.N), dtype=torch.float32, device=x.device) for w in ws_list]
    else:
        outs = [out] if single else list(out)
    if clip is None:
        clip = ws_list[0].clip()
    if act_group is None:
        act_group = lib().rq_w4a4_act_group()
    if workspace is None:
        workspace = new_workspace(K, M, x.device)
    pd = ctypes.POINTER(WeightDesc)
    descs = (pd * n_w)(*[ctypes.pointer(w.desc) for w in ws_list])
    ys = (ctypes.c_void_p * n_w)(*[o.data_ptr() for o in outs])
    ldy = (ctypes.c_int64 * n_w)(*[o.stride(0) for o in outs])
    with torch.cuda.device(x.device):
        _check(lib().rq_w4a4_mul_mat(descs, n_w, x.data_ptr(), x.stride(0), M, ys, ldy, clip, act_group, path,
                                     workspace.data_ptr(), workspace.numel(), _stream_ptr(stream)), "rq_w4a4_mul_mat")
    return outs[0] if single else outs


def _mul_mat_push_quantized(ws_list, M, dst_ptrs, ldy, act_group, workspace, stream):
    import torch
    n_w, n_dst = len(ws_list), len(dst_ptrs)
    if act_group is None:
        act_group = lib().rq_w4a4_act_group()
    with torch.cuda.device(workspace.device):
        pd = ctypes.POINTER(WeightDesc)
        descs = (pd * n_w)(*[ctypes.pointer(w.desc) for w in ws_list])
        ys = (ctypes.c_void_p * (n_w * n_dst))(*[dst_ptrs[d][i] for d in range(n_dst) for i in range(n_w)])
        lds = (ctypes.c_int64 * n_w)(*ldy)
        _check(lib().rq_w4a4_mul_mat_push(descs, n_w, None, 0, M, ys, n_dst, lds, 1.0, act_group, workspace.data_ptr(),
                                          workspace.numel(), _stream_ptr(stream)), "rq_w4a4_mul_mat_push")
    return workspace


def quantize_rows(x_rows, M_total, first, n_rot, clip, group, fmt, workspace, stream=None):
    """Rotate and quantize the tokens x_rows [count, K] into rows first .. first+count of a workspace laid out for M_total."""
    import torch
    count, K = x_rows.shape
    with torch.cuda.device(x_rows.device):
        _check(lib().rq_w4a4_quantize_rows(x_rows.data_ptr(), x_rows.stride(0), M_total, first, count, K, n_rot, clip, group, fmt,
                                           workspace.data_ptr(), workspace.numel(), _stream_ptr(stream)), "rq_w4a4_quantize_rows")


def mul_mat_push(weights, x, dst_ptrs, ldy, clip=None, act_group=None, workspace=None, stream=None, M=None):
    """The decode-path node writing every output into several buffers: dst_ptrs[d][i] is the device address of weight
    i's output in destination d (this rank's own buffer first, then the peer-mapped buffers of the other ranks)."""
    import torch
    ws_list = [weights] if isinstance(weights, Weight) else list(weights)
    n_w, n_dst = len(ws_list), len(dst_ptrs)
    if x is None:        # the workspace already holds the quantized activation of M tokens
        return _mul_mat_push_quantized(ws_list, M, dst_ptrs, ldy, act_group, workspace, stream)
    K, M = ws_list[0].K, x.shape[0]
    if clip is None:
        clip = ws_list[0].clip()
    if act_group is None:
        act_group = lib().rq_w4a4_act_group()
    with torch.cuda.device(x.device):
        if workspace is None:
            workspace = new_workspace(K, M, x.device)
        pd = ctypes.POINTER(WeightDesc)
        descs = (pd * n_w)(*[ctypes.pointer(w.desc) for w in ws_list])
        ys = (ctypes.c_void_p * (n_w * n_dst))(*[dst_ptrs[d][i] for d in range(n_dst) for i in range(n_w)])
        lds = (ctypes.c_int64 * n_w)(*ldy)
        _check(lib().rq_w4a4_mul_mat_push(descs, n_w, x.data_ptr(), x.stride(0), M, ys, n_dst, lds, clip, act_group,
                                          workspace.data_ptr(), workspace.numel(), _stream_ptr(stream)), "rq_w4a4_mul_mat_push")
    return workspace


def rank_barrier(flag_ptrs, rank, epoch, status=None, stream=None):
    """flag_ptrs[p]: device address (as mapped on this rank) of rank p's flag array; epoch: a zero-initialised uint32
    tensor on this device; status: an int32 tensor that becomes 3 if the bounded wait expires."""
    n = len(flag_ptrs)
    arr = (ctypes.c_void_p * n)(*flag_ptrs)
    _check(lib().rq_rank_barrier(arr, rank, n, epoch.data_ptr(), status.data_ptr() if status is not None else None,
                                 _stream_ptr(stream)), "rq_rank_barrier")


def share_rows(workspace_ptrs, rank, workspace_bytes_, K, M_total, group, first, count, stream=None):
    """Ranks that share the quantizer: rows first .. first+count of this rank's workspace (codes, multipliers, units) into
    the same rows of every other rank's.  workspace_ptrs[r]: rank r's workspace as mapped on this device."""
    n = len(workspace_ptrs)
    arr = (ctypes.c_void_p * n)(*workspace_ptrs)
    _check(lib().rq_w4a4_share_rows(arr, rank, n, workspace_bytes_, K, M_total, group, first, count, _stream_ptr(stream)),
           "rq_w4a4_share_rows")


def sum_partials(partial_ptrs, rank, count, y_ptrs, two_shot=False, stream=None):
    """K-split ranks: the rank-ordered sum of the ranks' partial outputs.  partial_ptrs[r] / y_ptrs[r]: device addresses,
    as mapped on this rank, of rank r's partial and output (one shot needs only y_ptrs[rank])."""
    n = len(partial_ptrs)
    parts = (ctypes.c_void_p * n)(*partial_ptrs)
    ys = (ctypes.c_void_p * n)(*[p if p else None for p in y_ptrs])
    _check(lib().rq_w4a4_sum_partials(parts, rank, n, count, ys, 1 if two_shot else 0, _stream_ptr(stream)), "rq_w4a4_sum_partials")


def mul_mat_static(weight, x, out=None, clip=None, act_group=None, path=PATH_AUTO, stream=None):
    """MUL_MAT without a caller workspace and without any allocation by the library: the scratch is a fixed array
    inside librq_b200.so (one weight, at most 16 tokens).  For hosts that cannot allocate device memory; calls on one
    device share the array, so do not let two of them overlap on the GPU."""
    import torch
    M, K = x.shape
    if out is None:
        out = torch.empty((M, weight.N), dtype=torch.float32, device=x.device)
    if clip is None:
        clip = weight.clip()
    if act_group is None:
        act_group = lib().rq_w4a4_act_group()
    with torch.cuda.device(x.device):
        _check(lib().rq_w4a4_mul_mat_static(ctypes.byref(weight.desc), x.data_ptr(), x.stride(0), M, out.data_ptr(),
                                            out.stride(0), clip, act_group, path, _stream_ptr(stream)), "rq_w4a4_mul_mat_static")
    return out


def rotate(x, n_rot, stream=None):
    """Rows of x (f32 CUDA [M, K]) times diag(H, H, ...), H of length n_rot: the online Hadamard alone."""
    import torch
    M, K = x.shape
    out = torch.empty((M, K), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib().rq_w4a4_rotate(x.data_ptr(), x.stride(0), M, K, n_rot, out.data_ptr(), out.stride(0),
                                    _stream_ptr(stream)), "rq_w4a4_rotate")
    return out


def act_format(weights, M, path=PATH_AUTO):
    """The activation format (FMT_*) the contraction of these weights at M tokens consumes."""
    ws_list = [weights] if isinstance(weights, Weight) else list(weights)
    pd = ctypes.POINTER(WeightDesc)
    descs = (pd * len(ws_list))(*[ctypes.pointer(w.desc) for w in ws_list])
    fmt = lib().rq_w4a4_act_format(descs, len(ws_list), M, path)
    _check(min(fmt, 0), "rq_w4a4_act_format")
    return fmt


def quantize_weights(w, type_, wgroup=0, rot_blocks=1, stream=None):
    """Rows of fp32 weights (CUDA, [N, K]) -> the reference's blocks as a uint8 tensor [N, K/256*144]."""
    import torch
    if not w.is_cuda or w.dtype != torch.float32 or w.dim() != 2 or w.stride(1) != 1:
        raise ValueError("w must be a 2-D float32 CUDA tensor with unit inner stride")
    N, K = w.shape
    nbytes = lib().rq_w4a4_quantize_weights_scratch_bytes(type_, K, N, wgroup)
    if nbytes == 0:
        raise RqError(-2, "rq_w4a4_quantize_weights_scratch_bytes")
    with torch.cuda.device(w.device):
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
        out = torch.empty((N, K // BLOCK_CODES * BLOCK_BYTES), dtype=torch.uint8, device=w.device)
        _check(lib().rq_w4a4_quantize_weights(w.data_ptr(), w.stride(0), type_, K, N, wgroup, rot_blocks, out.data_ptr(),
                                              scratch.data_ptr(), nbytes, _stream_ptr(stream)), "rq_w4a4_quantize_weights")
    return out


def quantize(x, n_rot, clip, group=64, workspace=None, stream=None, fmt=FMT_I8):
    """Rotate (n_rot > 0) and quantize; returns (workspace, a8, msh, u) (the views decode the FMT_I8 layout)."""
    M, K = x.shape
    if workspace is None:
        workspace = new_workspace(K, M, x.device)
    import torch
    with torch.cuda.device(x.device):
        _check(lib().rq_w4a4_quantize(x.data_ptr(), x.stride(0), M, K, n_rot, clip, group, fmt, workspace.data_ptr(),
                                      workspace.numel(), _stream_ptr(stream)), "rq_w4a4_quantize")
    return (workspace,) + workspace_views(workspace, K, M, group)


def mul_mat_quantized(weight, M, workspace, out=None, act_group=64, path=PATH_AUTO, stream=None):
    """The contraction stage alone, on an activation already quantized into `workspace` (a Weight, or a list of up to
    three sharing that activation, which at decode widths become one launch)."""
    import torch
    if not isinstance(weight, Weight):
        ws_list = list(weight)
        outs = list(out) if out is not None else [torch.empty((M, w.N), dtype=torch.float32, device=workspace.device)
                                                  for w in ws_list]
        n_w = len(ws_list)
        pd = ctypes.POINTER(WeightDesc)
        descs = (pd * n_w)(*[ctypes.pointer(w.desc) for w in ws_list])
        ys = (ctypes.c_void_p * n_w)(*[o.data_ptr() for o in outs])
        ldy = (ctypes.c_int64 * n_w)(*[o.stride(0) for o in outs])
        with torch.cuda.device(workspace.device):
            _check(lib().rq_w4a4_mul_mat_quantized_n(descs, n_w, M, ys, ldy, act_group, path, workspace.data_ptr(),
                                                     workspace.numel(), _stream_ptr(stream)), "rq_w4a4_mul_mat_quantized_n")
        return outs
    if out is None:
        out = torch.empty((M, weight.N), dtype=torch.float32, device=workspace.device)
    with torch.cuda.device(workspace.device):
        _check(lib().rq_w4a4_mul_mat_quantized(ctypes.byref(weight.desc), M, out.data_ptr(), out.stride(0), act_group, path,
                                               workspace.data_ptr(), workspace.numel(), _stream_ptr(stream)),
               "rq_w4a4_mul_mat_quantized")
    return out


def tc_nofold_probe(weight, M, workspace, out, stream=None):
    """Measurement aid: the tcgen05 kernel with all of K in one accumulator (no per-group fold); `out` gets no MUL_MAT."""
    import torch
    with torch.cuda.device(workspace.device):
        _check(lib().rq_w4a4_tc_nofold_probe(ctypes.byref(weight.desc), M, out.data_ptr(), out.stride(0), workspace.data_ptr(),
                                             workspace.numel(), _stream_ptr(stream)), "rq_w4a4_tc_nofold_probe")
    return out


def device_status(workspace, K, M, stream=None):
    """Synchronises and raises if a kernel of any earlier call on this workspace gave up on a bounded wait or met an
    activation in the wrong format (the report is sticky until read)."""
    _check(lib().rq_w4a4_device_status(workspace.data_ptr(), K, M, _stream_ptr(stream)), "rq_w4a4_device_status")
