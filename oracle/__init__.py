"""CPU checker for the W4A4 / W4A4H MUL_MAT path.  TEST INFRASTRUCTURE ONLY.

`rq_oracle.c` restates the reference's CPU arithmetic; `build_ref.py` compiles the reference's own lines into
`_ref/libruquant_ref.so` when the reference tree is present.  Only the tests, the smoke check and the benchmark's
CPU-baseline leg may import this package; the product (`ruquant_b200`) never does.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "librq_oracle.so")
PORT_SRC = os.path.join(HERE, "rq_oracle.c")
REF_SO = os.path.join(HERE, "_ref", "libruquant_ref.so")

TYPE_W4A4, TYPE_W4A4H = 44, 45
BLOCK_BYTES, QK = 144, 256

_c_f32p = ctypes.POINTER(ctypes.c_float)


def build(force=False):
    """Compiles rq_oracle.c (gcc, a second or two).  Rebuilt when the source is newer than the library."""
    if not force and os.path.exists(PORT_SO) and (not os.path.exists(PORT_SRC) or
                                                  os.path.getmtime(PORT_SO) >= os.path.getmtime(PORT_SRC)):
        return PORT_SO
    cmd = ["gcc", "-O3", "-std=gnu11", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", PORT_SRC, "-o", PORT_SO, "-lm"]
    subprocess.check_call(cmd)
    return PORT_SO


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


class Port:
    """ctypes face of librq_oracle.so (our restatement)."""

    def __init__(self):
        self.lib = ctypes.CDLL(build())
        L = self.lib
        L.rqo_hadamard_factor.argtypes = [ctypes.c_int64, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        L.rqo_hadamard.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        L.rqo_rotate_row.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        L.rqo_paley.argtypes = [ctypes.c_int, ctypes.c_void_p]
        L.rqo_quantize_weights.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.rqo_quantize_act.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int,
                                       ctypes.c_int64]
        L.rqo_vec_dot.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        L.rqo_vec_dot.restype = ctypes.c_float
        L.rqo_resolve_clip.argtypes = [ctypes.c_void_p, ctypes.c_float]
        L.rqo_resolve_clip.restype = ctypes.c_float
        L.rqo_resolve_rot.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        L.rqo_resolve_rot.restype = ctypes.c_int64
        L.rqo_mul_mat.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                  ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_float,
                                  ctypes.c_int, ctypes.c_int]

    def hadamard_factor(self, n):
        p, m = ctypes.c_int(0), ctypes.c_int(0)
        ok = self.lib.rqo_hadamard_factor(n, ctypes.byref(p), ctypes.byref(m))
        return (p.value, m.value) if ok else None

    def paley(self, p):
        A = np.zeros((p, p), dtype=np.int8)
        self.lib.rqo_paley(p, _ptr(A))
        return A

    def rotate(self, x, n_rot):
        """Rows of fp32 [M, K] rotated by blocks of n_rot; returns a new array."""
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        y2 = y.reshape(-1, y.shape[-1])
        for r in range(y2.shape[0]):
            if self.lib.rqo_rotate_row(_ptr(y2[r]), y2.shape[1], n_rot):
                raise ValueError("unfactorable rotation length %d" % n_rot)
        return y

    def quantize_weights(self, w, type_, wgroup=0, rot_blocks=1, threads=None):
        w = np.ascontiguousarray(w, dtype=np.float32)
        n, k = w.shape
        out = np.zeros((n, k // QK * BLOCK_BYTES), dtype=np.uint8)
        rc = self.lib.rqo_quantize_weights(_ptr(w), _ptr(out), n, k, int(type_ == TYPE_W4A4H), wgroup, rot_blocks,
                                           threads or os.cpu_count())
        if rc:
            raise ValueError("cannot quantize rows of %d" % k)
        return out

    def quantize_act(self, x, clip, group=64, n_rot=0):
        """[M, K] fp32 -> [M, K/256*144] uint8 activation blocks (the reference's A4 / A4H scratch layout)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        m, k = x.shape
        out = np.zeros((m, k // QK * BLOCK_BYTES), dtype=np.uint8)
        for t in range(m):
            if self.lib.rqo_quantize_act(_ptr(x[t]), _ptr(out[t]), k, clip, group, n_rot):
                raise ValueError("bad activation shape")
        return out

    def vec_dot(self, k, w_row, a_row):
        return self.lib.rqo_vec_dot(k, _ptr(w_row), _ptr(a_row))

    def mul_mat(self, w_blocks, type_, K, x, clip_override=0.0, group=64, threads=None):
        """w_blocks uint8 [N, K/256*144]; x fp32 [M, K] -> fp32 [M, N]."""
        w_blocks = np.ascontiguousarray(w_blocks)
        x = np.ascontiguousarray(x, dtype=np.float32)
        n, m = w_blocks.shape[0], x.shape[0]
        y = np.empty((m, n), dtype=np.float32)
        rc = self.lib.rqo_mul_mat(_ptr(w_blocks), type_, K, n, _ptr(x), x.shape[1], m, _ptr(y), n, clip_override, group,
                                  threads or os.cpu_count())
        if rc:
            raise ValueError("oracle rejected the shape")
        return y


class Ref:
    """ctypes face of _ref/libruquant_ref.so: the reference's own compiled lines.  Environment switches
    (RQ_ACT_GROUP, RQ_WGROUP, RQ_ROT_BLOCKS, RQ_ACT_CLIP[_H]) are read once per process by that code."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = ctypes.CDLL(REF_SO)
        L = self.lib
        L.rq_ref_mul_mat.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                     ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        L.rq_ref_quantize_act.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int64]
        L.rq_ref_quantize_weights.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
        L.rq_ref_quantize_weights.restype = ctypes.c_size_t
        L.rq_ref_vec_dot.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        L.rq_ref_vec_dot.restype = ctypes.c_float
        L.ggml_rq_hadamard.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_bool]
        L.ggml_rq_hadamard_factor.argtypes = [ctypes.c_int64, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        L.ggml_rq_hadamard_factor.restype = ctypes.c_bool

    def hadamard_factor(self, n):
        p, m = ctypes.c_int(0), ctypes.c_int(0)
        ok = self.lib.ggml_rq_hadamard_factor(n, ctypes.byref(p), ctypes.byref(m))
        return (p.value, m.value) if ok else None

    def rotate(self, x, n_rot):
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        y2 = y.reshape(-1, y.shape[-1])
        for r in range(y2.shape[0]):
            for o in range(0, y2.shape[1], n_rot):
                self.lib.ggml_rq_hadamard(_ptr(y2[r, o:]), n_rot, False)
        return y

    def quantize_weights(self, w, type_):
        w = np.ascontiguousarray(w, dtype=np.float32)
        n, k = w.shape
        out = np.zeros((n, k // QK * BLOCK_BYTES), dtype=np.uint8)
        self.lib.rq_ref_quantize_weights(_ptr(w), _ptr(out), n, k, type_)
        return out

    def quantize_act(self, x, clip, n_rot=0):
        x = np.ascontiguousarray(x, dtype=np.float32)
        m, k = x.shape
        out = np.zeros((m, k // QK * BLOCK_BYTES), dtype=np.uint8)
        for t in range(m):
            self.lib.rq_ref_quantize_act(_ptr(x[t]), _ptr(out[t]), k, clip, n_rot)
        return out

    def vec_dot(self, k, w_row, a_row):
        return self.lib.rq_ref_vec_dot(k, _ptr(w_row), _ptr(a_row))

    def mul_mat(self, w_blocks, type_, K, x, threads=None):
        w_blocks = np.ascontiguousarray(w_blocks)
        x = np.ascontiguousarray(x, dtype=np.float32)
        n, m = w_blocks.shape[0], x.shape[0]
        y = np.empty((m, n), dtype=np.float32)
        rc = self.lib.rq_ref_mul_mat(_ptr(w_blocks), type_, K, n, _ptr(x), x.shape[1], m, _ptr(y), n,
                                     threads or os.cpu_count())
        if rc:
            raise RuntimeError("reference mul_mat failed")
        return y


def have_ref():
    return os.path.exists(REF_SO)


# ---- helpers over the 144-byte block layout (header: d, sum, pad[0], pad[1]; then 32 code words) ----

def set_clip(w_blocks, clip):
    """Writes the activation clip (fp32 bits) into pad[1] of every block, as `ruquant setclip` does."""
    v = w_blocks.reshape(w_blocks.shape[0], -1, BLOCK_BYTES)
    v[:, :, 12:16] = np.frombuffer(np.float32(clip).tobytes(), dtype=np.uint8)
    return w_blocks


def act_fields(a_blocks, group=64):
    """Decodes activation blocks [M, nb*144] into (u[M], m[M, K/G], z[M, K/G], q[M, K] in 0..15)."""
    M = a_blocks.shape[0]
    v = a_blocks.reshape(M, -1, BLOCK_BYTES)
    nb = v.shape[1]
    u = v[:, 0, 0:4].copy().view(np.float32).reshape(M)
    summ = v[:, :, 4:8].copy().view(np.int32).reshape(M, nb)
    pad0 = v[:, :, 8:12].copy().view(np.uint32).reshape(M, nb)
    S = QK // group
    z = np.stack([(summ >> (4 * s)) & 0xF for s in range(S)], axis=-1).reshape(M, nb * S)
    m = np.stack([(pad0 >> (8 * s)) & 0xFF for s in range(S)], axis=-1).reshape(M, nb * S).astype(np.int32)
    words = v[:, :, 16:].copy().view(np.uint32).reshape(M, nb, 32)
    nib = np.stack([(words >> (4 * j)) & 0xF for j in range(8)], axis=-1).reshape(M, nb * QK).astype(np.int32)
    code = np.where(nib >= 8, nib - 16, nib)
    return u, m, z.astype(np.int32), code + 8
