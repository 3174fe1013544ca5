"""Seeded synthetic inputs for the parity tests and the benchmark-shaped cases.

`reference_test_*` restate the adversarial initialiser of the reference's own backend test for these types
(tests/test-backend-ops.cpp hunk in patches/llama.cpp-ruquant.patch:2956-2999): weights from std::mt19937(1234) /
uniform(-1, 1) with 64-wide groups scaled by 2^((i/64 + r) % 5 - 2) and every 7th row flat +-1; activations uniform
with 64-wide groups scaled by 2^((i/64) % 7 - 3 + r % 3 - 1) and, for W4A4, every 5th token carrying the signs of
weight row 0 (aligned flat rows whose un-shifted integer dot product passes 2^31 at K = 17408).
"""
import numpy as np


def _std_uniform_pm1(raw_u32):
    """libstdc++ uniform_real_distribution<float>(-1, 1) over successive mt19937 outputs."""
    r = raw_u32.astype(np.float32) / np.float32(4294967296.0)
    r = np.where(r >= np.float32(1.0), np.nextafter(np.float32(1.0), np.float32(0.0)), r).astype(np.float32)
    return (r * np.float32(2.0) + np.float32(-1.0)).astype(np.float32)


def reference_test_weights(rows, k):
    bg = np.random.MT19937()
    bg._legacy_seeding(1234)            # the seeding of std::mt19937(1234)
    v = _std_uniform_pm1(bg.random_raw(rows * k).astype(np.uint32)).reshape(rows, k)
    i = np.arange(k)[None, :]
    r = np.arange(rows)[:, None]
    scaled = v * np.exp2(((i // 64 + r) % 5 - 2).astype(np.float32))
    flat = np.where(v < 0, np.float32(-1.0), np.float32(1.0))
    return np.where(r % 7 == 0, flat, scaled).astype(np.float32)


def reference_test_activations(tokens, k, w_fp32, aligned, seed):
    rng = np.random.default_rng(seed)
    v = rng.uniform(-1.0, 1.0, (tokens, k)).astype(np.float32)
    i = np.arange(k)[None, :]
    r = np.arange(tokens)[:, None]
    out = v * np.exp2(((i // 64) % 7 - 3 + (r % 3 - 1)).astype(np.float32))
    if aligned:
        signs = np.where(w_fp32[0] < 0, np.float32(-1.0), np.float32(1.0))[None, :]
        out = np.where(r % 5 == 0, signs, out)
    return out.astype(np.float32)


def normal_weights(n, k, seed):
    return np.random.default_rng(seed).normal(0.0, 0.02, (n, k)).astype(np.float32)


def outlier_activations(m, k, seed, n_outliers=8, scale=40.0):
    """N(0, 1) with a fixed, seeded set of outlier channels scaled up."""
    rng = np.random.default_rng(seed)
    x = rng.normal(0.0, 1.0, (m, k)).astype(np.float32)
    ch = rng.choice(k, size=n_outliers, replace=False)
    x[:, ch] *= np.float32(scale)
    return x


def student_t_activations(m, k, seed, n_outliers=16, scale=50.0):
    rng = np.random.default_rng(seed)
    x = rng.standard_t(3.0, (m, k)).astype(np.float32)
    ch = rng.choice(k, size=n_outliers, replace=False)
    x[:, ch] *= np.float32(scale)
    return x


def spiky_activations(m, k, seed, frac=0.01, value=30.0):
    """N(0, 1) with a seeded 1% of the entries set to +-value."""
    rng = np.random.default_rng(seed)
    x = rng.normal(0.0, 1.0, (m, k)).astype(np.float32)
    mask = rng.random((m, k)) < frac
    sign = np.where(rng.random((m, k)) < 0.5, np.float32(-1.0), np.float32(1.0))
    return np.where(mask, sign * np.float32(value), x).astype(np.float32)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
