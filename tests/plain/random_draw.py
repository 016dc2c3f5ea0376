"""The seeded random weights restated in numpy, from the definition in the header comment of
leone_b200/csrc/random_draw.h (this engine's own generator: the reference has no random-weight
mode, crates/leone/tests/common/cpu_fixture.rs:67-106).  Shares no code with the product path:
numpy's float64 +, -, *, / and sqrt round once to nearest, as the definition asks."""
import hashlib

import numpy as np

MASK52 = np.uint64((1 << 52) - 1)


def tensor_key(seed, name):
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def mix(z):
    z = z ^ (z >> np.uint64(30))
    z = z * np.uint64(0xbf58476d1ce4e5b9)
    z = z ^ (z >> np.uint64(27))
    z = z * np.uint64(0x94d049bb133111eb)
    return z ^ (z >> np.uint64(31))


def bits(key, n):
    with np.errstate(over="ignore"):
        return mix(np.uint64(key) + (n.astype(np.uint64) + np.uint64(1)) * np.uint64(0x9e3779b97f4a7c15))


def horner(w, coefficients):
    p = np.full_like(w, coefficients[0])
    for c in coefficients[1:]:
        p = p * w + c
    return p


def ln(u):
    b = u.view(np.uint64)
    e = ((b >> np.uint64(52)) & np.uint64(0x7ff)).astype(np.int64) - 1023
    m = ((b & np.uint64(0x000fffffffffffff)) | np.uint64(0x3ff0000000000000)).view(np.float64)
    big = m > 1.4142135623730951
    m = np.where(big, m * 0.5, m)
    e = e + big
    s = (m - 1.0) / (m + 1.0)
    w = s * s
    p = horner(w, [1.0 / k for k in range(23, 0, -2)])
    return e.astype(np.float64) * 0.6931471805599453 + 2.0 * (s * p)


def factorial(n):
    out = 1
    for i in range(2, n + 1):
        out *= i
    return out


def cos_turn(b):
    o = (b >> np.uint64(49)).astype(np.int64)
    rest = b & np.uint64((1 << 49) - 1)
    rest = np.where(o & 1, np.uint64((1 << 49) - 1) - rest, rest)
    x = (rest.astype(np.float64) + 0.5) * (0.7853981633974483 * (1.0 / float(1 << 49)))
    w = x * x
    sin_c = [(-1.0 if (k % 2) else 1.0) / float(factorial(2 * k + 1)) for k in range(9, -1, -1)]
    cos_c = [(-1.0 if (k % 2) else 1.0) / float(factorial(2 * k)) for k in range(9, -1, -1)]
    sin_v = x * horner(w, sin_c)
    cos_v = horner(w, cos_c)
    v = np.where(np.isin(o, (1, 2, 5, 6)), sin_v, cos_v)
    return np.where((o >= 2) & (o <= 5), -v, v)


def normal(key, index):
    index = np.asarray(index, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a = bits(key, np.uint64(2) * index) >> np.uint64(12)
        b = bits(key, np.uint64(2) * index + np.uint64(1)) >> np.uint64(12)
    u = (a.astype(np.float64) + 0.5) * (1.0 / float(1 << 52))
    r = np.sqrt(-2.0 * ln(u))
    return r * cos_turn(b)


def draw(seed, name, shape, role="matrix", std=0.02, start=0, count=None):
    """float32 values (int32 for role "int_table") of a tensor; a flat slice if count is given."""
    numel = int(np.prod(shape))
    whole = count is None and start == 0
    if count is None:
        count = numel - start
    index = np.arange(start, start + count, dtype=np.uint64)
    key = tensor_key(seed, name)
    if role == "int_table":
        out = (bits(key, index) >> np.uint64(49)).astype(np.int32)
    else:
        mean = 1.0 if role == "norm" else 0.0
        out = (mean + std * normal(key, index)).astype(np.float32)
    return out.reshape(shape) if whole else out
