"""Seeded synthetic operands, identical on the host and on the device.

The reference fills its test matrices with rand_init (uniform in [-1, 1],
reference src/util.cpp:259-267) and normalRandom (Box-Muller,
src/util.cpp:270-280) from the C library's rand(), which cannot be reproduced on
a GPU.  The benchmark configurations therefore use a counter-based generator:
element i of a stream is a function of (seed, i) only,

    u(seed, i) = (splitmix64(seed * 0x9E3779B97F4A7C15 + i) >> 40) * 2^-24,

uniform = 2 u - 1, Bernoulli mask = u(mask_seed, i) < density, normal = sigma *
sqrt(-2 ln u(seed, 2i)) * cos(2 pi u(seed, 2i + 1)).  The functions here compute
those streams with torch integer arithmetic on whatever device is asked for, so a
32768 x 32768 operand can be produced in HBM directly and still be equal, element
for element, to what a host loop over the same formula produces.
Seeds used by the benchmark configurations: A = 1, B = 2, sparsity mask = 3,
convolution input = 4, filters = 5.
"""
import torch

_GOLDEN = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB


def _s64(v):
    """A 64-bit pattern as the signed integer torch stores."""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(z, s):
    """Logical right shift of int64 lanes."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def _u24(seed, first, count, device):
    """The 24-bit integers splitmix64(seed * golden + i) >> 40 for i in [first, first + count)."""
    z = torch.arange(first, first + count, dtype=torch.int64, device=device)
    z += torch.tensor(_s64(seed * _GOLDEN + _GOLDEN), dtype=torch.int64, device=device)  # wraps modulo 2^64 like the unsigned sum
    z = (z ^ _lsr(z, 30)) * torch.tensor(_s64(_M1), dtype=torch.int64, device=device)
    z = (z ^ _lsr(z, 27)) * torch.tensor(_s64(_M2), dtype=torch.int64, device=device)
    z = z ^ _lsr(z, 31)
    return _lsr(z, 40)


def _chunks(total, step=1 << 26):
    for lo in range(0, total, step):
        yield lo, min(step, total - lo)


def uniform(shape, seed, device="cuda", out=None):
    """float32 uniform in [-1, 1): element i (row-major) is 2 u(seed, i) - 1."""
    n = 1
    for d in shape:
        n *= d
    x = torch.empty(n, dtype=torch.float32, device=device) if out is None else out.view(-1)
    for lo, cnt in _chunks(n):
        x[lo:lo + cnt] = _u24(seed, lo, cnt, device).to(torch.float32) * (1.0 / 16777216.0) * 2.0 - 1.0
    return x.view(*shape)


def sparse_uniform(shape, seed, mask_seed, density, device="cuda"):
    """uniform(seed) where u(mask_seed, i) < density, zero elsewhere."""
    n = 1
    for d in shape:
        n *= d
    x = torch.empty(n, dtype=torch.float32, device=device)
    for lo, cnt in _chunks(n):
        v = _u24(seed, lo, cnt, device).to(torch.float32) * (1.0 / 16777216.0) * 2.0 - 1.0
        m = (_u24(mask_seed, lo, cnt, device).to(torch.float32) * (1.0 / 16777216.0)).double() < density
        x[lo:lo + cnt] = torch.where(m, v, torch.zeros_like(v))
    return x.view(*shape)
