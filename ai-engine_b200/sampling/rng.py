"""The uniform draw of a request's n-th token: Philox4x32-10 keyed by the
request's seed, counter = n.  The reference re-seeds its generator on every call
(crates/ai-engine-runtime/src/sample.rs:41), so every step of a request draws
the same number; a counter-based generator keeps the seed's meaning (same seed,
same tokens) without that, and a request that is preempted and recomputed draws
the same numbers again."""
from __future__ import annotations

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32(counter: int, key: int):
    c = [(counter >> (32 * i)) & _MASK for i in range(4)]
    k0, k1 = key & _MASK, (key >> 32) & _MASK
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c[3] ^ k1) & _MASK, p0 & _MASK]
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c


def uniform(seed: int, n: int) -> float:
    """A float32-representable number in [0, 1) for the n-th draw of `seed`."""
    return (philox4x32(n, seed)[0] >> 8) * (1.0 / (1 << 24))
