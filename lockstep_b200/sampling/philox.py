"""Counter-based random numbers keyed on (seed, request id, position) and nothing else
(LockStep: engine/sampler/philox.py).  Philox-4x32 with ten rounds, multipliers
0xD2511F53 / 0xCD9E8D57 and Weyl increments 0x9E3779B9 / 0xBB67AE85; the draw
for a position is word 0 of the block with counter (pos_lo, pos_hi, index, 0) and
key seed ^ sha256(uid)[:8], times 2^-32.  The device sampler computes the same
words (csrc/sampling.cu)."""

from __future__ import annotations

import hashlib

_M32 = 0xFFFFFFFF
ROUNDS = 10


def uid_key(uid: str) -> int:
    return int.from_bytes(hashlib.sha256(uid.encode("utf-8")).digest()[:8], "big")


def key_words(seed: int, uid: str) -> tuple[int, int]:
    """(low, high) 32-bit words of the request's Philox key."""
    mixed = (int(seed) ^ uid_key(uid)) & 0xFFFFFFFFFFFFFFFF
    return mixed & _M32, (mixed >> 32) & _M32


def philox_4x32(counter, key, rounds: int = ROUNDS):
    c0, c1, c2, c3 = (int(x) & _M32 for x in counter)
    k0, k1 = (int(x) & _M32 for x in key)
    for r in range(rounds):
        p0, p1 = 0xD2511F53 * c0, 0xCD9E8D57 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _M32, p1 & _M32, ((p0 >> 32) ^ c3 ^ k1) & _M32, p0 & _M32
        if r < rounds - 1:
            k0, k1 = (k0 + 0x9E3779B9) & _M32, (k1 + 0xBB67AE85) & _M32
    return c0, c1, c2, c3


def uniform(seed: int, uid: str, position: int, index: int = 0) -> float:
    words = philox_4x32((position & _M32, (position >> 32) & _M32, index & _M32, 0), key_words(seed, uid))
    return words[0] * 2.0 ** -32
