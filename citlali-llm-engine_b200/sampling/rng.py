"""The uniform numbers temperature sampling draws: a counter-based generator keyed by
(seed, request index, index of the generated token).  A sequence's draws depend on nothing
else, so which other sequences share its batch, which slot it got and how many steps came
before cannot change them."""
from __future__ import annotations

_MASK = 0xFFFFFFFFFFFFFFFF


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, request: int, token_index: int) -> float:
    """A float in [0, 1) with 24 random bits (exactly representable in float32)."""
    h = _splitmix64(seed & _MASK)
    h = _splitmix64(h ^ ((request + 1) * 0xD1342543DE82EF95 & _MASK))
    h = _splitmix64(h ^ ((token_index + 1) * 0xA0761D6478BD642F & _MASK))
    return (h >> 40) / float(1 << 24)
