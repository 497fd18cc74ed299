"""Counter-based uniform numbers: u = f(seed, step).

The reference draws from one ``System.Random(seed)`` per request
(src/DotLLM.Engine/Samplers/SamplerPipeline.cs:57): two requests with the same seed see the same
stream.  Here the n-th draw of a request is a function of its seed and n alone, so a request's
samples do not depend on what else is in its batch, on its place in it, or on the order requests
are served in.  (A request without a seed gets one from the system's entropy.)
"""
from __future__ import annotations

_MASK = 0xFFFFFFFFFFFFFFFF


def _splitmix64(x):
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed, step):
    """A float in [0, 1) with 24 random bits (exact in float32)."""
    x = _splitmix64(int(seed) & _MASK)
    x = _splitmix64(x ^ ((int(step) + 1) * 0xA0761D6478BD642F & _MASK))
    return (x >> 40) / float(1 << 24)
