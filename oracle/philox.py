"""Philox4x32-10 counter-based generator (test infrastructure, CPU oracle).

Restates the published Philox4x32-10 algorithm (Salmon et al., "Parallel
random numbers: as easy as 1, 2, 3", SC'11; the Random123 library).  The
reference has no Philox generator (its samplers call
``np.random.default_rng()``: verse_nex/cometspark.py:880,
verse_inference/sampler.py:64), so the stream layout below is this
project's definition, shared bit-for-bit with the CUDA acceptance kernel:

    key     = (seed & 0xffffffff, seed >> 32)
    counter = (position, row, purpose, offset)
    uniform = (word0 >> 8) * 2**-24            # float32 in [0, 1)

``purpose`` 0 is the accept/reject test of draft position ``position``;
``purpose`` 1 is the inverse-CDF draw for the token emitted at ``position``
(residual resample, or the bonus token when position == k).  ``offset`` is a
per-call counter so successive decoding rounds use fresh numbers.

Pinned by the Random123 known-answer vectors in tests/test_oracle.py.
"""

from __future__ import annotations

import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = np.uint32(0x9E3779B9)
_W1 = np.uint32(0xBB67AE85)
_MASK = np.uint64(0xFFFFFFFF)

PURPOSE_ACCEPT = 0
PURPOSE_SAMPLE = 1


def philox4x32_10(counter, key):
    """Vectorised Philox4x32-10.

    counter: array-like (..., 4) uint32; key: array-like (..., 2) uint32
    (broadcastable against counter's leading dims).  Returns (..., 4) uint32.
    """
    c = np.asarray(counter, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    c0, c1, c2, c3 = (c[..., i].astype(np.uint64) for i in range(4))
    k0 = np.broadcast_to(k[..., 0], c0.shape).astype(np.uint32)
    k1 = np.broadcast_to(k[..., 1], c0.shape).astype(np.uint32)
    with np.errstate(over="ignore"):
        for r in range(10):
            p0 = _M0 * c0
            p1 = _M1 * c2
            hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK
            hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK
            n0 = hi1 ^ c1 ^ k0.astype(np.uint64)
            n2 = hi0 ^ c3 ^ k1.astype(np.uint64)
            c0, c1, c2, c3 = n0, lo1, n2, lo0
            if r != 9:
                k0 = (k0 + _W0).astype(np.uint32)
                k1 = (k1 + _W1).astype(np.uint32)
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def uniform(seed: int, offset: int, row, position, purpose) -> np.ndarray:
    """float32 uniforms in [0,1) for (row, position, purpose) triples."""
    row, position, purpose = np.broadcast_arrays(
        np.asarray(row, dtype=np.uint32),
        np.asarray(position, dtype=np.uint32),
        np.asarray(purpose, dtype=np.uint32),
    )
    ctr = np.stack(
        [position, row, purpose, np.full(row.shape, offset & 0xFFFFFFFF, dtype=np.uint32)],
        axis=-1,
    )
    key = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint32)
    w0 = philox4x32_10(ctr, key)[..., 0]
    return ((w0 >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)).astype(np.float32)


def uniforms_for_call(seed: int, offset: int, batch: int, k: int):
    """(u_accept [B,k], u_sample [B,k+1]) for one acceptance call."""
    rows = np.arange(batch)[:, None]
    u_acc = uniform(seed, offset, rows, np.arange(k)[None, :], PURPOSE_ACCEPT)
    u_smp = uniform(seed, offset, rows, np.arange(k + 1)[None, :], PURPOSE_SAMPLE)
    return u_acc, u_smp
