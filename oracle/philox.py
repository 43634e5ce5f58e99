"""TEST INFRASTRUCTURE ONLY — CPU oracle for the dropout bits.

Philox-4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",
SC'11), restated in numpy. The reference draws its dropout bits with Triton's `tl.rand`
(jax_flash_attn2/flash_attention_triton/_forward_triton.py:140-143), itself a Philox-4x32-10;
bit-equality with Triton's stream is not a requirement of the build, reproducibility from the
seed is. The mapping used by the CUDA kernels and restated here:

    counter = (key_index // 8, query_index, batch * heads_q_global + head, 0)
    key     = (seed & 0xffffffff, seed >> 32)
    word    = output[(key_index % 8) // 2]
    draw    = word & 0xffff if key_index is even else word >> 16        (16 bits)
    keep    = draw >= min(round(p * 2**16), 65535)

One call thus serves eight adjacent keys of a query row, and the drop probability is realised in
steps of 2**-16.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module.
"""
from __future__ import annotations

import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Vectorised Philox-4x32-10. c0..c3: uint32 arrays (broadcastable); k0, k1: python ints.
    Returns four uint32 arrays."""
    c0, c1, c2, c3 = np.broadcast_arrays(*(np.asarray(c, dtype=np.uint64) for c in (c0, c1, c2, c3)))
    for r in range(10):
        kk0 = np.uint64((k0 + r * _W0) & 0xFFFFFFFF)
        kk1 = np.uint64((k1 + r * _W1) & 0xFFFFFFFF)
        p0 = _M0 * c0
        p1 = _M1 * c2
        n0 = (p1 >> np.uint64(32)) ^ c1 ^ kk0
        n1 = p1 & _MASK
        n2 = (p0 >> np.uint64(32)) ^ c3 ^ kk1
        n3 = p0 & _MASK
        c0, c1, c2, c3 = n0, n1, n2, n3
    return tuple(c.astype(np.uint32) for c in (c0, c1, c2, c3))


def dropout_threshold(p: float) -> int:
    thr = int(np.floor(float(np.float32(p)) * 65536.0 + 0.5))
    return min(thr, 0xFFFF)


def keep_mask(seed: int, p: float, batch: int, heads: int, sq: int, sk: int,
              batch_offset: int = 0, head_offset: int = 0, heads_q_global: int | None = None) -> np.ndarray:
    """Boolean keep mask [batch, heads, sq, sk] for dropout probability p."""
    hq_glob = heads if heads_q_global is None else heads_q_global
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    thr = np.uint32(dropout_threshold(p))
    n8 = (sk + 7) // 8
    out = np.empty((batch, heads, sq, n8 * 8), dtype=bool)
    c0 = np.arange(n8, dtype=np.uint32)[None, :]
    c1 = np.arange(sq, dtype=np.uint32)[:, None]
    for b in range(batch):
        for h in range(heads):
            bh = (batch_offset + b) * hq_glob + head_offset + h
            r = philox4x32_10(c0, c1, np.uint32(bh), np.uint32(0), k0, k1)
            halves = []
            for word in r:                       # key % 8 = 2 * word index + (0: low, 1: high half)
                halves += [word & np.uint32(0xFFFF), word >> np.uint32(16)]
            draws = np.stack(halves, axis=-1).reshape(sq, n8 * 8)
            out[b, h] = draws >= thr
    return out[..., :sk]
