"""Seeded random blocks of the sibling formats (test data; any bytes are valid blocks as long
as the fp16 fields are finite)."""
import numpy as np

STRIDES = {1: (20, 36), 2: (22, 34), 3: (24, 36)}  # (weight, activation) block bytes


def _scales(rng, shape, lo, hi):
    return rng.uniform(lo, hi, size=shape).astype(np.float16).view(np.uint8).reshape(*shape, 2)


def make(fmt, nr, nc, nb, seed):
    """(weights (nr, nb*wb) uint8, activations (nc, nb*ab) uint8)."""
    rng = np.random.default_rng(seed)
    wb, ab = STRIDES[fmt]
    w = rng.integers(0, 256, size=(nr, nb, wb), dtype=np.uint8)
    w[:, :, 0:2] = _scales(rng, (nr, nb), 0.001, 0.05)
    if fmt in (1, 3):
        w[:, :, 2:4] = _scales(rng, (nr, nb), -0.5, 0.5)  # the per-block minimum
    x = rng.integers(0, 256, size=(nc, nb, ab), dtype=np.uint8)
    d = rng.uniform(0.005, 0.05, size=(nc, nb)).astype(np.float16)
    x[:, :, 0:2] = d.view(np.uint8).reshape(nc, nb, 2)
    if ab == 36:  # block_q8_1: s = d * sum(q), stored as fp16
        q = x[:, :, 4:36].view(np.int8).astype(np.int32).sum(axis=2)
        s = (d.astype(np.float32) * q.astype(np.float32)).astype(np.float16)
        x[:, :, 2:4] = s.view(np.uint8).reshape(nc, nb, 2)
    return w.reshape(nr, nb * wb), x.reshape(nc, nb * ab)


def block_sums_numpy(fmt, w_row, x_row):
    """Independent integer stage in numpy (no C): int32 per block."""
    wb, ab = STRIDES[fmt]
    w = w_row.reshape(-1, wb).astype(np.int64)
    x = x_row.reshape(-1, ab)
    wq, aq, qh_off = {1: (4, 4, None), 2: (6, 2, 2), 3: (8, 4, 4)}[fmt]
    qs = w[:, wq:wq + 16]
    lo, hi = qs & 15, qs >> 4
    if qh_off is not None:
        qh = w[:, qh_off] | (w[:, qh_off + 1] << 8) | (w[:, qh_off + 2] << 16) | (w[:, qh_off + 3] << 24)
        j = np.arange(16)
        lo = lo | (((qh[:, None] >> j) & 1) << 4)
        hi = hi | (((qh[:, None] >> (j + 16)) & 1) << 4)
    if fmt == 2:
        lo, hi = lo - 16, hi - 16
    y = x[:, aq:aq + 32].view(np.int8).astype(np.int64)
    return (lo * y[:, :16] + hi * y[:, 16:]).sum(axis=1).astype(np.int32)
