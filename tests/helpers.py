"""Shared test helpers: seeded synthetic inputs with the value distributions of the
benchmark configurations, and numpy <-> device plumbing."""
import numpy as np

try:
    import torch
except Exception:  # pragma: no cover
    torch = None


def rand_q4(rng, rows, bpr, dist="baseline"):
    """Random Q4_0 planes.  'baseline': nibbles U{0..15}, d = fp16(|N(0, 0.02)|);
    'ref': d ~ U(0.002, 0.03) as the reference's GEMM tests use."""
    qs = rng.integers(0, 256, size=(rows, bpr, 16), dtype=np.uint8)
    if dist == "ref":
        d = rng.uniform(0.002, 0.03, size=(rows, bpr)).astype(np.float16)
    else:
        d = np.abs(rng.normal(0.0, 0.02, size=(rows, bpr))).astype(np.float16)
    return qs, d.view(np.uint16)


def act_floats(rng, n, outliers=True):
    """~N(0,1) with a few x8 outliers (the reference's activation generator)."""
    v = rng.standard_normal(n).astype(np.float32)
    if outliers:
        m = rng.integers(0, 64, size=n) == 0
        v[m] *= 8.0
    return v


def dev(a):
    """numpy array -> CUDA tensor with the same bytes (structured/uint16 go as uint8/int16 views)."""
    a = np.ascontiguousarray(a)
    if a.dtype.fields is not None or a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32).copy()).cuda()
    return torch.from_numpy(a.copy()).cuda()


def host(t, dtype=None, shape=None):
    a = t.detach().cpu().numpy()
    if dtype is not None:
        a = a.view(np.uint8).reshape(-1).view(dtype)
    if shape is not None:
        a = a.reshape(shape)
    return a


def empty_blocks(n):
    """Device buffer for n 36-byte Q8_1 blocks, poisoned."""
    return torch.full((n * 36,), 0x5A, dtype=torch.uint8, device="cuda")


def nan_f32(*shape):
    return torch.full(shape, float("nan"), dtype=torch.float32, device="cuda")


def ulp_diff(a, b):
    """Distance in float32 units-in-the-last-place (same-sign finite values)."""
    ai = np.asarray(a, np.float32).view(np.int32).astype(np.int64)
    bi = np.asarray(b, np.float32).view(np.int32).astype(np.int64)
    return np.abs(ai - bi)


def zipf_bias(rng, n_exp=64, s=1.1, scale=1.0):
    """Router-logit bias that skews the load: log of a Zipf(s) law over a fixed
    random permutation of the experts."""
    ranks = rng.permutation(n_exp) + 1
    p = 1.0 / ranks.astype(np.float64) ** s
    p /= p.sum()
    return (scale * (np.log(p) - np.log(p).mean())).astype(np.float32)
