"""Shared helpers of the parity tests: seeded inputs, fp16 comparison rules, metric log."""
import json
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_METRICS = {}


def record(name, **kw):
    """Keeps the measured errors of the GPU parity tests in parity_metrics.json in the folder NEUS2B_METRICS_DIR names
    (nothing is written when the variable is unset)."""
    out = os.environ.get("NEUS2B_METRICS_DIR")
    if not out:
        return
    path = os.path.join(out, "parity_metrics.json")
    if not _METRICS and os.path.exists(path):
        try:
            _METRICS.update(json.load(open(path)))
        except (OSError, ValueError):
            pass
    _METRICS[name] = {k: (float(v) if np.isscalar(v) else v) for k, v in kw.items()}
    try:
        os.makedirs(out, exist_ok=True)
        with open(path, "w") as f:
            json.dump(_METRICS, f, indent=1, sort_keys=True)
    except OSError:
        pass


def cosine(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-300))


def fp16_close_fraction(a, b, rel=1e-3):
    """Fraction of elements with |a-b| <= rel*|b| + rel*rms(b) (fp16 tensors computed with a different fp32
    summation order differ by an ulp here and there, and an element that cancels to ~0 has no relative scale of its
    own)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    rms = np.sqrt(np.mean(b * b)) + 1e-30
    return float((np.abs(a - b) <= rel * np.abs(b) + rel * rms).mean())


def check_fp16(name, a, b, rel=1e-3, min_frac=0.999, min_cos=0.9999):
    frac, c, r = fp16_close_fraction(a, b, rel), cosine(a, b), rel_l2(a, b)
    record(name, frac_within=frac, cosine=c, rel_l2=r)
    assert frac >= min_frac, (name, "fraction within %g relative" % rel, frac, "cos", c, "rel_l2", r)
    assert c >= min_cos, (name, "cosine", c)


def check_grad(name, got, ref, min_cos=0.999, max_rel=None):
    c, r = cosine(got, ref), rel_l2(got, ref)
    record(name, cosine=c, rel_l2=r)
    assert c >= min_cos, (name, "cosine", c, "rel_l2", r)
    if max_rel is not None:
        assert r <= max_rel, (name, "rel_l2", r)


def model(O, seed=0, n=4096, L=16, log2T=19, base=16, scale=1.447, grid_amp=0.1, n_active=None, mlp_amp=None):
    """Seeded parameters (fp16 bit patterns) + coordinates for a NeuS model of the given grid geometry."""
    rng = np.random.default_rng(seed)
    d = O.grid_desc(n_levels=L, log2_hashmap_size=log2T, base_resolution=base, per_level_scale=scale, n_active_levels=n_active)
    ng = O.grid_n_params(d)
    p = np.zeros(O.model_n_params(d), np.float32)
    off = 0
    for (o, i) in ((64, 48), (16, 64), (64, 48), (64, 64), (16, 64)):
        lim = mlp_amp if mlp_amp is not None else np.sqrt(6.0 / (o + i))
        p[off:off + o * i] = rng.uniform(-lim, lim, o * i)
        off += o * i
    p[O.GRID_OFF:O.GRID_OFF + ng] = rng.uniform(-grid_amp, grid_amp, ng)
    p[O.GRID_OFF + ng:] = 0.3
    coords = np.zeros((n, 7), np.float32)
    coords[:, :3] = rng.random((n, 3), dtype=np.float32)
    coords[:, 3] = rng.random(n, dtype=np.float32) * 0.01
    coords[:, 4:] = rng.random((n, 3), dtype=np.float32)
    return d, O.f16_bits(p), coords, rng


def to_lib_desc(L, d):
    return L.GridDesc(d.n_levels, d.log2_hashmap_size, d.base_resolution, d.per_level_scale, d.n_active_levels)

