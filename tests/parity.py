"""Error metrics shared by the parity tests.

`rel_err` is the reference's own definition (tests/wgpu_parity.rs:50-58): elementwise
|x-y| / max(1e-6, |x|, |y|), maximum over elements. It is the bar (1e-5) wherever the GPU keeps the
reference's operation order. Where the GPU reassociates a sum (time chunks of the scan, parallel
reductions), an element that is itself a near-cancellation of large terms has no meaningful
elementwise relative error -- the reference's own two CPU scans (ordered vs Blelloch,
src/gpu_batch.rs:543-575 vs 622-680) differ by more than 1e-5 under it, see
tests/test_oracle_kat.py::test_reference_cpu_scans_differ_elementwise_at_cancellations. For those
paths the bar is `chan_err` <= 1e-5: the error relative to the largest magnitude the same channel
reaches over time, plus the 99th percentile of the elementwise error (with 64 time chunks the oracle itself,
re-run in fp32 with the same chunking on the CPU, shows elementwise p99 = 5e-6, p99.9 = 5e-5, max = 5e-3 while
the per-channel-scale error is 3e-7: the tail is cancellation, not kernel error).
"""
import numpy as np

REL_TOL = 1e-5


def rel_elems(x, y):
    x = np.asarray(x, np.float64)
    y = np.asarray(y, np.float64)
    return np.abs(x - y) / np.maximum(1e-6, np.maximum(np.abs(x), np.abs(y)))


def rel_err(x, y) -> float:
    return float(np.max(rel_elems(x, y))) if np.size(x) else 0.0


def rel_p99(x, y) -> float:
    return float(np.quantile(rel_elems(x, y), 0.99)) if np.size(x) else 0.0


def chan_err(x, y, time_axis: int) -> float:
    """max |x-y| / max(1e-6, max over `time_axis` of |y|)."""
    x = np.asarray(x, np.float64)
    y = np.asarray(y, np.float64)
    scale = np.maximum(1e-6, np.max(np.abs(y), axis=time_axis, keepdims=True))
    return float(np.max(np.abs(x - y) / scale)) if x.size else 0.0


def worst(x, y):
    e = rel_elems(x, y)
    idx = np.unravel_index(int(np.argmax(e)), e.shape)
    return float(e[idx]), tuple(int(i) for i in idx)


def scale_err(x, y) -> float:
    """max |x-y| / max |y|: the bar for vectors whose entries are dot products (logits, features): an entry that
    happens to cancel to ~0 carries the absolute roundoff of its terms, so it is measured against the vector."""
    x = np.asarray(x, np.float64)
    y = np.asarray(y, np.float64)
    return float(np.max(np.abs(x - y)) / max(1e-30, np.max(np.abs(y)))) if x.size else 0.0
