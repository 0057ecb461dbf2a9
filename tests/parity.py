"""Parity metrics shared by the GPU tests.

``headline`` is max|x - ref| / max|ref|, the tolerance the benchmark specification
states for y and the final state (1e-3 with bf16 inputs and fp32 accumulation).
``stats`` reports the per-tensor statistics of the reference's trace comparer
(crates/rwkv-test/src/main.rs:343-375).
"""
import numpy as np

BF16_ULP = 2.0 ** -8  # spacing of bf16 relative to the value (upper bound)


def headline(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))


def stats(x, ref, rel_eps=1e-12):
    x = np.asarray(x, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    d = np.abs(x - ref)
    rel = d / np.maximum(np.abs(ref), rel_eps)
    cos = float(x @ ref / max(np.linalg.norm(x) * np.linalg.norm(ref), 1e-300))
    return dict(max_abs=float(d.max()), mean_abs=float(d.mean()), max_rel=float(rel.max()),
                mean_rel=float(rel.mean()), cosine=cos)


def assert_close_f32(x, ref, tol=1e-3, what=""):
    """fp32 storage: headline error within ``tol`` and cosine >= 0.99999."""
    h = headline(x, ref)
    assert h <= tol, f"{what}: headline error {h:.3e} > {tol:.1e}"
    assert stats(x, ref)["cosine"] >= 0.99999, what


def assert_close_bf16_store(x, ref, tol=1e-3, what=""):
    """bf16 storage of an fp32 result: the arithmetic must be within ``tol`` of the
    reference in the headline norm; rounding the result to bf16 adds at most one
    bf16 spacing of the value itself."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    bound = tol * np.abs(ref).max() + BF16_ULP * np.abs(ref)
    bad = np.abs(x - ref) > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} elements beyond {tol:.1e}*max + 1 bf16 ulp; " \
                          f"headline {headline(x, ref):.3e}"
