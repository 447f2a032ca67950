"""Tolerances of the half-precision (bf16 / W4A16) paths, shared by the GPU parity tests.

The stated bar for logits is rtol 2e-2.  A logit is a d-term dot product whose terms largely cancel, so the
error that bf16 operand rounding and a different summation order leave on it does not shrink with the logit's
own magnitude: it scales with the typical magnitude of the row's logits.  A pure relative test would therefore
fail every logit that happens to land near zero.  The absolute floor used here is the same 2e-2 applied to
the root-mean-square logit of the row: |got - ref| <= 2e-2 * (|ref| + rms(ref_row))."""
import numpy as np

LOGIT_RTOL = 2e-2


def logit_band(ref, rtol=LOGIT_RTOL):
    """Per-element allowance for a [rows, vocab] logit matrix."""
    ref = np.asarray(ref, np.float64)
    rms = np.sqrt((ref * ref).mean(axis=1, keepdims=True))
    return rtol * (np.abs(ref) + rms)


def check_logits(got, ref, rtol=LOGIT_RTOL, what=""):
    """Assert the bar and return the worst error as a fraction of its allowance (for reporting)."""
    band = logit_band(ref, rtol)
    err = np.abs(np.asarray(got, np.float64) - np.asarray(ref, np.float64))
    worst = float((err / band).max())
    assert worst <= 1.0, (what, worst)
    return worst


def clear_winner(ref, rtol=LOGIT_RTOL):
    """Rows whose arg-max leads the runner-up by more than both allowances together: their greedy token must match."""
    ref = np.asarray(ref, np.float64)
    band = logit_band(ref, rtol)
    order = np.argsort(ref, axis=1)
    rows = np.arange(ref.shape[0])
    top, second = order[:, -1], order[:, -2]
    return (ref[rows, top] - ref[rows, second]) > (band[rows, top] + band[rows, second])
