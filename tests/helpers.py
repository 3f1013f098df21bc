"""Shared assertions for the parity tests."""

from __future__ import annotations

import torch

# Output tolerance of the forward path: max|err| <= 1e-2 * RMS(y_ref) on the fp32-accumulated
# value.  The result is then stored in the activation dtype, which by itself moves a value by
# up to half a unit in the last place of that dtype; the bound below adds exactly that.
OUT_TOL = 1e-2

# (label, max|err| / RMS(ref), how far the worst element is beyond its half-ulp allowance / RMS):
# filled by assert_output_close, printed at the end of the run so the margin under the
# tolerance is visible per case.
MARGINS: list[tuple[str, float, float]] = []


def half_ulp(ref64: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Half a unit in the last place of *dtype* at each |ref| (0 for fp32)."""
    if dtype == torch.float32:
        return torch.zeros_like(ref64)
    mant = 7 if dtype == torch.bfloat16 else 10
    a = ref64.abs().clamp_min(2.0 ** -14 if dtype == torch.float16 else 1e-30)
    return 0.5 * torch.exp2(torch.floor(torch.log2(a)) - mant)


def assert_output_close(y: torch.Tensor, ref64: torch.Tensor, dtype: torch.dtype, tol: float = OUT_TOL,
                        label: str | None = None):
    """|y - ref| <= tol * RMS(ref) + half an ulp of the output dtype, elementwise.  Returns
    max|err| / RMS(ref); with *label* the achieved figures are kept for the end-of-run table."""
    y = y.detach().cpu().double()
    ref64 = ref64.detach().cpu().double()
    assert y.shape == ref64.shape, (y.shape, ref64.shape)
    assert torch.isfinite(y).all()
    rms = float(torch.sqrt(torch.mean(ref64 * ref64)))
    err = (y - ref64).abs()
    bound = tol * rms + half_ulp(ref64, dtype)
    worst = float((err - bound).max())
    if label is not None:
        beyond = float((err - half_ulp(ref64, dtype)).clamp_min(0).max()) / max(rms, 1e-30)
        MARGINS.append((label, float(err.max()) / max(rms, 1e-30), beyond))
    assert worst <= 0, (
        f"max|err|={float(err.max()):.4g}, RMS(ref)={rms:.4g}, "
        f"max|err|/RMS={float(err.max()) / max(rms, 1e-30):.4g} exceeds the bound by {worst:.3g}"
    )
    return float(err.max()) / max(rms, 1e-30)
