"""Error statistics for comparing a 16-bit result with the oracle's.

Test infrastructure, like the rest of this folder: only tests/, the smoke check and the
benchmark's CPU legs import it.  For a 16-bit attention result the maximum absolute error
alone hides how close the bulk of the elements is, so the comparison reports three figures:
the max-abs error, how many elements exceed the stated tolerance, and the share of elements
within one unit in the last place of the expected value.
"""
import torch

_MANTISSA_BITS = {torch.bfloat16: 7, torch.float16: 10, torch.float32: 23}


def ulp_of(want: torch.Tensor) -> torch.Tensor:
    """Spacing of `want`'s dtype at each of its values (as float64); the spacing at the
    smallest normal number for zeros and subnormals."""
    bits = _MANTISSA_BITS[want.dtype]
    fi = torch.finfo(want.dtype)
    mag = want.double().abs().clamp(min=fi.tiny)
    return torch.exp2(torch.floor(torch.log2(mag)) - bits)


def report(got: torch.Tensor, want: torch.Tensor, tol: float = 2e-2) -> dict:
    """{'max_abs', 'over_tol', 'within_1ulp', 'bit_equal', 'n'} for got vs want (same shape;
    NaNs must coincide and are left out of the figures)."""
    got, want = got.detach().cpu(), want.detach().cpu()
    assert got.shape == want.shape, (tuple(got.shape), tuple(want.shape))
    g, w = got.double(), want.double()
    nan = torch.isnan(w)
    assert torch.equal(torch.isnan(g), nan), "NaN pattern differs"
    err = (g - w).abs().masked_fill(nan, 0.0)
    n = int(want.numel())
    if n == 0:
        return {"max_abs": 0.0, "over_tol": 0, "within_1ulp": 1.0, "bit_equal": 1.0, "n": 0}
    return {"max_abs": float(err.max()), "over_tol": int((err > tol).sum()),
            "within_1ulp": float((err <= ulp_of(want)).double().mean()),
            "bit_equal": float((err == 0).double().mean()), "n": n}


def fmt(r: dict) -> str:
    return (f"max-abs {r['max_abs']:.3e}, {r['over_tol']} of {r['n']} over tolerance, "
            f"{100 * r['within_1ulp']:.2f}% within 1 ulp, {100 * r['bit_equal']:.2f}% bit-equal")
