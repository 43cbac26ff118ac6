"""Fit the odd polynomial used by adop_atan_core() in adop_math.h.

atan(x) ~= x + x^3 * (c0 + c1 z + c2 z^2 + c3 z^3 + c4 z^4),  z = x^2,  |x| <= tan(pi/8).
Least squares on Chebyshev nodes in float64; prints the coefficients and the max relative error.
Run:  python tests/golden/fit_atan_poly.py
"""
import numpy as np

def main():
    xmax = np.tan(np.pi / 8) * 1.0001
    k = np.arange(4000)
    x = xmax * np.cos(np.pi * (k + 0.5) / 4000)
    x = x[np.abs(x) > 1e-6]
    z = x * x
    target = (np.arctan(x) - x) / x**3
    A = np.stack([z**i for i in range(5)], axis=1)
    # weight by x^3/atan(x) so the fit minimises relative error of the final value
    w = np.abs(x**3 / np.arctan(x))
    c, *_ = np.linalg.lstsq(A * w[:, None], target * w, rcond=None)
    approx = x + x**3 * (A @ c)
    err = np.max(np.abs(approx / np.arctan(x) - 1))
    for i, ci in enumerate(c):
        print(f"c{i} = {np.float32(ci)!r:>16}  ({ci:.12e})")
    print("max rel err (f64 eval):", err)

if __name__ == "__main__":
    main()
