"""Elementwise acceptance of 16-bit attention outputs against the fp64 oracle.

The bound every element must hold is 2e-3 abs + 1e-2 rel against the exact
(fp64) result.  The reference's GPU kernels round the probabilities P and the
score gradients dS to the I/O dtype before the second GEMM of each product and
take delta from the rounded O; with bf16 (8 bits) and key sets of a few dozen
tokens that rounding alone moves single elements past the bound (the oracle's
`roundings="reference"` mode, exact arithmetic plus exactly those roundings,
shows 7 to 14 such elements per 43 200 on the shortest lists tested).  So an
element may pass the plain bound only by what those roundings can contribute in
the worst case, element by element (the oracle's first-order `envelope`), and the
error of a whole tensor may not be larger, in the root mean square, than the
error of the reference's rounding recipe itself.  No fraction of elements is
exempt and no bound is multiplied.
"""

import numpy as np

ATOL, RTOL = 2e-3, 1e-2


def rel_err(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return np.abs(got - want) / (ATOL + RTOL * np.abs(want))


def check_rounded(got, exact, rounded, envelope, what=""):
    """`got` (GPU) against `exact` (fp64 oracle); `rounded` = the oracle with the
    reference's roundings, `envelope` = worst-case contribution of those
    roundings per element.  Returns the number of elements beyond the plain
    bound (for reports)."""
    got = np.asarray(got, np.float64)
    exact = np.asarray(exact, np.float64)
    fin = np.isfinite(exact)
    assert (np.isfinite(got) == fin).all(), f"{what}: finiteness differs"
    err = np.abs(got[fin] - exact[fin])
    tol = ATOL + RTOL * np.abs(exact[fin])
    over = err > tol + np.asarray(envelope, np.float64)[fin]
    assert not over.any(), (f"{what}: {int(over.sum())} elements beyond bound + rounding envelope, "
                            f"worst {float((err / tol).max()):.2f} x bound")
    mine = np.sqrt(np.mean((err / tol) ** 2)) if err.size else 0.0
    ref = np.sqrt(np.mean(rel_err(np.asarray(rounded)[fin], exact[fin]) ** 2)) if err.size else 0.0
    assert mine <= 1.2 * ref + 3e-3, (f"{what}: rms error {mine:.4f} of the bound, the reference's "
                                      f"rounding recipe gives {ref:.4f}")
    return int((err > tol).sum())


def attention_oracles(orc, x, merged, H, g, kvb, dtype, o_gpu, q_padding=(0, 0),
                      kv_padding=(0, 0), kx=None, vx=None):
    """Exact results, reference-rounded results and envelopes for O, dQ, dK, dV
    (per query head; fold grouped kv heads with `fold_groups`).  `o_gpu` is the
    stored forward output the gradient kernels took delta from."""
    k = x["k"] if kx is None else kx
    v = x["v"] if vx is None else vx
    a = (x["q"], k, v, merged, H, g, kvb, None, q_padding, kv_padding)
    wo, wl = orc.sparse_attn_fwd(*a)
    ro, _, eo = orc.sparse_attn_fwd(*a, roundings="reference", io_dtype=dtype, envelope=True)
    b = (merged, H, g, kvb, None, q_padding, kv_padding)
    wq, wk, wv = orc.sparse_attn_bwd(x["q"], k, v, o_gpu, wl, x["do"], *b)
    rq, rk, rv, (eq, ek, ev) = orc.sparse_attn_bwd(
        x["q"], k, v, ro, wl, x["do"], *b, roundings="reference", io_dtype=dtype, envelope=True,
        o_envelope=eo)
    return dict(lse=wl, exact=dict(O=wo, dQ=wq, dK=wk, dV=wv), rounded=dict(O=ro, dQ=rq, dK=rk, dV=rv),
                envelope=dict(O=eo, dQ=eq, dK=ek, dV=ev))
