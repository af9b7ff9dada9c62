"""Shared builders for the GPU parity tests: seeded logical caches, permuted page tables, tolerances."""
import numpy as np

# north_star tolerance for bf16 attention outputs
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def have_gpu():
    try:
        from relux_b200 import lib as L
        import ctypes as C
        n = C.c_int32()
        return L.load().relux_cuda_device_count(C.byref(n)) == 0 and n.value > 0
    except Exception:
        return False


def check_attention(got, ref, what="", bf16_output=False, max_tol=MAX_ABS_TOL, mean_tol=MEAN_ABS_TOL):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    if bf16_output:
        # an output stored as bf16 carries half an ulp (2^-8 relative) of its own magnitude
        err = np.maximum(err - np.abs(ref) * 2.0 ** -8, 0.0)
    rel = np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30)
    assert np.isfinite(got).all(), "%s: non-finite output" % what
    assert err.max() <= max_tol, "%s: max-abs %g > %g (rel %g)" % (what, err.max(), max_tol, rel)
    assert err.mean() <= mean_tol, "%s: mean-abs %g > %g (rel %g)" % (what, err.mean(), mean_tol, rel)
    # the outputs are small numbers; the relative error gives the check teeth
    assert rel <= 5e-2, "%s: relative error %g" % (what, rel)
    return err.max(), err.mean(), rel


def permuted_tables(rng, n_seqs, pages_per_seq, num_pages=None):
    num_pages = num_pages or n_seqs * pages_per_seq
    perm = rng.permutation(num_pages).astype(np.int32)
    return perm[: n_seqs * pages_per_seq].reshape(n_seqs, pages_per_seq)


def ragged_to_padded(rows, lens, width_shape):
    """rows: [sum(lens), ...] -> [B, max(lens), ...] zero padded."""
    B, Tm = len(lens), int(max(lens))
    out = np.zeros((B, Tm) + tuple(width_shape), rows.dtype)
    o = 0
    for b, n in enumerate(lens):
        out[b, :n] = rows[o:o + n]
        o += n
    return out
