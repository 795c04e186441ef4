"""Shared comparison helpers for the parity tests."""
from __future__ import annotations

import numpy as np

TIE_EPS = 1e-6       # a differing code is a tie when the rotated coordinate is this close to a boundary
MAX_TIE_RATE = 1e-5  # parity bar for packed codes and sign bits on full-size inputs


def code_mismatches(orc, packed, packed_ref, rotated, boundaries, bits, dim):
    """Returns (mismatch_rate, worst_distance_to_boundary).  Asserts that every differing code is a
    neighbouring bin and sits within TIE_EPS of a decision boundary of the ORACLE's coordinates."""
    a = orc.unpack_codes(np.ascontiguousarray(packed), bits, dim)
    b = orc.unpack_codes(np.ascontiguousarray(packed_ref), bits, dim)
    bad = np.argwhere(a != b)
    worst = 0.0
    for r, j in bad:
        dist = float(np.min(np.abs(boundaries.astype(np.float64) - float(rotated[r, j]))))
        assert dist < TIE_EPS, f"row {r} dim {j}: codes {a[r, j]} vs {b[r, j]} at {dist:.3e} from a boundary"
        assert abs(int(a[r, j]) - int(b[r, j])) == 1
        worst = max(worst, dist)
    return len(bad) / max(a.size, 1), worst


def attention_close(out, ref, max_abs=1e-2, min_cos=0.9999):
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = float(np.abs(out - ref).max())
    cos = float((out * ref).sum() / np.sqrt((out * out).sum() * (ref * ref).sum()))
    assert err <= max_abs, f"max-abs {err:.3e} > {max_abs}"
    assert cos >= min_cos, f"cosine {cos:.6f} < {min_cos}"
    return err, cos


def topk_ids_match(ids, ref_ids, all_scores, rel_tie=4e-6):
    """ids equal, or every disagreement is between scores closer than float32 summation noise."""
    ids, ref_ids = np.asarray(ids), np.asarray(ref_ids)
    ties = 0
    for qi in range(ids.shape[0]):
        if np.array_equal(ids[qi], ref_ids[qi]):
            continue
        for a, b in zip(ids[qi], ref_ids[qi]):
            if a != b:
                sa, sb = all_scores[qi, a], all_scores[qi, b]
                assert abs(sa - sb) <= rel_tie * max(abs(sa), abs(sb)), (qi, a, b, sa, sb)
                ties += 1
    return ties
