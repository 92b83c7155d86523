"""Index arithmetic of the one-launch reduction kernels, restated in NumPy: the partial-row layout, the tickets and
the fixed-order folds of csrc/kernels/norm_bwd_onepass.cu and csrc/kernels/colsum_fused.cu give the plain column sums
for any order in which the CTAs finish, and leave their counters at zero."""
import numpy as np
import pytest


@pytest.mark.parametrize("C,rms", [(8, False), (16, True), (768, False), (1024, True)])
def test_norm_backward_group_folds(C, rms):
    ctas, per_group, groups = 148, 4, 37
    rng = np.random.default_rng(C)
    w2 = C if rms else 2 * C
    part = rng.standard_normal((ctas, 2 * C)).astype(np.float32)          # what each CTA holds after its warp fold
    for trial in range(3):
        scratch = np.full((ctas + groups) * 2 * C, np.nan, np.float32)
        counters = np.zeros(1 + groups, np.uint32)
        dw, db = np.zeros(C, np.float32), np.zeros(C, np.float32)
        finals = 0
        for b in rng.permutation(ctas):
            scratch[b * 2 * C: b * 2 * C + w2] = part[b, :w2]
            g = b // per_group
            ticket = counters[1 + g]
            counters[1 + g] += 1
            if ticket != per_group - 1:
                continue
            base, first = ctas * 2 * C, g * per_group * 2 * C
            for c in range(0, w2, 4):
                t = scratch[first + c: first + c + 4].copy()
                for j in range(1, per_group):
                    t += scratch[first + j * 2 * C + c: first + j * 2 * C + c + 4]
                scratch[base + g * 2 * C + c: base + g * 2 * C + c + 4] = t
            counters[1 + g] = 0
            ticket = counters[0]
            counters[0] += 1
            if ticket != groups - 1:
                continue
            finals += 1
            for c in range(0, w2, 4):
                t = scratch[base + c: base + c + 4].copy()
                for j in range(1, groups):
                    t += scratch[base + j * 2 * C + c: base + j * 2 * C + c + 4]
                if c < C:
                    dw[c:c + 4] = t
                else:
                    db[c - C:c - C + 4] = t
            counters[0] = 0
        assert finals == 1 and not counters.any()
        assert np.allclose(dw, part[:, :C].sum(0), atol=2e-3)
        if not rms:
            assert np.allclose(db, part[:, C:].sum(0), atol=2e-3)


@pytest.mark.parametrize("rows,C,vn", [(8192, 768, 8), (1000, 2304, 8), (37, 264, 8), (5, 8, 4), (4099, 132, 4)])
def test_column_sum_partition_and_fold(rows, C, vn):
    w = 32 * vn                                   # columns per strip
    strips = (C + w - 1) // w
    parts = min((148 * 4 + strips - 1) // strips, (rows + 31) // 32, 256)
    parts = max(parts, 1)
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, C)).astype(np.float32)
    scratch = np.full((parts, C), np.nan, np.float32)
    counters = np.zeros(strips, np.uint32)
    out = np.zeros(C, np.float32)
    seen = np.zeros(rows, np.int32)
    blocks = [(s, p) for s in range(strips) for p in range(parts)]
    for s, p in (blocks[i] for i in rng.permutation(len(blocks))):
        c0 = s * w
        acc = np.zeros((8, w), np.float32)
        step = parts * 8
        for ty in range(8):
            r = p * 8 + ty
            while r < rows:
                if s == 0:
                    seen[r] += 1
                cols = min(w, C - c0)
                acc[ty, :cols] += x[r, c0:c0 + cols]
                r += step
        cols = min(w, C - c0)
        scratch[p, c0:c0 + cols] = acc.sum(0)[:cols]
        ticket = counters[s]
        counters[s] += 1
        if ticket != parts - 1:
            continue
        fold = np.zeros((8, w), np.float32)
        for ty in range(8):
            for q in range(ty, parts, 8):
                fold[ty, :cols] += scratch[q, c0:c0 + cols]
        out[c0:c0 + cols] = fold.sum(0)[:cols]
        counters[s] = 0
    assert (seen == 1).all() and not counters.any()
    assert np.allclose(out, x.sum(0), atol=1e-2)
