"""Host-side helpers that need neither a GPU nor the CUDA library."""


def test_trace_summary_reads_a_fabricated_table():
    """paroatten_b200.trace_attention.summarise on a table with known segment lengths (no GPU)."""
    import numpy as np
    from paroatten_b200.trace_attention import EVENTS, ROLES, STEPS, summarise
    t = np.zeros((ROLES, STEPS, EVENTS), dtype=np.int64)
    for i in range(STEPS):
        base = 1000 + 2000 * i
        for r in (2, 3):       # two tiles per step: polls 100, issue 400 each, loop 1000
            t[r, i] = [base, base + 100, 0, base + 500, base + 500, base + 600, 0, base + 1000]
        for w in range(8):
            if (i & 1) == (w >> 2):
                t[4 + w, i, :6] = [base, base + 300, base + 380, base + 1500, base + 1700, base + 1800]
    text = summarise(t, 60, 150)
    assert "period 2000" in text
    assert "tile 0 polls 100, issue+commit 400; tile 1 polls 100, issue+commit 400; loop 1000" in text
    assert "softmax warp 5: waits for scores 300, TMEM load 80, exponentials 1120" in text
