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


def test_pairing_by_overlap_is_a_permutation_and_saves_tiles():
    """plan.pair_rows_by_overlap on CPU tensors: every q-block appears once per slice, and the pairs it forms
    need fewer tiles (union of the two lists) than pairs of adjacent q-blocks on a Bernoulli mask."""
    import torch
    from paroatten_b200.plan import pair_rows_by_overlap
    g = torch.Generator().manual_seed(3)
    for nb in (9, 64, 131):
        m = (torch.rand(3, nb, nb, generator=g) < 0.25)
        m[:, torch.arange(nb), torch.arange(nb)] = True
        order = pair_rows_by_overlap(m.to(torch.uint8))
        assert order.shape == (3, nb)
        for s in range(3):
            assert sorted(order[s].tolist()) == list(range(nb))

        def tiles(rows):     # rows: [S, nb] order; pairs (rows[2p], rows[2p+1])
            mm = torch.gather(m, 1, rows.unsqueeze(-1).expand(-1, -1, nb))
            even, odd = mm[:, 0:2 * (nb // 2):2], mm[:, 1:2 * (nb // 2):2]
            t = (even | odd).sum().item()
            return t + (mm[:, nb - 1].sum().item() if nb % 2 else 0)

        adjacent = tiles(torch.arange(nb).expand(3, nb))
        assert tiles(order) <= adjacent
        if nb >= 64:
            assert tiles(order) < 0.99 * adjacent
