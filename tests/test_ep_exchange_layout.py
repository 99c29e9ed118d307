"""The receive-buffer layout of the peer-memory exchange, as restated in torch
(deepgemm.ep_exchange.layout_from_counts; the GPU tests hold dg_ep_plan to it): for random counts
tables every rank derives a consistent view -- each expert's block starts on a multiple of the
alignment, the ranges of the source ranks inside a block follow one another without gap or
overlap, and m_indices names exactly the rows in use."""
import torch

from deepgemm.ep_exchange import layout_from_counts


def test_layouts_of_all_ranks_are_consistent():
    gen = torch.Generator().manual_seed(11)
    for world, experts, align in ((1, 4, 256), (2, 8, 256), (4, 16, 128), (8, 64, 256)):
        e_local = experts // world
        counts = torch.randint(0, 700, (world, experts), generator=gen)
        counts[:, 1] = 0                                        # an expert nobody routes to
        views = [layout_from_counts(counts, r, align) for r in range(world)]
        tot = counts.sum(dim=0)
        for owner in range(world):
            m_indices, m_total = views[owner][1], views[owner][2]
            assert m_total % align == 0 and m_indices.numel() == m_total
            row = 0
            for el in range(e_local):
                e = owner * e_local + el
                assert row % align == 0
                # source ranks in order, back to back, starting at the block's first row
                for s in range(world):
                    assert int(views[s][0][e]) == row + int(counts[:s, e].sum())
                block = (int(tot[e]) + align - 1) // align * align
                assert bool((m_indices[row:row + int(tot[e])] == el).all())
                assert bool((m_indices[row + int(tot[e]):row + block] == -1).all())
                row += block
            assert row == m_total
