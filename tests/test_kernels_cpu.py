

def test_grouped_layout_capacity_bound_drops_the_overflow_and_counts_it():
    """Rows past the capacity bound are dropped (dest_row -1), counted, and the expert ranges are clipped to the buffer."""
    import torch

    from lm_engine.ops.moe import TILE, build_grouped_layout

    torch.manual_seed(0)
    experts = torch.randint(0, 8, (9000,), dtype=torch.int32)
    free = build_grouped_layout(experts, 8, first_expert=4, num_local_experts=4)
    assert int(free.dropped.item()) == 0 and (free.dest_row >= 0).sum().item() == ((experts >= 4).sum().item())
    bound = build_grouped_layout(experts, 8, first_expert=4, num_local_experts=4, capacity_rows=3000)
    assert bound.rows == 3072 and bound.rows % TILE == 0
    placed = int((bound.dest_row >= 0).sum().item())
    assert placed + int(bound.dropped.item()) == int((experts >= 4).sum().item()) and int(bound.dropped.item()) > 0
    assert int(bound.dest_row.max().item()) < bound.rows and int(bound.padded_offsets[-1].item()) <= bound.rows
    # every placed entry is found again through src_entry, and the kept prefix matches the unbounded layout
    rows = bound.dest_row[bound.dest_row >= 0].long()
    assert torch.equal(bound.src_entry[rows].long(), torch.nonzero(bound.dest_row >= 0).flatten())
    keep = bound.dest_row >= 0
    assert torch.equal(bound.dest_row[keep], free.dest_row[keep])
