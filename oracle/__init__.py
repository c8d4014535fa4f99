"""CPU oracle of the AlignedKV decode hot path (test infrastructure only; never imported by the product)."""
