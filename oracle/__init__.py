"""CPU oracle of the sparse hot path - test infrastructure, never imported by the product."""
