"""CPU oracle of the per-step token loop — test infrastructure, never part of the product path."""
