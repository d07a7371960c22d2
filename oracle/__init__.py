"""CPU oracle of the hot path - test infrastructure, never imported by the shipped package."""
