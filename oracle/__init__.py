"""CPU oracle of the MoE hot path: test infrastructure, never imported by the product package."""
