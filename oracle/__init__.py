"""CPU checker for g4b_b200 (test infrastructure; never imported by the product)."""
