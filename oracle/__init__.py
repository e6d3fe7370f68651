"""CPU oracle of the wide-row hot path: test infrastructure, never imported by credit_b200."""
