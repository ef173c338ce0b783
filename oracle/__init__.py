"""CPU oracles for the hot path — test infrastructure, never imported by the product package."""
