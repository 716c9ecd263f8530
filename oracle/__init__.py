"""CPU oracle of the paged KV path: test infrastructure, never imported by the product."""
