"""CPU oracle of the hinge tree evaluation path: test infrastructure, never part of the product."""
