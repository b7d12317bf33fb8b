"""CPU oracle of the augmentation hot path — test infrastructure, never imported by the product."""
