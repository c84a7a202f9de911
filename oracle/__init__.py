"""CPU checkers for the hot path. Test infrastructure: the product never imports this package."""
