"""CPU checkers for the SOCKET decode path (test infrastructure, not a product path)."""
