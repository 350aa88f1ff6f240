"""Test-only CPU checkers for the compound-optree path (never imported by the product)."""
