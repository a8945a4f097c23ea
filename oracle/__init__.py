"""Test-only CPU checkers for the sparse-MLA path (never imported by the shipped package)."""
