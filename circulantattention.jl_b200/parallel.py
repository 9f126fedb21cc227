"""Multi-GPU plumbing (filled in below)."""
