"""Stand-in for flash-linear-attention's package root (only the entry the reference calls)."""
