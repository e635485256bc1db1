"""Stand-in for the reference's ``kernel`` package: same module and function names, this library underneath."""
