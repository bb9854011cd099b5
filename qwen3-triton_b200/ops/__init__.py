"""Stand-alone operator package (same public names as the reference ops/triton)."""
