"""Weight loading and artifact tooling for the quantized-linear path."""
