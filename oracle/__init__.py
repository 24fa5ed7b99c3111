"""CPU oracle of the quantized-linear path.  TEST INFRASTRUCTURE ONLY: imported by
tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline leg, never by the
product package."""
