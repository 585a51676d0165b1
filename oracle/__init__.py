"""CPU oracle for the lm2exp / lt2exp hot path.  TEST INFRASTRUCTURE ONLY: imported by tests/, by
__graft_entry__.smoke() and by bench.py's CPU-baseline legs, never by the triturus_b200 package."""
