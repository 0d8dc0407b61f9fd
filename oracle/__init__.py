"""CPU restatement of the reference's block-sparse attention path.  TEST INFRASTRUCTURE ONLY: it may be
imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline leg, never by the product."""
