"""CPU oracle of the Vesta GPT-2 decode step. TEST INFRASTRUCTURE ONLY: imported by tests/,
by __graft_entry__.smoke() and by bench.py's CPU-baseline legs as the checker and the timed
baseline; never by the product path (vesta_gpu_b200)."""
