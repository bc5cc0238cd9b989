"""TEST INFRASTRUCTURE: CPU oracles for the attention path.  Nothing under af3_kernels_b200/
imports this package; only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs do."""
