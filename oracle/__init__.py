"""CPU oracle for the fused norm ops: TEST INFRASTRUCTURE, never the product path.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
legs import this package.
"""
