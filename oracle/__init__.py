"""CPU restatement of the reference's GEMM path. TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline leg import it, and only as the checker or the reported baseline.
"""
