"""CPU checker for the TN GEMM path.  TEST INFRASTRUCTURE ONLY: imported by tests/,
__graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py, never by the
product package."""
