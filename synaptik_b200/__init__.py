"""B200 (sm_100a) CUDA backend for Synaptik: C-ABI shim plus the Python mirror of its callers."""
