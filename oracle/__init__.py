"""CPU checker for the CUDA backend (test infrastructure only; see oracle.py)."""
