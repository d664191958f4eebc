"""CPU oracle (test infrastructure): see oracle.c for the parity status."""
