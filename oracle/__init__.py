"""CPU oracle of the fused embedding-bag forward: test infrastructure only (see oracle/eb_oracle.c)."""
