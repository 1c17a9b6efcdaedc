"""CPU oracle (test infrastructure only): see nvfp4_oracle.py."""
