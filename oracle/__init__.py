"""CPU oracle (test infrastructure only): see oracle/duq_oracle.c and oracle/oracle.py."""
