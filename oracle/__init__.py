"""CPU restatement of the reference algorithm.  Test infrastructure only: nothing
that ships imports this package (see semblo_oracle.py for the parity status)."""
