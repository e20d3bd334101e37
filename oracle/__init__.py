"""CPU oracle of the paged KV-cache path: test infrastructure only (see tk_oracle.h)."""
