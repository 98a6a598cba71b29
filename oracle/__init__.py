"""CPU oracles for DSQG attention: test infrastructure, never imported by dwarf_b200."""
