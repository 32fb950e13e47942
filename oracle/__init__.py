"""CPU checker for the MLA decode path (test infrastructure, never product code)."""
