"""CPU oracle for the rosa_soft operator family (test infrastructure only)."""
