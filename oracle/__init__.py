"""CPU oracle for the compressed-weight path: test infrastructure, not product code."""
