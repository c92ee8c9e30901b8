"""CPU oracle for the UltraQuant verify-attention path (test infrastructure only)."""
