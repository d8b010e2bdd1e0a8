"""CPU oracle for the scatter path.  Test infrastructure, never a product path."""
