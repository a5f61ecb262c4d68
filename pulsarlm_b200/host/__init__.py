"""Python face of the C++ host core (page pools, block tables, scheduler decisions)."""
