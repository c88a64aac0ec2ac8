"""Import stand-in (see package docstring)."""
