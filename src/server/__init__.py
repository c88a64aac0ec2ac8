"""Import-compatible face of the reference's ``server`` package."""
