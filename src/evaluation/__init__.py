"""Import-compatible face of the reference's ``evaluation`` package."""
