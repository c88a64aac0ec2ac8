"""Import-compatible face of the reference's ``modeling`` package, backed by ``allie_b200``."""
