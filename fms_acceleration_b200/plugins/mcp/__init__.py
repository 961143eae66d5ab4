"""Plugin package (filled in below)."""
