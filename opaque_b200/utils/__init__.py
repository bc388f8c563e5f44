"""Build helpers and small utilities shared by the package."""
