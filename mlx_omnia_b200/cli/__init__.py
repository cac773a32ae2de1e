"""The `omnia` command line."""
