"""Op-level and model-level benchmark drivers (run as `python -m benchmarks.<name>` from the repository root)."""
