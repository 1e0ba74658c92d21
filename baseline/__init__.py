"""Reference arm of the benchmark (the unmodified reference engine on the same job)."""
