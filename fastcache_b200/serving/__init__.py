"""Serving layer: HTTP server, load-test harness, command lines, datasets, analytic profiler."""
