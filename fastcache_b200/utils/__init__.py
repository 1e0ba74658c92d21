"""Process-wide helpers: step context, weight loading, memory queries, streams, tracing, watchdogs."""
