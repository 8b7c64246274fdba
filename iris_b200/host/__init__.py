"""Host runtime: context, symmetric heap, distributed helpers, platform queries, tracing, logging."""
