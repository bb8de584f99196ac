"""Fixtures for the tests and the benchmark (synthetic quantised models, a GGUF writer).  Nothing in the product path
(backend.py, tp.py, csrc/) imports this package."""
