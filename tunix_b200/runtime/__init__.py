"""Host runtime: native helpers (packing, parallel reads, asynchronous writes) with Python fallbacks."""
