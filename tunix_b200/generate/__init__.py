"""Text generation: tokenizer adapters, the KV-cached sampler, beam search and weight-transfer helpers."""
