"""Serving engine: paged KV, scheduling, sampling, speculative decoding."""
