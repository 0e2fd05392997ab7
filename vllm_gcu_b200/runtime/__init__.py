"""Adapters that plug this package into vLLM's own engine (platform plugin path)."""
